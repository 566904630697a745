// Kernel body and host launch of the tensor-core attention backward. Included by attention_bwd_tc.cu only.
#pragma once

// One CTA's work: work item `item` of the dQ kernel (MODE_DQ) or of the dK/dV kernel (MODE_DKV).
template <typename T, int D, int MODE>
__device__ __forceinline__ void bwd_cta(const CUtensorMap& map_x1, const CUtensorMap& map_x2, const CUtensorMap& map_y1,
                                        const CUtensorMap& map_y2, T* __restrict__ out1, T* __restrict__ out2,
                                        const float* __restrict__ lse2_t, const float* __restrict__ delta_t, const AttnDims& dm,
                                        int accumulate, unsigned int* __restrict__ status, unsigned long long* trace, int item,
                                        int items) {
    using L = BwdSmem<D>;
    extern __shared__ unsigned char bwd_smem_raw[];
    const std::uint32_t raw = smem_u32(bwd_smem_raw);
    const std::uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
    if (pad > static_cast<std::uint32_t>(L::kAlignSlack)) {   // uniform over the CTA; nothing is allocated or armed yet
        if (threadIdx.x == 0) atomicExch(status, 2u);
        return;
    }
    unsigned char* smem = bwd_smem_raw + pad;
    std::uint64_t* bar = reinterpret_cast<std::uint64_t*>(smem + L::kBars);
    BwdBars bars;
    bars.x_full = bar + 0;
    constexpr int kYStages = L::kStages;
    bars.y_full = bar + 1;                      // [kYStages]
    bars.stat_full = bar + 1 + kYStages;        // [kYStages]
    bars.y_free = bar + 1 + 2 * kYStages;       // [kYStages]
    bars.uw_free = bar + 1 + 3 * kYStages;      // [1]
    constexpr int kTBufs = BwdTmem<D, MODE>::kTBufs;
    bars.t_full = bars.uw_free + 1;             // [3]
    bars.w_full = bars.uw_free + 4;             // [3]
    bars.acc_done = bars.uw_free + 7;
    static_assert((1 + 3 * kYStages + 8) * 8 + 4 <= 256, "barrier area");
    bars.trace = (trace != nullptr && item == items / 4) ? trace : nullptr;
    std::uint32_t* tmem_slot = reinterpret_cast<std::uint32_t*>(bars.acc_done + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // 1-D grid, heaviest tiles first over ALL (head, batch) pairs: CTAs start in blockIdx order, so the light tiles of
    // the causal triangle fill the tail of the launch instead of a heavy tile starting last.
    const int heads_here = MODE == MODE_DQ ? dm.hq : dm.hkv;
    const int pairs = heads_here * dm.batch;
    const int tile_rank = item / pairs;           // 0 = most streaming tiles
    const int pair = item % pairs;
    BwdGeom g;
    g.b = pair / heads_here;
    g.ratio = dm.hq / dm.hkv;
    g.i0 = 0;
    g.n_q = 0;
    if (MODE == MODE_DQ) {
        const int q_tiles = (dm.sq + kRows - 1) / kRows;
        g.x0 = (q_tiles - 1 - tile_rank) * kRows;   // the last query tile sees the most keys
        g.h = pair % heads_here;
        g.kvh = g.h / g.ratio;
        int q_last = g.x0 + kRows - 1;
        if (q_last > dm.sq - 1) q_last = dm.sq - 1;
        int last_key = dm.causal ? dm.offset + q_last : dm.sk - 1;
        if (last_key > dm.sk - 1) last_key = dm.sk - 1;
        g.n_it = last_key / kCols + 1;
    } else {
        g.x0 = tile_rank * kRows;                   // the first key tile is seen by the most queries (causal)
        g.kvh = pair % heads_here;
        g.h = g.kvh * g.ratio;
        int first_q = dm.causal ? g.x0 - dm.offset : 0;
        if (first_q < 0) first_q = 0;
        g.i0 = first_q / kCols;
        g.n_q = (dm.sq - 1) / kCols - g.i0 + 1;
        if (g.n_q < 0) g.n_q = 0;
        g.n_it = g.ratio * g.n_q;
    }

    if (threadIdx.x == 0) {
        mbar_init(bars.x_full, 1);
        for (int s = 0; s < kYStages; ++s) {
            mbar_init(&bars.y_full[s], 1);
            mbar_init(&bars.stat_full[s], 32);
            mbar_init(&bars.y_free[s], 1);
        }
        mbar_init(bars.uw_free, 1);
        for (int s = 0; s < kTBufs; ++s) {
            mbar_init(&bars.t_full[s], 1);
            mbar_init(&bars.w_full[s], kRows);          // the 128 threads of the warpgroup that took the tile arrive
        }
        mbar_init(bars.acc_done, 1);
        mbar_init_fence();
        tma_prefetch_desc(&map_x1); tma_prefetch_desc(&map_x2); tma_prefetch_desc(&map_y1); tma_prefetch_desc(&map_y2);
    }
    if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const std::uint32_t tmem = *tmem_slot;

    bool ok = true;
    if (warp == 8) {
        if (g.n_it > 0) ok = bwd_producer<D, MODE>(smem, bars, g, dm, &map_x1, &map_x2, &map_y1, &map_y2, lse2_t, delta_t, lane);
    } else if (warp == 9) {
        if (lane == 0 && g.n_it > 0) ok = bwd_mma_issuer<T, D, MODE>(smem, bars, g, tmem);
    } else {
        ok = bwd_compute<T, D, MODE>(smem, bars, g, dm, tmem, lse2_t, delta_t, out1, out2, accumulate);
    }
    if (!ok) {
        atomicExch(status, 2u);
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

template <typename T, int D, int MODE>
__global__ void __launch_bounds__(kBwdThreads, 1)
attention_bwd_tc_kernel(const __grid_constant__ CUtensorMap map_x1, const __grid_constant__ CUtensorMap map_x2,
                        const __grid_constant__ CUtensorMap map_y1, const __grid_constant__ CUtensorMap map_y2,
                        T* __restrict__ out1, T* __restrict__ out2, const float* __restrict__ lse2_t,
                        const float* __restrict__ delta_t, AttnDims dm, int accumulate, unsigned int* __restrict__ status,
                        unsigned long long* trace) {
    bwd_cta<T, D, MODE>(map_x1, map_x2, map_y1, map_y2, out1, out2, lse2_t, delta_t, dm, accumulate, status, trace,
                        static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x));
}

// dK/dV and dQ in ONE launch: the first items_kv CTAs are the (few, long) dK/dV items, the rest the (many, short) dQ
// items, each list heaviest first. The short dQ items fill the SMs that the last wave of dK/dV items would leave idle,
// and one launch tail replaces two.
template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attention_bwd_tc_both_kernel(const __grid_constant__ CUtensorMap k128, const __grid_constant__ CUtensorMap v128,
                             const __grid_constant__ CUtensorMap q64, const __grid_constant__ CUtensorMap do64,
                             const __grid_constant__ CUtensorMap q128, const __grid_constant__ CUtensorMap do128,
                             const __grid_constant__ CUtensorMap k64, const __grid_constant__ CUtensorMap v64, T* __restrict__ dq,
                             T* __restrict__ dk, T* __restrict__ dv, const float* __restrict__ lse2_t,
                             const float* __restrict__ delta_t, AttnDims dm, int items_kv, int accumulate,
                             unsigned int* __restrict__ status) {
    const int item = static_cast<int>(blockIdx.x);
    if (item < items_kv) {
        bwd_cta<T, D, MODE_DKV>(k128, v128, q64, do64, dk, dv, lse2_t, delta_t, dm, accumulate, status, nullptr, item, items_kv);
    } else {
        bwd_cta<T, D, MODE_DQ>(q128, do128, k64, v64, dq, static_cast<T*>(nullptr), lse2_t, delta_t, dm, accumulate, status, nullptr,
                               item - items_kv, static_cast<int>(gridDim.x) - items_kv);
    }
}

// 4D tensor map over a [batch, seq, heads, D] tensor: box = 64 columns x 1 head x `rows` positions.
inline int make_bshd_map_rows(CUtensorMap* map, const void* base, int dtype, int batch, int seq, int heads, int d, int rows) {
    const std::uint64_t dims[4] = {static_cast<std::uint64_t>(d), static_cast<std::uint64_t>(heads), static_cast<std::uint64_t>(seq),
                                   static_cast<std::uint64_t>(batch)};
    const std::uint64_t strides[3] = {static_cast<std::uint64_t>(d) * 2, static_cast<std::uint64_t>(heads) * d * 2,
                                      static_cast<std::uint64_t>(seq) * heads * d * 2};
    const std::uint32_t box[4] = {64, 1, static_cast<std::uint32_t>(rows), 1};
    return make_tensor_map(map, dtype, base, 4, dims, strides, box);
}

template <typename T, int D>
int launch_backward(void* dq, void* dk, void* dv, const void* dout, const void* out, const float* lse, const void* q,
                    const void* k, const void* v, const AttnDims& dm, int accumulate, int dtype, cudaStream_t s) {
    using L = BwdSmem<D>;
    const long long qrows = static_cast<long long>(dm.batch) * dm.sq * dm.hq;
    void* scratch = nullptr;
    CGPT_TRY(scratch_get(&scratch, static_cast<std::size_t>(qrows) * 2 * sizeof(float), s));
    float* delta_t = static_cast<float*>(scratch);
    float* lse2_t = delta_t + qrows;
    if (qrows >= (1ll << 31)) return CGPT_ERR_UNSUPPORTED;      // 32-bit row indices in the preparation pass
    const long long prep_rows_per_cta = 8LL * (32 / (D / 8)) * kPrepUnroll;
    const long long prep_need = (qrows + prep_rows_per_cta - 1) / prep_rows_per_cta;
    const long long prep_cap = static_cast<long long>(kNumSMs) *
                               resident_ctas_per_sm(reinterpret_cast<const void*>(attention_bwd_prep_kernel<T, D>), 256, 0);
    attention_bwd_prep_kernel<T, D><<<static_cast<unsigned>(prep_need < prep_cap ? prep_need : prep_cap), 256, 0, s>>>(
        delta_t, lse2_t, static_cast<const T*>(dout), static_cast<const T*>(out), lse, static_cast<unsigned>(qrows), dm.sq, dm.hq,
        FastDiv(static_cast<unsigned>(dm.hq)), FastDiv(static_cast<unsigned>(dm.sq)));
    count_launch();
    CGPT_LAUNCH_CHECK();

    CUtensorMap q128, do128, k64, v64, k128, v128, q64, do64;
    CGPT_TRY(make_bshd_map_rows(&q128, q, dtype, dm.batch, dm.sq, dm.hq, D, kRows));
    CGPT_TRY(make_bshd_map_rows(&do128, dout, dtype, dm.batch, dm.sq, dm.hq, D, kRows));
    CGPT_TRY(make_bshd_map_rows(&k64, k, dtype, dm.batch, dm.sk, dm.hkv, D, kCols));
    CGPT_TRY(make_bshd_map_rows(&v64, v, dtype, dm.batch, dm.sk, dm.hkv, D, kCols));
    CGPT_TRY(make_bshd_map_rows(&k128, k, dtype, dm.batch, dm.sk, dm.hkv, D, kRows));
    CGPT_TRY(make_bshd_map_rows(&v128, v, dtype, dm.batch, dm.sk, dm.hkv, D, kRows));
    CGPT_TRY(make_bshd_map_rows(&q64, q, dtype, dm.batch, dm.sq, dm.hq, D, kCols));
    CGPT_TRY(make_bshd_map_rows(&do64, dout, dtype, dm.batch, dm.sq, dm.hq, D, kCols));

    auto kq = attention_bwd_tc_kernel<T, D, MODE_DQ>;
    auto kkv = attention_bwd_tc_kernel<T, D, MODE_DKV>;
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
        CGPT_CUDA_TRY(cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
        attr_once.done();
    }
    unsigned int* status = tc_status_device_ptr();
    if (status == nullptr) return CGPT_ERR_STATE;
    const int items_q = ((dm.sq + kRows - 1) / kRows) * dm.hq * dm.batch;
    const int items_kv = ((dm.sk + kRows - 1) / kRows) * dm.hkv * dm.batch;
    static const bool split_launches = [] { const char* e = diagnosis_env("CGPT_B200_ATTN_SPLIT"); return e && e[0] == '1'; }();
    if (!split_launches && diagnosis_env("CGPT_B200_ATTN_TRACE") == nullptr) {
        auto kboth = attention_bwd_tc_both_kernel<T, D>;
        static PerDeviceOnce both_once;
        if (both_once.needed()) {
            CGPT_CUDA_TRY(cudaFuncSetAttribute(kboth, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
            both_once.done();
        }
        kboth<<<static_cast<unsigned>(items_q + items_kv), kBwdThreads, L::kBytes, s>>>(
            k128, v128, q64, do64, q128, do128, k64, v64, static_cast<T*>(dq), static_cast<T*>(dk), static_cast<T*>(dv), lse2_t, delta_t, dm,
            items_kv, accumulate, status);
        count_launch();
        CGPT_LAUNCH_CHECK();
        return CGPT_OK;
    }
    const dim3 grid_q(static_cast<unsigned>(items_q));
    // Diagnosis builds only: CGPT_B200_ATTN_TRACE=<device pointer of 2*64*8 uint64> records per-iteration timestamps of one
    // CTA per kernel. The shipped build never takes a pointer from the environment.
    unsigned long long* trace = nullptr;
    if (const char* e = diagnosis_env("CGPT_B200_ATTN_TRACE")) trace = reinterpret_cast<unsigned long long*>(std::strtoull(e, nullptr, 0));
    kq<<<grid_q, kBwdThreads, L::kBytes, s>>>(q128, do128, k64, v64, static_cast<T*>(dq), static_cast<T*>(nullptr), lse2_t, delta_t, dm,
                                              accumulate, status, trace);
    count_launch();
    CGPT_LAUNCH_CHECK();
    const dim3 grid_kv(static_cast<unsigned>(((dm.sk + kRows - 1) / kRows) * dm.hkv * dm.batch));
    kkv<<<grid_kv, kBwdThreads, L::kBytes, s>>>(k128, v128, q64, do64, static_cast<T*>(dk), static_cast<T*>(dv), lse2_t, delta_t, dm,
                                                accumulate, status, trace ? trace + 64 * 8 : nullptr);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}
