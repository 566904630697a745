// Persistent variant of the tcgen05 GEMM. Included by gemm.cu only (inside its anonymous namespace).
//
// One CTA per SM walks a list of work units (output tile x K split). The TMA ring and its phase counters
// run on across units; the fp32 accumulator is double-buffered in TMEM (2 x BN columns) so that the four
// epilogue warps drain tile j (tcgen05.ld -> convert -> global stores) while the MMA warp already
// accumulates tile j+1. Units are ordered tile_n fastest so that CTAs running at the same time share the
// same rows of A through L2.
#pragma once

// One 32-column chunk of an accumulator row -> global memory.
template <typename T>
__device__ __forceinline__ void gemm_store_chunk(const std::uint32_t (&r)[32], T* __restrict__ C, float* __restrict__ partial,
                                                 int row, int col0, int M, int N, int split, int epilogue) {
    if (row >= M || col0 >= N || epilogue == 3) return;
    if (epilogue == kEpiPartial) {
        float* dst = partial + (static_cast<long long>(split) * M + row) * N + col0;
        if (col0 + 32 <= N && (N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                  __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < N) dst[j] = __uint_as_float(r[j]);
        }
        return;
    }
    T* dst = C + static_cast<long long>(row) * N + col0;
    if (col0 + 32 <= N && (N & 7) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
            if (epilogue == kEpiAccumulate) {
                float old[8];
                load_vec<T, 8>(old, dst + j);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += old[e];
            }
            store_vec<T, 8>(dst + j, v);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (col0 + j < N) {
                float v = __uint_as_float(r[j]);
                if (epilogue == kEpiAccumulate) v += to_f32<T>(dst[j]);
                dst[j] = from_f32<T>(v);
            }
        }
    }
}

// Operands of C = sum_i A_i * B_i: up to kMaxKSegments (A_i, B_i) pairs that share M and N and are chained along K
// (the input gradient of several projections that read the same input: dX = dQ Wq + dK Wk + dV Wv in one pass).
// Segment i covers K blocks [kb_end[i-1], kb_end[i]); a segment whose K is not a multiple of BK is zero-filled by TMA.
constexpr int kMaxKSegments = 3;
struct GemmOperands {
    CUtensorMap a[kMaxKSegments];
    CUtensorMap b[kMaxKSegments];
    int kb_end[kMaxKSegments];
    int segments;
    // Output groups (exclusive with K segments): several products that share A, each with its own B_g and C_g, run as
    // one launch (Q, K and V projections of the same input). The N tiles of the groups are numbered consecutively;
    // group g owns tiles [tile_end[g-1], tile_end[g]). groups == 1: the plain case.
    int groups;
    int group_dim;                 // 0: groups split the N tiles (own B_g, C_g); 1: they split the M tiles (own A_g, C_g)
    int tile_end[kMaxKSegments];
};
struct GemmOutputs {
    CUtensorMap c[kMaxKSegments];   // TMA-store maps, one per output group
};

template <typename T, int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ GemmOperands ops, const __grid_constant__ GemmOutputs outs,
                               T* __restrict__ C, float* __restrict__ partial, int M, int N, int total_kb, int tiles_m,
                               int tiles_n, int splits, int kb_per_split, int epilogue) {
    using Cfg = GemmCfg<BN>;
    extern __shared__ unsigned char gemm_smem_raw[];
    const std::uint32_t raw = smem_u32(gemm_smem_raw);
    unsigned char* smem = gemm_smem_raw + ((1024u - (raw & 1023u)) & 1023u);
    unsigned char* staging = smem + Cfg::kStages * Cfg::kStageBytes;   // kStoreBufs x [128 rows][128 B], 1024-byte aligned
    std::uint64_t* bars = reinterpret_cast<std::uint64_t*>(staging + Cfg::kStoreBufs * BM * 128);
    std::uint64_t* full = bars;
    std::uint64_t* empty = bars + Cfg::kStages;
    std::uint64_t* acc_full = bars + 2 * Cfg::kStages;       // [2]
    std::uint64_t* acc_empty = bars + 2 * Cfg::kStages + 2;  // [2]
    std::uint32_t* tmem_slot = reinterpret_cast<std::uint32_t*>(bars + 2 * Cfg::kStages + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles = tiles_m * tiles_n;
    const int units = tiles * splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        mbar_init_fence();
        for (int i = 0; i < ops.segments; ++i) { tma_prefetch_desc(&ops.a[i]); tma_prefetch_desc(&ops.b[i]); }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const std::uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int u = blockIdx.x; u < units && !failed; u += gridDim.x) {
                const int split = u / tiles, t = u % tiles;
                const int tile_m = t / tiles_n, tile_n = t % tiles_n;
                const int kb_begin = split * kb_per_split;
                int nkb = total_kb - kb_begin;
                if (nkb > kb_per_split) nkb = kb_per_split;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % Cfg::kStages;
                    const std::uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1u)) { failed = true; break; }
                    mbar_expect_tx(&full[s], Cfg::kStageBytes);
                    unsigned char* a_dst = smem + s * Cfg::kStageBytes;
                    unsigned char* b_dst = a_dst + Cfg::kABytes;
                    const int kb = kb_begin + i;
                    int seg = 0, kb_first = 0;
                    if (ops.segments > 1 && kb >= ops.kb_end[0]) { seg = 1; kb_first = ops.kb_end[0]; }
                    if (ops.segments > 2 && kb >= ops.kb_end[1]) { seg = 2; kb_first = ops.kb_end[1]; }
                    const int tile_g = ops.group_dim ? tile_m : tile_n;
                    int group = 0, tile_first = 0;
                    if (ops.groups > 1 && tile_g >= ops.tile_end[0]) { group = 1; tile_first = ops.tile_end[0]; }
                    if (ops.groups > 2 && tile_g >= ops.tile_end[1]) { group = 2; tile_first = ops.tile_end[1]; }
                    const int tile_n_b = ops.group_dim ? tile_n : tile_n - tile_first;   // N tile inside the group's own B
                    const int tile_m_a = ops.group_dim ? tile_m - tile_first : tile_m;   // M tile inside the group's own A
                    const CUtensorMap* tmap_a = &ops.a[ops.groups > 1 ? group : seg];
                    const CUtensorMap* tmap_b = &ops.b[ops.groups > 1 ? group : seg];
                    const int k0 = (kb - kb_first) * BK;
                    if (!A_MN) {
                        tma_load_2d(a_dst, tmap_a, &full[s], k0, tile_m_a * BM);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), tmap_a, &full[s], tile_m_a * BM + j * 64, k0);
                    }
                    if (!B_MN) {
                        tma_load_2d(b_dst, tmap_b, &full[s], k0, tile_n_b * BN);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), tmap_b, &full[s], tile_n_b * BN + j * 64, k0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr std::uint32_t idesc = idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
            int it = 0, j = 0;
            for (int u = blockIdx.x; u < units && !failed; u += gridDim.x, ++j) {
                const int split = u / tiles;
                const int kb_begin = split * kb_per_split;
                int nkb = total_kb - kb_begin;
                if (nkb > kb_per_split) nkb = kb_per_split;
                const int buf = j & 1;
                if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1u)) { failed = true; break; }
                tc_fence_after_sync();
                const std::uint32_t tmem_acc = tmem_base + buf * BN;
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % Cfg::kStages;
                    const std::uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!mbar_wait(&full[s], ph)) { failed = true; break; }
                    tc_fence_after_sync();
                    const std::uint32_t a_base = smem_u32(smem + s * Cfg::kStageBytes);
                    const std::uint32_t b_base = a_base + Cfg::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const std::uint64_t adesc = A_MN ? smem_desc_sw128(a_base + k * (UMMA_K * 128), BK * 128, 1024)
                                                         : smem_desc_sw128(a_base + k * (UMMA_K * 2), 16, 1024);
                        const std::uint64_t bdesc = B_MN ? smem_desc_sw128(b_base + k * (UMMA_K * 128), BK * 128, 1024)
                                                         : smem_desc_sw128(b_base + k * (UMMA_K * 2), 16, 1024);
                        mma_f16_ss(tmem_acc, adesc, bdesc, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(&empty[s]);
                }
                tc_commit(&acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;
        int j = 0;
        int stage_buf = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, ++j) {
            const int split = u / tiles, t = u % tiles;
            const int tile_m = t / tiles_n, tile_n = t % tiles_n;
            const int buf = j & 1;
            if (!mbar_wait(&acc_full[buf], (j >> 1) & 1)) failed = true;
            failed = __any_sync(0xffffffffu, failed);
            if (failed) break;
            tc_fence_after_sync();
            const int row = tile_m * BM + quarter * 32 + lane;
            const std::uint32_t tmem_acc = tmem_base + buf * BN + (static_cast<std::uint32_t>(quarter * 32) << 16);
            if (epilogue == kEpiStoreTma || epilogue == kEpiStageOnly || epilogue == kEpiStoreTmaFixed) {
                // Stage 64 columns of the tile as 16-bit values in 128B-swizzled shared memory and let TMA write
                // them out as full lines (a direct store would give every lane a different row: 16-byte pieces).
                const int et = threadIdx.x - 64;              // 0..127 within the epilogue warps
                const int trow = quarter * 32 + lane;         // row inside the tile
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    unsigned char* buf_s = staging + stage_buf * (BM * 128);
                    if (et == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // buffer used 2 stores ago is free
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    std::uint32_t r0[32], r1[32];
                    tmem_ld_32x32_x2(tmem_acc + c0, r0, tmem_acc + c0 + 32, r1);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const std::uint32_t* src = j < 4 ? &r0[8 * j] : &r1[8 * (j - 4)];
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(src[e]);
                        store_vec<T, 8>(reinterpret_cast<T*>(buf_s + trow * 128 + ((j ^ (trow & 7)) << 4)), v);
                    }
                    fence_proxy_async_smem();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (et == 0 && epilogue != kEpiStageOnly) {
                        const bool fixed = epilogue == kEpiStoreTmaFixed;   // diagnosis: every store lands on the same 16 KB
                        const int tile_g = ops.group_dim ? tile_m : tile_n;
                        int group = 0, tile_first = 0;
                        if (ops.groups > 1 && tile_g >= ops.tile_end[0]) { group = 1; tile_first = ops.tile_end[0]; }
                        if (ops.groups > 2 && tile_g >= ops.tile_end[1]) { group = 2; tile_first = ops.tile_end[1]; }
                        const int cx = (ops.group_dim ? tile_n : tile_n - tile_first) * BN + c0;
                        const int cy = (ops.group_dim ? tile_m - tile_first : tile_m) * BM;
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(reinterpret_cast<std::uint64_t>(&outs.c[group])), "r"(smem_u32(buf_s)),
                                       "r"(fixed ? 0 : cx), "r"(fixed ? 0 : cy)
                                     : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    stage_buf ^= 1;
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 64) {
                    std::uint32_t r0[32], r1[32];
                    tmem_ld_32x32_x2(tmem_acc + c0, r0, tmem_acc + c0 + 32, r1);
                    gemm_store_chunk<T>(r0, C, partial, row, tile_n * BN + c0, M, N, split, epilogue);
                    gemm_store_chunk<T>(r1, C, partial, row, tile_n * BN + c0 + 32, M, N, split, epilogue);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }

    if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the staging buffers have been read; the writes drain on their own
    if (failed) {
        atomicExch(&g_gemm_status, 1u);
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}
