// Gate/up projections with the SwiGLU activation in the epilogue. Included by gemm.cu only (inside its anonymous
// namespace, after gemm_persistent.cuh).
//
//   gate = X Wg^T,  up = X Wu^T,  act = gate / (1 + exp(-gate)) * up        (X [M,K], Wg/Wu [N,K], outputs [M,N])
//
// The reference runs two linear_forward calls and swiglu_forward (src/core/transformer_block.cu:566-579, src/ops/swiglu.cu:
// 69-71): the activation pass re-reads both projections from HBM. Here one CTA tile covers 128 rows x 128 output columns
// of BOTH projections: the B stage holds 128 rows of Wg followed by 128 rows of Wu, one 128x256x16 tcgen05.mma per K
// step fills accumulator columns [0,128) with gate and [128,256) with up, and the epilogue writes gate, up (both are
// saved for the backward pass) and act from the same accumulator. gate and up are rounded to the storage dtype first
// and act is computed from the rounded values, exactly what the separate activation kernel reads.
// Same persistent structure as gemm_tcgen05_persistent_kernel: TMA ring, two accumulators in TMEM, staged TMA stores.
#pragma once

struct SwigluMaps {
    CUtensorMap x, wg, wu;        // loads: box {BK, 128}
    CUtensorMap gate, up, act;    // stores: box {64, 128}
};

// Writes 64 accumulator columns (two 32-column register chunks, fp32 bit patterns) as one 16-bit [128 x 64] block:
// swizzled staging buffer -> TMA store. All 128 epilogue threads call this together.
template <typename T>
__device__ __forceinline__ void staged_store_64(unsigned char* staging, int& stage_buf, int et, int trow, const CUtensorMap* map,
                                                int x, int y, const std::uint32_t (&r0)[32], const std::uint32_t (&r1)[32]) {
    unsigned char* buf_s = staging + stage_buf * (BM * 128);
    if (et == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the buffer used two stores ago is free
    asm volatile("bar.sync 1, 128;" ::: "memory");
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
    if (et == 0) {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                     ::"l"(reinterpret_cast<std::uint64_t>(map)), "r"(smem_u32(buf_s)), "r"(x), "r"(y)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    stage_buf ^= 1;
}

template <typename T>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_swiglu_persistent_kernel(const __grid_constant__ SwigluMaps maps, int total_kb, int tiles_m, int tiles_n) {
    constexpr int BN = 256;          // MMA width: 128 gate + 128 up columns
    constexpr int BNH = 128;         // output columns per tile
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
    const int units = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        mbar_init_fence();
        tma_prefetch_desc(&maps.x); tma_prefetch_desc(&maps.wg); tma_prefetch_desc(&maps.wu);
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
                const int tile_m = u / tiles_n, tile_n = u % tiles_n;
                for (int i = 0; i < total_kb; ++i, ++it) {
                    const int s = it % Cfg::kStages;
                    const std::uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1u)) { failed = true; break; }
                    mbar_expect_tx(&full[s], Cfg::kStageBytes);
                    unsigned char* a_dst = smem + s * Cfg::kStageBytes;
                    unsigned char* b_dst = a_dst + Cfg::kABytes;
                    tma_load_2d(a_dst, &maps.x, &full[s], i * BK, tile_m * BM);
                    tma_load_2d(b_dst, &maps.wg, &full[s], i * BK, tile_n * BNH);                  // B rows 0..127
                    tma_load_2d(b_dst + BNH * BK * 2, &maps.wu, &full[s], i * BK, tile_n * BNH);  // B rows 128..255
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr std::uint32_t idesc = idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, 0, 0, BM, BN);
            int it = 0, j = 0;
            for (int u = blockIdx.x; u < units && !failed; u += gridDim.x, ++j) {
                const int buf = j & 1;
                if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1u)) { failed = true; break; }
                tc_fence_after_sync();
                const std::uint32_t tmem_acc = tmem_base + buf * BN;
                for (int i = 0; i < total_kb; ++i, ++it) {
                    const int s = it % Cfg::kStages;
                    const std::uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!mbar_wait(&full[s], ph)) { failed = true; break; }
                    tc_fence_after_sync();
                    const std::uint32_t a_base = smem_u32(smem + s * Cfg::kStageBytes);
                    const std::uint32_t b_base = a_base + Cfg::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_f16_ss(tmem_acc, smem_desc_sw128(a_base + k * (UMMA_K * 2), 16, 1024),
                                   smem_desc_sw128(b_base + k * (UMMA_K * 2), 16, 1024), idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit(&empty[s]);
                }
                tc_commit(&acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;
        const int et = threadIdx.x - 64;              // 0..127 within the epilogue warps
        const int trow = quarter * 32 + lane;         // row inside the tile
        int j = 0;
        int stage_buf = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, ++j) {
            const int tile_m = u / tiles_n, tile_n = u % tiles_n;
            const int buf = j & 1;
            if (!mbar_wait(&acc_full[buf], (j >> 1) & 1)) failed = true;
            failed = __any_sync(0xffffffffu, failed);
            if (failed) break;
            tc_fence_after_sync();
            const std::uint32_t tmem_acc = tmem_base + buf * BN + (static_cast<std::uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BNH; c0 += 64) {
                const int x = tile_n * BNH + c0, y = tile_m * BM;
                std::uint32_t g0[32], g1[32], u0[32], u1[32];
                tmem_ld_32x32_x2(tmem_acc + c0, g0, tmem_acc + c0 + 32, g1);
                staged_store_64<T>(staging, stage_buf, et, trow, &maps.gate, x, y, g0, g1);
                tmem_ld_32x32_x2(tmem_acc + BNH + c0, u0, tmem_acc + BNH + c0 + 32, u1);
                staged_store_64<T>(staging, stage_buf, et, trow, &maps.up, x, y, u0, u1);
                // act from the ROUNDED gate and up, in place over the gate registers
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float ga = __uint_as_float(g0[e]), gb = __uint_as_float(g0[e + 1]);
                    float ua = __uint_as_float(u0[e]), ub = __uint_as_float(u0[e + 1]);
                    round_pair_to_storage<T>(ga, gb);
                    round_pair_to_storage<T>(ua, ub);
                    g0[e] = __float_as_uint(ga / (1.0f + __expf(-ga)) * ua);
                    g0[e + 1] = __float_as_uint(gb / (1.0f + __expf(-gb)) * ub);
                    ga = __uint_as_float(g1[e]); gb = __uint_as_float(g1[e + 1]);
                    ua = __uint_as_float(u1[e]); ub = __uint_as_float(u1[e + 1]);
                    round_pair_to_storage<T>(ga, gb);
                    round_pair_to_storage<T>(ua, ub);
                    g1[e] = __float_as_uint(ga / (1.0f + __expf(-ga)) * ua);
                    g1[e + 1] = __float_as_uint(gb / (1.0f + __expf(-gb)) * ub);
                }
                staged_store_64<T>(staging, stage_buf, et, trow, &maps.act, x, y, g0, g1);
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

// Launch; returns CGPT_ERR_UNSUPPORTED when the operands cannot be addressed by TMA (the caller then runs the three
// separate kernels).
template <typename T>
int launch_gemm_swiglu(T* gate, T* up, T* act, const T* x, const T* wg, const T* wu, int M, int N, int K, int dtype, cudaStream_t s) {
    using Cfg = GemmCfg<256>;
    if (!aligned16(gate) || !aligned16(up) || !aligned16(act) || !aligned16(x) || !aligned16(wg) || !aligned16(wu) || N % 8 != 0 ||
        K % 8 != 0 || K < 32 || static_cast<long long>(M) * N < 64 * 64)
        return CGPT_ERR_UNSUPPORTED;
    SwigluMaps maps;
    const std::uint64_t xd[2] = {static_cast<std::uint64_t>(K), static_cast<std::uint64_t>(M)};
    const std::uint64_t wd[2] = {static_cast<std::uint64_t>(K), static_cast<std::uint64_t>(N)};
    const std::uint64_t kst[1] = {static_cast<std::uint64_t>(K) * 2};
    const std::uint32_t in_box[2] = {BK, 128};
    CGPT_TRY(make_tensor_map(&maps.x, dtype, x, 2, xd, kst, in_box));
    CGPT_TRY(make_tensor_map(&maps.wg, dtype, wg, 2, wd, kst, in_box));
    CGPT_TRY(make_tensor_map(&maps.wu, dtype, wu, 2, wd, kst, in_box));
    const std::uint64_t od[2] = {static_cast<std::uint64_t>(N), static_cast<std::uint64_t>(M)};
    const std::uint64_t ost[1] = {static_cast<std::uint64_t>(N) * 2};
    const std::uint32_t out_box[2] = {64, BM};
    CGPT_TRY(make_tensor_map(&maps.gate, dtype, gate, 2, od, ost, out_box));
    CGPT_TRY(make_tensor_map(&maps.up, dtype, up, 2, od, ost, out_box));
    CGPT_TRY(make_tensor_map(&maps.act, dtype, act, 2, od, ost, out_box));
    auto kernel = gemm_swiglu_persistent_kernel<T>;
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_once.done();
    }
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + 127) / 128;
    const long long units = static_cast<long long>(tiles_m) * tiles_n;
    const unsigned grid = static_cast<unsigned>(units < kNumSMs ? units : kNumSMs);
    const bool timed = g_timing.enabled && g_timing.used + 2 <= g_timing.events.size();
    if (timed) CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used], s));
    kernel<<<grid, kGemmThreads, Cfg::kSmemBytes, s>>>(maps, (K + BK - 1) / BK, tiles_m, tiles_n);
    count_launch();
    CGPT_LAUNCH_CHECK();
    if (timed) {
        CGPT_CUDA_TRY(cudaEventRecord(g_timing.events[g_timing.used + 1], s));
        g_timing.used += 2;
        g_timing.flops.push_back(4.0 * M * N * K);
    }
    return CGPT_OK;
}
