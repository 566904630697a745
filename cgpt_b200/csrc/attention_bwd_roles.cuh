// Producer (TMA) and MMA-issuer roles of attention_bwd_tc_kernel. Included by attention_bwd_tc.cu only.
#pragma once

// Geometry of one CTA's work, computed identically by every thread.
struct BwdGeom {
    int b;        // batch index
    int h;        // MODE_DQ: query head of this CTA
    int kvh;      // kv head
    int x0;       // first stationary row: query index (dQ) or key index (dKV)
    int n_it;     // streaming tiles to process
    int i0;       // MODE_DKV: first 64-query tile that can see this key tile
    int n_q;      // MODE_DKV: 64-query tiles per query head
    int ratio;    // query heads per kv head
};

struct BwdBars {
    std::uint64_t *x_full, *y_full, *stat_full, *y_free, *uw_free, *t_full, *w_full, *acc_done;
    unsigned long long* trace;   // diagnosis: per-iteration timestamps of one CTA (nullptr = off)
};

__device__ __forceinline__ void bwd_trace(const BwdBars& b, int it, int slot) {
    if (b.trace != nullptr && it < 64) b.trace[it * 8 + slot] = globaltimer_ns();
}

// Streaming tile `it` -> (head, first row of the streaming tile).
template <int MODE>
__device__ __forceinline__ void bwd_stream_coords(const BwdGeom& g, int it, int* head, int* row0) {
    if (MODE == MODE_DQ) {
        *head = g.kvh;             // K / V tiles of the kv head
        *row0 = it * kCols;
    } else {
        *head = g.kvh * g.ratio + it / g.n_q;
        *row0 = (g.i0 + it % g.n_q) * kCols;
    }
}

template <int D, int MODE>
__device__ __forceinline__ bool bwd_producer(unsigned char* smem, const BwdBars& bars, const BwdGeom& g, const AttnDims& dm,
                                             const CUtensorMap* map_x1, const CUtensorMap* map_x2, const CUtensorMap* map_y1,
                                             const CUtensorMap* map_y2, const float* __restrict__ lse2_t,
                                             const float* __restrict__ delta_t, int lane) {
    using L = BwdSmem<D>;
    if (lane == 0) {
        const int xh = MODE == MODE_DQ ? g.h : g.kvh;
        mbar_expect_tx(bars.x_full, 2 * L::kXBytes);
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c) {
            tma_load_4d(smem + L::kX1 + c * kRows * 128, map_x1, bars.x_full, c * 64, xh, g.x0, g.b);
            tma_load_4d(smem + L::kX2 + c * kRows * 128, map_x2, bars.x_full, c * 64, xh, g.x0, g.b);
        }
    }
    constexpr int kYStages = L::kStages;
    // MODE_DKV: the statistics of tile it + 1 (lse2 and delta * scale of its 64 queries, two per lane) are fetched into
    // registers while this warp waits for tile it's ring stage, so the loads' latency never stalls the TMA issue
    float next_lse2[2] = {1.0e30f, 1.0e30f}, next_delta[2] = {0.f, 0.f};
    auto fetch_stats = [&](int it) {
        int head, row0;
        bwd_stream_coords<MODE>(g, it, &head, &row0);
        const long long base = (static_cast<long long>(g.b) * dm.hq + head) * dm.sq;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int q = row0 + lane + 32 * u;
            next_lse2[u] = q < dm.sq ? lse2_t[base + q] : 1.0e30f;          // rows past the end: P = 0
            next_delta[u] = q < dm.sq ? delta_t[base + q] * dm.scale : 0.f;  // the compute warps use delta * scale
        }
    };
    if (MODE == MODE_DKV) fetch_stats(0);
    int s = 0;                  // ring stage = it % kYStages
    std::uint32_t par = 0;      // its phase = (it / kYStages) & 1
    for (int it = 0; it < g.n_it; ++it) {
        if (!mbar_wait(&bars.y_free[s], par ^ 1u)) return false;
        if (lane == 0) bwd_trace(bars, it, 0);
        int head, row0;
        bwd_stream_coords<MODE>(g, it, &head, &row0);
        if (lane == 0) {
            unsigned char* y1 = smem + L::kY + s * 2 * L::kYBytes;
            unsigned char* y2 = y1 + L::kYBytes;
            mbar_expect_tx(&bars.y_full[s], 2 * L::kYBytes);
#pragma unroll
            for (int c = 0; c < L::kChunks; ++c) {
                tma_load_4d(y1 + c * kCols * 128, map_y1, &bars.y_full[s], c * 64, head, row0, g.b);
                tma_load_4d(y2 + c * kCols * 128, map_y2, &bars.y_full[s], c * 64, head, row0, g.b);
            }
        }
        if (MODE == MODE_DKV) {
            // per-query statistics of the streaming tile, fetched one iteration ago
            float* st = reinterpret_cast<float*>(smem + L::kStats) + s * 2 * kCols;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                st[lane + 32 * u] = next_lse2[u];
                st[kCols + lane + 32 * u] = next_delta[u];
            }
            mbar_arrive(&bars.stat_full[s]);
            if (it + 1 < g.n_it) fetch_stats(it + 1);
        }
        if (++s == kYStages) { s = 0; par ^= 1u; }
    }
    return true;
}

// The MMA-issuing thread is a single scalar instruction stream, so every instruction between two tcgen05.mma
// counts: all shared-memory descriptors are loop-invariant per ring stage and are built once; a K step only adds
// a constant to the 14-bit address field.
__device__ __forceinline__ std::uint64_t desc_advance(std::uint64_t desc, std::uint32_t bytes) { return desc + (bytes >> 4); }

template <typename T, int D, int MODE>
__device__ __forceinline__ bool bwd_mma_issuer(unsigned char* smem, const BwdBars& bars, const BwdGeom& g, std::uint32_t tmem) {
    using L = BwdSmem<D>;
    constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr std::uint32_t idesc_t = idesc_f16(fmt, 0, 0, kRows, kCols);   // T = X Y^T: both K-major
    constexpr std::uint32_t idesc_acc = idesc_f16(fmt, 0, 1, kRows, D);     // acc += U/W (K-major) * Y (N-major)
    constexpr std::uint32_t kYStage16 = (2 * L::kYBytes) >> 4;              // ring stage stride in descriptor units
    using TM = BwdTmem<D, MODE>;
    constexpr int kTBufs = TM::kTBufs;
    const std::uint32_t tmem_acc1 = tmem + TM::kAcc, tmem_acc2 = tmem + TM::kAcc + D;
    const std::uint64_t dx1 = smem_desc_sw128(smem_u32(smem + L::kX1), 16, 1024);
    const std::uint64_t dx2 = smem_desc_sw128(smem_u32(smem + L::kX2), 16, 1024);
    const std::uint32_t y_base = smem_u32(smem + L::kY);
    const std::uint64_t dy1k = smem_desc_sw128(y_base, 16, 1024);                       // as K-major B of T1
    const std::uint64_t dy2k = smem_desc_sw128(y_base + L::kYBytes, 16, 1024);
    const std::uint64_t dy1n = smem_desc_sw128(y_base, kCols * 128, 1024);              // as N-major B of the accumulations
    const std::uint64_t dy2n = smem_desc_sw128(y_base + L::kYBytes, kCols * 128, 1024);

    // T1/T2 of tile `it` (TMEM buffer tb) whose streaming pair sits in ring stage ys (phase ypar)
    auto issue_t = [&](int it, int tb, int ys, std::uint32_t ypar) -> bool {
        if (!mbar_wait(&bars.y_full[ys], ypar)) return false;
        bwd_trace(bars, it, 1);
        tc_fence_after_sync();
        const int s = tb;
        const std::uint32_t t1 = tmem + TM::kT1 + s * kCols, t2 = tmem + TM::kT2 + s * kCols;
        const std::uint64_t y1 = dy1k + ys * kYStage16, y2 = dy2k + ys * kYStage16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
            const std::uint32_t xo = (k >> 2) * (kRows * 128) + (k & 3) * 32, yo = (k >> 2) * (kCols * 128) + (k & 3) * 32;
            mma_f16_ss(t1, desc_advance(dx1, xo), desc_advance(y1, yo), idesc_t, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
            const std::uint32_t xo = (k >> 2) * (kRows * 128) + (k & 3) * 32, yo = (k >> 2) * (kCols * 128) + (k & 3) * 32;
            mma_f16_ss(t2, desc_advance(dx2, xo), desc_advance(y2, yo), idesc_t, k > 0 ? 1u : 0u);
        }
        tc_commit(&bars.t_full[s]);
        return true;
    };

    if (!mbar_wait(bars.x_full, 0)) return false;
    // The T products run kTBufs - 1 tiles ahead of the accumulating products. `ahead` = the next tile whose T products
    // have not been issued, with its TMEM buffer, ring stage and phase kept as counters (no divisions in this thread).
    int ahead = 0, ahead_tb = 0, ahead_ys = 0;
    std::uint32_t ahead_par = 0;
    auto issue_next_t = [&]() -> bool {
        if (!issue_t(ahead, ahead_tb, ahead_ys, ahead_par)) return false;
        ++ahead;
        if (++ahead_tb == kTBufs) ahead_tb = 0;
        if (++ahead_ys == L::kStages) { ahead_ys = 0; ahead_par ^= 1u; }
        return true;
    };
    for (int p = 0; p < kTBufs - 1 && p < g.n_it; ++p)
        if (!issue_next_t()) return false;
    int ys = 0;                  // ring stage of tile `it`
    int tb = 0;                  // its TMEM buffer = it % kTBufs
    std::uint32_t tpar = 0;      // phase of that buffer's barriers = (it / kTBufs) & 1
    for (int it = 0; it < g.n_it; ++it) {
        const int s = tb;
        if (ahead < g.n_it && !issue_next_t()) return false;
        if (!mbar_wait(&bars.w_full[s], tpar)) return false;
        bwd_trace(bars, it, 2);
        tc_fence_after_sync();
        const std::uint32_t acc = it > 0 ? 1u : 0u;
        const std::uint64_t y1 = dy1n + ys * kYStage16, y2 = dy2n + ys * kYStage16;
        const std::uint32_t u_tmem = tmem + TM::kT1 + s * kCols, w_tmem = tmem + TM::kT2 + s * kCols;   // over T1 / T2 of this tile
#pragma unroll
        for (int k = 0; k < kCols / 16; ++k) {
            // A: TMEM, lanes = stationary rows, 16 streaming rows (one K step) = 8 packed columns; the tile's compute
            // warpgroup wrote streaming rows 0-31 at columns [0,16) and rows 32-63 at columns [32,48).
            // B: streaming tile as N-major: 16 rows of 128 B per K step, 64-column chunks of D kCols*128 bytes apart.
            const std::uint32_t a_col = (k >> 1) * 32 + (k & 1) * 8;
            if (MODE == MODE_DKV) {
                mma_f16_ts(tmem_acc1, u_tmem + a_col, desc_advance(y2, k * (16 * 128)), idesc_acc,
                           k > 0 ? 1u : acc);                                            // dV += P^T dO
                mma_f16_ts(tmem_acc2, w_tmem + a_col, desc_advance(y1, k * (16 * 128)), idesc_acc,
                           k > 0 ? 1u : acc);                                            // dK += dS^T Q
            } else {
                mma_f16_ts(tmem_acc1, w_tmem + a_col, desc_advance(y1, k * (16 * 128)), idesc_acc,
                           k > 0 ? 1u : acc);                                            // dQ += dS K
            }
        }
        tc_commit(&bars.y_free[ys]);     // the streaming tile's ring stage may be refilled ...
        if (++ys == L::kStages) ys = 0;
        if (++tb == kTBufs) { tb = 0; tpar ^= 1u; }
    }
    tc_commit(bars.acc_done);
    return true;
}
