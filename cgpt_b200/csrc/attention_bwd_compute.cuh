// Compute role (warps 0-7) of attention_bwd_tc_kernel. The two warpgroups take the streaming tiles in turn: warpgroup w
// owns the tiles with (it & 1) == w, i.e. always the same one of the two T1/T2 buffers in TMEM, and thread t of a
// warpgroup owns stationary row t = TMEM lane t of its tile (all 64 columns, in two chunks of 32). While one warpgroup
// waits for its tile's products, for a TMEM load or for its stores to land, the other is in its arithmetic, so the
// per-tile latencies of the chain (T products -> load -> exponentials -> store -> accumulating products) overlap
// instead of adding up in every tile period. Included by attention_bwd_tc.cu only.
#pragma once

// One thread's 32 columns of a tile: P = 2^(S*scale2 - lse2) (0 where masked), W = P * (dP*scale - delta*scale), both packed
// to the storage dtype. Straight-line per variant: the masked form (tiles on the diagonal or past the end) pays a compare
// and a select per element, the common form nothing. dKV reads the streaming rows' statistics (lse2 and delta*scale, 32
// floats each at st and st + kCols) as 16-byte shared-memory loads; dQ has them in registers.
template <typename T, int MODE, bool MASK>
__device__ __forceinline__ void bwd_tile_math(const std::uint32_t* t1, const std::uint32_t* t2, std::uint32_t* pu, std::uint32_t* pw,
                                              const float* st, float my_lse2, float my_delta_s, float scale2, float scale, int thr) {
#pragma unroll
    for (int j4 = 0; j4 < 32; j4 += 4) {
        float lse2[4] = {my_lse2, my_lse2, my_lse2, my_lse2}, dls[4] = {my_delta_s, my_delta_s, my_delta_s, my_delta_s};
        if (MODE == MODE_DKV) {
            const float4 a = *reinterpret_cast<const float4*>(st + j4), b = *reinterpret_cast<const float4*>(st + kCols + j4);
            lse2[0] = a.x; lse2[1] = a.y; lse2[2] = a.z; lse2[3] = a.w;
            dls[0] = b.x; dls[1] = b.y; dls[2] = b.z; dls[3] = b.w;
        }
        float p[4], ds[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = j4 + e;
            float pe = fast_exp2(fmaf(__uint_as_float(t1[j]), scale2, -lse2[e]));
            if (MASK) pe = (MODE == MODE_DQ ? j <= thr : j >= thr) ? pe : 0.f;
            p[e] = pe;
            ds[e] = pe * fmaf(__uint_as_float(t2[j]), scale, -dls[e]);
        }
        pu[j4 >> 1] = pack2<T>(p[0], p[1]);
        pu[(j4 >> 1) + 1] = pack2<T>(p[2], p[3]);
        pw[j4 >> 1] = pack2<T>(ds[0], ds[1]);
        pw[(j4 >> 1) + 1] = pack2<T>(ds[2], ds[3]);
    }
}

template <typename T, int D, int MODE>
__device__ __forceinline__ bool bwd_compute(unsigned char* smem, const BwdBars& bars, const BwdGeom& g, const AttnDims& dm,
                                            std::uint32_t tmem, const float* __restrict__ lse2_t,
                                            const float* __restrict__ delta_t, T* __restrict__ out1, T* __restrict__ out2,
                                            int accumulate) {
    using L = BwdSmem<D>;
    const int row = threadIdx.x & (kRows - 1);         // 0..127: TMEM lane; two threads (one per warpgroup) share a row
    const int half = threadIdx.x >> 7;                 // warpgroup: owns the tiles with (it & 1) == half; half of the epilogue's columns
    const int warp = (threadIdx.x >> 5) & 3;           // lane quarter of this warp
    const std::uint32_t lane_base = static_cast<std::uint32_t>(warp * 32) << 16;
    const float scale2 = dm.scale * kLog2e;
    const int x_idx = g.x0 + row;                      // query index (dQ) or key index (dKV) of this thread

    // MODE_DQ: this thread's own statistics; rows past the end get lse2 = +1e30 so that P = 0.
    float my_lse2 = 1.0e30f, my_delta = 0.f;
    int limit = 0;                                     // MODE_DQ: last visible key of this query
    if (MODE == MODE_DQ) {
        if (x_idx < dm.sq) {
            const long long t = (static_cast<long long>(g.b) * dm.hq + g.h) * dm.sq + x_idx;
            my_lse2 = lse2_t[t];
            my_delta = delta_t[t];
        }
        limit = dm.causal ? dm.offset + x_idx : dm.sk - 1;
        if (limit > dm.sk - 1) limit = dm.sk - 1;
    }
    const float my_delta_s = my_delta * dm.scale;
    bool failed = false;

    constexpr int kYStages = L::kStages;
    using TM = BwdTmem<D, MODE>;
    constexpr int kTBufs = TM::kTBufs;
    for (int it = half; it < g.n_it; it += 2) {
        const int s = it % kTBufs;                                 // the tile's T1/T2 buffer in TMEM
        const std::uint32_t par = (it / kTBufs) & 1;               // and the phase of its barriers
        const int ys = it % kYStages;                              // ring stage of the streaming tile
        const std::uint32_t ypar = (it / kYStages) & 1;            // and its phase
        int head, y0;
        bwd_stream_coords<MODE>(g, it, &head, &y0);
        if (!mbar_wait(&bars.t_full[s], par)) failed = true;
        if (MODE == MODE_DKV && !failed && !mbar_wait(&bars.stat_full[ys], ypar)) failed = true;
        failed = __any_sync(0xffffffffu, failed);
        if (failed) break;
        if (threadIdx.x == 0) bwd_trace(bars, it, 3);
        tc_fence_after_sync();
        const float* st = reinterpret_cast<const float*>(smem + L::kStats) + ys * 2 * kCols;
        // does any element of this tile need the visibility test?
        bool need_mask;
        if (MODE == MODE_DQ) need_mask = (y0 + kCols > dm.sk) || (dm.causal && y0 + kCols - 1 > dm.offset + g.x0);
        else need_mask = dm.causal && (g.x0 + kRows - 1 > dm.offset + y0);
#pragma unroll 1
        for (int c0 = 0; c0 < kCols; c0 += 32) {
            std::uint32_t t1[32], t2[32];
            tmem_ld_32x32_x2(tmem + TM::kT1 + s * kCols + lane_base + c0, t1, tmem + TM::kT2 + s * kCols + lane_base + c0, t2);
            std::uint32_t pu[16], pw[16];
            // column j of this thread's 32 is visible iff j <= thr (dQ: key <= limit) or j >= thr (dKV: query >= key - offset)
            const int thr = MODE == MODE_DQ ? limit - y0 - c0 : x_idx - dm.offset - y0 - c0;
            if (need_mask) bwd_tile_math<T, MODE, true>(t1, t2, pu, pw, st + c0, my_lse2, my_delta_s, scale2, dm.scale, thr);
            else bwd_tile_math<T, MODE, false>(t1, t2, pu, pw, st + c0, my_lse2, my_delta_s, scale2, dm.scale, thr);
            // U (P^T) and W (dS or dS^T) go back into TMEM over this thread's own, already read, columns of T1 and T2:
            // 16 packed words at columns [c0, c0 + 16) of the tile's buffer. The accumulating products read them from
            // there as their A operands, so neither the stores nor the operand reads touch shared memory.
            if (MODE == MODE_DKV) tmem_st_32x16(tmem + TM::kT1 + s * kCols + lane_base + c0, pu);
            tmem_st_32x16(tmem + TM::kT2 + s * kCols + lane_base + c0, pw);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(&bars.w_full[s]);
        if (threadIdx.x == 0) bwd_trace(bars, it, 4);
    }

    // ---- epilogue: accumulators -> global
    if (g.n_it > 0) {
        if (!failed && !mbar_wait(bars.acc_done, 0)) failed = true;
        failed = __any_sync(0xffffffffu, failed);
        if (failed) return false;
        tc_fence_after_sync();
    }
    const int x_limit = MODE == MODE_DQ ? dm.sq : dm.sk;
    const int heads = MODE == MODE_DQ ? dm.hq : dm.hkv;
    const int xh = MODE == MODE_DQ ? g.h : g.kvh;
    const long long dst_off = ((static_cast<long long>(g.b) * x_limit + x_idx) * heads + xh) * D;
    constexpr int kOuts = MODE == MODE_DKV ? 2 : 1;
#pragma unroll
    for (int o = 0; o < kOuts; ++o) {
        // dKV: acc1 = dV -> out2 (grad_value), acc2 = dK -> out1 (grad_key); dQ: acc1 -> out1
        T* dst = (MODE == MODE_DKV ? (o == 0 ? out2 : out1) : out1) + dst_off;
        const std::uint32_t acc = tmem + TM::kAcc + o * D;
#pragma unroll
        for (int cc = 0; cc < D / 2; cc += 32) {
            const int c0 = half * (D / 2) + cc;
            std::uint32_t r[32];
            if (g.n_it > 0) {
                tmem_ld_32x32(acc + lane_base + c0, r);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
            if (x_idx < x_limit) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    float v8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v8[e] = __uint_as_float(r[j + e]);
                    if (accumulate) {
                        float old[8];
                        load_vec<T, 8>(old, dst + c0 + j);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v8[e] += old[e];
                    }
                    store_vec<T, 8>(dst + c0 + j, v8);
                }
            }
        }
    }
    tc_fence_before_sync();
    return true;
}
