// Softmax gradient and loss from per-tile row statistics. Included by cross_entropy.cu only.
//
// The LM-head logits product can leave, for every row and every tile of 256 vocabulary columns, the pair
// (m_t, s_t) = (max of the tile's logits, sum exp(l - m_t)) and the target's logit (gemm_pair.cuh, softmax epilogues).
// From those a row's maximum and sum need no pass over the logits:
//     m = max_t m_t,    sum = sum_t s_t * exp(m_t - m)      (tiles combined in a fixed order)
// so the gradient is ONE streaming pass: read 16 bytes of logits, write 16 bytes of gradient, no block-wide
// reduction and no second sweep of the row (the row kernel of cross_entropy_ring.cuh needs both).
// Per element the arithmetic is that kernel's: e = ex2.approx.ftz((l - m) * log2 e), non-target gradient
// e * (1/sum * out_scale), target (e * 1/sum - 1) * out_scale, row loss (log sum + m - l_target) / total rows.
#pragma once

constexpr int kTileGradThreads = 256;
constexpr int kTileGradUnroll = 4;     // 16-byte chunks a thread has in flight

// (max, 1 / sum) of one row from its tile statistics, computed redundantly by every lane group of a warp: lanes
// stride over the tiles, then a butterfly (same value, same order in every warp).
__device__ __forceinline__ float2 row_stats_from_tiles(const float2* __restrict__ partial, long long row, int tiles, int lane,
                                                       float* sum_out) {
    const float2* mine = partial + row * tiles;     // [rows][tiles]: a row's statistics are contiguous
    float m = -3.0e38f;
    for (int t = lane; t < tiles; t += 32) m = fmaxf(m, __ldg(&mine[t]).x);
    m = warp_max(m);
    float sum = 0.f;
    for (int t = lane; t < tiles; t += 32) {
        const float2 p = __ldg(&mine[t]);
        sum += p.y * fast_exp(p.x - m);
    }
    sum = warp_sum(sum);
    *sum_out = sum;
    return make_float2(m, __frcp_rn(sum));
}

template <typename T>
__global__ void __launch_bounds__(kTileGradThreads)
softmax_grad_rows_kernel(float* __restrict__ row_loss, T* grad, const float2* __restrict__ partial,
                         const float* __restrict__ target_logit, const std::uint32_t* __restrict__ targets, long long rows, int vocab,
                         int tiles, float inv_rows, float gradient_scale) {
    const int lane = threadIdx.x & 31;
    const int chunks = vocab / 8;
    const float out_scale = inv_rows * gradient_scale;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        float sum;
        const float2 st = row_stats_from_tiles(partial, row, tiles, lane, &sum);
        const std::uint32_t target = targets[row];
        const bool valid = target < static_cast<std::uint32_t>(vocab);
        const float l_target = valid ? target_logit[row] : 0.f;
        if (threadIdx.x == 0) row_loss[row] = valid ? (__logf(sum) + st.x - l_target) * inv_rows : 0.f;
        const float k = st.y * out_scale;
        T* dst = grad + row * vocab;
        for (int c0 = threadIdx.x; c0 < chunks; c0 += kTileGradThreads * kTileGradUnroll) {
            uint4 raw[kTileGradUnroll];
#pragma unroll
            for (int u = 0; u < kTileGradUnroll; ++u) {
                const int c = c0 + u * kTileGradThreads;
                if (c < chunks) raw[u] = __ldcs(reinterpret_cast<const uint4*>(dst + c * 8));
            }
#pragma unroll
            for (int u = 0; u < kTileGradUnroll; ++u) {
                const int c = c0 + u * kTileGradThreads;
                if (c < chunks) {
                    Pack<T, 8> pk;
                    *reinterpret_cast<uint4*>(&pk) = raw[u];
                    float p[8];
                    unpack_pack(p, pk);
#pragma unroll
                    for (int e = 0; e < 8; ++e) p[e] = fast_exp(p[e] - st.x) * k;
                    store_vec<T, 8>(dst + c * 8, p);
                }
            }
        }
        // The element that carries the -1 is rewritten by the thread that owns its chunk (same thread, same address,
        // program order: this store lands after that thread's vector store).
        if (valid && static_cast<int>((target >> 3) % kTileGradThreads) == static_cast<int>(threadIdx.x))
            dst[target] = from_f32<T>((fast_exp(l_target - st.x) * st.y - 1.0f) * out_scale);
    }
}

// One thread group per row: row statistics for the gradient epilogue of the recomputed logits product, and the row loss.
__global__ void __launch_bounds__(256)
softmax_stats_reduce_kernel(float2* __restrict__ row_stats, float* __restrict__ row_loss, const float2* __restrict__ partial,
                            const float* __restrict__ target_logit, const std::uint32_t* __restrict__ targets, long long rows,
                            int vocab, int tiles, float inv_rows) {
    const int lane = threadIdx.x & 31;
    const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
    for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
        float sum;
        const float2 st = row_stats_from_tiles(partial, row, tiles, lane, &sum);
        if (lane == 0) {
            const std::uint32_t target = targets[row];
            const bool valid = target < static_cast<std::uint32_t>(vocab);
            row_stats[row] = st;
            row_loss[row] = valid ? (__logf(sum) + st.x - target_logit[row]) * inv_rows : 0.f;
        }
    }
}
