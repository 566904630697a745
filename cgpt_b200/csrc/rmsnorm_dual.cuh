// Two RMSNorms of the SAME input in one pass, forward and backward, warp per row. Included by rmsnorm.cu only, after
// rmsnorm_warp.cuh (same namespace, same packing helpers).
//
// CGPT's block is a parallel-residual block: the attention branch and the MLP branch each start with their own RMSNorm
// of the block input x (src/core/transformer_block.cu:483-487 and :556-560), and the backward ends with
//     grad_in = grad_out + rmsnorm_backward(d_ffn_norm_out; x, w_ffn) + rmsnorm_backward(d_attn_norm_out; x, w_attn)
// (:678-681 and :745-747: a copy, two backward calls and two in-place adds in the reference). Both norms share x and
// therefore rsqrt(mean(x^2) + eps):
//   forward   reads x once and writes both normalised tensors            (3 tensor passes instead of 4)
//   backward  reads dy_a, dy_b, x and the residual once, writes dx once  (5 tensor passes instead of 8)
// and the three terms of grad_in are summed in fp32 with ONE rounding to the storage dtype. Same per-element expression
// trees as the single-norm kernels; the dw partial sums of both norms are combined in a fixed order (deterministic).
#pragma once

namespace warp_rows {

// y_a = x * inv * w_a, y_b = x * inv * w_b; two rows per warp per trip.
// EXACT: hidden == CPT * 256, so every chunk of every lane is inside the row (no column checks, no zero fills).
template <typename T, int CPT, bool EXACT>
__global__ void __launch_bounds__(kThreads, 2)
rmsnorm_forward_dual_warp_kernel(T* __restrict__ y_a, T* __restrict__ y_b, const T* __restrict__ x, const T* __restrict__ w_a,
                                 const T* __restrict__ w_b, long long rows, int hidden, float epsilon) {
    constexpr int R = 2;
    const int lane = threadIdx.x & 31;
    const long long warp_id = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const long long warps_total = static_cast<long long>(gridDim.x) * kWarps;
    const float inv_hidden = 1.0f / static_cast<float>(hidden);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    uint4 wa[CPT], wb[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int col = (c * 32 + lane) * 8;
        wa[c] = (EXACT || col < hidden) ? *reinterpret_cast<const uint4*>(w_a + col) : zero;
        wb[c] = (EXACT || col < hidden) ? *reinterpret_cast<const uint4*>(w_b + col) : zero;
    }
    for (long long row0 = warp_id * R; row0 < rows; row0 += warps_total * R) {
        uint4 xp[R][CPT];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const long long row = row0 + r;
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int col = (c * 32 + lane) * 8;
                xp[r][c] = (row < rows && (EXACT || col < hidden)) ? __ldcs(reinterpret_cast<const uint4*>(x + row * hidden + col)) : zero;
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const long long row = row0 + r;
            float ss = 0.f;
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float xv[8];
                unpack8<T>(xv, xp[r][c]);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(xv[i], xv[i], ss);
            }
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss * inv_hidden + epsilon);
#pragma unroll
            for (int c = 0; c < CPT; ++c) keep_packed(xp[r][c]);
            if (row < rows) {
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    const int col = (c * 32 + lane) * 8;
                    if (EXACT || col < hidden) {
                        float xv[8], wv[8], out[8];
                        unpack8<T>(xv, xp[r][c]);
                        unpack8<T>(wv, wa[c]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) out[i] = xv[i] * inv * wv[i];
                        *reinterpret_cast<uint4*>(y_a + row * hidden + col) = pack8<T>(out);
                        unpack8<T>(wv, wb[c]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) out[i] = xv[i] * inv * wv[i];
                        *reinterpret_cast<uint4*>(y_b + row * hidden + col) = pack8<T>(out);
                    }
                }
            }
        }
    }
}

// dx = res + (dy_a*w_a*inv - x*c_a) + (dy_b*w_b*inv - x*c_b); per-CTA dw partial rows in dw_partial[blockIdx.x][2][hidden]
// (norm a first). dx may alias res. Shared memory: the thread's running dw sums ([2][CPT*2][kThreads] float4, its own
// slots: no conflicts, no synchronisation) and both weight vectors ([2][CPT*32] uint4).
template <typename T, int CPT, bool EXACT>
__global__ void __launch_bounds__(kThreads, 2)
rmsnorm_backward_dual_warp_kernel(T* dx, float* __restrict__ dw_partial, const T* __restrict__ dy_a, const T* __restrict__ dy_b,
                                  const T* __restrict__ x, const T* __restrict__ w_a, const T* __restrict__ w_b, const T* res,
                                  long long rows, int hidden, float epsilon) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long warp_id = static_cast<long long>(blockIdx.x) * kWarps + warp;
    const long long warps_total = static_cast<long long>(gridDim.x) * kWarps;
    const float inv_hidden = 1.0f / static_cast<float>(hidden);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    extern __shared__ float4 dual_smem[];
    float4* slots_a = dual_smem;                                   // [CPT*2][kThreads]
    float4* slots_b = dual_smem + CPT * 2 * kThreads;
    uint4* w_s = reinterpret_cast<uint4*>(dual_smem + 2 * CPT * 2 * kThreads);   // [2][CPT*32]
    for (int i = threadIdx.x; i < 2 * CPT * 32; i += kThreads) {
        const int n = i / (CPT * 32), col = (i % (CPT * 32)) * 8;
        w_s[i] = col < hidden ? *reinterpret_cast<const uint4*>((n == 0 ? w_a : w_b) + col) : zero;
    }
#pragma unroll
    for (int c = 0; c < CPT * 2; ++c) {
        slots_a[c * kThreads + threadIdx.x] = make_float4(0.f, 0.f, 0.f, 0.f);
        slots_b[c * kThreads + threadIdx.x] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();

    for (long long row = warp_id; row < rows; row += warps_total) {
        const long long off = row * hidden + lane * 8;
        uint4 xp[CPT], ap[CPT], bp[CPT], rp[CPT];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const bool in = EXACT || c * 256 + lane * 8 < hidden;
            xp[c] = in ? __ldcs(reinterpret_cast<const uint4*>(x + off + c * 256)) : zero;
            ap[c] = in ? __ldcs(reinterpret_cast<const uint4*>(dy_a + off + c * 256)) : zero;
            bp[c] = in ? __ldcs(reinterpret_cast<const uint4*>(dy_b + off + c * 256)) : zero;
        }
        float sx = 0.f, sa = 0.f, sb = 0.f;   // sum x^2, sum dy_a*w_a*x, sum dy_b*w_b*x
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            float xv[8], gv[8], wv[8];
            unpack8<T>(xv, xp[c]);
            unpack8<T>(gv, ap[c]);
            unpack8<T>(wv, w_s[c * 32 + lane]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sx = fmaf(xv[i], xv[i], sx);
                sa = fmaf(gv[i] * wv[i], xv[i], sa);
            }
            unpack8<T>(gv, bp[c]);
            unpack8<T>(wv, w_s[CPT * 32 + c * 32 + lane]);
#pragma unroll
            for (int i = 0; i < 8; ++i) sb = fmaf(gv[i] * wv[i], xv[i], sb);
        }
        // the residual is only needed for the output: fetch it while the shuffles of the row sums run
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            keep_packed(xp[c]);
            keep_packed(ap[c]);
            keep_packed(bp[c]);
            rp[c] = (res != nullptr && (EXACT || c * 256 + lane * 8 < hidden)) ? __ldcs(reinterpret_cast<const uint4*>(res + off + c * 256)) : zero;
        }
        sx = warp_sum(sx);
        sa = warp_sum(sa);
        sb = warp_sum(sb);
        const float inv = rsqrtf(sx * inv_hidden + epsilon);
        const float scale3 = inv_hidden * inv * inv * inv;
        const float corr_a = sa * scale3, corr_b = sb * scale3;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            if (EXACT || c * 256 + lane * 8 < hidden) {
                float xv[8], gv[8], wv[8], out[8], xn[8];
                unpack8<T>(xv, xp[c]);
                unpack8<T>(out, rp[c]);                       // zeros without a residual
#pragma unroll
                for (int i = 0; i < 8; ++i) xn[i] = xv[i] * inv;
                {
                    unpack8<T>(gv, ap[c]);
                    unpack8<T>(wv, w_s[c * 32 + lane]);
                    float4 a0 = slots_a[(c * 2) * kThreads + threadIdx.x], a1 = slots_a[(c * 2 + 1) * kThreads + threadIdx.x];
#pragma unroll
                    for (int i = 0; i < 8; ++i) out[i] += fmaf(-xv[i], corr_a, gv[i] * wv[i] * inv);
                    a0.x = fmaf(gv[0], xn[0], a0.x); a0.y = fmaf(gv[1], xn[1], a0.y);
                    a0.z = fmaf(gv[2], xn[2], a0.z); a0.w = fmaf(gv[3], xn[3], a0.w);
                    a1.x = fmaf(gv[4], xn[4], a1.x); a1.y = fmaf(gv[5], xn[5], a1.y);
                    a1.z = fmaf(gv[6], xn[6], a1.z); a1.w = fmaf(gv[7], xn[7], a1.w);
                    slots_a[(c * 2) * kThreads + threadIdx.x] = a0;
                    slots_a[(c * 2 + 1) * kThreads + threadIdx.x] = a1;
                }
                {
                    unpack8<T>(gv, bp[c]);
                    unpack8<T>(wv, w_s[CPT * 32 + c * 32 + lane]);
                    float4 b0 = slots_b[(c * 2) * kThreads + threadIdx.x], b1 = slots_b[(c * 2 + 1) * kThreads + threadIdx.x];
#pragma unroll
                    for (int i = 0; i < 8; ++i) out[i] += fmaf(-xv[i], corr_b, gv[i] * wv[i] * inv);
                    b0.x = fmaf(gv[0], xn[0], b0.x); b0.y = fmaf(gv[1], xn[1], b0.y);
                    b0.z = fmaf(gv[2], xn[2], b0.z); b0.w = fmaf(gv[3], xn[3], b0.w);
                    b1.x = fmaf(gv[4], xn[4], b1.x); b1.y = fmaf(gv[5], xn[5], b1.y);
                    b1.z = fmaf(gv[6], xn[6], b1.z); b1.w = fmaf(gv[7], xn[7], b1.w);
                    slots_b[(c * 2) * kThreads + threadIdx.x] = b0;
                    slots_b[(c * 2 + 1) * kThreads + threadIdx.x] = b1;
                }
                *reinterpret_cast<uint4*>(dx + off + c * 256) = pack8<T>(out);
            }
        }
    }

    // Combine the CTA's 8 warps in a fixed order: one fp32 partial row per CTA and norm.
    __syncthreads();
    for (int n = 0; n < 2; ++n) {
        const float* slots = reinterpret_cast<const float*>(n == 0 ? slots_a : slots_b);
        for (int col = threadIdx.x; col < hidden; col += kThreads) {
            const int c = col >> 8, l = (col >> 3) & 31, i = col & 7;
            float acc = 0.f;
#pragma unroll
            for (int wi = 0; wi < kWarps; ++wi) acc += slots[(((c * 2 + (i >> 2)) * kThreads) + wi * 32 + l) * 4 + (i & 3)];
            dw_partial[(static_cast<long long>(blockIdx.x) * 2 + n) * hidden + col] = acc;
        }
    }
}

// dw_a[col], dw_b[col] = sums over `parts` partial rows ([parts][2][hidden]) in a fixed order.
template <typename T>
__global__ void __launch_bounds__(1024)
dw_reduce_dual_kernel(T* __restrict__ dw_a, T* __restrict__ dw_b, const float* __restrict__ partial, int parts, int hidden) {
    __shared__ float tile[32][33];
    const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + cl;      // 0 .. 2*hidden: norm a's columns first
    float acc = 0.f;
    if (col < 2 * hidden)
        for (int p = rl; p < parts; p += 32) acc += partial[static_cast<long long>(p) * 2 * hidden + col];
    tile[rl][cl] = acc;
    __syncthreads();
    if (rl == 0 && col < 2 * hidden) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) total += tile[r][cl];
        if (col < hidden) dw_a[col] = from_f32<T>(total);
        else dw_b[col - hidden] = from_f32<T>(total);
    }
}

}  // namespace warp_rows
