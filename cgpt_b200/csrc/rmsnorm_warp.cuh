// Warp-per-row RMSNorm kernels for 16-bit rows of 256..1024 elements. Included by rmsnorm.cu only.
//
// One warp owns a whole row: lane l holds the 16-byte chunks l, l+32, l+64, l+96 of the row (CPT of them), kept
// PACKED in registers (4 registers per chunk instead of 8 fp32), so that a thread has CPT (forward: 2*CPT, two rows
// per trip) independent 16-byte loads in flight and the row reduction is a pure shuffle: no shared memory and no
// CTA barrier inside the row loop. That is what keeps enough bytes in flight per SM to cover HBM latency.
// Same fp32 expression trees as the general kernels in rmsnorm.cu.
#pragma once

namespace warp_rows {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <typename T>
__device__ __forceinline__ void unpack8(float (&out)[8], const uint4& raw) {
    Pack<T, 8> pk;
    *reinterpret_cast<uint4*>(&pk) = raw;
    unpack_pack(out, pk);
}

// Makes the packed registers opaque to the optimiser, so that it unpacks them again where they are used next
// instead of keeping the fp32 copies of an earlier use alive (8 registers instead of 4 per chunk).
__device__ __forceinline__ void keep_packed(uint4& v) { asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)); }

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&in)[8]) {
    Pack<T, 8> pk;
#pragma unroll
    for (int i = 0; i < 8; ++i) pk.v[i] = from_f32<T>(in[i]);
    return *reinterpret_cast<const uint4*>(&pk);
}

// y = x * rsqrt(mean(x^2) + eps) * w, two rows per warp per trip.
template <typename T, int CPT>
__global__ void __launch_bounds__(kThreads)
rmsnorm_forward_warp_kernel(T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ w, long long rows, int hidden,
                            float epsilon) {
    constexpr int R = 2;
    const int lane = threadIdx.x & 31;
    const long long warp_id = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const long long warps_total = static_cast<long long>(gridDim.x) * kWarps;
    const float inv_hidden = 1.0f / static_cast<float>(hidden);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    uint4 wp[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int col = (c * 32 + lane) * 8;
        wp[c] = col < hidden ? *reinterpret_cast<const uint4*>(w + col) : zero;
    }
    for (long long row0 = warp_id * R; row0 < rows; row0 += warps_total * R) {
        uint4 xp[R][CPT];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const long long row = row0 + r;
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int col = (c * 32 + lane) * 8;
                xp[r][c] = (row < rows && col < hidden) ? __ldcs(reinterpret_cast<const uint4*>(x + row * hidden + col)) : zero;
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
                    if (col < hidden) {
                        float xv[8], wv[8], out[8];
                        unpack8<T>(xv, xp[r][c]);
                        unpack8<T>(wv, wp[c]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) out[i] = xv[i] * inv * wv[i];
                        *reinterpret_cast<uint4*>(y + row * hidden + col) = pack8<T>(out);
                    }
                }
            }
        }
    }
}

// dx = dy*w*inv - x*c (+ residuals), per-CTA dw partial row in dw_partial[blockIdx.x][hidden].
template <typename T, int CPT>
__global__ void __launch_bounds__(kThreads, 2)
rmsnorm_backward_warp_kernel(T* dx, float* __restrict__ dw_partial, const T* __restrict__ dy,   // dx may alias res_a / res_b
                             const T* __restrict__ x, const T* __restrict__ w, const T* res_a,
                             const T* res_b, long long rows, int hidden, float epsilon) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long warp_id = static_cast<long long>(blockIdx.x) * kWarps + warp;
    const long long warps_total = static_cast<long long>(gridDim.x) * kWarps;
    const float inv_hidden = 1.0f / static_cast<float>(hidden);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // The thread's CPT*8 running dw sums live in shared memory (its own float4 slots: conflict-free, no
    // synchronisation): 32 fp32 registers fewer, which is what lets two CTAs of 256 threads share an SM.
    extern __shared__ float4 dw_slots[];   // [CPT * 2][kThreads]
    uint4 wp[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int col = (c * 32 + lane) * 8;
        wp[c] = col < hidden ? *reinterpret_cast<const uint4*>(w + col) : zero;
        dw_slots[(c * 2) * kThreads + threadIdx.x] = make_float4(0.f, 0.f, 0.f, 0.f);
        dw_slots[(c * 2 + 1) * kThreads + threadIdx.x] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (long long row = warp_id; row < rows; row += warps_total) {
        // one 64-bit offset per row; the chunk index only adds a compile-time constant to each address
        const long long off = row * hidden + lane * 8;
        const T* xr = x + off;
        const T* gr = dy + off;
        const T* ar = res_a != nullptr ? res_a + off : nullptr;
        const T* br = res_b != nullptr ? res_b + off : nullptr;
        T* outr = dx + off;
        uint4 xp[CPT], gp[CPT], rp[CPT];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const bool in = c * 256 + lane * 8 < hidden;
            xp[c] = in ? __ldcs(reinterpret_cast<const uint4*>(xr + c * 256)) : zero;
            gp[c] = in ? __ldcs(reinterpret_cast<const uint4*>(gr + c * 256)) : zero;
        }
        float sx = 0.f, sg = 0.f;   // sum x^2, sum dy*w*x
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            float xv[8], gv[8], wv[8];
            unpack8<T>(xv, xp[c]);
            unpack8<T>(gv, gp[c]);
            unpack8<T>(wv, wp[c]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sx = fmaf(xv[i], xv[i], sx);
                sg = fmaf(gv[i] * wv[i], xv[i], sg);
            }
        }
        // the residual is only needed for the output: fetch it while the shuffles of the row sums run
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            keep_packed(xp[c]);
            keep_packed(gp[c]);
            rp[c] = (ar != nullptr && c * 256 + lane * 8 < hidden) ? __ldcs(reinterpret_cast<const uint4*>(ar + c * 256)) : zero;
        }
        sx = warp_sum(sx);
        sg = warp_sum(sg);
        const float inv = rsqrtf(sx * inv_hidden + epsilon);
        const float corr = sg * inv_hidden * inv * inv * inv;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            if (c * 256 + lane * 8 < hidden) {
                float xv[8], gv[8], wv[8], out[8];
                unpack8<T>(xv, xp[c]);
                unpack8<T>(gv, gp[c]);
                unpack8<T>(wv, wp[c]);
                float4 a0 = dw_slots[(c * 2) * kThreads + threadIdx.x], a1 = dw_slots[(c * 2 + 1) * kThreads + threadIdx.x];
#pragma unroll
                for (int i = 0; i < 8; ++i) out[i] = fmaf(-xv[i], corr, gv[i] * wv[i] * inv);
                a0.x = fmaf(gv[0], xv[0] * inv, a0.x); a0.y = fmaf(gv[1], xv[1] * inv, a0.y);
                a0.z = fmaf(gv[2], xv[2] * inv, a0.z); a0.w = fmaf(gv[3], xv[3] * inv, a0.w);
                a1.x = fmaf(gv[4], xv[4] * inv, a1.x); a1.y = fmaf(gv[5], xv[5] * inv, a1.y);
                a1.z = fmaf(gv[6], xv[6] * inv, a1.z); a1.w = fmaf(gv[7], xv[7] * inv, a1.w);
                dw_slots[(c * 2) * kThreads + threadIdx.x] = a0;
                dw_slots[(c * 2 + 1) * kThreads + threadIdx.x] = a1;
                if (ar != nullptr) {
                    float rv[8];
                    unpack8<T>(rv, rp[c]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) out[i] += rv[i];
                }
                if (br != nullptr) {
                    float rv[8];
                    unpack8<T>(rv, __ldcs(reinterpret_cast<const uint4*>(br + c * 256)));
#pragma unroll
                    for (int i = 0; i < 8; ++i) out[i] += rv[i];
                }
                *reinterpret_cast<uint4*>(outr + c * 256) = pack8<T>(out);
            }
        }
    }

    // Combine the CTA's 8 warps in a fixed order: one fp32 partial row per CTA. Column (c*32 + l)*8 + i is element
    // i of slot pair c of lane l in every warp.
    __syncthreads();
    const float* slots = reinterpret_cast<const float*>(dw_slots);
    for (int col = threadIdx.x; col < hidden; col += kThreads) {
        const int c = col >> 8, l = (col >> 3) & 31, i = col & 7;
        float acc = 0.f;
#pragma unroll
        for (int wi = 0; wi < kWarps; ++wi) acc += slots[(((c * 2 + (i >> 2)) * kThreads) + wi * 32 + l) * 4 + (i & 3)];
        dw_partial[static_cast<long long>(blockIdx.x) * hidden + col] = acc;
    }
}

// dw[col] = sum over `parts` partial rows in a fixed order: 32 row lanes per column, then a shared-memory combine.
template <typename T>
__global__ void __launch_bounds__(1024)
dw_reduce_wide_kernel(T* __restrict__ dw, const float* __restrict__ partial, int parts, int hidden) {
    __shared__ float tile[32][33];
    const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + cl;
    float acc = 0.f;
    if (col < hidden)
        for (int p = rl; p < parts; p += 32) acc += partial[static_cast<long long>(p) * hidden + col];
    tile[rl][cl] = acc;
    __syncthreads();
    if (rl == 0 && col < hidden) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) total += tile[r][cl];
        dw[col] = from_f32<T>(total);
    }
}

// Diagnosis builds only: CGPT_B200_RMS_WARP=0 routes these shapes through the general kernels instead.
inline bool applicable(std::size_t hidden, int vec, std::size_t elem_size) {
    static const bool enabled = [] {
        const char* e = diagnosis_env("CGPT_B200_RMS_WARP");
        return !(e != nullptr && e[0] == '0');
    }();
    return enabled && elem_size == 2 && vec == 8 && hidden >= 256 && hidden <= 1024;
}

}  // namespace warp_rows
