// Generic (any dtype, any head_dim <= 256, any GQA ratio, causal or not, Sq != Sk with an offset)
// attention forward and backward: the correctness path behind the tensor-core kernels, which only take
// 16-bit tensors with head_dim 64 or 128. One warp owns one row; all sums are fp32 and nothing is
// accumulated with atomics, so results are bit-reproducible.
//
// Reference semantics (src/ops/attention.cu:669-690, src/ops/backward/attention_backward.cu:352-504):
//   visible keys of query q: k <= offset + q (causal) or all; scale = attention_scale > 0 ? it : 1/sqrt(D)
//   P = exp(scale*QK^T - LSE), LSE = max + log(sum exp(s - max)) (natural log, scale included)
//   delta = rowsum(dO * O); dS = P * (dP - delta), dP = dO V^T
//   dQ = scale * dS K;  dK = scale * dS^T Q;  dV = P^T dO
#include <math_constants.h>

#include "attention.h"
#include "launch_counter.h"

namespace cgpt {
namespace {

constexpr int kMaxRegs = 8;  // head_dim <= 256: each lane holds ceil(D/32) <= 8 elements
constexpr int kWarpsPerCta = 4;

template <typename T>
__device__ __forceinline__ void load_row(float (&r)[kMaxRegs], const T* __restrict__ p, int d, int lane) {
#pragma unroll
    for (int i = 0; i < kMaxRegs; ++i) {
        const int c = lane + 32 * i;
        r[i] = c < d ? to_f32<T>(p[c]) : 0.f;
    }
}
__device__ __forceinline__ float dot_rows(const float (&a)[kMaxRegs], const float (&b)[kMaxRegs]) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxRegs; ++i) s = fmaf(a[i], b[i], s);
    return warp_sum(s);
}

// Forward: O (type TO) and LSE for one (b, q, h) row per warp.
template <typename T, typename TO>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
attention_forward_generic(TO* __restrict__ out, float* __restrict__ lse, const T* __restrict__ q,
                          const T* __restrict__ k, const T* __restrict__ v, AttnDims dm) {
    const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const long long rows = static_cast<long long>(dm.batch) * dm.sq * dm.hq;
    if (row >= rows) return;
    const int h = static_cast<int>(row % dm.hq);
    const int qi = static_cast<int>((row / dm.hq) % dm.sq);
    const int b = static_cast<int>(row / (static_cast<long long>(dm.hq) * dm.sq));
    const int kvh = h / (dm.hq / dm.hkv);
    int visible = dm.causal ? dm.offset + qi + 1 : dm.sk;
    if (visible > dm.sk) visible = dm.sk;
    float qr[kMaxRegs], acc[kMaxRegs];
    load_row(qr, q + row * dm.d, dm.d, lane);
#pragma unroll
    for (int i = 0; i < kMaxRegs; ++i) acc[i] = 0.f;
    float m = -CUDART_INF_F, l = 0.f;
    const long long kv_base = (static_cast<long long>(b) * dm.sk * dm.hkv + kvh) * dm.d;
    const long long kv_step = static_cast<long long>(dm.hkv) * dm.d;
    for (int kp = 0; kp < visible; ++kp) {
        float kr[kMaxRegs], vr[kMaxRegs];
        load_row(kr, k + kv_base + kp * kv_step, dm.d, lane);
        load_row(vr, v + kv_base + kp * kv_step, dm.d, lane);
        const float s = dot_rows(qr, kr) * dm.scale;
        const float m_new = fmaxf(m, s);
        const float alpha = __expf(m - m_new);
        const float p = __expf(s - m_new);
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < kMaxRegs; ++i) acc[i] = fmaf(p, vr[i], acc[i] * alpha);
        m = m_new;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < kMaxRegs; ++i) {
        const int c = lane + 32 * i;
        if (c < dm.d) out[row * dm.d + c] = from_f32<TO>(acc[i] * inv);
    }
    if (lane == 0 && lse != nullptr) lse[row] = l > 0.f ? m + logf(l) : -CUDART_INF_F;
}

// delta[row] = sum_d dO * O
template <typename T, typename TO>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
attention_delta_generic(float* __restrict__ delta, const T* __restrict__ dout, const TO* __restrict__ out,
                        long long rows, int d) {
    const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) s = fmaf(to_f32<T>(dout[row * d + c]), to_f32<TO>(out[row * d + c]), s);
    s = warp_sum(s);
    if (lane == 0) delta[row] = s;
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
attention_dq_generic(T* __restrict__ dq, const T* __restrict__ dout, const float* __restrict__ lse,
                     const float* __restrict__ delta, const T* __restrict__ q, const T* __restrict__ k,
                     const T* __restrict__ v, AttnDims dm, int accumulate) {
    const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const long long rows = static_cast<long long>(dm.batch) * dm.sq * dm.hq;
    if (row >= rows) return;
    const int h = static_cast<int>(row % dm.hq);
    const int qi = static_cast<int>((row / dm.hq) % dm.sq);
    const int b = static_cast<int>(row / (static_cast<long long>(dm.hq) * dm.sq));
    const int kvh = h / (dm.hq / dm.hkv);
    int visible = dm.causal ? dm.offset + qi + 1 : dm.sk;
    if (visible > dm.sk) visible = dm.sk;
    float qr[kMaxRegs], gr[kMaxRegs], acc[kMaxRegs];
    load_row(qr, q + row * dm.d, dm.d, lane);
    load_row(gr, dout + row * dm.d, dm.d, lane);
#pragma unroll
    for (int i = 0; i < kMaxRegs; ++i) acc[i] = 0.f;
    const float row_lse = lse[row], row_delta = delta[row];
    const long long kv_base = (static_cast<long long>(b) * dm.sk * dm.hkv + kvh) * dm.d;
    const long long kv_step = static_cast<long long>(dm.hkv) * dm.d;
    for (int kp = 0; kp < visible; ++kp) {
        float kr[kMaxRegs], vr[kMaxRegs];
        load_row(kr, k + kv_base + kp * kv_step, dm.d, lane);
        load_row(vr, v + kv_base + kp * kv_step, dm.d, lane);
        const float s = dot_rows(qr, kr) * dm.scale;
        const float p = __expf(s - row_lse);
        const float dp = dot_rows(gr, vr);
        const float ds = p * (dp - row_delta) * dm.scale;
#pragma unroll
        for (int i = 0; i < kMaxRegs; ++i) acc[i] = fmaf(ds, kr[i], acc[i]);
    }
#pragma unroll
    for (int i = 0; i < kMaxRegs; ++i) {
        const int c = lane + 32 * i;
        if (c < dm.d) {
            float val = acc[i];
            if (accumulate) val += to_f32<T>(dq[row * dm.d + c]);
            dq[row * dm.d + c] = from_f32<T>(val);
        }
    }
}

// One warp per (b, key position, kv head): sums over the query heads of its group and the query rows
// that can see the key, in a fixed order.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
attention_dkv_generic(T* __restrict__ dk, T* __restrict__ dv, const T* __restrict__ dout,
                      const float* __restrict__ lse, const float* __restrict__ delta, const T* __restrict__ q,
                      const T* __restrict__ k, const T* __restrict__ v, AttnDims dm, int accumulate) {
    const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const long long rows = static_cast<long long>(dm.batch) * dm.sk * dm.hkv;
    if (row >= rows) return;
    const int kvh = static_cast<int>(row % dm.hkv);
    const int kp = static_cast<int>((row / dm.hkv) % dm.sk);
    const int b = static_cast<int>(row / (static_cast<long long>(dm.hkv) * dm.sk));
    const int ratio = dm.hq / dm.hkv;
    float kr[kMaxRegs], vr[kMaxRegs], acc_k[kMaxRegs], acc_v[kMaxRegs];
    load_row(kr, k + row * dm.d, dm.d, lane);
    load_row(vr, v + row * dm.d, dm.d, lane);
#pragma unroll
    for (int i = 0; i < kMaxRegs; ++i) { acc_k[i] = 0.f; acc_v[i] = 0.f; }
    int q_first = dm.causal ? kp - dm.offset : 0;
    if (q_first < 0) q_first = 0;
    for (int qi = q_first; qi < dm.sq; ++qi) {
        for (int g = 0; g < ratio; ++g) {
            const int h = kvh * ratio + g;
            const long long qrow = (static_cast<long long>(b) * dm.sq + qi) * dm.hq + h;
            float qr[kMaxRegs], gr[kMaxRegs];
            load_row(qr, q + qrow * dm.d, dm.d, lane);
            load_row(gr, dout + qrow * dm.d, dm.d, lane);
            const float s = dot_rows(qr, kr) * dm.scale;
            const float p = __expf(s - lse[qrow]);
            const float dp = dot_rows(gr, vr);
            const float ds = p * (dp - delta[qrow]) * dm.scale;
#pragma unroll
            for (int i = 0; i < kMaxRegs; ++i) {
                acc_k[i] = fmaf(ds, qr[i], acc_k[i]);
                acc_v[i] = fmaf(p, gr[i], acc_v[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kMaxRegs; ++i) {
        const int c = lane + 32 * i;
        if (c < dm.d) {
            float a = acc_k[i], bb = acc_v[i];
            if (accumulate) { a += to_f32<T>(dk[row * dm.d + c]); bb += to_f32<T>(dv[row * dm.d + c]); }
            dk[row * dm.d + c] = from_f32<T>(a);
            dv[row * dm.d + c] = from_f32<T>(bb);
        }
    }
}

inline unsigned warp_grid(long long rows) { return static_cast<unsigned>((rows + kWarpsPerCta - 1) / kWarpsPerCta); }

}  // namespace

int attention_forward_generic_launch(void* out, float* lse, const void* q, const void* k, const void* v,
                                     const AttnDims& dm, int dtype, cudaStream_t s) {
    const long long rows = static_cast<long long>(dm.batch) * dm.sq * dm.hq;
    CGPT_DISPATCH_DTYPE(dtype, T, {
        attention_forward_generic<T, T><<<warp_grid(rows), kWarpsPerCta * 32, 0, s>>>(
            static_cast<T*>(out), lse, static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), dm);
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}

int attention_backward_generic_launch(void* dq, void* dk, void* dv, const void* dout, const void* out,
                                      const float* lse, const void* q, const void* k, const void* v,
                                      const AttnDims& dm, int accumulate, int dtype, cudaStream_t s) {
    const long long qrows = static_cast<long long>(dm.batch) * dm.sq * dm.hq;
    const long long krows = static_cast<long long>(dm.batch) * dm.sk * dm.hkv;
    // scratch: delta[qrows] (+ lse[qrows] + fp32 O[qrows, d] when no saved statistics were given)
    const bool need_stats = out == nullptr || lse == nullptr;
    std::size_t bytes = static_cast<std::size_t>(qrows) * sizeof(float);
    if (need_stats) bytes += static_cast<std::size_t>(qrows) * sizeof(float) * (1 + dm.d);
    void* scratch = nullptr;
    CGPT_TRY(scratch_get(&scratch, bytes, s));
    float* delta = static_cast<float*>(scratch);
    float* lse_buf = delta + qrows;
    float* o_buf = lse_buf + qrows;
    CGPT_DISPATCH_DTYPE(dtype, T, {
        if (need_stats) {
            attention_forward_generic<T, float><<<warp_grid(qrows), kWarpsPerCta * 32, 0, s>>>(
                o_buf, lse_buf, static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), dm);
            count_launch();
            CGPT_LAUNCH_CHECK();
            attention_delta_generic<T, float><<<warp_grid(qrows), kWarpsPerCta * 32, 0, s>>>(
                delta, static_cast<const T*>(dout), o_buf, qrows, dm.d);
            lse = lse_buf;
        } else {
            attention_delta_generic<T, T><<<warp_grid(qrows), kWarpsPerCta * 32, 0, s>>>(
                delta, static_cast<const T*>(dout), static_cast<const T*>(out), qrows, dm.d);
        }
        count_launch();
        CGPT_LAUNCH_CHECK();
        attention_dq_generic<T><<<warp_grid(qrows), kWarpsPerCta * 32, 0, s>>>(
            static_cast<T*>(dq), static_cast<const T*>(dout), lse, delta, static_cast<const T*>(q),
            static_cast<const T*>(k), static_cast<const T*>(v), dm, accumulate);
        count_launch();
        CGPT_LAUNCH_CHECK();
        attention_dkv_generic<T><<<warp_grid(krows), kWarpsPerCta * 32, 0, s>>>(
            static_cast<T*>(dk), static_cast<T*>(dv), static_cast<const T*>(dout), lse, delta, static_cast<const T*>(q),
            static_cast<const T*>(k), static_cast<const T*>(v), dm, accumulate);
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}

}  // namespace cgpt
