// RoPE forward (in place) and backward (inverse rotation) on adjacent pairs, for sm_100a.
//
// Pair convention and fp32 expression trees follow the reference:
//   forward   y0 = fma(-x1, s, x0*c),  y1 = fma(x0, s, x1*c)        (src/ops/rope.cu:133-134)
//   backward  dx0 = fma(dy1, s, dy0*c), dx1 = fma(-dy0, s, dy1*c)   (src/ops/backward/rope_backward.cu:94-105)
// with c/s read from tables [max_seq, rotary_dim/2] stored in the tensors' dtype at row
// (position_offset + s). Dims >= rotary_dim are copied (backward) or left alone (forward).
//
// Memory-bound: one thread moves one 16-byte chunk (8 halves = 4 pairs, or 4 floats = 2 pairs) of a
// head and reads the matching 8 (4) table bytes; q and k heads of a token are covered by the same
// launch. A scalar kernel handles unaligned shapes. Algorithmic HBM bytes: 2 * elements * sizeof(T)
// (+ the tables, which stay in L2).
#include "common.cuh"
#include "launch_counter.h"

namespace cgpt {
namespace {

template <typename T, int VEC, bool BACKWARD>
__global__ void __launch_bounds__(256)
rope_vec_kernel(T* out_q, T* out_k, const T* in_q,
                const T* in_k, const T* __restrict__ cos_t, const T* __restrict__ sin_t,
                long long tokens, int seq, int q_heads, int kv_heads, int head_dim, int rotary_dim,
                int position_offset) {
    const int chunks_per_head = head_dim / VEC;
    const int heads = q_heads + kv_heads;
    const long long total = tokens * heads * chunks_per_head;
    const int half_rot = rotary_dim / 2;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int chunk = static_cast<int>(idx % chunks_per_head);
        const long long th = idx / chunks_per_head;
        const int head = static_cast<int>(th % heads);
        const long long token = th / heads;
        const int d0 = chunk * VEC;
        const bool is_q = head < q_heads;
        const long long off = is_q
            ? (token * q_heads + head) * static_cast<long long>(head_dim) + d0
            : (token * kv_heads + (head - q_heads)) * static_cast<long long>(head_dim) + d0;
        const T* src = (is_q ? in_q : in_k) + off;
        T* dst = (is_q ? out_q : out_k) + off;
        if (d0 >= rotary_dim) {
            if (BACKWARD && src != dst) {
                float v[VEC];
                load_vec_stream<T, VEC>(v, src);
                store_vec<T, VEC>(dst, v);
            }
            continue;
        }
        const int pos = static_cast<int>(token % seq) + position_offset;
        float v[VEC], c[VEC / 2], s[VEC / 2], o[VEC];
        load_vec_stream<T, VEC>(v, src);
        load_vec<T, VEC / 2>(c, cos_t + static_cast<long long>(pos) * half_rot + d0 / 2);
        load_vec<T, VEC / 2>(s, sin_t + static_cast<long long>(pos) * half_rot + d0 / 2);
#pragma unroll
        for (int p = 0; p < VEC / 2; ++p) {
            const float a = v[2 * p], b = v[2 * p + 1];
            if (BACKWARD) {
                o[2 * p] = fmaf(b, s[p], a * c[p]);
                o[2 * p + 1] = fmaf(-a, s[p], b * c[p]);
            } else {
                o[2 * p] = fmaf(-b, s[p], a * c[p]);
                o[2 * p + 1] = fmaf(a, s[p], b * c[p]);
            }
        }
        store_vec<T, VEC>(dst, o);
    }
}

// One thread per pair (or per tail element). Any head_dim, any even rotary_dim.
template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(256)
rope_scalar_kernel(T* out_q, T* out_k, const T* in_q,
                   const T* in_k, const T* __restrict__ cos_t, const T* __restrict__ sin_t,
                   long long tokens, int seq, int q_heads, int kv_heads, int head_dim, int rotary_dim,
                   int position_offset) {
    const int half_rot = rotary_dim / 2;
    const int units = half_rot + (head_dim - rotary_dim);  // pairs, then single tail elements
    const int heads = q_heads + kv_heads;
    const long long total = tokens * heads * units;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int unit = static_cast<int>(idx % units);
        const long long th = idx / units;
        const int head = static_cast<int>(th % heads);
        const long long token = th / heads;
        const bool is_q = head < q_heads;
        const long long base = is_q ? (token * q_heads + head) * static_cast<long long>(head_dim)
                                    : (token * kv_heads + (head - q_heads)) * static_cast<long long>(head_dim);
        const T* src = (is_q ? in_q : in_k) + base;
        T* dst = (is_q ? out_q : out_k) + base;
        if (unit >= half_rot) {
            const int d = rotary_dim + (unit - half_rot);
            if (BACKWARD && src != dst) dst[d] = src[d];
            continue;
        }
        const int pos = static_cast<int>(token % seq) + position_offset;
        const float c = to_f32<T>(cos_t[static_cast<long long>(pos) * half_rot + unit]);
        const float s = to_f32<T>(sin_t[static_cast<long long>(pos) * half_rot + unit]);
        const float a = to_f32<T>(src[2 * unit]), b = to_f32<T>(src[2 * unit + 1]);
        if (BACKWARD) {
            dst[2 * unit] = from_f32<T>(fmaf(b, s, a * c));
            dst[2 * unit + 1] = from_f32<T>(fmaf(-a, s, b * c));
        } else {
            dst[2 * unit] = from_f32<T>(fmaf(-b, s, a * c));
            dst[2 * unit + 1] = from_f32<T>(fmaf(a, s, b * c));
        }
    }
}

template <bool BACKWARD>
int rope_dispatch(void* oq, void* ok, const void* iq, const void* ik, const void* cos_t, const void* sin_t,
                  size_t batch, size_t seq, size_t q_heads, size_t kv_heads, size_t head_dim,
                  size_t rotary_dim, size_t position_offset, size_t max_seq, int dtype, cudaStream_t s) {
    if (!oq || !ok || !iq || !ik || !cos_t || !sin_t) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rotary_dim == 0) rotary_dim = head_dim;
    if (batch == 0 || seq == 0 || q_heads == 0 || kv_heads == 0 || head_dim == 0) return CGPT_ERR_SHAPE;
    if (rotary_dim > head_dim || (rotary_dim & 1u) != 0) return CGPT_ERR_OPTION;
    if (position_offset + seq > max_seq) return CGPT_ERR_SHAPE;
    if (seq > 0x7fffffffull || head_dim > 0x7fffffffull || q_heads + kv_heads > 0x7fffffffull ||
        max_seq > 0x7fffffffull || batch > (1ull << 40) / seq)
        return CGPT_ERR_SHAPE;
    const long long tokens = static_cast<long long>(batch * seq);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        constexpr int VEC = 16 / sizeof(T);
        const bool vec_ok = head_dim % VEC == 0 && rotary_dim % VEC == 0 && aligned16(oq) && aligned16(ok) &&
                            aligned16(iq) && aligned16(ik) &&
                            (reinterpret_cast<std::uintptr_t>(cos_t) % (sizeof(T) * VEC / 2)) == 0 &&
                            (reinterpret_cast<std::uintptr_t>(sin_t) % (sizeof(T) * VEC / 2)) == 0;
        const long long units = vec_ok
            ? tokens * static_cast<long long>(q_heads + kv_heads) * static_cast<long long>(head_dim / VEC)
            : tokens * static_cast<long long>(q_heads + kv_heads) *
                  static_cast<long long>(rotary_dim / 2 + head_dim - rotary_dim);
        long long blocks = (units + 255) / 256;
        const long long cap = static_cast<long long>(kNumSMs) * 16;
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        if (vec_ok) {
            rope_vec_kernel<T, VEC, BACKWARD><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
                static_cast<T*>(oq), static_cast<T*>(ok), static_cast<const T*>(iq), static_cast<const T*>(ik),
                static_cast<const T*>(cos_t), static_cast<const T*>(sin_t), tokens, static_cast<int>(seq),
                static_cast<int>(q_heads), static_cast<int>(kv_heads), static_cast<int>(head_dim),
                static_cast<int>(rotary_dim), static_cast<int>(position_offset));
        } else {
            rope_scalar_kernel<T, BACKWARD><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
                static_cast<T*>(oq), static_cast<T*>(ok), static_cast<const T*>(iq), static_cast<const T*>(ik),
                static_cast<const T*>(cos_t), static_cast<const T*>(sin_t), tokens, static_cast<int>(seq),
                static_cast<int>(q_heads), static_cast<int>(kv_heads), static_cast<int>(head_dim),
                static_cast<int>(rotary_dim), static_cast<int>(position_offset));
        }
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}

}  // namespace
}  // namespace cgpt

extern "C" int cgpt_rope_forward(void* q, void* k, const void* cos_table, const void* sin_table, size_t batch,
                                 size_t seq, size_t q_heads, size_t kv_heads, size_t head_dim,
                                 size_t rotary_dim, size_t position_offset, size_t max_seq, int dtype,
                                 cgpt_stream_t stream) {
    return cgpt::rope_dispatch<false>(q, k, q, k, cos_table, sin_table, batch, seq, q_heads, kv_heads, head_dim,
                                      rotary_dim, position_offset, max_seq, dtype,
                                      static_cast<cudaStream_t>(stream));
}

extern "C" int cgpt_rope_backward(void* dq, void* dk, const void* dq_rot, const void* dk_rot,
                                  const void* cos_table, const void* sin_table, size_t batch, size_t seq,
                                  size_t q_heads, size_t kv_heads, size_t head_dim, size_t rotary_dim,
                                  size_t position_offset, size_t max_seq, int dtype, cgpt_stream_t stream) {
    return cgpt::rope_dispatch<true>(dq, dk, dq_rot, dk_rot, cos_table, sin_table, batch, seq, q_heads,
                                     kv_heads, head_dim, rotary_dim, position_offset, max_seq, dtype,
                                     static_cast<cudaStream_t>(stream));
}
