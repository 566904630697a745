// Fused per-head QK-RMSNorm + RoPE, forward and backward, for sm_100a.
//
// The reference runs these as separate passes over the [tokens*heads, head_dim] query/key tensors
// (src/core/transformer_block.cu:496-521 forward: rmsnorm_forward on q and k, then rope_forward; :705-720 backward:
// rope_backward, then rmsnorm_backward for q and for k). Fused, every element is read and written once:
//   forward   y = RoPE(x * rsqrt(mean(x^2)+eps) * w)
//   backward  g = RoPE^-1(dy);  c = sum(g*w*x)/D * inv^3;  dx = g*w*inv - x*c;  dw += g * x * inv
// with the same fp32 expression trees as rmsnorm.cu and rope.cu. Memory-bound: 2 x 16-bit bytes per element
// forward, 3 x backward (dy, x read; dx written). head_dim/8 lanes own one row (16-byte chunks), so a warp
// handles 32/(head_dim/8) rows at a time; the per-lane dw partial sums stay in registers over the row loop and are
// combined in a fixed order (CTA partials in scratch, then a small reduce kernel): deterministic.
// Fast path only: 16-bit dtype, head_dim a power of two in [8, 256], rotary_dim a multiple of 8.
#include "common.cuh"
#include "launch_counter.h"

namespace cgpt {
namespace {

constexpr int kQkThreads = 256;

__device__ __forceinline__ float group_sum(float v, int lanes_per_row) {
    for (int o = lanes_per_row >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct QkDims {
    long long tokens;   // batch * seq
    int seq, q_heads, kv_heads, head_dim, rotary_dim, offset;
    float eps;
};

// Row r in [0, tokens*(q_heads+kv_heads)): token = r / heads, head = r % heads; heads < q_heads are query heads.
template <typename T, bool BACKWARD>
__global__ void __launch_bounds__(kQkThreads)
qknorm_rope_kernel(T* __restrict__ out_q, T* __restrict__ out_k, const T* __restrict__ in_q, const T* __restrict__ in_k,
                   const T* __restrict__ x_q, const T* __restrict__ x_k, const T* __restrict__ w_q, const T* __restrict__ w_k,
                   const T* __restrict__ cos_t, const T* __restrict__ sin_t, float* __restrict__ dw_partial, QkDims dm) {
    const int lpr = dm.head_dim / 8;                 // lanes per row
    const int rows_per_warp = 32 / lpr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / lpr, l = lane % lpr;      // row slot inside the warp, chunk inside the row
    const int heads = dm.q_heads + dm.kv_heads;
    const long long rows = dm.tokens * heads;
    const int d0 = l * 8;
    const float inv_d = 1.0f / static_cast<float>(dm.head_dim);
    const int half_rot = dm.rotary_dim / 2;

    float wq[8], wk[8], dwq[8], dwk[8];
    load_vec<T, 8>(wq, w_q + d0);
    load_vec<T, 8>(wk, w_k + d0);
#pragma unroll
    for (int i = 0; i < 8; ++i) { dwq[i] = 0.f; dwk[i] = 0.f; }

    const long long warps_total = static_cast<long long>(gridDim.x) * (kQkThreads / 32);
    const long long warp_id = static_cast<long long>(blockIdx.x) * (kQkThreads / 32) + warp;
    for (long long base = warp_id * rows_per_warp; base < rows; base += warps_total * rows_per_warp) {
        const long long r = base + sub;
        const bool active = r < rows;
        const long long token = active ? r / heads : 0;
        const int head = active ? static_cast<int>(r % heads) : 0;
        const bool is_q = head < dm.q_heads;
        const long long off = is_q ? (token * dm.q_heads + head) * dm.head_dim + d0
                                   : (token * dm.kv_heads + (head - dm.q_heads)) * dm.head_dim + d0;
        float c[4], s[4];
        const bool rotate = d0 < dm.rotary_dim;
        if (active && rotate) {
            const int pos = static_cast<int>(token % dm.seq) + dm.offset;
            load_vec<T, 4>(c, cos_t + static_cast<long long>(pos) * half_rot + d0 / 2);
            load_vec<T, 4>(s, sin_t + static_cast<long long>(pos) * half_rot + d0 / 2);
        }
        if (!BACKWARD) {
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = 0.f;
            if (active) load_vec_stream<T, 8>(x, (is_q ? in_q : in_k) + off);
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
            ss = group_sum(ss, lpr);
            const float inv = rsqrtf(ss * inv_d + dm.eps);
            float y[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                // the reference rounds the normalised value to the storage dtype before RoPE reads it
                y[i] = to_f32<T>(from_f32<T>(x[i] * inv * (is_q ? wq[i] : wk[i])));
            }
            if (rotate) {
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float a = y[2 * p], b = y[2 * p + 1];
                    y[2 * p] = fmaf(-b, s[p], a * c[p]);
                    y[2 * p + 1] = fmaf(a, s[p], b * c[p]);
                }
            }
            if (active) store_vec<T, 8>((is_q ? out_q : out_k) + off, y);
        } else {
            float g[8], x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { g[i] = 0.f; x[i] = 0.f; }
            if (active) {
                load_vec_stream<T, 8>(g, (is_q ? in_q : in_k) + off);
                load_vec_stream<T, 8>(x, (is_q ? x_q : x_k) + off);
            }
            if (rotate) {
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float a = g[2 * p], b = g[2 * p + 1];
                    // the reference rounds the un-rotated gradient to the storage dtype (output of rope_backward)
                    g[2 * p] = to_f32<T>(from_f32<T>(fmaf(b, s[p], a * c[p])));
                    g[2 * p + 1] = to_f32<T>(from_f32<T>(fmaf(-a, s[p], b * c[p])));
                }
            }
            float sx = 0.f, sg = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sx = fmaf(x[i], x[i], sx);
                sg = fmaf(g[i] * (is_q ? wq[i] : wk[i]), x[i], sg);
            }
            sx = group_sum(sx, lpr);
            sg = group_sum(sg, lpr);
            const float inv = rsqrtf(sx * inv_d + dm.eps);
            const float corr = sg * inv_d * inv * inv * inv;
            float dx[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                dx[i] = fmaf(-x[i], corr, g[i] * (is_q ? wq[i] : wk[i]) * inv);
                const float contrib = g[i] * (x[i] * inv);
                if (is_q) dwq[i] += contrib; else dwk[i] += contrib;
            }
            if (active) store_vec<T, 8>((is_q ? out_q : out_k) + off, dx);
        }
    }

    if (BACKWARD) {
        // Combine lanes that own the same columns (fixed order), then one partial row per CTA: [grid][2][head_dim].
        __shared__ float red[kQkThreads][9];
        for (int which = 0; which < 2; ++which) {
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; ++i) red[threadIdx.x][i] = which == 0 ? dwq[i] : dwk[i];
            __syncthreads();
            if (threadIdx.x < lpr) {
                for (int i = 0; i < 8; ++i) {
                    float acc = 0.f;
                    for (int t = threadIdx.x; t < kQkThreads; t += lpr) acc += red[t][i];
                    dw_partial[(static_cast<long long>(blockIdx.x) * 2 + which) * dm.head_dim + threadIdx.x * 8 + i] = acc;
                }
            }
        }
    }
}

// dw[col] = sum of the per-CTA partials in a fixed order: 8 row lanes per column, then a shared-memory combine.
template <typename T>
__global__ void __launch_bounds__(256)
qknorm_dw_reduce_kernel(T* __restrict__ dw_q, T* __restrict__ dw_k, const float* __restrict__ partial, int parts, int head_dim) {
    __shared__ float tile[8][33];
    const int col = blockIdx.x * 32 + (threadIdx.x & 31);      // 0 .. 2*head_dim
    const int rl = threadIdx.x >> 5;
    float acc = 0.f;
    if (col < 2 * head_dim)
        for (int p = rl; p < parts; p += 8) acc += partial[static_cast<long long>(p) * 2 * head_dim + col];
    tile[rl][threadIdx.x & 31] = acc;
    __syncthreads();
    if (rl == 0 && col < 2 * head_dim) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) total += tile[r][threadIdx.x & 31];
        if (col < head_dim) dw_q[col] = from_f32<T>(total);
        else dw_k[col - head_dim] = from_f32<T>(total);
    }
}

bool fast_path_ok(size_t head_dim, size_t rotary_dim, int dtype, std::initializer_list<const void*> ptrs) {
    if (dtype == CGPT_DTYPE_F32) return false;
    if (head_dim < 8 || head_dim > 256 || (head_dim & (head_dim - 1)) != 0 || rotary_dim % 8 != 0) return false;
    for (const void* p : ptrs)
        if (!aligned16(p)) return false;
    return true;
}

}  // namespace
}  // namespace cgpt

using namespace cgpt;

extern "C" int cgpt_qknorm_rope_forward(void* q, void* k, const void* q_pre, const void* k_pre, const void* q_norm,
                                        const void* k_norm, const void* cos_table, const void* sin_table, size_t batch,
                                        size_t seq, size_t q_heads, size_t kv_heads, size_t head_dim, size_t rotary_dim,
                                        size_t position_offset, size_t max_seq, float epsilon, int dtype,
                                        cgpt_stream_t stream) {
    if (!q || !k || !q_pre || !k_pre || !q_norm || !k_norm || !cos_table || !sin_table) return CGPT_ERR_NULL;
    if (rotary_dim == 0) rotary_dim = head_dim;
    if (batch == 0 || seq == 0 || q_heads == 0 || kv_heads == 0 || head_dim == 0 || rotary_dim > head_dim ||
        position_offset + seq > max_seq || batch * seq > (1ull << 40))
        return CGPT_ERR_SHAPE;
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    if (!fast_path_ok(head_dim, rotary_dim, dtype, {q, k, q_pre, k_pre, q_norm, k_norm, cos_table, sin_table}))
        return CGPT_ERR_UNSUPPORTED;
    auto s = static_cast<cudaStream_t>(stream);
    const QkDims dm{static_cast<long long>(batch * seq), static_cast<int>(seq), static_cast<int>(q_heads),
                    static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<int>(rotary_dim),
                    static_cast<int>(position_offset), epsilon};
    const unsigned grid = kNumSMs * 8;
    if (dtype == CGPT_DTYPE_F16)
        qknorm_rope_kernel<__half, false><<<grid, kQkThreads, 0, s>>>(
            static_cast<__half*>(q), static_cast<__half*>(k), static_cast<const __half*>(q_pre), static_cast<const __half*>(k_pre),
            nullptr, nullptr, static_cast<const __half*>(q_norm), static_cast<const __half*>(k_norm),
            static_cast<const __half*>(cos_table), static_cast<const __half*>(sin_table), nullptr, dm);
    else
        qknorm_rope_kernel<__nv_bfloat16, false><<<grid, kQkThreads, 0, s>>>(
            static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(q_pre),
            static_cast<const __nv_bfloat16*>(k_pre), nullptr, nullptr, static_cast<const __nv_bfloat16*>(q_norm),
            static_cast<const __nv_bfloat16*>(k_norm), static_cast<const __nv_bfloat16*>(cos_table),
            static_cast<const __nv_bfloat16*>(sin_table), nullptr, dm);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

extern "C" int cgpt_qknorm_rope_backward(void* dq_pre, void* dk_pre, void* dq_norm, void* dk_norm, const void* dq_rot,
                                         const void* dk_rot, const void* q_pre, const void* k_pre, const void* q_norm,
                                         const void* k_norm, const void* cos_table, const void* sin_table, size_t batch,
                                         size_t seq, size_t q_heads, size_t kv_heads, size_t head_dim, size_t rotary_dim,
                                         size_t position_offset, size_t max_seq, float epsilon, int dtype,
                                         cgpt_stream_t stream) {
    if (!dq_pre || !dk_pre || !dq_norm || !dk_norm || !dq_rot || !dk_rot || !q_pre || !k_pre || !q_norm || !k_norm ||
        !cos_table || !sin_table)
        return CGPT_ERR_NULL;
    if (rotary_dim == 0) rotary_dim = head_dim;
    if (batch == 0 || seq == 0 || q_heads == 0 || kv_heads == 0 || head_dim == 0 || rotary_dim > head_dim ||
        position_offset + seq > max_seq || batch * seq > (1ull << 40))
        return CGPT_ERR_SHAPE;
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    if (!fast_path_ok(head_dim, rotary_dim, dtype, {dq_pre, dk_pre, dq_rot, dk_rot, q_pre, k_pre, q_norm, k_norm, cos_table, sin_table}))
        return CGPT_ERR_UNSUPPORTED;
    auto s = static_cast<cudaStream_t>(stream);
    const QkDims dm{static_cast<long long>(batch * seq), static_cast<int>(seq), static_cast<int>(q_heads),
                    static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<int>(rotary_dim),
                    static_cast<int>(position_offset), epsilon};
    const unsigned grid = kNumSMs * 4;
    void* scratch = nullptr;
    CGPT_TRY(scratch_get(&scratch, static_cast<std::size_t>(grid) * 2 * head_dim * sizeof(float), s));
    float* partial = static_cast<float*>(scratch);
    const unsigned rgrid = static_cast<unsigned>((2 * head_dim + 31) / 32);
    if (dtype == CGPT_DTYPE_F16) {
        qknorm_rope_kernel<__half, true><<<grid, kQkThreads, 0, s>>>(
            static_cast<__half*>(dq_pre), static_cast<__half*>(dk_pre), static_cast<const __half*>(dq_rot),
            static_cast<const __half*>(dk_rot), static_cast<const __half*>(q_pre), static_cast<const __half*>(k_pre),
            static_cast<const __half*>(q_norm), static_cast<const __half*>(k_norm), static_cast<const __half*>(cos_table),
            static_cast<const __half*>(sin_table), partial, dm);
        count_launch();
        CGPT_LAUNCH_CHECK();
        qknorm_dw_reduce_kernel<__half><<<rgrid, 256, 0, s>>>(static_cast<__half*>(dq_norm), static_cast<__half*>(dk_norm), partial,
                                                             static_cast<int>(grid), static_cast<int>(head_dim));
    } else {
        qknorm_rope_kernel<__nv_bfloat16, true><<<grid, kQkThreads, 0, s>>>(
            static_cast<__nv_bfloat16*>(dq_pre), static_cast<__nv_bfloat16*>(dk_pre), static_cast<const __nv_bfloat16*>(dq_rot),
            static_cast<const __nv_bfloat16*>(dk_rot), static_cast<const __nv_bfloat16*>(q_pre),
            static_cast<const __nv_bfloat16*>(k_pre), static_cast<const __nv_bfloat16*>(q_norm),
            static_cast<const __nv_bfloat16*>(k_norm), static_cast<const __nv_bfloat16*>(cos_table),
            static_cast<const __nv_bfloat16*>(sin_table), partial, dm);
        count_launch();
        CGPT_LAUNCH_CHECK();
        qknorm_dw_reduce_kernel<__nv_bfloat16><<<rgrid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(dq_norm),
                                                                    static_cast<__nv_bfloat16*>(dk_norm), partial,
                                                                    static_cast<int>(grid), static_cast<int>(head_dim));
    }
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}
