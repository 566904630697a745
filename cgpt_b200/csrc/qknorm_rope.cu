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
// Rows a lane group has in flight per trip. Measured at 32768 tokens, 8 + 2 heads of 128: forward 8 rows (80 registers, 3 CTAs
// per SM) 38.5 us, 4 rows (55 registers, 4 CTAs) 32.7 us, 2 rows 33.1 us; backward 4 rows (126 registers, 2 CTAs) 62.2 us,
// 2 rows (74 registers, 3 CTAs) 61.3 us: the kernels are bound by instruction issue, so resident warps beat loads in flight.
constexpr int kFwdUnroll = 4;
constexpr int kBwdUnroll = 2;

// Sum over the lanes that share a row. LPR (lanes per row) known at compile time: an unrolled butterfly; LPR == 0: the
// run-time width (a real loop: shift, compare and branch around every shuffle).
template <int LPR>
__device__ __forceinline__ float group_sum(float v, int lanes_per_row) {
    if constexpr (LPR > 0) {
#pragma unroll
        for (int o = LPR >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    } else {
        for (int o = lanes_per_row >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

struct QkDims {
    long long tokens;   // batch * seq
    int seq, q_heads, kv_heads, head_dim, rotary_dim, offset;
    float eps;
};

template <typename T>
__device__ __forceinline__ void unpack8(float (&out)[8], const uint4& raw) {
    Pack<T, 8> pk;
    *reinterpret_cast<uint4*>(&pk) = raw;
    unpack_pack(out, pk);
}
template <typename T>
__device__ __forceinline__ void unpack4(float (&out)[4], const uint2& raw) {
    Pack<T, 4> pk;
    *reinterpret_cast<uint2*>(&pk) = raw;
    unpack_pack(out, pk);
}

// Two phases per thread, query rows then key rows, so that a phase has one source tensor, one weight vector and one dw
// accumulator (no per-element selects). Row r of a phase: token = r / heads_of_phase, head = r % heads_of_phase; both
// tensors are [tokens, heads, head_dim] contiguous, so the row's offset is simply r * head_dim.
// A warp works on 32/(head_dim/8) runs of U CONSECUTIVE rows per trip (a lane group owns one run); every 16-byte row load
// of the trip (x, and dy in the backward pass) is issued before the first value is used: U (2U) independent loads in
// flight per thread. Consecutive rows are the heads of one token, so a lane converts its slice of the rotary tables once
// per token instead of once per row (8 query heads: one table fetch and conversion per 8 rows), and the token / head of
// a row follow from the run's first row by counting: one division per run, none per row.
// Row indices fit 31 bits (checked by the host); divisions by heads and seq use precomputed multipliers.
// LPR: head_dim / 8 when the host knows it at compile time (8 or 16: head_dim 64 or 128), else 0 = read from dm.
template <typename T, bool BACKWARD, int U, int LPR>
__global__ void __launch_bounds__(kQkThreads)
qknorm_rope_kernel(T* __restrict__ out_q, T* __restrict__ out_k, const T* __restrict__ in_q, const T* __restrict__ in_k,
                   const T* __restrict__ x_q, const T* __restrict__ x_k, const T* __restrict__ w_q, const T* __restrict__ w_k,
                   const T* __restrict__ cos_t, const T* __restrict__ sin_t, float* __restrict__ dw_partial, QkDims dm,
                   FastDiv div_qh, FastDiv div_kh, FastDiv div_seq) {
    const int hd = LPR > 0 ? LPR * 8 : dm.head_dim;    // head_dim (a compile-time constant for the common sizes)
    const int lpr = LPR > 0 ? LPR : dm.head_dim / 8;   // lanes per row
    const int rows_per_warp = 32 / lpr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / lpr, l = lane % lpr;      // row slot inside the warp, chunk inside the row
    const int d0 = l * 8;
    const float inv_d = 1.0f / static_cast<float>(hd);
    const int half_rot = dm.rotary_dim / 2;
    const bool rotate = d0 < dm.rotary_dim;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    const unsigned group = static_cast<unsigned>(rows_per_warp) * U;
    const unsigned warps_total = gridDim.x * (kQkThreads / 32);
    const unsigned warp_id = blockIdx.x * (kQkThreads / 32) + warp;
    __shared__ float red[BACKWARD ? kQkThreads : 1][9];

    for (int which = 0; which < 2; ++which) {
        const T* __restrict__ in = which == 0 ? in_q : in_k;
        const T* __restrict__ xs = which == 0 ? x_q : x_k;
        T* __restrict__ out = which == 0 ? out_q : out_k;
        const FastDiv div_heads = which == 0 ? div_qh : div_kh;
        const unsigned rows = static_cast<unsigned>(dm.tokens) * div_heads.d;
        float w[8], dw[8];
        load_vec<T, 8>(w, (which == 0 ? w_q : w_k) + d0);
#pragma unroll
        for (int i = 0; i < 8; ++i) dw[i] = 0.f;

        const unsigned trips = (rows + group * warps_total - 1) / (group * warps_total);
        for (unsigned trip = 0; trip < trips; ++trip) {
            const unsigned r0 = (trip * warps_total + warp_id) * group + sub * U;   // first row of this lane group's run
            const long long off0 = static_cast<long long>(r0) * hd + d0;
            uint4 raw_in[U], raw_x[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool active = r0 + u < rows;
                raw_in[u] = active ? __ldcs(reinterpret_cast<const uint4*>(in + off0 + u * hd)) : zero4;
                if (BACKWARD) raw_x[u] = active ? __ldcs(reinterpret_cast<const uint4*>(xs + off0 + u * hd)) : zero4;
            }
            unsigned token = div_heads.div(r0);
            unsigned head = r0 - token * div_heads.d;
            bool fetch_tables = true;           // the run's first row, then every row that starts a new token
            float c[4] = {0.f, 0.f, 0.f, 0.f}, s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const bool active = r0 + u < rows;
                const long long off = off0 + u * hd;
                // the rotary tables are small and stay in L1/L2: fetched here, not ahead, to keep registers for the row data
                if (fetch_tables && active && rotate) {
                    const unsigned pos = token - div_seq.div(token) * div_seq.d + dm.offset;
                    const long long t = static_cast<long long>(pos) * half_rot + d0 / 2;
                    unpack4<T>(c, __ldg(reinterpret_cast<const uint2*>(cos_t + t)));
                    unpack4<T>(s, __ldg(reinterpret_cast<const uint2*>(sin_t + t)));
                }
                fetch_tables = false;
                if (++head == div_heads.d) { head = 0; ++token; fetch_tables = true; }
                if (!BACKWARD) {
                    float x[8];
                    unpack8<T>(x, raw_in[u]);
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
                    ss = group_sum<LPR>(ss, lpr);
                    const float inv = rsqrtf(ss * inv_d + dm.eps);
                    float y[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) y[i] = x[i] * inv * w[i];
                    // the reference rounds the normalised value to the storage dtype before RoPE reads it
#pragma unroll
                    for (int i = 0; i < 8; i += 2) round_pair_to_storage<T>(y[i], y[i + 1]);
                    if (rotate) {
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const float a = y[2 * p], b = y[2 * p + 1];
                            y[2 * p] = fmaf(-b, s[p], a * c[p]);
                            y[2 * p + 1] = fmaf(a, s[p], b * c[p]);
                        }
                    }
                    if (active) store_vec<T, 8>(out + off, y);
                } else {
                    float g[8], x[8];
                    unpack8<T>(g, raw_in[u]);
                    unpack8<T>(x, raw_x[u]);
                    if (rotate) {
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const float a = g[2 * p], b = g[2 * p + 1];
                            // the reference rounds the un-rotated gradient to the storage dtype (output of rope_backward)
                            g[2 * p] = fmaf(b, s[p], a * c[p]);
                            g[2 * p + 1] = fmaf(-a, s[p], b * c[p]);
                            round_pair_to_storage<T>(g[2 * p], g[2 * p + 1]);
                        }
                    }
                    float sx = 0.f, sg = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        sx = fmaf(x[i], x[i], sx);
                        sg = fmaf(g[i] * w[i], x[i], sg);
                    }
                    sx = group_sum<LPR>(sx, lpr);
                    sg = group_sum<LPR>(sg, lpr);
                    const float inv = rsqrtf(sx * inv_d + dm.eps);
                    const float corr = sg * inv_d * inv * inv * inv;
                    float dx[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        dx[i] = fmaf(-x[i], corr, g[i] * w[i] * inv);
                        dw[i] += g[i] * (x[i] * inv);    // inactive rows hold zeros
                    }
                    if (active) store_vec<T, 8>(out + off, dx);
                }
            }
        }

        if (BACKWARD) {
            // Combine lanes that own the same columns (fixed order), then one partial row per CTA: [grid][2][head_dim].
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; ++i) red[threadIdx.x][i] = dw[i];
            __syncthreads();
            for (int col = threadIdx.x; col < hd; col += kQkThreads) {
                float acc = 0.f;
                for (int t = col >> 3; t < kQkThreads; t += lpr) acc += red[t][col & 7];
                dw_partial[(static_cast<long long>(blockIdx.x) * 2 + which) * hd + col] = acc;
            }
        }
    }
}

// dw[col] = sum of the per-CTA partials in a fixed order: 32 row lanes per column, then a shared-memory combine.
template <typename T>
__global__ void __launch_bounds__(1024)
qknorm_dw_reduce_kernel(T* __restrict__ dw_q, T* __restrict__ dw_k, const float* __restrict__ partial, int parts, int head_dim) {
    __shared__ float tile[32][33];
    const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + cl;      // 0 .. 2*head_dim
    float acc = 0.f;
    if (col < 2 * head_dim)
        for (int p = rl; p < parts; p += 32) acc += partial[static_cast<long long>(p) * 2 * head_dim + col];
    tile[rl][cl] = acc;
    __syncthreads();
    if (rl == 0 && col < 2 * head_dim) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) total += tile[r][cl];
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
    if (batch * seq * (q_heads + kv_heads) >= (1ull << 31)) return CGPT_ERR_UNSUPPORTED;   // 32-bit row indices in the kernel
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    if (!fast_path_ok(head_dim, rotary_dim, dtype, {q, k, q_pre, k_pre, q_norm, k_norm, cos_table, sin_table}))
        return CGPT_ERR_UNSUPPORTED;
    auto s = static_cast<cudaStream_t>(stream);
    const QkDims dm{static_cast<long long>(batch * seq), static_cast<int>(seq), static_cast<int>(q_heads),
                    static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<int>(rotary_dim),
                    static_cast<int>(position_offset), epsilon};
    const FastDiv div_qh(static_cast<unsigned>(q_heads)), div_kh(static_cast<unsigned>(kv_heads)), div_seq(static_cast<unsigned>(seq));
#define CGPT_QK_FWD(T, LPR)                                                                                                    \
    {                                                                                                                          \
        auto* kernel = qknorm_rope_kernel<T, false, kFwdUnroll, LPR>;                                                         \
        const unsigned grid = kNumSMs * resident_ctas_per_sm(reinterpret_cast<const void*>(kernel), kQkThreads, 0);           \
        kernel<<<grid, kQkThreads, 0, s>>>(static_cast<T*>(q), static_cast<T*>(k), static_cast<const T*>(q_pre),              \
                                           static_cast<const T*>(k_pre), nullptr, nullptr, static_cast<const T*>(q_norm),     \
                                           static_cast<const T*>(k_norm), static_cast<const T*>(cos_table),                   \
                                           static_cast<const T*>(sin_table), nullptr, dm, div_qh, div_kh, div_seq);           \
    }
    // every CTA resident (no partial last wave); lanes per row as a compile-time constant for the common head sizes
    if (dtype == CGPT_DTYPE_F16) {
        if (head_dim == 128) CGPT_QK_FWD(__half, 16) else if (head_dim == 64) CGPT_QK_FWD(__half, 8) else CGPT_QK_FWD(__half, 0)
    } else {
        if (head_dim == 128) CGPT_QK_FWD(__nv_bfloat16, 16) else if (head_dim == 64) CGPT_QK_FWD(__nv_bfloat16, 8) else CGPT_QK_FWD(__nv_bfloat16, 0)
    }
#undef CGPT_QK_FWD
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
    if (batch * seq * (q_heads + kv_heads) >= (1ull << 31)) return CGPT_ERR_UNSUPPORTED;   // 32-bit row indices in the kernel
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    if (!fast_path_ok(head_dim, rotary_dim, dtype, {dq_pre, dk_pre, dq_rot, dk_rot, q_pre, k_pre, q_norm, k_norm, cos_table, sin_table}))
        return CGPT_ERR_UNSUPPORTED;
    auto s = static_cast<cudaStream_t>(stream);
    const QkDims dm{static_cast<long long>(batch * seq), static_cast<int>(seq), static_cast<int>(q_heads),
                    static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<int>(rotary_dim),
                    static_cast<int>(position_offset), epsilon};
    const FastDiv div_qh(static_cast<unsigned>(q_heads)), div_kh(static_cast<unsigned>(kv_heads)), div_seq(static_cast<unsigned>(seq));
    // the same grid for every instantiation of a dtype (the partial buffer is sized by it): the smallest residency
    unsigned grid = 0;
    void* scratch = nullptr;
    const unsigned rgrid = static_cast<unsigned>((2 * head_dim + 31) / 32);
#define CGPT_QK_BWD(T, LPR)                                                                                                    \
    {                                                                                                                          \
        auto* kernel = qknorm_rope_kernel<T, true, kBwdUnroll, LPR>;                                                          \
        grid = kNumSMs * resident_ctas_per_sm(reinterpret_cast<const void*>(kernel), kQkThreads, 0);                          \
        CGPT_TRY(scratch_get(&scratch, static_cast<std::size_t>(grid) * 2 * head_dim * sizeof(float), s));                    \
        kernel<<<grid, kQkThreads, 0, s>>>(static_cast<T*>(dq_pre), static_cast<T*>(dk_pre), static_cast<const T*>(dq_rot),   \
                                           static_cast<const T*>(dk_rot), static_cast<const T*>(q_pre),                       \
                                           static_cast<const T*>(k_pre), static_cast<const T*>(q_norm),                       \
                                           static_cast<const T*>(k_norm), static_cast<const T*>(cos_table),                   \
                                           static_cast<const T*>(sin_table), static_cast<float*>(scratch), dm, div_qh, div_kh, \
                                           div_seq);                                                                          \
        count_launch();                                                                                                        \
        CGPT_LAUNCH_CHECK();                                                                                                   \
        qknorm_dw_reduce_kernel<T><<<rgrid, 1024, 0, s>>>(static_cast<T*>(dq_norm), static_cast<T*>(dk_norm),                 \
                                                          static_cast<const float*>(scratch), static_cast<int>(grid),         \
                                                          static_cast<int>(head_dim));                                        \
    }
    if (dtype == CGPT_DTYPE_F16) {
        if (head_dim == 128) CGPT_QK_BWD(__half, 16) else if (head_dim == 64) CGPT_QK_BWD(__half, 8) else CGPT_QK_BWD(__half, 0)
    } else {
        if (head_dim == 128) CGPT_QK_BWD(__nv_bfloat16, 16) else if (head_dim == 64) CGPT_QK_BWD(__nv_bfloat16, 8) else CGPT_QK_BWD(__nv_bfloat16, 0)
    }
#undef CGPT_QK_BWD
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}
