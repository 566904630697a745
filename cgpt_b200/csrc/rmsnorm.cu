// RMSNorm forward and fused backward (dx + dw in one pass over x and dy) for sm_100a.
//
// Math follows the reference kernels: forward  y = x * inv * w  with inv = rsqrtf(mean(x^2) + eps)
// (src/ops/rmsnorm.cu:60,122-125 of the reference); backward
//   c  = sum(dy*w*x) / hidden * inv^3,  dx = fma(-x, c, dy*w*inv)      (rmsnorm_backward.cu:276-293)
//   dw = sum_rows dy * (x*inv)                                          (rmsnorm_backward.cu:374-398)
//
// Memory-bound. Layout of work: a row is owned by `wpr` whole warps (1, 2, 4 or 8); a CTA of 256
// threads therefore works on 8/wpr rows at a time and walks the rows with a grid stride. Each thread
// keeps its CPT*VEC elements of x and dy in registers (one 16-byte load each for 16-bit types), so x
// and dy are read from HBM exactly once. The thread's columns are the same for every row it visits,
// which lets it accumulate its dw contributions in registers over the whole row loop; per-CTA
// partials go to a [grid, hidden] fp32 scratch and a second, tiny kernel sums them in a fixed order
// (deterministic, no atomics). Algorithmic HBM bytes per row: 3 * hidden * sizeof(T)
// (+ hidden * sizeof(T) per residual operand).
#include <cstdlib>
#include <initializer_list>
#include <mutex>

#include "common.cuh"
#include "launch_counter.h"

namespace cgpt {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// Sum over the `wpr` warps that share a row. `slot` is this row group's index inside the CTA.
// All threads of the CTA must call this (it contains __syncthreads()).
template <int NV>
__device__ __forceinline__ void row_group_sum(float (&vals)[NV], int wpr, int warp_in_row, int slot,
                                              float* smem /* [kWarps * NV] */) {
#pragma unroll
    for (int i = 0; i < NV; ++i) vals[i] = warp_sum(vals[i]);
    if (wpr == 1) return;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    __syncthreads();  // protect smem reuse across successive calls
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) smem[warp * NV + i] = vals[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        float acc = 0.f;
        for (int w = 0; w < wpr; ++w) acc += smem[(slot * wpr + w) * NV + i];
        vals[i] = acc;
    }
    (void)warp_in_row;
}

template <typename T, int VEC, int CPT>
__global__ void __launch_bounds__(kThreads)
rmsnorm_forward_kernel(T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ w,
                       long long rows, int hidden, float epsilon, int wpr) {
    __shared__ float red[kWarps];
    const int tpr = wpr * 32;
    const int rows_per_cta = kWarps / wpr;
    const int slot = threadIdx.x / tpr;
    const int tid_in_row = threadIdx.x % tpr;
    const float inv_hidden = 1.0f / static_cast<float>(hidden);

    float wv[CPT][VEC];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int col = (c * tpr + tid_in_row) * VEC;
        if (col < hidden) load_vec<T, VEC>(wv[c], w + col);
        else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) wv[c][i] = 0.f;
        }
    }
    const long long row_step = static_cast<long long>(gridDim.x) * rows_per_cta;
    const long long iters = (rows + row_step - 1) / row_step;
    for (long long it = 0; it < iters; ++it) {
        const long long row = it * row_step + static_cast<long long>(blockIdx.x) * rows_per_cta + slot;
        const bool active = row < rows;
        float xv[CPT][VEC];
        float ss[1] = {0.f};
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int col = (c * tpr + tid_in_row) * VEC;
            if (active && col < hidden) {
                load_vec_stream<T, VEC>(xv[c], x + row * hidden + col);
#pragma unroll
                for (int i = 0; i < VEC; ++i) ss[0] = fmaf(xv[c][i], xv[c][i], ss[0]);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) xv[c][i] = 0.f;
            }
        }
        row_group_sum<1>(ss, wpr, 0, slot, red);
        const float inv = rsqrtf(ss[0] * inv_hidden + epsilon);
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int col = (c * tpr + tid_in_row) * VEC;
            if (active && col < hidden) {
                float out[VEC];
#pragma unroll
                for (int i = 0; i < VEC; ++i) out[i] = xv[c][i] * inv * wv[c][i];
                store_vec<T, VEC>(y + row * hidden + col, out);
            }
        }
    }
}

template <typename T, int VEC, int CPT>
__global__ void __launch_bounds__(kThreads)
rmsnorm_backward_kernel(T* dx, float* __restrict__ dw_partial,   // dx may alias res_a / res_b (element-wise in place)
                        const T* __restrict__ dy, const T* __restrict__ x,
                        const T* __restrict__ w, const T* res_a,
                        const T* res_b, long long rows, int hidden, float epsilon,
                        int wpr) {
    __shared__ float red[kWarps * 2];
    const int tpr = wpr * 32;
    const int rows_per_cta = kWarps / wpr;
    const int slot = threadIdx.x / tpr;
    const int tid_in_row = threadIdx.x % tpr;
    const float inv_hidden = 1.0f / static_cast<float>(hidden);

    float wv[CPT][VEC], dwacc[CPT][VEC];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int col = (c * tpr + tid_in_row) * VEC;
        if (col < hidden) load_vec<T, VEC>(wv[c], w + col);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            if (col >= hidden) wv[c][i] = 0.f;
            dwacc[c][i] = 0.f;
        }
    }

    const long long row_step = static_cast<long long>(gridDim.x) * rows_per_cta;
    const long long iters = (rows + row_step - 1) / row_step;
    for (long long it = 0; it < iters; ++it) {
        const long long row = it * row_step + static_cast<long long>(blockIdx.x) * rows_per_cta + slot;
        const bool active = row < rows;
        float xv[CPT][VEC], gv[CPT][VEC];
        float sums[2] = {0.f, 0.f};  // sum x^2, sum dy*w*x
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int col = (c * tpr + tid_in_row) * VEC;
            if (active && col < hidden) {
                load_vec_stream<T, VEC>(xv[c], x + row * hidden + col);
                load_vec_stream<T, VEC>(gv[c], dy + row * hidden + col);
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    sums[0] = fmaf(xv[c][i], xv[c][i], sums[0]);
                    sums[1] = fmaf(gv[c][i] * wv[c][i], xv[c][i], sums[1]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) { xv[c][i] = 0.f; gv[c][i] = 0.f; }
            }
        }
        row_group_sum<2>(sums, wpr, 0, slot, red);
        const float inv = rsqrtf(sums[0] * inv_hidden + epsilon);
        const float corr = sums[1] * inv_hidden * inv * inv * inv;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int col = (c * tpr + tid_in_row) * VEC;
            if (active && col < hidden) {
                float out[VEC];
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    out[i] = fmaf(-xv[c][i], corr, gv[c][i] * wv[c][i] * inv);
                    dwacc[c][i] = fmaf(gv[c][i], xv[c][i] * inv, dwacc[c][i]);
                }
                if (res_a != nullptr) {
                    float r[VEC];
                    load_vec_stream<T, VEC>(r, res_a + row * hidden + col);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) out[i] += r[i];
                }
                if (res_b != nullptr) {
                    float r[VEC];
                    load_vec_stream<T, VEC>(r, res_b + row * hidden + col);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) out[i] += r[i];
                }
                store_vec<T, VEC>(dx + row * hidden + col, out);
            }
        }
    }

    // Combine the CTA's row slots (fixed order) and publish one fp32 partial row per CTA.
    __shared__ float slots[kThreads];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            __syncthreads();
            slots[threadIdx.x] = dwacc[c][i];
            __syncthreads();
            if (slot == 0) {
                const int col = (c * tpr + tid_in_row) * VEC + i;
                if (col < hidden) {
                    float acc = 0.f;
                    for (int s = 0; s < rows_per_cta; ++s) acc += slots[s * tpr + tid_in_row];
                    dw_partial[static_cast<long long>(blockIdx.x) * hidden + col] = acc;
                }
            }
        }
    }
}

// dw[col] = sum over partial rows, in a fixed tree order: each thread sums a strided subset, then the
// CTA's 8 row-lanes are combined through shared memory.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_dw_reduce_kernel(T* __restrict__ dw, const float* __restrict__ partial, int parts, int hidden) {
    __shared__ float tile[8][33];
    const int col = blockIdx.x * 32 + (threadIdx.x & 31);
    const int lane_row = threadIdx.x >> 5;
    float acc = 0.f;
    if (col < hidden) {
        for (int p = lane_row; p < parts; p += 8) acc += partial[static_cast<long long>(p) * hidden + col];
    }
    tile[lane_row][threadIdx.x & 31] = acc;
    __syncthreads();
    if (lane_row == 0 && col < hidden) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) total += tile[r][threadIdx.x & 31];
        dw[col] = from_f32<T>(total);
    }
}

#include "rmsnorm_warp.cuh"
#include "rmsnorm_dual.cuh"

struct Plan {
    int vec, cpt, wpr;
};

// 16-byte chunks a thread should hold before a row is spread over more warps (diagnosis builds: CGPT_B200_RMS_CPT = 1, 2 or 4 overrides).
// More chunks per thread = more loads in flight per thread but more registers (fewer resident CTAs).
inline int chunks_per_thread_target() {
    static const int v = [] {
        const char* e = diagnosis_env("CGPT_B200_RMS_CPT");
        const int x = e ? std::atoi(e) : 1;
        return (x == 1 || x == 2 || x == 4) ? x : 1;
    }();
    return v;
}

// Chooses vector width, chunks per thread and warps per row. Returns false if hidden is too large
// for the register-cached layout.
template <typename T>
bool make_plan(std::size_t hidden, bool all_aligned16, Plan* plan) {
    constexpr int kMaxVec = 16 / sizeof(T);
    int vec = (all_aligned16 && hidden % kMaxVec == 0) ? kMaxVec : 1;
    if (vec == 8 && hidden <= 128 && hidden % 4 == 0) vec = 4;  // keep all 32 lanes busy on head_dim rows
    const std::size_t chunks = (hidden + vec - 1) / vec;
    // Prefer up to four 16-byte chunks per thread before spreading a row over more warps: a row owned by one
    // warp needs no block-level synchronisation and keeps more loads in flight per thread.
    int wpr = 1;
    while (wpr < kWarps && chunks > static_cast<std::size_t>(wpr) * 32 * chunks_per_thread_target()) wpr *= 2;
    const std::size_t per_thread = (chunks + wpr * 32 - 1) / (wpr * 32);
    int cpt = 1;
    while (cpt < static_cast<int>(per_thread)) cpt *= 2;
    if (cpt > 4) return false;
    *plan = {vec, cpt, wpr};
    return true;
}

int grid_for(std::size_t rows, int wpr, int ctas_per_sm) {
    const std::size_t rows_per_cta = kWarps / wpr;
    const std::size_t need = (rows + rows_per_cta - 1) / rows_per_cta;
    const std::size_t cap = static_cast<std::size_t>(kNumSMs) * ctas_per_sm;
    return static_cast<int>(need < cap ? (need == 0 ? 1 : need) : cap);
}

template <typename T, int VEC>
int launch_forward(void* y, const void* x, const void* w, std::size_t rows, std::size_t hidden,
                   float eps, const Plan& p, cudaStream_t s) {
    if constexpr (sizeof(T) == 2 && VEC == 8) {
        if (warp_rows::applicable(hidden, VEC, sizeof(T))) {
            const int cpt = static_cast<int>((hidden / 8 + 31) / 32);
            const std::size_t need = (rows + 2 * warp_rows::kWarps - 1) / (2 * warp_rows::kWarps);
            const std::size_t cap = static_cast<std::size_t>(kNumSMs) * 4;
            const int grid = static_cast<int>(need < cap ? need : cap);
#define CGPT_RMS_FWD_WARP(CPT)                                                                              \
    warp_rows::rmsnorm_forward_warp_kernel<T, CPT><<<grid, warp_rows::kThreads, 0, s>>>(                    \
        static_cast<T*>(y), static_cast<const T*>(x), static_cast<const T*>(w), static_cast<long long>(rows), \
        static_cast<int>(hidden), eps)
            switch (cpt) {
                case 1: CGPT_RMS_FWD_WARP(1); break;
                case 2: CGPT_RMS_FWD_WARP(2); break;
                case 3: CGPT_RMS_FWD_WARP(3); break;
                default: CGPT_RMS_FWD_WARP(4); break;
            }
#undef CGPT_RMS_FWD_WARP
            count_launch();
            CGPT_LAUNCH_CHECK();
            return CGPT_OK;
        }
    }
    const int grid = grid_for(rows, p.wpr, 8);
#define CGPT_RMS_FWD(CPT)                                                                      \
    rmsnorm_forward_kernel<T, VEC, CPT><<<grid, kThreads, 0, s>>>(                              \
        static_cast<T*>(y), static_cast<const T*>(x), static_cast<const T*>(w),               \
        static_cast<long long>(rows), static_cast<int>(hidden), eps, p.wpr)
    switch (p.cpt) {
        case 1: CGPT_RMS_FWD(1); break;
        case 2: CGPT_RMS_FWD(2); break;
        default: CGPT_RMS_FWD(4); break;
    }
#undef CGPT_RMS_FWD
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

template <typename T, int VEC>
int launch_backward(void* dx, void* dw, const void* dy, const void* x, const void* w,
                    const void* ra, const void* rb, std::size_t rows, std::size_t hidden, float eps,
                    const Plan& p, cudaStream_t s, float* fixed_scratch = nullptr, std::size_t fixed_floats = 0) {
    // fixed_scratch != nullptr: the per-CTA partial rows go there (capacity fixed_floats) and the grid is capped to fit;
    // otherwise they come from the library's arena.
    const std::size_t fit = fixed_scratch != nullptr ? fixed_floats / hidden : ~std::size_t{0};
    if (fit == 0) return CGPT_ERR_SHAPE;
    if constexpr (sizeof(T) == 2 && VEC == 8) {
        if (warp_rows::applicable(hidden, VEC, sizeof(T))) {
            const int cpt = static_cast<int>((hidden / 8 + 31) / 32);
            const std::size_t need = (rows + warp_rows::kWarps - 1) / warp_rows::kWarps;
            const std::size_t cap = static_cast<std::size_t>(kNumSMs) * 2;
            int grid = static_cast<int>(need < cap ? need : cap);
            if (static_cast<std::size_t>(grid) > fit) grid = static_cast<int>(fit);
            void* partial = fixed_scratch;
            if (partial == nullptr) CGPT_TRY(scratch_get(&partial, static_cast<std::size_t>(grid) * hidden * sizeof(float), s));
            const std::size_t smem = static_cast<std::size_t>(cpt) * 2 * warp_rows::kThreads * sizeof(float4);
#define CGPT_RMS_BWD_WARP(CPT)                                                                                 \
    warp_rows::rmsnorm_backward_warp_kernel<T, CPT><<<grid, warp_rows::kThreads, smem, s>>>(                   \
        static_cast<T*>(dx), static_cast<float*>(partial), static_cast<const T*>(dy), static_cast<const T*>(x), \
        static_cast<const T*>(w), static_cast<const T*>(ra), static_cast<const T*>(rb),                        \
        static_cast<long long>(rows), static_cast<int>(hidden), eps)
            switch (cpt) {
                case 1: CGPT_RMS_BWD_WARP(1); break;
                case 2: CGPT_RMS_BWD_WARP(2); break;
                case 3: CGPT_RMS_BWD_WARP(3); break;
                default: CGPT_RMS_BWD_WARP(4); break;
            }
#undef CGPT_RMS_BWD_WARP
            count_launch();
            CGPT_LAUNCH_CHECK();
            warp_rows::dw_reduce_wide_kernel<T><<<static_cast<unsigned>((hidden + 31) / 32), 1024, 0, s>>>(
                static_cast<T*>(dw), static_cast<const float*>(partial), grid, static_cast<int>(hidden));
            count_launch();
            CGPT_LAUNCH_CHECK();
            return CGPT_OK;
        }
    }
    int grid = grid_for(rows, p.wpr, 4);
    if (static_cast<std::size_t>(grid) > fit) grid = static_cast<int>(fit);
    void* scratch = fixed_scratch;
    if (scratch == nullptr) CGPT_TRY(scratch_get(&scratch, static_cast<std::size_t>(grid) * hidden * sizeof(float), s));
#define CGPT_RMS_BWD(CPT)                                                                       \
    rmsnorm_backward_kernel<T, VEC, CPT><<<grid, kThreads, 0, s>>>(                              \
        static_cast<T*>(dx), static_cast<float*>(scratch), static_cast<const T*>(dy),          \
        static_cast<const T*>(x), static_cast<const T*>(w), static_cast<const T*>(ra),         \
        static_cast<const T*>(rb), static_cast<long long>(rows), static_cast<int>(hidden), eps, p.wpr)
    switch (p.cpt) {
        case 1: CGPT_RMS_BWD(1); break;
        case 2: CGPT_RMS_BWD(2); break;
        default: CGPT_RMS_BWD(4); break;
    }
#undef CGPT_RMS_BWD
    count_launch();
    CGPT_LAUNCH_CHECK();
    rmsnorm_dw_reduce_kernel<T><<<static_cast<unsigned>((hidden + 31) / 32), 256, 0, s>>>(
        static_cast<T*>(dw), static_cast<const float*>(scratch), grid, static_cast<int>(hidden));
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

}  // namespace
}  // namespace cgpt

using namespace cgpt;

extern "C" int cgpt_rmsnorm_forward(void* y, const void* x, const void* w, size_t rows, size_t hidden,
                                    float epsilon, int dtype, cgpt_stream_t stream) {
    if (!y || !x || !w) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rows == 0 || hidden == 0 || hidden > 0x7fffffffull || rows > (1ull << 40)) return CGPT_ERR_SHAPE;
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    auto s = static_cast<cudaStream_t>(stream);
    const bool al = aligned16(y) && aligned16(x) && aligned16(w);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        Plan p;
        if (!make_plan<T>(hidden, al, &p)) return CGPT_ERR_UNSUPPORTED;
        constexpr int kMaxVec = 16 / sizeof(T);
        if (p.vec == kMaxVec) return launch_forward<T, kMaxVec>(y, x, w, rows, hidden, epsilon, p, s);
        if (p.vec == 4) return launch_forward<T, 4>(y, x, w, rows, hidden, epsilon, p, s);
        return launch_forward<T, 1>(y, x, w, rows, hidden, epsilon, p, s);
    });
    return CGPT_OK;
}

extern "C" int cgpt_rmsnorm_backward(void* dx, void* dw, const void* dy, const void* x, const void* w,
                                     const void* residual_a, const void* residual_b, size_t rows,
                                     size_t hidden, float epsilon, int dtype, cgpt_stream_t stream) {
    if (!dx || !dw || !dy || !x || !w) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rows == 0 || hidden == 0 || hidden > 0x7fffffffull || rows > (1ull << 40)) return CGPT_ERR_SHAPE;
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    auto s = static_cast<cudaStream_t>(stream);
    const bool al = aligned16(dx) && aligned16(dy) && aligned16(x) && aligned16(w) &&
                    aligned16(residual_a) && aligned16(residual_b);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        Plan p;
        if (!make_plan<T>(hidden, al, &p)) return CGPT_ERR_UNSUPPORTED;
        constexpr int kMaxVec = 16 / sizeof(T);
        if (p.vec == kMaxVec)
            return launch_backward<T, kMaxVec>(dx, dw, dy, x, w, residual_a, residual_b, rows, hidden, epsilon, p, s);
        if (p.vec == 4)
            return launch_backward<T, 4>(dx, dw, dy, x, w, residual_a, residual_b, rows, hidden, epsilon, p, s);
        return launch_backward<T, 1>(dx, dw, dy, x, w, residual_a, residual_b, rows, hidden, epsilon, p, s);
    });
    return CGPT_OK;
}

// Two norms of the same input in one pass (rmsnorm_dual.cuh). Fast path: 16-bit rows of 256..1024 elements, 16-byte
// aligned; every other shape runs the two single-norm operators one after the other (same results up to the one
// rounding the fused backward saves).
namespace cgpt {
namespace {
template <typename T>
int launch_forward_dual(void* y_a, void* y_b, const void* x, const void* w_a, const void* w_b, std::size_t rows, std::size_t hidden,
                        float eps, cudaStream_t s) {
    const int cpt = static_cast<int>((hidden / 8 + 31) / 32);
    const std::size_t need = (rows + 2 * warp_rows::kWarps - 1) / (2 * warp_rows::kWarps);
    const std::size_t cap = static_cast<std::size_t>(kNumSMs) * 2;      // __launch_bounds__(kThreads, 2): two resident CTAs per SM
    const int grid = static_cast<int>(need < cap ? need : cap);
    const bool exact = hidden == static_cast<std::size_t>(cpt) * 256;      // no column checks in the kernel
#define CGPT_RMS_FWD_DUAL(CPT, EXACT)                                                                                     \
    warp_rows::rmsnorm_forward_dual_warp_kernel<T, CPT, EXACT><<<grid, warp_rows::kThreads, 0, s>>>(                      \
        static_cast<T*>(y_a), static_cast<T*>(y_b), static_cast<const T*>(x), static_cast<const T*>(w_a),                \
        static_cast<const T*>(w_b), static_cast<long long>(rows), static_cast<int>(hidden), eps)
    switch (cpt) {
        case 1: if (exact) CGPT_RMS_FWD_DUAL(1, true); else CGPT_RMS_FWD_DUAL(1, false); break;
        case 2: if (exact) CGPT_RMS_FWD_DUAL(2, true); else CGPT_RMS_FWD_DUAL(2, false); break;
        case 3: if (exact) CGPT_RMS_FWD_DUAL(3, true); else CGPT_RMS_FWD_DUAL(3, false); break;
        default: if (exact) CGPT_RMS_FWD_DUAL(4, true); else CGPT_RMS_FWD_DUAL(4, false); break;
    }
#undef CGPT_RMS_FWD_DUAL
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

template <typename T, int CPT, bool EXACT>
int launch_backward_dual_cpt(void* dx, float* partial, const void* dy_a, const void* dy_b, const void* x, const void* w_a,
                             const void* w_b, const void* res, std::size_t rows, std::size_t hidden, float eps, int grid,
                             cudaStream_t s) {
    constexpr std::size_t smem = static_cast<std::size_t>(2 * CPT * 2 * warp_rows::kThreads) * sizeof(float4) + 2 * CPT * 32 * sizeof(uint4);
    static PerDeviceOnce attr_once;
    if (attr_once.needed()) {
        CGPT_CUDA_TRY(cudaFuncSetAttribute(warp_rows::rmsnorm_backward_dual_warp_kernel<T, CPT, EXACT>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_once.done();
    }
    warp_rows::rmsnorm_backward_dual_warp_kernel<T, CPT, EXACT><<<grid, warp_rows::kThreads, smem, s>>>(
        static_cast<T*>(dx), partial, static_cast<const T*>(dy_a), static_cast<const T*>(dy_b), static_cast<const T*>(x),
        static_cast<const T*>(w_a), static_cast<const T*>(w_b), static_cast<const T*>(res), static_cast<long long>(rows),
        static_cast<int>(hidden), eps);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

template <typename T>
int launch_backward_dual(void* dx, void* dw_a, void* dw_b, const void* dy_a, const void* dy_b, const void* x, const void* w_a,
                         const void* w_b, const void* res, std::size_t rows, std::size_t hidden, float eps, cudaStream_t s) {
    const int cpt = static_cast<int>((hidden / 8 + 31) / 32);
    const std::size_t need = (rows + warp_rows::kWarps - 1) / warp_rows::kWarps;
    const std::size_t cap = static_cast<std::size_t>(kNumSMs) * 2;
    const int grid = static_cast<int>(need < cap ? need : cap);
    void* scratch = nullptr;
    CGPT_TRY(scratch_get(&scratch, static_cast<std::size_t>(grid) * 2 * hidden * sizeof(float), s));
    float* partial = static_cast<float*>(scratch);
    const bool exact = hidden == static_cast<std::size_t>(cpt) * 256;      // no column checks in the kernel
#define CGPT_RMS_BWD_DUAL(CPT)                                                                                                    \
    CGPT_TRY((exact ? launch_backward_dual_cpt<T, CPT, true>(dx, partial, dy_a, dy_b, x, w_a, w_b, res, rows, hidden, eps, grid, s) \
                    : launch_backward_dual_cpt<T, CPT, false>(dx, partial, dy_a, dy_b, x, w_a, w_b, res, rows, hidden, eps, grid, s)))
    switch (cpt) {
        case 1: CGPT_RMS_BWD_DUAL(1); break;
        case 2: CGPT_RMS_BWD_DUAL(2); break;
        case 3: CGPT_RMS_BWD_DUAL(3); break;
        default: CGPT_RMS_BWD_DUAL(4); break;
    }
#undef CGPT_RMS_BWD_DUAL
    warp_rows::dw_reduce_dual_kernel<T><<<static_cast<unsigned>((2 * hidden + 31) / 32), 1024, 0, s>>>(
        static_cast<T*>(dw_a), static_cast<T*>(dw_b), partial, grid, static_cast<int>(hidden));
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

bool dual_fast_path(std::size_t hidden, int dtype, std::initializer_list<const void*> ptrs) {
    if (dtype != CGPT_DTYPE_F16 && dtype != CGPT_DTYPE_BF16) return false;
    if (hidden % 8 != 0 || !warp_rows::applicable(hidden, 8, 2)) return false;
    for (const void* p : ptrs)
        if (!aligned16(p)) return false;
    return true;
}
}  // namespace
}  // namespace cgpt

extern "C" int cgpt_rmsnorm_forward_dual(void* y_a, void* y_b, const void* x, const void* w_a, const void* w_b, size_t rows,
                                         size_t hidden, float epsilon, int dtype, cgpt_stream_t stream) {
    if (!y_a || !y_b || !x || !w_a || !w_b) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rows == 0 || hidden == 0 || hidden > 0x7fffffffull || rows > (1ull << 40)) return CGPT_ERR_SHAPE;
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    auto s = static_cast<cudaStream_t>(stream);
    if (dual_fast_path(hidden, dtype, {y_a, y_b, x, w_a, w_b})) {
        if (dtype == CGPT_DTYPE_F16) return launch_forward_dual<__half>(y_a, y_b, x, w_a, w_b, rows, hidden, epsilon, s);
        return launch_forward_dual<__nv_bfloat16>(y_a, y_b, x, w_a, w_b, rows, hidden, epsilon, s);
    }
    CGPT_TRY(cgpt_rmsnorm_forward(y_a, x, w_a, rows, hidden, epsilon, dtype, stream));
    return cgpt_rmsnorm_forward(y_b, x, w_b, rows, hidden, epsilon, dtype, stream);
}

extern "C" int cgpt_rmsnorm_backward_dual(void* dx, void* dw_a, void* dw_b, const void* dy_a, const void* dy_b, const void* x,
                                          const void* w_a, const void* w_b, const void* residual, size_t rows, size_t hidden,
                                          float epsilon, int dtype, cgpt_stream_t stream) {
    if (!dx || !dw_a || !dw_b || !dy_a || !dy_b || !x || !w_a || !w_b) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rows == 0 || hidden == 0 || hidden > 0x7fffffffull || rows > (1ull << 40)) return CGPT_ERR_SHAPE;
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    auto s = static_cast<cudaStream_t>(stream);
    if (dual_fast_path(hidden, dtype, {dx, dy_a, dy_b, x, w_a, w_b, residual})) {
        if (dtype == CGPT_DTYPE_F16)
            return launch_backward_dual<__half>(dx, dw_a, dw_b, dy_a, dy_b, x, w_a, w_b, residual, rows, hidden, epsilon, s);
        return launch_backward_dual<__nv_bfloat16>(dx, dw_a, dw_b, dy_a, dy_b, x, w_a, w_b, residual, rows, hidden, epsilon, s);
    }
    // dx = residual + backward a, then dx += backward b (dx is its own residual in the second call)
    CGPT_TRY(cgpt_rmsnorm_backward(dx, dw_a, dy_a, x, w_a, residual, nullptr, rows, hidden, epsilon, dtype, stream));
    return cgpt_rmsnorm_backward(dx, dw_b, dy_b, x, w_b, dx, nullptr, rows, hidden, epsilon, dtype, stream);
}

// ------------------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate.
//
// Some hosts embed this library where device allocation is off limits at call time: a process that
// handed all device memory to its own pool allocator at start-up, a real-time loop that may not take the
// allocator's lock, or a sandbox that only lets pre-approved entry points touch the driver's allocator.
// cgpt_rmsnorm_backward takes its [grid, hidden] fp32 partial-sum buffer from the library's arena, which
// calls cudaMalloc the first time (or whenever a larger size is needed). This variant instead keeps that
// buffer in a fixed array in the library's own device image: it exists from the moment the library is
// loaded on a GPU until the process exits, costs kNoAllocFloats * 4 bytes on every GPU that loads the
// library, and is never resized.
// ------------------------------------------------------------------------------------------------
namespace cgpt {
namespace {

constexpr std::size_t kNoAllocFloats = std::size_t{1} << 20;   // 4 MiB of fp32 partial sums per GPU
static __device__ __align__(256) float g_noalloc_partials[kNoAllocFloats];

constexpr int kNoAllocMaxDevices = 64;
float* g_noalloc_address[kNoAllocMaxDevices] = {};   // device address of the array, per device
std::mutex g_noalloc_mutex;

// In host code the array's name is only a handle for the runtime, not an address the GPU can use:
// ask the runtime for the device address once per device (with that device current) and cache it.
int noalloc_scratch(float** out) {
    int device = 0;
    CGPT_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kNoAllocMaxDevices) return CGPT_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_address[device] == nullptr) {
        float* p = nullptr;
        CGPT_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials));
        if (p == nullptr) return CGPT_ERR_STATE;
        g_noalloc_address[device] = p;
    }
    *out = g_noalloc_address[device];
    return CGPT_OK;
}

}  // namespace
}  // namespace cgpt

// Same contract and results as cgpt_rmsnorm_backward, but no cudaMalloc / cudaFree / allocating library
// routine is ever called: the partial sums live in a 4 MiB array that is part of the library image.
//  * Limit: hidden <= 8192 (and within what the register-cached kernel supports); larger sizes return
//    CGPT_ERR_SHAPE. When rows are many and hidden is large the grid is capped so that grid * hidden
//    floats fit in the array.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
//    that first call outside of any stream capture.
//  * All calls on a device share the one array, which still holds the previous call's partial sums.
//    Nothing needs to start at zero (every partial that is read was written by the same call), but
//    two calls that overlap on the GPU (different streams) would overwrite each other's partials:
//    issue them on one stream or otherwise order them.
extern "C" int cgpt_rmsnorm_backward_noalloc(void* dx, void* dw, const void* dy, const void* x, const void* w,
                                             const void* residual_a, const void* residual_b, size_t rows,
                                             size_t hidden, float epsilon, int dtype, cgpt_stream_t stream) {
    if (!dx || !dw || !dy || !x || !w) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rows == 0 || hidden == 0 || rows > (1ull << 40)) return CGPT_ERR_SHAPE;
    if (hidden > 8192) return CGPT_ERR_SHAPE;   // beyond the fixed scratch this entry point is built for
    if (!(epsilon > 0.f)) return CGPT_ERR_OPTION;
    float* scratch = nullptr;
    CGPT_TRY(noalloc_scratch(&scratch));
    auto s = static_cast<cudaStream_t>(stream);
    const bool al = aligned16(dx) && aligned16(dy) && aligned16(x) && aligned16(w) && aligned16(residual_a) &&
                    aligned16(residual_b);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        Plan p;
        if (!make_plan<T>(hidden, al, &p)) return CGPT_ERR_UNSUPPORTED;
        constexpr int kMaxVec = 16 / sizeof(T);
        if (p.vec == kMaxVec)
            return launch_backward<T, kMaxVec>(dx, dw, dy, x, w, residual_a, residual_b, rows, hidden, epsilon, p, s, scratch, kNoAllocFloats);
        if (p.vec == 4)
            return launch_backward<T, 4>(dx, dw, dy, x, w, residual_a, residual_b, rows, hidden, epsilon, p, s, scratch, kNoAllocFloats);
        return launch_backward<T, 1>(dx, dw, dy, x, w, residual_a, residual_b, rows, hidden, epsilon, p, s, scratch, kNoAllocFloats);
    });
    return CGPT_OK;
}
