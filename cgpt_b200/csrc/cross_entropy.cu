// Softmax cross-entropy on materialised logits (loss + gradient) for sm_100a.
//
// Math follows the reference kernel (src/ops/cross_entropy.cu:134-245): per row max, sum of
// __expf(logit - max), loss_row = __logf(sum) + max - logit[target], grad = (__expf(logit - max) *
// __frcp_rn(sum) - onehot) * (1/rows) * gradient_scale; a row whose target is outside the vocabulary
// contributes no loss and gets no -1. The reference adds row losses with a float atomicAdd; here row
// losses go to scratch and one CTA sums them in a fixed order, so the loss is reproducible.
//
// Memory-bound: the row is staged once in shared memory (up to 200 KB) so logits are read from HBM
// once and the gradient written once: 2 * rows * vocab * sizeof(T) algorithmic bytes.
#include <math_constants.h>

#include <cstdlib>

#include "common.cuh"
#include "launch_counter.h"
#include "sm100.cuh"

namespace cgpt {

unsigned int* tc_status_device_ptr();   // gemm.cu: status word raised when a bounded device-side wait runs out

namespace {

constexpr int kCeThreads = 512;
constexpr int kCeWarps = kCeThreads / 32;

__device__ __forceinline__ float block_max_512(float v, float* red) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int i = 1; i < kCeWarps; ++i) r = fmaxf(r, red[i]);
    return r;
}
__device__ __forceinline__ float block_sum_512(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < kCeWarps; ++i) r += red[i];
    return r;
}

// VEC = elements moved per access (16 bytes when the row pitch and pointers allow it, else 1).
template <typename T, bool STAGED, int VEC>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(float* __restrict__ row_loss, T* grad, const T* logits,
                     const std::uint32_t* __restrict__ targets, long long rows, int vocab, float inv_rows,
                     float gradient_scale) {
    extern __shared__ __align__(16) unsigned char ce_smem[];
    __shared__ float red[kCeWarps];
    T* staged = reinterpret_cast<T*>(ce_smem);
    const int chunks = vocab / VEC;   // VEC > 1 only when vocab % VEC == 0
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* src = logits + row * vocab;
        float local_max = -CUDART_INF_F;
        for (int c = threadIdx.x; c < chunks; c += kCeThreads) {
            float v[VEC];
            load_vec_stream<T, VEC>(v, src + c * VEC);
            if (STAGED) {
                using Raw = typename RawVec<sizeof(T) * VEC>::type;
                *reinterpret_cast<Raw*>(staged + c * VEC) = *reinterpret_cast<const Raw*>(src + c * VEC);
            }
#pragma unroll
            for (int i = 0; i < VEC; ++i) local_max = fmaxf(local_max, v[i]);
        }
        const float maximum = block_max_512(local_max, red);  // also orders the staging writes
        const T* cached = STAGED ? staged : src;
        float local_sum = 0.f;
        for (int c = threadIdx.x; c < chunks; c += kCeThreads) {
            float v[VEC];
            load_vec<T, VEC>(v, cached + c * VEC);
#pragma unroll
            for (int i = 0; i < VEC; ++i) local_sum += __expf(v[i] - maximum);
        }
        const float denominator = block_sum_512(local_sum, red);
        const float inv_denominator = __frcp_rn(denominator);
        const std::uint32_t target = targets[row];
        const bool valid = target < static_cast<std::uint32_t>(vocab);
        if (threadIdx.x == 0) {
            row_loss[row] = valid ? (__logf(denominator) + maximum - to_f32<T>(cached[target])) * inv_rows : 0.f;
        }
        if (grad != nullptr) {
            T* dst = grad + row * vocab;
            const float out_scale = inv_rows * gradient_scale;
            for (int c = threadIdx.x; c < chunks; c += kCeThreads) {
                float v[VEC];
                load_vec<T, VEC>(v, cached + c * VEC);
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    float p = __expf(v[i] - maximum) * inv_denominator;
                    if (valid && static_cast<std::uint32_t>(c * VEC + i) == target) p -= 1.0f;
                    v[i] = p * out_scale;
                }
                store_vec<T, VEC>(dst + c * VEC, v);
            }
        }
        __syncthreads();  // staged row is reused by the next iteration
    }
}

// Fixed-order sum of n floats by one CTA.
__global__ void __launch_bounds__(1024)
sum_floats_kernel(float* __restrict__ out, const float* __restrict__ in, long long n) {
    __shared__ float red[32];
    float acc = 0.f;
    for (long long i = threadIdx.x; i < n; i += 1024) acc += in[i];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = red[threadIdx.x];
        v = warp_sum(v);
        if (threadIdx.x == 0) *out = v;
    }
}

}  // namespace

// Shared with the fused LM-head loss: deterministic sum of per-row losses into loss[0].
int sum_floats(float* out, const float* in, long long n, cudaStream_t s) {
    sum_floats_kernel<<<1, 1024, 0, s>>>(out, in, n);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

}  // namespace cgpt

using namespace cgpt;

namespace cgpt {
// Per-row losses (already divided by total_rows) and, when grad != nullptr, the scaled gradient for
// `rows` rows. grad may alias logits (every thread rewrites exactly the elements it read).
namespace {
template <typename T, bool STAGED, int VEC>
int ce_launch(float* row_loss, void* grad, const void* logits, const std::uint32_t* targets, long long rows, long long vocab,
              float inv_total_rows, float gradient_scale, unsigned grid, std::size_t smem, cudaStream_t s) {
    if (STAGED) {
        static PerDeviceOnce attr_once;
        if (attr_once.needed()) {
            CGPT_CUDA_TRY(cudaFuncSetAttribute(cross_entropy_kernel<T, STAGED, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               200 * 1024));
            attr_once.done();
        }
    }
    cross_entropy_kernel<T, STAGED, VEC><<<grid, kCeThreads, smem, s>>>(row_loss, static_cast<T*>(grad), static_cast<const T*>(logits),
                                                                        targets, rows, static_cast<int>(vocab), inv_total_rows,
                                                                        gradient_scale);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

#include "cross_entropy_ring.cuh"
#include "cross_entropy_tiles.cuh"
}  // namespace

int softmax_grad_rows(float* row_loss, void* logits_to_grad, const float2* partial, const float* target_logit,
                      const std::uint32_t* targets, long long rows, long long vocab, int tiles, float inv_total_rows,
                      float gradient_scale, int dtype, cudaStream_t s) {
    if (dtype != CGPT_DTYPE_F16 && dtype != CGPT_DTYPE_BF16) return CGPT_ERR_UNSUPPORTED;
    if (vocab % 8 != 0 || !aligned16(logits_to_grad) || vocab > 0x7fffffffll || tiles < 1) return CGPT_ERR_UNSUPPORTED;
    const void* kernel = dtype == CGPT_DTYPE_F16 ? reinterpret_cast<const void*>(softmax_grad_rows_kernel<__half>)
                                                 : reinterpret_cast<const void*>(softmax_grad_rows_kernel<__nv_bfloat16>);
    const long long resident = static_cast<long long>(kNumSMs) * resident_ctas_per_sm(kernel, kTileGradThreads, 0);
    const unsigned grid = static_cast<unsigned>(rows < resident ? rows : resident);
    if (dtype == CGPT_DTYPE_F16)
        softmax_grad_rows_kernel<__half><<<grid, kTileGradThreads, 0, s>>>(row_loss, static_cast<__half*>(logits_to_grad), partial,
                                                                          target_logit, targets, rows, static_cast<int>(vocab), tiles,
                                                                          inv_total_rows, gradient_scale);
    else
        softmax_grad_rows_kernel<__nv_bfloat16><<<grid, kTileGradThreads, 0, s>>>(row_loss, static_cast<__nv_bfloat16*>(logits_to_grad),
                                                                                 partial, target_logit, targets, rows,
                                                                                 static_cast<int>(vocab), tiles, inv_total_rows,
                                                                                 gradient_scale);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

int softmax_stats_reduce(float2* row_stats, float* row_loss, const float2* partial, const float* target_logit,
                         const std::uint32_t* targets, long long rows, long long vocab, int tiles, float inv_total_rows,
                         cudaStream_t s) {
    if (vocab > 0x7fffffffll || tiles < 1) return CGPT_ERR_UNSUPPORTED;
    const long long blocks = (rows + 7) / 8;
    softmax_stats_reduce_kernel<<<static_cast<unsigned>(blocks < kNumSMs * 8ll ? blocks : kNumSMs * 8ll), 256, 0, s>>>(
        row_stats, row_loss, partial, target_logit, targets, rows, static_cast<int>(vocab), tiles, inv_total_rows);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}

int cross_entropy_rows(float* row_loss, void* grad, const void* logits, const std::uint32_t* targets, long long rows,
                       long long vocab, float inv_total_rows, float gradient_scale, int dtype, cudaStream_t s) {
    const std::size_t row_bytes = static_cast<std::size_t>(vocab) * dtype_size(dtype);
    const bool staged = row_bytes <= 200 * 1024;
    const unsigned grid = static_cast<unsigned>(rows < kNumSMs * 4ll ? rows : kNumSMs * 4ll);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        const bool vec = vocab % V == 0 && aligned16(logits) && aligned16(grad);
        if constexpr (sizeof(T) == 2) {
            unsigned pitch = 0;
            const int stages = ring_stages<T>(vocab, logits, grad, &pitch);
            if (stages > 0)
                return ce_ring_launch<T>(row_loss, grad, logits, targets, rows, vocab, inv_total_rows, gradient_scale, stages, pitch, s);
        }
        if (staged && vec) return ce_launch<T, true, V>(row_loss, grad, logits, targets, rows, vocab, inv_total_rows, gradient_scale, grid, row_bytes, s);
        if (staged) return ce_launch<T, true, 1>(row_loss, grad, logits, targets, rows, vocab, inv_total_rows, gradient_scale, grid, row_bytes, s);
        if (vec) return ce_launch<T, false, V>(row_loss, grad, logits, targets, rows, vocab, inv_total_rows, gradient_scale, grid, 0, s);
        return ce_launch<T, false, 1>(row_loss, grad, logits, targets, rows, vocab, inv_total_rows, gradient_scale, grid, 0, s);
    });
    return CGPT_OK;
}
}  // namespace cgpt

extern "C" int cgpt_cross_entropy(float* loss, void* grad, const void* logits, const uint32_t* targets,
                                  size_t rows, size_t vocab, float gradient_scale, int dtype,
                                  cgpt_stream_t stream) {
    if (!loss || !logits || !targets) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rows == 0 || vocab == 0 || vocab > 0x7fffffffull || rows > (1ull << 40)) return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    void* scratch = nullptr;
    CGPT_TRY(scratch_get(&scratch, rows * sizeof(float), s));
    CGPT_TRY(cross_entropy_rows(static_cast<float*>(scratch), grad, logits, targets, static_cast<long long>(rows),
                                static_cast<long long>(vocab), 1.0f / static_cast<float>(rows), gradient_scale, dtype, s));
    return sum_floats(loss, static_cast<const float*>(scratch), static_cast<long long>(rows), s);
}
