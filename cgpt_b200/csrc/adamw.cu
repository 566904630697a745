// Multi-tensor AdamW for sm_100a: three launches per step regardless of the number of tensors.
//
//   1. statistics  - one pass over the gradients only: sum of (g/loss_scale)^2 and a non-finite flag
//                    (reference: gradient_statistics_kernel, src/optim/adamw.cu:74-109, launched once
//                    per tensor there). Per-CTA partial sums go to a small buffer.
//   2. prepare     - one CTA: fixed-order sum of the partials, skip decision, step+1, bias corrections
//                    1 - powf(beta, float(step)), clip factor (reference: adamw_prepare_step_kernel,
//                    adamw.cu:166-187).
//   3. update      - one pass over grad/master/m/v/param with 16-byte accesses; expression tree as in
//                    adamw_batch_kernel (adamw.cu:147-163) so that results agree to fp32 rounding.
//
// Work is expressed as fixed-size chunks of consecutive elements of one tensor; a device table built
// at workspace creation maps chunk -> (tensor, offset). CTAs walk the chunk list with a grid stride,
// so 90 tensors of very different sizes load all SMs evenly. HBM bytes per element: 2 (statistics,
// 16-bit grads) + 28 (update: grad 2r, master/m/v 12r + 12w, param 2w).
#include <cmath>
#include <vector>

#include "common.cuh"
#include "launch_counter.h"

namespace cgpt {
namespace {

constexpr int kChunk = 4096;     // elements per work item
constexpr int kAdamThreads = 256;

struct DevTensor {
    void* param;
    const void* grad;
    float* master;
    float* m;
    float* v;
    unsigned long long count;
    int dtype;
    int pad;
};
struct Chunk {
    unsigned int tensor;
    unsigned int pad;
    unsigned long long offset;
};

// g / loss_scale as the reference writes it. POW2: loss_scale is a power of two, so multiplying by its (exact) reciprocal
// gives the same correctly rounded value as the division, bit for bit, at a tenth of the instructions; the statistics
// pass reads 2 bytes per element and is bound by those divisions otherwise.
template <bool POW2>
__device__ __forceinline__ float unscale(float g, float loss_scale, float inv_loss_scale) {
    return POW2 ? g * inv_loss_scale : g / loss_scale;
}

template <typename T, bool POW2>
__device__ __forceinline__ void stats_chunk(const T* __restrict__ g, unsigned long long n, float loss_scale, float inv_loss_scale,
                                            float& sum, bool& bad) {
    constexpr int V = 16 / sizeof(T);
    const bool vec = (reinterpret_cast<std::uintptr_t>(g) & 15u) == 0;
    if (vec) {
        for (unsigned long long i = threadIdx.x * V; i < n; i += kAdamThreads * V) {
            if (i + V <= n) {
                float x[V];
                load_vec<T, V>(x, g + i);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const float u = unscale<POW2>(x[k], loss_scale, inv_loss_scale);
                    if (isfinite(u)) sum = fmaf(u, u, sum); else bad = true;
                }
            } else {
                for (unsigned long long j = i; j < n; ++j) {
                    const float u = unscale<POW2>(to_f32<T>(g[j]), loss_scale, inv_loss_scale);
                    if (isfinite(u)) sum = fmaf(u, u, sum); else bad = true;
                }
            }
        }
    } else {
        for (unsigned long long i = threadIdx.x; i < n; i += kAdamThreads) {
            const float u = unscale<POW2>(to_f32<T>(g[i]), loss_scale, inv_loss_scale);
            if (isfinite(u)) sum = fmaf(u, u, sum); else bad = true;
        }
    }
}

template <bool POW2>
__global__ void __launch_bounds__(kAdamThreads)
adamw_stats_kernel(const DevTensor* __restrict__ tensors, const Chunk* __restrict__ chunks, unsigned int n_chunks,
                   float loss_scale, float inv_loss_scale, float* __restrict__ partial_sums, unsigned int* __restrict__ partial_bad) {
    __shared__ float red[kAdamThreads / 32];
    __shared__ int any_bad;
    if (threadIdx.x == 0) any_bad = 0;
    __syncthreads();
    float sum = 0.f;
    bool bad = false;
    for (unsigned int c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const Chunk ch = chunks[c];
        const DevTensor t = tensors[ch.tensor];
        unsigned long long n = t.count - ch.offset;
        if (n > kChunk) n = kChunk;
        switch (t.dtype) {
            case CGPT_DTYPE_F16: stats_chunk<__half, POW2>(static_cast<const __half*>(t.grad) + ch.offset, n, loss_scale, inv_loss_scale, sum, bad); break;
            case CGPT_DTYPE_BF16: stats_chunk<__nv_bfloat16, POW2>(static_cast<const __nv_bfloat16*>(t.grad) + ch.offset, n, loss_scale, inv_loss_scale, sum, bad); break;
            default: stats_chunk<float, POW2>(static_cast<const float*>(t.grad) + ch.offset, n, loss_scale, inv_loss_scale, sum, bad); break;
        }
    }
    if (bad) any_bad = 1;
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
#pragma unroll
        for (int i = 0; i < kAdamThreads / 32; ++i) total += red[i];
        partial_sums[blockIdx.x] = total;
        partial_bad[blockIdx.x] = any_bad ? 1u : 0u;
    }
}

// state[0] = non_finite (this step), state[1] = observed_non_finite (sticky)
// scalars[0] = bc1, [1] = bc2, [2] = clip, [3] = squared norm of the last step
__global__ void __launch_bounds__(256)
adamw_prepare_kernel(const float* __restrict__ partial_sums, const unsigned int* __restrict__ partial_bad, int parts,
                     unsigned int* __restrict__ state, unsigned long long* __restrict__ step,
                     float* __restrict__ scalars, float beta1, float beta2, float max_grad_norm) {
    __shared__ float red[8];
    __shared__ unsigned int bad_any;
    if (threadIdx.x == 0) bad_any = 0;
    __syncthreads();
    float acc = 0.f;
    unsigned int bad = 0;
    for (int i = threadIdx.x; i < parts; i += 256) { acc += partial_sums[i]; bad |= partial_bad[i]; }
    if (bad) atomicOr(&bad_any, 1u);
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x != 0) return;
    float squared = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) squared += red[i];
    scalars[3] = squared;
    if (bad_any != 0u || !isfinite(squared)) {
        state[0] = 1u;
        state[1] = 1u;
        return;
    }
    state[0] = 0u;
    const unsigned long long next_step = *step + 1ULL;
    *step = next_step;
    scalars[0] = 1.0F - powf(beta1, static_cast<float>(next_step));
    scalars[1] = 1.0F - powf(beta2, static_cast<float>(next_step));
    if (isinf(max_grad_norm)) {
        scalars[2] = 1.0F;
    } else {
        const float norm = sqrtf(squared);
        scalars[2] = norm > max_grad_norm ? max_grad_norm / norm : 1.0F;
    }
}

struct Hyper {
    float beta1, beta2, lr, eps, wd, loss_scale;
};

__device__ __forceinline__ void adamw_element(float g_raw, float& master, float& m, float& v, const Hyper& h,
                                              float bc1, float bc2, float clip) {
    const float grad = g_raw / h.loss_scale * clip;
    m = h.beta1 * m + (1.0f - h.beta1) * grad;
    v = h.beta2 * v + (1.0f - h.beta2) * grad * grad;
    const float normalized = m / bc1 / (sqrtf(v / bc2) + h.eps);
    master = master * (1.0f - h.lr * h.wd) - h.lr * normalized;
}

template <typename T>
__device__ __forceinline__ void update_chunk(T* __restrict__ p, const T* __restrict__ g, float* __restrict__ master,
                                             float* __restrict__ m, float* __restrict__ v, unsigned long long n,
                                             const Hyper& h, float bc1, float bc2, float clip) {
    constexpr int V = 4;  // 4 fp32 = 16 bytes for the state tensors; 8 bytes for 16-bit param/grad
    const bool vec = ((reinterpret_cast<std::uintptr_t>(p) | reinterpret_cast<std::uintptr_t>(g)) % (sizeof(T) * V) == 0) &&
                     ((reinterpret_cast<std::uintptr_t>(master) | reinterpret_cast<std::uintptr_t>(m) |
                       reinterpret_cast<std::uintptr_t>(v)) & 15u) == 0;
    if (vec) {
        for (unsigned long long i = threadIdx.x * V; i < n; i += kAdamThreads * V) {
            if (i + V <= n) {
                float gr[V], w[V], mm[V], vv[V];
                load_vec_stream<T, V>(gr, g + i);
                load_vec_stream<float, V>(w, master + i);
                load_vec_stream<float, V>(mm, m + i);
                load_vec_stream<float, V>(vv, v + i);
#pragma unroll
                for (int k = 0; k < V; ++k) adamw_element(gr[k], w[k], mm[k], vv[k], h, bc1, bc2, clip);
                store_vec_stream<float, V>(m + i, mm);
                store_vec_stream<float, V>(v + i, vv);
                store_vec_stream<float, V>(master + i, w);
                store_vec<T, V>(p + i, w);
            } else {
                for (unsigned long long j = i; j < n; ++j) {
                    float w = master[j], mm = m[j], vv = v[j];
                    adamw_element(to_f32<T>(g[j]), w, mm, vv, h, bc1, bc2, clip);
                    m[j] = mm; v[j] = vv; master[j] = w; p[j] = from_f32<T>(w);
                }
            }
        }
    } else {
        for (unsigned long long j = threadIdx.x; j < n; j += kAdamThreads) {
            float w = master[j], mm = m[j], vv = v[j];
            adamw_element(to_f32<T>(g[j]), w, mm, vv, h, bc1, bc2, clip);
            m[j] = mm; v[j] = vv; master[j] = w; p[j] = from_f32<T>(w);
        }
    }
}

__global__ void __launch_bounds__(kAdamThreads)
adamw_update_kernel(const DevTensor* __restrict__ tensors, const Chunk* __restrict__ chunks, unsigned int n_chunks,
                    Hyper h, const unsigned int* __restrict__ state, const float* __restrict__ scalars,
                    const float* __restrict__ lr_device) {
    if (state[0] != 0u) return;  // non-finite gradients: the whole step is skipped
    if (lr_device != nullptr) h.lr = *lr_device;   // the step's learning rate as a device scalar (captured graphs)
    const float bc1 = scalars[0], bc2 = scalars[1], clip = scalars[2];
    for (unsigned int c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const Chunk ch = chunks[c];
        const DevTensor t = tensors[ch.tensor];
        unsigned long long n = t.count - ch.offset;
        if (n > kChunk) n = kChunk;
        float* master = t.master + ch.offset;
        float* m = t.m + ch.offset;
        float* v = t.v + ch.offset;
        switch (t.dtype) {
            case CGPT_DTYPE_F16:
                update_chunk(static_cast<__half*>(t.param) + ch.offset, static_cast<const __half*>(t.grad) + ch.offset,
                             master, m, v, n, h, bc1, bc2, clip);
                break;
            case CGPT_DTYPE_BF16:
                update_chunk(static_cast<__nv_bfloat16*>(t.param) + ch.offset,
                             static_cast<const __nv_bfloat16*>(t.grad) + ch.offset, master, m, v, n, h, bc1, bc2, clip);
                break;
            default:
                update_chunk(static_cast<float*>(t.param) + ch.offset, static_cast<const float*>(t.grad) + ch.offset,
                             master, m, v, n, h, bc1, bc2, clip);
                break;
        }
    }
}

}  // namespace
}  // namespace cgpt

using namespace cgpt;

struct cgpt_adamw_workspace {
    DevTensor* d_tensors = nullptr;
    Chunk* d_chunks = nullptr;
    unsigned int n_chunks = 0;
    int grid = 0;
    float* d_partial_sums = nullptr;
    unsigned int* d_partial_bad = nullptr;
    unsigned int* d_state = nullptr;      // [2]
    unsigned long long* d_step = nullptr; // [1]
    float* d_scalars = nullptr;           // [4]
    std::size_t n_tensors = 0;
};

extern "C" int cgpt_adamw_destroy(cgpt_adamw_workspace* ws) {
    if (!ws) return CGPT_OK;
    cudaFree(ws->d_tensors);
    cudaFree(ws->d_chunks);
    cudaFree(ws->d_partial_sums);
    cudaFree(ws->d_partial_bad);
    cudaFree(ws->d_state);
    cudaFree(ws->d_step);
    cudaFree(ws->d_scalars);
    delete ws;
    return CGPT_OK;
}

extern "C" int cgpt_adamw_create(cgpt_adamw_workspace** out, const cgpt_adamw_tensor* tensors, size_t count,
                                 uint64_t initial_step, cgpt_stream_t stream) {
    if (!out || !tensors) return CGPT_ERR_NULL;
    if (count == 0 || count > 0x7fffffffull) return CGPT_ERR_SHAPE;
    std::vector<DevTensor> host_tensors(count);
    std::vector<Chunk> host_chunks;
    for (size_t i = 0; i < count; ++i) {
        const cgpt_adamw_tensor& t = tensors[i];
        if (!t.param || !t.grad || !t.master || !t.m || !t.v) return CGPT_ERR_NULL;
        if (!valid_float_dtype(t.dtype)) return CGPT_ERR_DTYPE;
        if (t.count == 0) return CGPT_ERR_SHAPE;
        host_tensors[i] = DevTensor{t.param, t.grad, t.master, t.m, t.v, t.count, t.dtype, 0};
        for (unsigned long long off = 0; off < t.count; off += kChunk)
            host_chunks.push_back(Chunk{static_cast<unsigned int>(i), 0u, off});
    }
    if (host_chunks.size() > 0xffffffffull) return CGPT_ERR_SHAPE;
    auto* ws = new cgpt_adamw_workspace();
    ws->n_tensors = count;
    ws->n_chunks = static_cast<unsigned int>(host_chunks.size());
    // every CTA of the chunk loops resident from the start (the smaller of what the two kernels fit per SM)
    int per_sm = resident_ctas_per_sm(reinterpret_cast<const void*>(adamw_update_kernel), kAdamThreads, 0);
    const int per_sm_stats = resident_ctas_per_sm(reinterpret_cast<const void*>(adamw_stats_kernel<false>), kAdamThreads, 0);
    if (per_sm_stats < per_sm) per_sm = per_sm_stats;
    const unsigned int cap = static_cast<unsigned int>(kNumSMs * per_sm);
    ws->grid = static_cast<int>(ws->n_chunks < cap ? ws->n_chunks : cap);
    auto s = static_cast<cudaStream_t>(stream);
    auto fail = [&](cudaError_t e) { cgpt_adamw_destroy(ws); return -static_cast<int>(e); };
    cudaError_t e;
    if ((e = cudaMalloc(&ws->d_tensors, count * sizeof(DevTensor))) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&ws->d_chunks, host_chunks.size() * sizeof(Chunk))) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&ws->d_partial_sums, ws->grid * sizeof(float))) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&ws->d_partial_bad, ws->grid * sizeof(unsigned int))) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&ws->d_state, 2 * sizeof(unsigned int))) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&ws->d_step, sizeof(unsigned long long))) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&ws->d_scalars, 4 * sizeof(float))) != cudaSuccess) return fail(e);
    // Synchronous copies from pageable host vectors: creation is a set-up call, not part of the step.
    if ((e = cudaMemcpy(ws->d_tensors, host_tensors.data(), count * sizeof(DevTensor), cudaMemcpyHostToDevice)) != cudaSuccess) return fail(e);
    if ((e = cudaMemcpy(ws->d_chunks, host_chunks.data(), host_chunks.size() * sizeof(Chunk), cudaMemcpyHostToDevice)) != cudaSuccess) return fail(e);
    const unsigned long long step0 = initial_step;
    if ((e = cudaMemcpy(ws->d_step, &step0, sizeof(step0), cudaMemcpyHostToDevice)) != cudaSuccess) return fail(e);
    if ((e = cudaMemset(ws->d_state, 0, 2 * sizeof(unsigned int))) != cudaSuccess) return fail(e);
    if ((e = cudaMemset(ws->d_scalars, 0, 4 * sizeof(float))) != cudaSuccess) return fail(e);
    (void)s;
    *out = ws;
    return CGPT_OK;
}

namespace {
int adamw_step_impl(cgpt_adamw_workspace* ws, const cgpt_adamw_options* o, const float* lr_device, cgpt_stream_t stream);
}

extern "C" int cgpt_adamw_step(cgpt_adamw_workspace* ws, const cgpt_adamw_options* o, cgpt_stream_t stream) {
    return adamw_step_impl(ws, o, nullptr, stream);
}

extern "C" int cgpt_adamw_step_device_lr(cgpt_adamw_workspace* ws, const cgpt_adamw_options* o, const float* learning_rate_device,
                                         cgpt_stream_t stream) {
    if (!learning_rate_device) return CGPT_ERR_NULL;
    return adamw_step_impl(ws, o, learning_rate_device, stream);
}

namespace {
int adamw_step_impl(cgpt_adamw_workspace* ws, const cgpt_adamw_options* o, const float* lr_device, cgpt_stream_t stream) {
    if (!ws || !o) return CGPT_ERR_NULL;
    // Same validation as the reference's validate_options (src/optim/adamw.cu:28-45).
    if (!(o->learning_rate >= 0.f) || !(o->beta1 >= 0.f && o->beta1 < 1.f) || !(o->beta2 >= 0.f && o->beta2 < 1.f) ||
        !(o->epsilon > 0.f) || !(o->weight_decay >= 0.f) || !(o->loss_scale > 0.f) || !(o->max_grad_norm > 0.f))
        return CGPT_ERR_OPTION;
    auto s = static_cast<cudaStream_t>(stream);
    {   // a power-of-two loss scale (the trainer's 1024) is divided out by an exact multiplication
        int exponent = 0;
        const bool pow2 = std::frexp(o->loss_scale, &exponent) == 0.5f && exponent > -100 && exponent < 100;
        const float inv = 1.0f / o->loss_scale;
        if (pow2)
            adamw_stats_kernel<true><<<ws->grid, kAdamThreads, 0, s>>>(ws->d_tensors, ws->d_chunks, ws->n_chunks, o->loss_scale, inv,
                                                                      ws->d_partial_sums, ws->d_partial_bad);
        else
            adamw_stats_kernel<false><<<ws->grid, kAdamThreads, 0, s>>>(ws->d_tensors, ws->d_chunks, ws->n_chunks, o->loss_scale, inv,
                                                                       ws->d_partial_sums, ws->d_partial_bad);
    }
    count_launch();
    CGPT_LAUNCH_CHECK();
    adamw_prepare_kernel<<<1, 256, 0, s>>>(ws->d_partial_sums, ws->d_partial_bad, ws->grid, ws->d_state, ws->d_step,
                                           ws->d_scalars, o->beta1, o->beta2, o->max_grad_norm);
    count_launch();
    CGPT_LAUNCH_CHECK();
    const Hyper h{o->beta1, o->beta2, o->learning_rate, o->epsilon, o->weight_decay, o->loss_scale};
    adamw_update_kernel<<<ws->grid, kAdamThreads, 0, s>>>(ws->d_tensors, ws->d_chunks, ws->n_chunks, h, ws->d_state,
                                                         ws->d_scalars, lr_device);
    count_launch();
    CGPT_LAUNCH_CHECK();
    return CGPT_OK;
}
}  // namespace

extern "C" int cgpt_adamw_check(cgpt_adamw_workspace* ws, uint64_t* step_out, int* non_finite_out,
                                cgpt_stream_t stream) {
    if (!ws) return CGPT_ERR_NULL;
    auto s = static_cast<cudaStream_t>(stream);
    unsigned int state[2] = {0, 0};
    unsigned long long step = 0;
    CGPT_CUDA_TRY(cudaMemcpyAsync(state, ws->d_state, sizeof(state), cudaMemcpyDeviceToHost, s));
    CGPT_CUDA_TRY(cudaMemcpyAsync(&step, ws->d_step, sizeof(step), cudaMemcpyDeviceToHost, s));
    CGPT_CUDA_TRY(cudaStreamSynchronize(s));
    CGPT_CUDA_TRY(cudaMemsetAsync(ws->d_state + 1, 0, sizeof(unsigned int), s));
    if (step_out) *step_out = step;
    if (non_finite_out) *non_finite_out = state[1] != 0u ? 1 : 0;
    return CGPT_OK;
}

extern "C" int cgpt_adamw_last_stats(cgpt_adamw_workspace* ws, float* squared_norm, float* clip,
                                     cgpt_stream_t stream) {
    if (!ws) return CGPT_ERR_NULL;
    auto s = static_cast<cudaStream_t>(stream);
    float sc[4] = {0, 0, 0, 0};
    CGPT_CUDA_TRY(cudaMemcpyAsync(sc, ws->d_scalars, sizeof(sc), cudaMemcpyDeviceToHost, s));
    CGPT_CUDA_TRY(cudaStreamSynchronize(s));
    if (squared_norm) *squared_norm = sc[3];
    if (clip) *clip = sc[2];
    return CGPT_OK;
}
