// SwiGLU forward/backward and residual adds for sm_100a: pure streaming kernels, one 16-byte vector
// per thread per tensor per iteration, grid = a multiple of the SM count with a grid-stride loop.
//
// Math follows the reference:
//   forward   y = g / (1 + __expf(-g)) * up                               (src/ops/swiglu.cu:69-71)
//   backward  s = 1/(1+expf(-g)); dgate = dy*up*s*(1+g*(1-s)); dup = dy*g*s
//                                                                          (src/ops/backward/swiglu_backward.cu:61-74)
// Algorithmic HBM bytes per element: forward 3*sizeof(T); backward 5*sizeof(T) (+1 per accumulate flag).
#include "common.cuh"
#include "launch_counter.h"

namespace cgpt {
namespace {

__device__ __forceinline__ float sigmoid_accurate(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
swiglu_forward_kernel(T* __restrict__ y, const T* __restrict__ gate, const T* __restrict__ up, long long count) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * VEC;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC; i < count; i += stride) {
        if (i + VEC <= count) {
            float g[VEC], u[VEC], o[VEC];
            load_vec_stream<T, VEC>(g, gate + i);
            load_vec_stream<T, VEC>(u, up + i);
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = g[k] / (1.0f + __expf(-g[k])) * u[k];
            store_vec<T, VEC>(y + i, o);
        } else {
            for (long long j = i; j < count; ++j) {
                const float g = to_f32<T>(gate[j]);
                y[j] = from_f32<T>(g / (1.0f + __expf(-g)) * to_f32<T>(up[j]));
            }
        }
    }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
swiglu_backward_kernel(T* dgate, T* dup, const T* __restrict__ dy, const T* __restrict__ gate,
                       const T* __restrict__ up, long long count, int acc_gate, int acc_up) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * VEC;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC; i < count; i += stride) {
        if (i + VEC <= count) {
            float g[VEC], u[VEC], d[VEC], og[VEC], ou[VEC];
            load_vec_stream<T, VEC>(d, dy + i);
            load_vec_stream<T, VEC>(g, gate + i);
            load_vec_stream<T, VEC>(u, up + i);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                const float s = sigmoid_accurate(g[k]);
                og[k] = d[k] * u[k] * (s * (1.0f + g[k] * (1.0f - s)));
                ou[k] = d[k] * (g[k] * s);
            }
            if (acc_gate) {
                float old[VEC];
                load_vec<T, VEC>(old, dgate + i);
#pragma unroll
                for (int k = 0; k < VEC; ++k) og[k] += old[k];
            }
            if (acc_up) {
                float old[VEC];
                load_vec<T, VEC>(old, dup + i);
#pragma unroll
                for (int k = 0; k < VEC; ++k) ou[k] += old[k];
            }
            store_vec<T, VEC>(dgate + i, og);
            store_vec<T, VEC>(dup + i, ou);
        } else {
            for (long long j = i; j < count; ++j) {
                const float g = to_f32<T>(gate[j]), u = to_f32<T>(up[j]), d = to_f32<T>(dy[j]);
                const float s = sigmoid_accurate(g);
                float a = d * u * (s * (1.0f + g * (1.0f - s)));
                float b = d * (g * s);
                if (acc_gate) a += to_f32<T>(dgate[j]);
                if (acc_up) b += to_f32<T>(dup[j]);
                dgate[j] = from_f32<T>(a);
                dup[j] = from_f32<T>(b);
            }
        }
    }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
add_kernel(T* out, const T* a, const T* b, const T* c, long long count) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * VEC;
    for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC; i < count; i += stride) {
        if (i + VEC <= count) {
            float x[VEC], y[VEC];
            load_vec<T, VEC>(x, a + i);
            load_vec<T, VEC>(y, b + i);
#pragma unroll
            for (int k = 0; k < VEC; ++k) x[k] += y[k];
            if (c != nullptr) {
                load_vec<T, VEC>(y, c + i);
#pragma unroll
                for (int k = 0; k < VEC; ++k) x[k] += y[k];
            }
            store_vec<T, VEC>(out + i, x);
        } else {
            for (long long j = i; j < count; ++j) {
                float v = to_f32<T>(a[j]) + to_f32<T>(b[j]);
                if (c != nullptr) v += to_f32<T>(c[j]);
                out[j] = from_f32<T>(v);
            }
        }
    }
}

// Grid of a grid-stride kernel of 256 threads: enough CTAs for the elements, at most what the SMs hold at a time.
template <typename Kernel>
inline unsigned stream_grid(Kernel kernel, long long count, int vec) {
    long long blocks = (count + 256ll * vec - 1) / (256ll * vec);
    const long long cap = static_cast<long long>(kNumSMs) * resident_ctas_per_sm(reinterpret_cast<const void*>(kernel), 256, 0);
    if (blocks > cap) blocks = cap;
    return static_cast<unsigned>(blocks < 1 ? 1 : blocks);
}

}  // namespace
}  // namespace cgpt

using namespace cgpt;

extern "C" int cgpt_swiglu_forward(void* y, const void* gate, const void* up, size_t count, int dtype,
                                   cgpt_stream_t stream) {
    if (!y || !gate || !up) return CGPT_ERR_NULL;
    if (count == 0 || count > (1ull << 46)) return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    const bool al = aligned16(y) && aligned16(gate) && aligned16(up);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (al)
            swiglu_forward_kernel<T, V><<<stream_grid(swiglu_forward_kernel<T, V>, count, V), 256, 0, s>>>(
                static_cast<T*>(y), static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<long long>(count));
        else
            swiglu_forward_kernel<T, 1><<<stream_grid(swiglu_forward_kernel<T, 1>, count, 1), 256, 0, s>>>(
                static_cast<T*>(y), static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<long long>(count));
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}

extern "C" int cgpt_swiglu_backward(void* dgate, void* dup, const void* dy, const void* gate, const void* up,
                                    size_t count, int accumulate_gate, int accumulate_up, int dtype,
                                    cgpt_stream_t stream) {
    if (!dgate || !dup || !dy || !gate || !up) return CGPT_ERR_NULL;
    if (count == 0 || count > (1ull << 46)) return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    const bool al = aligned16(dgate) && aligned16(dup) && aligned16(dy) && aligned16(gate) && aligned16(up);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (al)
            swiglu_backward_kernel<T, V><<<stream_grid(swiglu_backward_kernel<T, V>, count, V), 256, 0, s>>>(
                static_cast<T*>(dgate), static_cast<T*>(dup), static_cast<const T*>(dy), static_cast<const T*>(gate),
                static_cast<const T*>(up), static_cast<long long>(count), accumulate_gate, accumulate_up);
        else
            swiglu_backward_kernel<T, 1><<<stream_grid(swiglu_backward_kernel<T, 1>, count, 1), 256, 0, s>>>(
                static_cast<T*>(dgate), static_cast<T*>(dup), static_cast<const T*>(dy), static_cast<const T*>(gate),
                static_cast<const T*>(up), static_cast<long long>(count), accumulate_gate, accumulate_up);
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}

extern "C" int cgpt_add(void* out, const void* a, const void* b, const void* c, size_t count, int dtype,
                        cgpt_stream_t stream) {
    if (!out || !a || !b) return CGPT_ERR_NULL;
    if (count == 0 || count > (1ull << 46)) return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    const bool al = aligned16(out) && aligned16(a) && aligned16(b) && aligned16(c);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (al)
            add_kernel<T, V><<<stream_grid(add_kernel<T, V>, count, V), 256, 0, s>>>(
                static_cast<T*>(out), static_cast<const T*>(a), static_cast<const T*>(b), static_cast<const T*>(c),
                static_cast<long long>(count));
        else
            add_kernel<T, 1><<<stream_grid(add_kernel<T, 1>, count, 1), 256, 0, s>>>(
                static_cast<T*>(out), static_cast<const T*>(a), static_cast<const T*>(b), static_cast<const T*>(c),
                static_cast<long long>(count));
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}
