// Shared device/host helpers for the cgpt_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstdlib>

#include "../../include/cgpt_b200.h"

namespace cgpt {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this.

// ---------------------------------------------------------------------------------------------
// Status helpers. Every C-ABI entry point returns 0, a positive CGPT_ERR_* argument class, or
// the negated cudaError_t of the failing runtime call. Nothing throws and nothing exits.
// ---------------------------------------------------------------------------------------------
inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? CGPT_OK : -static_cast<int>(e); }

#define CGPT_CUDA_TRY(expr)                                        \
    do {                                                           \
        cudaError_t cgpt_err__ = (expr);                           \
        if (cgpt_err__ != cudaSuccess) return -static_cast<int>(cgpt_err__); \
    } while (0)

#define CGPT_TRY(expr)                      \
    do {                                    \
        int cgpt_rc__ = (expr);             \
        if (cgpt_rc__ != CGPT_OK) return cgpt_rc__; \
    } while (0)

#define CGPT_LAUNCH_CHECK() CGPT_CUDA_TRY(cudaGetLastError())

inline bool valid_float_dtype(int dtype) {
    return dtype == CGPT_DTYPE_F16 || dtype == CGPT_DTYPE_BF16 || dtype == CGPT_DTYPE_F32;
}
inline std::size_t dtype_size(int dtype) { return dtype == CGPT_DTYPE_F32 ? 4 : 2; }

// Diagnosis switches (kernel variants that skip stores, trace buffers, forced fall-backs) are read from the environment
// only in a library built with -DCGPT_B200_DIAGNOSIS. The shipped build does not define it: there the switches do not
// exist, so no environment variable can change a result or hand a kernel a pointer.
inline const char* diagnosis_env(const char* name) {
#ifdef CGPT_B200_DIAGNOSIS
    return std::getenv(name);
#else
    (void)name;
    return nullptr;
#endif
}

inline bool aligned16(const void* p) { return (reinterpret_cast<std::uintptr_t>(p) & 15u) == 0; }

// Per-device scratch arena owned by the library. Grown with cudaMalloc on first use (never during
// stream capture: a growth request while the stream is capturing returns an error instead).
// Every kernel that needs global scratch and was not handed a caller workspace takes it from here.
int scratch_get(void** out, std::size_t bytes, cudaStream_t stream);
// CTAs of `kernel` (with this block size and dynamic shared memory) that one SM holds at a time, from the occupancy
// calculator, cached per (kernel, device). Grid-stride kernels size their grid as kNumSMs * this, so that every CTA is
// resident from the start: a grid of, say, 4 CTAs per SM on a kernel that fits 3 runs a last third of the work at a third
// of the occupancy.
int resident_ctas_per_sm(const void* kernel, int threads, std::size_t dynamic_smem);

// Holds `bytes` of the arena for the lifetime of the object, so that ops called meanwhile (which use
// scratch_get themselves) are placed behind it. `inner_headroom` is the most scratch those inner ops may
// ask for; the arena is grown to bytes + inner_headroom up front because it cannot move while held.
struct ScratchFrame {
    ScratchFrame(std::size_t bytes, std::size_t inner_headroom, cudaStream_t stream);
    ~ScratchFrame();
    ScratchFrame(const ScratchFrame&) = delete;
    ScratchFrame& operator=(const ScratchFrame&) = delete;
    void* ptr = nullptr;
    int status = CGPT_OK;

private:
    std::size_t held_ = 0;
};

// "Done once per device" flag for per-kernel attributes (cudaFuncSetAttribute applies to the current device only).
// Usage: static PerDeviceOnce once; if (once.needed()) { ...set attributes...; once.done(); }
struct PerDeviceOnce {
    bool flags[64] = {};
    int device = 0;
    bool needed() {
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) { device = 0; return true; }
        return !flags[device];
    }
    void done() { flags[device] = true; }
};

// While alive, scratch_get calls of this thread are served from arena `lane` (1 = ops issued on the side stream).
struct ScratchLane {
    explicit ScratchLane(int lane);
    ~ScratchLane();
    ScratchLane(const ScratchLane&) = delete;
    ScratchLane& operator=(const ScratchLane&) = delete;

private:
    int previous_;
};

// Two-stream execution of the block's independent branches (runtime.cu).
bool branch_streams_enabled();
int side_stream_get(cudaStream_t main, cudaStream_t* side, cudaEvent_t* fork, cudaEvent_t* join);

// ---------------------------------------------------------------------------------------------
// Scalar conversion
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------------------
// Vector access: N consecutive elements of T moved with the widest possible single instruction
// (16 bytes for N*sizeof(T) == 16). The address must be aligned to N*sizeof(T).
// ---------------------------------------------------------------------------------------------
template <int BYTES> struct RawVec;
template <> struct RawVec<2> { using type = unsigned short; };
template <> struct RawVec<4> { using type = unsigned int; };
template <> struct RawVec<8> { using type = uint2; };
template <> struct RawVec<16> { using type = uint4; };
template <> struct RawVec<32> { using type = ulonglong4; };

template <typename T, int N>
struct alignas(sizeof(T) * N) Pack {
    T v[N];
};

// Pack -> fp32. 16-bit types convert two values per packed register (the pair intrinsics select the half inside the
// conversion instead of extracting it first): same values as the scalar conversions, fewer instructions.
template <typename T, int N>
__device__ __forceinline__ void unpack_pack(float (&out)[N], const Pack<T, N>& pk) {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = to_f32<T>(pk.v[i]);
}
template <int N>
__device__ __forceinline__ void unpack_pack(float (&out)[N], const Pack<__half, N>& pk) {
    if constexpr (N % 2 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pk.v[i]));
            out[i] = f.x;
            out[i + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = __half2float(pk.v[i]);
    }
}
template <int N>
__device__ __forceinline__ void unpack_pack(float (&out)[N], const Pack<__nv_bfloat16, N>& pk) {
    if constexpr (N % 2 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 2) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk.v[i]));
            out[i] = f.x;
            out[i + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = __bfloat162float(pk.v[i]);
    }
}

template <typename T, int N>
__device__ __forceinline__ void load_vec(float (&out)[N], const T* __restrict__ p) {
    using Raw = typename RawVec<sizeof(T) * N>::type;
    Pack<T, N> pk;
    *reinterpret_cast<Raw*>(&pk) = *reinterpret_cast<const Raw*>(p);
    unpack_pack(out, pk);
}

// Streaming (read-once) variant: bypasses L1 allocation.
template <typename T, int N>
__device__ __forceinline__ void load_vec_stream(float (&out)[N], const T* __restrict__ p) {
    using Raw = typename RawVec<sizeof(T) * N>::type;
    Pack<T, N> pk;
    *reinterpret_cast<Raw*>(&pk) = __ldcs(reinterpret_cast<const Raw*>(p));
    unpack_pack(out, pk);
}

// Round-to-nearest conversion of N floats into a Pack. 16-bit types convert two values per instruction
// (cvt.rn.f16x2.f32 / cvt.rn.bf16x2.f32): same results as the scalar conversions, half the instructions.
template <typename T, int N>
__device__ __forceinline__ void convert_pack(Pack<T, N>& pk, const float (&in)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) pk.v[i] = from_f32<T>(in[i]);
}
template <int N>
__device__ __forceinline__ void convert_pack(Pack<__half, N>& pk, const float (&in)[N]) {
    if constexpr (N % 2 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 2) *reinterpret_cast<__half2*>(&pk.v[i]) = __floats2half2_rn(in[i], in[i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) pk.v[i] = __float2half_rn(in[i]);
    }
}
template <int N>
__device__ __forceinline__ void convert_pack(Pack<__nv_bfloat16, N>& pk, const float (&in)[N]) {
    if constexpr (N % 2 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 2) *reinterpret_cast<__nv_bfloat162*>(&pk.v[i]) = __floats2bfloat162_rn(in[i], in[i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) pk.v[i] = __float2bfloat16_rn(in[i]);
    }
}

template <typename T, int N>
__device__ __forceinline__ void store_vec(T* __restrict__ p, const float (&in)[N]) {
    using Raw = typename RawVec<sizeof(T) * N>::type;
    Pack<T, N> pk;
    convert_pack(pk, in);
    *reinterpret_cast<Raw*>(p) = *reinterpret_cast<const Raw*>(&pk);
}

template <typename T, int N>
__device__ __forceinline__ void store_vec_stream(T* __restrict__ p, const float (&in)[N]) {
    using Raw = typename RawVec<sizeof(T) * N>::type;
    Pack<T, N> pk;
    convert_pack(pk, in);
    __stcs(reinterpret_cast<Raw*>(p), *reinterpret_cast<const Raw*>(&pk));
}

// Rounds a pair of fp32 values to the storage dtype and back (where the reference stores an intermediate tensor).
template <typename T>
__device__ __forceinline__ void round_pair_to_storage(float& a, float& b) {
    a = to_f32<T>(from_f32<T>(a));
    b = to_f32<T>(from_f32<T>(b));
}
template <>
__device__ __forceinline__ void round_pair_to_storage<__half>(float& a, float& b) {
    const float2 f = __half22float2(__floats2half2_rn(a, b));
    a = f.x;
    b = f.y;
}
template <>
__device__ __forceinline__ void round_pair_to_storage<__nv_bfloat16>(float& a, float& b) {
    const float2 f = __bfloat1622float2(__floats2bfloat162_rn(a, b));
    a = f.x;
    b = f.y;
}

// Division of a 31-bit dividend by a run-time constant: q = (n * mul) >> (31 + shift), exact for n < 2^31
// (mul = floor(2^(31+shift) / d) + 1 with shift = ceil(log2 d) fits 32 bits).
struct FastDiv {
    unsigned d, mul, shift;
    FastDiv() : d(1), mul(0x80000001u), shift(0) {}
    explicit FastDiv(unsigned divisor) : d(divisor) {
        shift = 0;
        while ((1ull << shift) < divisor) ++shift;
        mul = static_cast<unsigned>((1ull << (31 + shift)) / divisor + 1);
    }
    __host__ __device__ __forceinline__ unsigned div(unsigned n) const {
        return static_cast<unsigned>((static_cast<unsigned long long>(n) * mul) >> (31 + shift));
    }
    __host__ __device__ __forceinline__ void divmod(unsigned n, unsigned& q, unsigned& r) const {
        q = div(n);
        r = n - q * d;
    }
};

// ---------------------------------------------------------------------------------------------
// Reductions
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// exp as the reference's fast-math build computes __expf: ex2.approx.ftz(x * log2 e).
__device__ __forceinline__ float fast_exp(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
    return y;
}

// Dispatch a lambda-like macro body over the storage dtype.
#define CGPT_DISPATCH_DTYPE(dtype, T, ...)                       \
    switch (dtype) {                                             \
        case CGPT_DTYPE_F16: { using T = __half; __VA_ARGS__; break; }        \
        case CGPT_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
        case CGPT_DTYPE_F32: { using T = float; __VA_ARGS__; break; }          \
        default: return CGPT_ERR_DTYPE;                          \
    }

}  // namespace cgpt
