// Embedding gather and deterministic embedding backward for sm_100a.
//
// Reference semantics (src/ops/backward/embedding_backward.cu:39-92,207-254): after an optional
// memset, grad_weight[ids[t], :] += grad_output[t, :] for every token whose id is inside the table.
// The reference adds with storage-dtype atomics in arrival order, which makes the fp16 rounding
// order-dependent. Here tokens are grouped by id with a stable radix sort (keys: ids, values: token
// index) so each table row has exactly one owner CTA that sums its tokens in ascending token order in
// fp32 and rounds once; identical inputs give identical bits on every run.
//
// Memory-bound: reads grad_output once (tokens*hidden*sizeof(T)), writes (and, when accumulating,
// reads) only the touched table rows, plus the memset of the table when not accumulating.
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"
#include "launch_counter.h"

namespace cgpt {
namespace {

template <typename T, int VEC>
__global__ void __launch_bounds__(128)
embedding_forward_kernel(T* __restrict__ out, const std::uint32_t* __restrict__ ids,
                         const T* __restrict__ weight, long long tokens, int vocab, int hidden) {
    for (long long t = blockIdx.x; t < tokens; t += gridDim.x) {
        const std::uint32_t id = ids[t];
        const bool ok = id < static_cast<std::uint32_t>(vocab);
        for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC) {
            float v[VEC];
            if (ok) load_vec<T, VEC>(v, weight + static_cast<long long>(id) * hidden + c);
            else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[i] = 0.f;
            }
            store_vec<T, VEC>(out + t * hidden + c, v);
        }
    }
}

__global__ void embedding_keys_kernel(std::uint32_t* __restrict__ keys, std::uint32_t* __restrict__ vals,
                                      const std::uint32_t* __restrict__ ids, long long tokens, std::uint32_t vocab) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t < tokens) {
        const std::uint32_t id = ids[t];
        keys[t] = id < vocab ? id : vocab;  // every out-of-table id sorts behind the table
        vals[t] = static_cast<std::uint32_t>(t);
    }
}

// One CTA per sorted position; only the first position of each id run does work.
template <typename T, int VEC>
__global__ void __launch_bounds__(128)
embedding_backward_kernel(T* __restrict__ grad_weight, const T* __restrict__ grad_output,
                          const std::uint32_t* __restrict__ sorted_ids,
                          const std::uint32_t* __restrict__ sorted_tokens, long long tokens, std::uint32_t vocab,
                          int hidden, int accumulate) {
    const long long pos = blockIdx.x;
    const std::uint32_t id = sorted_ids[pos];
    if (id >= vocab) return;
    if (pos > 0 && sorted_ids[pos - 1] == id) return;
    for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC) {
        float acc[VEC];
        if (accumulate) load_vec<T, VEC>(acc, grad_weight + static_cast<long long>(id) * hidden + c);
        else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
        }
        for (long long p = pos; p < tokens && sorted_ids[p] == id; ++p) {
            float g[VEC];
            load_vec_stream<T, VEC>(g, grad_output + static_cast<long long>(sorted_tokens[p]) * hidden + c);
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] += g[i];
        }
        store_vec<T, VEC>(grad_weight + static_cast<long long>(id) * hidden + c, acc);
    }
}

inline int bit_length(std::uint64_t v) {
    int b = 0;
    while (v) { ++b; v >>= 1; }
    return b;
}

}  // namespace
}  // namespace cgpt

using namespace cgpt;

extern "C" int cgpt_embedding_forward(void* out, const uint32_t* ids, const void* weight, size_t tokens,
                                      size_t vocab, size_t hidden, int dtype, cgpt_stream_t stream) {
    if (!out || !ids || !weight) return CGPT_ERR_NULL;
    if (tokens == 0 || vocab == 0 || hidden == 0 || vocab > 0x7fffffffull || hidden > 0x7fffffffull ||
        tokens > 0xffffffffull)
        return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>(tokens < kNumSMs * 16ull ? tokens : kNumSMs * 16ull);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (hidden % V == 0 && aligned16(out) && aligned16(weight))
            embedding_forward_kernel<T, V><<<grid, 128, 0, s>>>(static_cast<T*>(out), ids, static_cast<const T*>(weight),
                                                             static_cast<long long>(tokens), static_cast<int>(vocab),
                                                             static_cast<int>(hidden));
        else
            embedding_forward_kernel<T, 1><<<grid, 128, 0, s>>>(static_cast<T*>(out), ids, static_cast<const T*>(weight),
                                                             static_cast<long long>(tokens), static_cast<int>(vocab),
                                                             static_cast<int>(hidden));
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}

extern "C" int cgpt_embedding_backward(void* grad_weight, const void* grad_output, const uint32_t* ids,
                                       size_t tokens, size_t vocab, size_t hidden, int bounds_check,
                                       int accumulate, int dtype, cgpt_stream_t stream) {
    (void)bounds_check;  // ids outside the table are always skipped (the reference's unchecked mode is UB)
    if (!grad_weight || !grad_output || !ids) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (tokens == 0 || vocab == 0 || hidden == 0 || vocab > 0x7ffffffeull || hidden > 0x7fffffffull ||
        tokens > 0x7fffffffull)
        return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);

    const int end_bit = bit_length(vocab);  // keys are in [0, vocab]
    std::size_t cub_bytes = 0;
    std::uint32_t* null_u32 = nullptr;
    CGPT_CUDA_TRY(cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, null_u32, null_u32, null_u32, null_u32,
                                                  static_cast<int>(tokens), 0, end_bit, s));
    const std::size_t arr = (tokens * sizeof(std::uint32_t) + 255) & ~std::size_t{255};
    void* scratch = nullptr;
    CGPT_TRY(scratch_get(&scratch, 4 * arr + cub_bytes + 256, s));
    auto* base = static_cast<unsigned char*>(scratch);
    auto* keys_in = reinterpret_cast<std::uint32_t*>(base);
    auto* vals_in = reinterpret_cast<std::uint32_t*>(base + arr);
    auto* keys_out = reinterpret_cast<std::uint32_t*>(base + 2 * arr);
    auto* vals_out = reinterpret_cast<std::uint32_t*>(base + 3 * arr);
    void* cub_tmp = base + 4 * arr;

    if (!accumulate) CGPT_CUDA_TRY(cudaMemsetAsync(grad_weight, 0, vocab * hidden * dtype_size(dtype), s));
    embedding_keys_kernel<<<static_cast<unsigned>((tokens + 255) / 256), 256, 0, s>>>(
        keys_in, vals_in, ids, static_cast<long long>(tokens), static_cast<std::uint32_t>(vocab));
    count_launch();
    CGPT_LAUNCH_CHECK();
    CGPT_CUDA_TRY(cub::DeviceRadixSort::SortPairs(cub_tmp, cub_bytes, keys_in, keys_out, vals_in, vals_out,
                                                  static_cast<int>(tokens), 0, end_bit, s));
    count_launch(3);
    CGPT_DISPATCH_DTYPE(dtype, T, {
        constexpr int V = 16 / sizeof(T);
        if (hidden % V == 0 && aligned16(grad_weight) && aligned16(grad_output))
            embedding_backward_kernel<T, V><<<static_cast<unsigned>(tokens), 128, 0, s>>>(
                static_cast<T*>(grad_weight), static_cast<const T*>(grad_output), keys_out, vals_out,
                static_cast<long long>(tokens), static_cast<std::uint32_t>(vocab), static_cast<int>(hidden), accumulate);
        else
            embedding_backward_kernel<T, 1><<<static_cast<unsigned>(tokens), 128, 0, s>>>(
                static_cast<T*>(grad_weight), static_cast<const T*>(grad_output), keys_out, vals_out,
                static_cast<long long>(tokens), static_cast<std::uint32_t>(vocab), static_cast<int>(hidden), accumulate);
        count_launch();
        CGPT_LAUNCH_CHECK();
    });
    return CGPT_OK;
}
