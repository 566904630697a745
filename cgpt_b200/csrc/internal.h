// Functions shared between translation units of the library (not part of the C ABI).
#pragma once
#include "common.cuh"

namespace cgpt {

// gemm.cu
int gemm_dispatch(void* C, const void* A, const void* B, long long M, long long N, long long K, int a_mn, int b_mn,
                  int accumulate, int dtype, bool force_simt, cudaStream_t s);
int column_sum(void* out, const void* in, long long rows, long long cols, int accumulate, int dtype, cudaStream_t s);

// cross_entropy.cu
int cross_entropy_rows(float* row_loss, void* grad, const void* logits, const std::uint32_t* targets, long long rows,
                       long long vocab, float inv_total_rows, float gradient_scale, int dtype, cudaStream_t s);
int sum_floats(float* out, const float* in, long long n, cudaStream_t s);

}  // namespace cgpt
