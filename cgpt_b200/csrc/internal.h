// Functions shared between translation units of the library (not part of the C ABI).
#pragma once
#include "common.cuh"

namespace cgpt {

// gemm.cu
int gemm_dispatch(void* C, const void* A, const void* B, long long M, long long N, long long K, int a_mn, int b_mn,
                  int accumulate, int dtype, bool force_simt, cudaStream_t s);
// The LM-head logits product x [M,K] * c [N,K]^T with a softmax epilogue (16-bit tensors, CTA-pair kernel; returns
// CGPT_ERR_UNSUPPORTED where that kernel does not apply). mode 1: out = logits, and per tile of 256 columns and row the
// pair (max, sum exp(l - max)) -> partial [M][ceil(N/256)], the target's logit -> target_logit [M]; mode 2: the same
// without storing the logits; mode 3: out = (exp(l - row_stats.x) * row_stats.y - onehot) * out_scale.
int gemm_logits_softmax(int mode, void* out, const void* x, const void* c, long long M, long long N, long long K,
                        float2* partial, float* target_logit, const std::uint32_t* targets, const float2* row_stats,
                        float out_scale, int dtype, cudaStream_t s);
int column_sum(void* out, const void* in, long long rows, long long cols, int accumulate, int dtype, cudaStream_t s);

// cross_entropy.cu
int cross_entropy_rows(float* row_loss, void* grad, const void* logits, const std::uint32_t* targets, long long rows,
                       long long vocab, float inv_total_rows, float gradient_scale, int dtype, cudaStream_t s);
int sum_floats(float* out, const float* in, long long n, cudaStream_t s);
// Softmax gradient from per-tile statistics (gemm_logits_softmax mode 1): G = (softmax - onehot) * inv_total_rows *
// gradient_scale written over the 16-bit logits [rows, vocab] in one pass, row losses to row_loss.
int softmax_grad_rows(float* row_loss, void* logits_to_grad, const float2* partial, const float* target_logit,
                      const std::uint32_t* targets, long long rows, long long vocab, int tiles, float inv_total_rows,
                      float gradient_scale, int dtype, cudaStream_t s);
// Row statistics (max, 1 / sum) and row losses from the per-tile statistics (before gemm_logits_softmax mode 3).
int softmax_stats_reduce(float2* row_stats, float* row_loss, const float2* partial, const float* target_logit,
                         const std::uint32_t* targets, long long rows, long long vocab, int tiles, float inv_total_rows,
                         cudaStream_t s);

}  // namespace cgpt
