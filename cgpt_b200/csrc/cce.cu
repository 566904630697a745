// Cut cross-entropy: LM-head GEMM + softmax cross-entropy + both LM-head gradient GEMMs without a
// [rows, vocab] tensor in memory.
//
// Rows (tokens) are processed in chunks. For each chunk
//   1. logits_chunk = X_chunk C^T                      tensor-core GEMM into scratch [chunk, vocab]
//   2. G = (softmax - onehot)/rows * gradient_scale    in place over the logits, row losses to scratch
//   3. dX_chunk = G C                                  tensor-core GEMM, complete (reduction over vocab)
//   4. dC (+)= G^T X_chunk                             tensor-core GEMM, accumulated over chunks
// and finally loss = fixed-order sum of the row losses. Because whole rows of logits exist inside a chunk
// the softmax needs no second pass over the vocabulary and no recomputation of the logits GEMM: the
// arithmetic is the three GEMMs 2*rows*vocab*hidden each, the same as with materialised logits, while the
// scratch is chunk_rows*vocab elements instead of rows*vocab.
//
// Reference semantics: src/ops/cut_cross_entropy.cu:97-160 (F32 tensors; same loss and gradients, no
// gradient_scale there) and, for what CGPT's trainer computes on fp16 logits, src/ops/cross_entropy.cu:
// 134-245 between linear_forward and linear_backward (train/train.cpp:536-544).
#include "internal.h"
#include "launch_counter.h"

using namespace cgpt;

extern "C" int cgpt_cut_cross_entropy(float* loss, void* dx, void* dc, const void* x, const void* c,
                                      const uint32_t* targets, size_t rows, size_t vocab, size_t hidden,
                                      float gradient_scale, int accumulate_dc, size_t chunk_rows, int dtype,
                                      cgpt_stream_t stream) {
    if (!loss || !dx || !dc || !x || !c || !targets) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rows == 0 || vocab == 0 || hidden == 0 || vocab > 0x7fffffffull || hidden > 0x7fffffffull ||
        rows > 0x7fffffffull)
        return CGPT_ERR_SHAPE;
    auto s = static_cast<cudaStream_t>(stream);
    if (chunk_rows == 0) chunk_rows = 8192;
    if (chunk_rows > rows) chunk_rows = rows;
    const std::size_t esz = dtype_size(dtype);
    const std::size_t loss_bytes = (rows * sizeof(float) + 255) & ~std::size_t{255};
    // The GEMMs below take their split-K scratch from the same arena: hold this call's buffers in a frame
    // so they are placed behind it, with headroom for the largest split-K workspace they can ask for.
    ScratchFrame frame(loss_bytes + chunk_rows * vocab * esz, std::size_t{128} << 20, s);
    CGPT_TRY(frame.status);
    float* row_loss = static_cast<float*>(frame.ptr);
    void* chunk = static_cast<unsigned char*>(frame.ptr) + loss_bytes;
    const float inv_rows = 1.0f / static_cast<float>(rows);
    const long long V = static_cast<long long>(vocab), H = static_cast<long long>(hidden);
    for (std::size_t r0 = 0; r0 < rows; r0 += chunk_rows) {
        const long long n = static_cast<long long>(rows - r0 < chunk_rows ? rows - r0 : chunk_rows);
        const unsigned char* xc = static_cast<const unsigned char*>(x) + r0 * hidden * esz;
        unsigned char* dxc = static_cast<unsigned char*>(dx) + r0 * hidden * esz;
        CGPT_TRY(gemm_dispatch(chunk, xc, c, n, V, H, 0, 0, 0, dtype, false, s));                 // logits
        CGPT_TRY(cross_entropy_rows(row_loss + r0, chunk, chunk, targets + r0, n, V, inv_rows, gradient_scale, dtype, s));
        CGPT_TRY(gemm_dispatch(dxc, chunk, c, n, H, V, 0, 1, 0, dtype, false, s));                // dX = G C
        CGPT_TRY(gemm_dispatch(dc, chunk, xc, V, H, n, 1, 1, (accumulate_dc || r0 > 0) ? 1 : 0, dtype, false, s));  // dC += G^T X
    }
    return sum_floats(loss, row_loss, static_cast<long long>(rows), s);
}
