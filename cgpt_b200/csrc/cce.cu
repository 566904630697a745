// Cut cross-entropy: LM-head GEMM + softmax cross-entropy + both LM-head gradient GEMMs without a
// [rows, vocab] tensor in memory.
//
// Rows (tokens) are processed in chunks. Three forms of a chunk are built; all end with
//   dX_chunk = G C  (reduction over vocab)   and   dC (+)= G^T X_chunk  (accumulated over chunks)
// on tensor cores, with G = (softmax - onehot)/rows * gradient_scale in a [chunk, vocab] 16-bit scratch:
//   kCceRows (1)       logits = X_chunk C^T into the scratch; one row kernel (row max, exp, row sum, gradient in place).
//   kCceTiles (2)      the logits product's epilogue also leaves per-row statistics of every 256-column tile
//                      (gemm_pair.cuh), so the gradient is ONE streaming pass over the scratch with no row reduction.
//   kCceRecompute (3)  the logits are never stored: product 1 leaves only the tile statistics, a small kernel combines
//                      them per row, product 2 recomputes the logits and its epilogue writes G straight from TMEM.
//                      Four products instead of three; the scratch holds the gradient only.
// A kernel that also kept G on chip would need the dX accumulator of a row block (128 x hidden fp32) or the dC
// accumulator of a vocabulary block beside the logits tile in tensor memory: at hidden 1024 either alone is twice the
// 512 columns an SM has, so G goes through the (L2-sized) scratch in all three forms.
// The default form is the fastest measured one (kCceDefault below); all three give the same loss and gradients
// up to the rounding of the row sums (tests compare them).
//
// Reference semantics: src/ops/cut_cross_entropy.cu:97-160 (F32 tensors; same loss and gradients, no
// gradient_scale there) and, for what CGPT's trainer computes on fp16 logits, src/ops/cross_entropy.cu:
// 134-245 between linear_forward and linear_backward (train/train.cpp:536-544).
#include <cstdlib>

#include "internal.h"
#include "launch_counter.h"

using namespace cgpt;

namespace {
enum : int { kCceAuto = 0, kCceRows = 1, kCceTiles = 2, kCceRecompute = 3 };
// Measured at 32768 x 1024 x 32000 fp16 on one B200, 8192-row chunks: tiles 5.43 ms, rows 5.51-5.53 ms, recompute 6.36 ms per
// call (per chunk under a profiler: logits product 412 us, with the statistics epilogue 445 us; row kernel 218 us, streaming
// gradient pass 185 us; statistics-only product 402 us + gradient-writing product 435 us).
constexpr int kCceDefault = kCceTiles;

int cut_cross_entropy_form(int form, float* loss, void* dx, void* dc, const void* x, const void* c, const uint32_t* targets,
                           size_t rows, size_t vocab, size_t hidden, float gradient_scale, int accumulate_dc, size_t chunk_rows,
                           int dtype, cudaStream_t s) {
    if (!loss || !dx || !dc || !x || !c || !targets) return CGPT_ERR_NULL;
    if (!valid_float_dtype(dtype)) return CGPT_ERR_DTYPE;
    if (rows == 0 || vocab == 0 || hidden == 0 || vocab > 0x7fffffffull || hidden > 0x7fffffffull ||
        rows > 0x7fffffffull)
        return CGPT_ERR_SHAPE;
    if (form < kCceAuto || form > kCceRecompute) return CGPT_ERR_OPTION;
    const bool explicit_form = form != kCceAuto;
    if (form == kCceAuto) {
        // diagnosis builds: CGPT_B200_CCE_FORM=1|2|3 replaces the default form (same-box comparisons inside a training step)
        static const int forced = [] { const char* e = diagnosis_env("CGPT_B200_CCE_FORM"); return e ? std::atoi(e) : 0; }();
        form = forced >= kCceRows && forced <= kCceRecompute ? forced : kCceDefault;
    }
    // Default chunk: 74 row tiles of 256 (one tile per CTA pair of the GPU), so that the dX product of a chunk, whose work
    // list is (row tiles) x (hidden / 256 column tiles), is a whole number of waves for any hidden size. Measured at
    // 32768 x 1024 x 32000: 5.30-5.32 ms against 5.42-5.44 ms with 8192-row chunks (128 units on 74 pairs = 2 waves, the
    // second one a quarter empty); scratch 1.2 GB instead of 0.5 GB.
    if (chunk_rows == 0) chunk_rows = static_cast<size_t>(kNumSMs / 2) * 256;
    if (chunk_rows > rows) chunk_rows = rows;
    const std::size_t esz = dtype_size(dtype);
    auto pad = [](std::size_t b) { return (b + 255) & ~std::size_t{255}; };
    const int tiles = static_cast<int>((vocab + 255) / 256);
    const std::size_t loss_bytes = pad(rows * sizeof(float));
    const std::size_t chunk_bytes = pad(chunk_rows * vocab * esz);
    const std::size_t partial_bytes = form == kCceRows ? 0 : pad(chunk_rows * tiles * sizeof(float2));
    const std::size_t target_bytes = form == kCceRows ? 0 : pad(chunk_rows * sizeof(float));
    const std::size_t stats_bytes = form == kCceRecompute ? pad(chunk_rows * sizeof(float2)) : 0;
    // The GEMMs below take their split-K scratch from the same arena: hold this call's buffers in a frame
    // so they are placed behind it, with headroom for the largest split-K workspace they can ask for.
    ScratchFrame frame(loss_bytes + chunk_bytes + partial_bytes + target_bytes + stats_bytes, std::size_t{128} << 20, s);
    CGPT_TRY(frame.status);
    unsigned char* base = static_cast<unsigned char*>(frame.ptr);
    float* row_loss = reinterpret_cast<float*>(base);
    void* chunk = base + loss_bytes;
    float2* partial = reinterpret_cast<float2*>(base + loss_bytes + chunk_bytes);
    float* target_logit = reinterpret_cast<float*>(base + loss_bytes + chunk_bytes + partial_bytes);
    float2* row_stats = reinterpret_cast<float2*>(base + loss_bytes + chunk_bytes + partial_bytes + target_bytes);
    const float inv_rows = 1.0f / static_cast<float>(rows);
    const long long V = static_cast<long long>(vocab), H = static_cast<long long>(hidden);
    for (std::size_t r0 = 0; r0 < rows; r0 += chunk_rows) {
        const long long n = static_cast<long long>(rows - r0 < chunk_rows ? rows - r0 : chunk_rows);
        const unsigned char* xc = static_cast<const unsigned char*>(x) + r0 * hidden * esz;
        unsigned char* dxc = static_cast<unsigned char*>(dx) + r0 * hidden * esz;
        int chunk_form = form;
        if (chunk_form == kCceTiles) {
            const int rc = gemm_logits_softmax(1, chunk, xc, c, n, V, H, partial, target_logit, targets + r0, nullptr, 0.f, dtype, s);
            if (rc == CGPT_ERR_UNSUPPORTED) {
                if (explicit_form) return rc;
                chunk_form = kCceRows;     // e.g. a short last chunk: the row kernel handles every shape
            } else {
                CGPT_TRY(rc);
                CGPT_TRY(softmax_grad_rows(row_loss + r0, chunk, partial, target_logit, targets + r0, n, V, tiles, inv_rows,
                                           gradient_scale, dtype, s));
            }
        } else if (chunk_form == kCceRecompute) {
            const int rc = gemm_logits_softmax(2, nullptr, xc, c, n, V, H, partial, target_logit, targets + r0, nullptr, 0.f, dtype, s);
            if (rc == CGPT_ERR_UNSUPPORTED) {
                if (explicit_form) return rc;
                chunk_form = kCceRows;
            } else {
                CGPT_TRY(rc);
                CGPT_TRY(softmax_stats_reduce(row_stats, row_loss + r0, partial, target_logit, targets + r0, n, V, tiles, inv_rows, s));
                CGPT_TRY(gemm_logits_softmax(3, chunk, xc, c, n, V, H, nullptr, nullptr, targets + r0, row_stats,
                                             inv_rows * gradient_scale, dtype, s));
            }
        }
        if (chunk_form == kCceRows) {
            CGPT_TRY(gemm_dispatch(chunk, xc, c, n, V, H, 0, 0, 0, dtype, false, s));                 // logits
            CGPT_TRY(cross_entropy_rows(row_loss + r0, chunk, chunk, targets + r0, n, V, inv_rows, gradient_scale, dtype, s));
        }
        CGPT_TRY(gemm_dispatch(dxc, chunk, c, n, H, V, 0, 1, 0, dtype, false, s));                // dX = G C
        CGPT_TRY(gemm_dispatch(dc, chunk, xc, V, H, n, 1, 1, (accumulate_dc || r0 > 0) ? 1 : 0, dtype, false, s));  // dC += G^T X
    }
    return sum_floats(loss, row_loss, static_cast<long long>(rows), s);
}
}  // namespace

extern "C" int cgpt_cut_cross_entropy(float* loss, void* dx, void* dc, const void* x, const void* c,
                                      const uint32_t* targets, size_t rows, size_t vocab, size_t hidden,
                                      float gradient_scale, int accumulate_dc, size_t chunk_rows, int dtype,
                                      cgpt_stream_t stream) {
    return cut_cross_entropy_form(kCceAuto, loss, dx, dc, x, c, targets, rows, vocab, hidden, gradient_scale, accumulate_dc,
                                  chunk_rows, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int cgpt_cut_cross_entropy_form(int form, float* loss, void* dx, void* dc, const void* x, const void* c,
                                           const uint32_t* targets, size_t rows, size_t vocab, size_t hidden,
                                           float gradient_scale, int accumulate_dc, size_t chunk_rows, int dtype,
                                           cgpt_stream_t stream) {
    return cut_cross_entropy_form(form, loss, dx, dc, x, c, targets, rows, vocab, hidden, gradient_scale, accumulate_dc,
                                  chunk_rows, dtype, static_cast<cudaStream_t>(stream));
}
