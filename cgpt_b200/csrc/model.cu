// Host-side orchestration of one transformer block and of the whole model, forward and backward, on
// top of the kernels of this library. Pure C++ host code: it only sequences launches on the caller's
// stream, never synchronises and never allocates (scratch comes from the caller's workspace), so a whole
// step can be captured into a CUDA graph.
//
// The operator graph is the reference's (src/core/transformer_block.cu:466-595 forward, :644-748 backward;
// src/core/transformer_model.cu:170-218, :336-381), with these differences in how it is executed:
//   * projections are written straight into the tensors that the backward needs (no D2D copies of
//     query/key into *_pre_norm, no copy of the hidden state into layer_inputs);
//   * the two residual adds of the forward are one three-input add; the two add_inplace passes and two D2D
//     copies of the backward are folded into the RMSNorm-backward kernels (residual operands);
//   * bias gradients are not computed (the model has no biases; the reference reduces them anyway);
//   * one backward workspace serves all layers (the reference allocates one per layer).
#include <cstdlib>

#include "internal.h"

using namespace cgpt;

namespace {

struct Dims {
    std::size_t rows, d, inter, hq, hkv, hd, qdim, kvdim, esz;
};

int check_cfg(const cgpt_model_config* c, std::size_t batch, std::size_t seq, Dims* out) {
    if (!c) return CGPT_ERR_NULL;
    if (!valid_float_dtype(c->dtype)) return CGPT_ERR_DTYPE;
    if (batch == 0 || seq == 0 || c->hidden == 0 || c->intermediate == 0 || c->q_heads == 0 || c->kv_heads == 0 ||
        c->head_dim == 0 || c->q_heads % c->kv_heads != 0)
        return CGPT_ERR_SHAPE;
    if (c->rotary_dim > c->head_dim || (c->rotary_dim & 1) != 0 || !(c->rms_epsilon > 0.f)) return CGPT_ERR_OPTION;
    // The reference's block requires hidden == q_heads * head_dim (it reshapes the attention output to
    // [rows, hidden], transformer_block.cu:571).
    if (c->q_heads * c->head_dim != c->hidden) return CGPT_ERR_SHAPE;
    *out = Dims{batch * seq, static_cast<std::size_t>(c->hidden), static_cast<std::size_t>(c->intermediate),
                static_cast<std::size_t>(c->q_heads), static_cast<std::size_t>(c->kv_heads),
                static_cast<std::size_t>(c->head_dim), static_cast<std::size_t>(c->q_heads * c->head_dim),
                static_cast<std::size_t>(c->kv_heads * c->head_dim), dtype_size(c->dtype)};
    return CGPT_OK;
}

// Bump allocator over the caller's workspace.
struct Carver {
    unsigned char* p;
    std::size_t used = 0;
    explicit Carver(void* base) : p(static_cast<unsigned char*>(base)) {}
    void* take(std::size_t bytes) {
        void* r = p ? p + used : nullptr;
        used += (bytes + 255) & ~std::size_t{255};
        return r;
    }
};

struct BlockScratch {
    void *attn_proj, *ffn_out, *norm_f;              // forward (norm_f: attention-norm output, not kept)
    void *d_act, *d_gate, *d_up, *d_ffn_norm_in;     // backward, MLP branch
    void *d_attn_out, *dq, *dk, *dv, *dq_pre, *dk_pre, *norm_a, *d_attn_norm_in;
    void *grad_a, *grad_b;                           // model backward ping-pong
    std::size_t bytes;
};

BlockScratch carve(void* base, const Dims& m) {
    Carver c(base);
    BlockScratch s;
    const std::size_t rd = m.rows * m.d * m.esz, ri = m.rows * m.inter * m.esz, rq = m.rows * m.qdim * m.esz,
                      rk = m.rows * m.kvdim * m.esz;
    // forward and backward scratch never live at the same time, so they overlay each other
    s.attn_proj = c.take(rd);
    s.ffn_out = c.take(rd);
    s.norm_f = c.take(rd);
    const std::size_t fwd_used = c.used;
    c.used = 0;
    s.d_act = c.take(ri);
    s.d_gate = c.take(ri);
    s.d_up = c.take(ri);
    s.d_ffn_norm_in = c.take(rd);
    s.d_attn_out = c.take(rq);
    s.dq = c.take(rq);
    s.dk = c.take(rk);
    s.dv = c.take(rk);
    s.dq_pre = c.take(rq);
    s.dk_pre = c.take(rk);
    s.norm_a = c.take(rd);
    s.d_attn_norm_in = c.take(rd);
    s.grad_a = c.take(rd);
    s.grad_b = c.take(rd);
    s.bytes = c.used > fwd_used ? c.used : fwd_used;
    return s;
}

// The block is a parallel-residual block: its attention branch and its MLP branch both start from the block input
// (forward) or from the output gradient (backward) and only meet again at the end. They are issued on two streams, the
// caller's and the library's side stream, so that the memory-bound kernels of one branch (norms, QK-norm/RoPE, SwiGLU,
// reductions) run underneath the tensor-core kernels of the other. Fork and join are event record/wait pairs, which
// stream capture turns into graph edges; everything issued on the side stream takes library scratch from lane 1.
struct Branches {
    cudaStream_t main = nullptr, side = nullptr;
    cudaEvent_t fork_event = nullptr, join_event = nullptr;
    bool two = false;
    int begin(cudaStream_t main_stream) {
        main = main_stream;
        side = main_stream;
        two = false;
        if (!branch_streams_enabled()) return CGPT_OK;
        const int rc = side_stream_get(main_stream, &side, &fork_event, &join_event);
        if (rc == CGPT_ERR_STATE) {   // first use inside a capture: run both branches on the caller's stream
            side = main_stream;
            return CGPT_OK;
        }
        CGPT_TRY(rc);
        two = true;
        return CGPT_OK;
    }
    int fork() const {
        if (!two) return CGPT_OK;
        CGPT_CUDA_TRY(cudaEventRecord(fork_event, main));
        CGPT_CUDA_TRY(cudaStreamWaitEvent(side, fork_event, 0));
        return CGPT_OK;
    }
    int join() const {
        if (!two) return CGPT_OK;
        CGPT_CUDA_TRY(cudaEventRecord(join_event, side));
        CGPT_CUDA_TRY(cudaStreamWaitEvent(main, join_event, 0));
        return CGPT_OK;
    }
    int lane() const { return two ? 1 : 0; }
};

// Diagnosis builds: CGPT_B200_DUAL_NORM=0 runs the two norms of the block input as separate passes (comparison runs).
bool dual_norm_enabled() {
    static const bool on = [] { const char* e = diagnosis_env("CGPT_B200_DUAL_NORM"); return !(e && e[0] == '0'); }();
    return on;
}

int mlp_forward(const void* in, const cgpt_block_params* w, const cgpt_block_saved* sv, const BlockScratch& ws, const Dims& m,
                int dt, float eps, bool with_norm, bool with_down, cudaStream_t stream) {
    if (with_norm) CGPT_TRY(cgpt_rmsnorm_forward(sv->norm, in, w->ffn_norm, m.rows, m.d, eps, dt, stream));
    // gate, up and the activation (two GEMMs and an activation pass in the reference, :566-579). The form with the
    // activation in the product's epilogue (cgpt_linear_swiglu_forward, same results bit for bit) measured 300 us against
    // 292 us for separate launches at the 104m shape (a third output stream costs the product what the activation pass
    // costs), so the block uses it only in diagnosis builds with CGPT_B200_FUSED_SWIGLU=1.
    static const bool fused_swiglu = [] { const char* e = diagnosis_env("CGPT_B200_FUSED_SWIGLU"); return e && e[0] == '1'; }();
    if (fused_swiglu) {
        CGPT_TRY(cgpt_linear_swiglu_forward(sv->gate, sv->up, sv->activated, sv->norm, w->gate_proj, w->up_proj, m.rows, m.d,
                                            m.inter, dt, stream));
    } else {
        {   // gate and up projections of the same input as one launch (it falls back to two where grouping does not apply)
            void* ys[2] = {sv->gate, sv->up};
            const void* wts[2] = {w->gate_proj, w->up_proj};
            const size_t outs[2] = {m.inter, m.inter};
            CGPT_TRY(cgpt_linear_forward_fused(ys, sv->norm, wts, outs, 2, m.rows, m.d, dt, stream));
        }
        CGPT_TRY(cgpt_swiglu_forward(sv->activated, sv->gate, sv->up, m.rows * m.inter, dt, stream));
    }
    if (!with_down) return CGPT_OK;     // the caller folds the down projection into the block's final product
    return cgpt_linear_forward(ws.ffn_out, sv->activated, w->down_proj, m.rows, m.inter, m.d, dt, stream);
}

// MLP branch of the backward (transformer_block.cu:663-681): ends with grad_in = grad_out + d(ffn_norm).
int mlp_backward(void* grad_in, const void* grad_out, const void* in, const cgpt_block_params* w, const cgpt_block_params* g,
                 const cgpt_block_saved* sv, const BlockScratch& ws, const Dims& m, int dt, float eps, bool with_norm,
                 cudaStream_t stream) {
    CGPT_TRY(cgpt_linear_backward(ws.d_act, g->down_proj, nullptr, grad_out, sv->activated, w->down_proj, m.rows, m.inter,
                                  m.d, 0, 0, 0, dt, stream));
    CGPT_TRY(cgpt_swiglu_backward(ws.d_gate, ws.d_up, ws.d_act, sv->gate, sv->up, m.rows * m.inter, 0, 0, dt, stream));
    {   // d(ffn norm output) = d_gate Wg + d_up Wu in one pass (the reference accumulates two GEMMs into the buffer)
        const void* dys[2] = {ws.d_gate, ws.d_up};
        const void* wts[2] = {w->gate_proj, w->up_proj};
        const size_t outs[2] = {m.inter, m.inter};
        CGPT_TRY(cgpt_linear_backward_input_fused(ws.d_ffn_norm_in, dys, wts, outs, 2, m.rows, m.d, 0, dt, stream));
    }
    {   // both weight gradients of the FFN input as one launch
        void* dws[2] = {g->gate_proj, g->up_proj};
        const void* dys[2] = {ws.d_gate, ws.d_up};
        const size_t outs[2] = {m.inter, m.inter};
        CGPT_TRY(cgpt_linear_backward_weight_fused(dws, dys, sv->norm, outs, 2, m.rows, m.d, 0, dt, stream));
    }
    if (!with_norm) return CGPT_OK;     // the caller runs the backward of both norms of the block input in one pass
    // grad_in = grad_out + d(ffn_norm)  (the reference's D2D copy + add_inplace, :678-681)
    return cgpt_rmsnorm_backward(grad_in, g->ffn_norm, ws.d_ffn_norm_in, in, w->ffn_norm, grad_out, nullptr, m.rows, m.d, eps,
                                 dt, stream);
}

}  // namespace

extern "C" size_t cgpt_block_workspace_bytes(const cgpt_model_config* cfg, size_t batch, size_t seq) {
    Dims m;
    if (check_cfg(cfg, batch, seq, &m) != CGPT_OK) return 0;
    return carve(nullptr, m).bytes;
}

extern "C" int cgpt_block_forward(void* out, const void* in, const cgpt_block_params* w, const cgpt_block_saved* sv,
                                  void* workspace, const void* cos_table, const void* sin_table,
                                  const cgpt_model_config* cfg, size_t batch, size_t seq, size_t position_offset,
                                  cgpt_stream_t stream) {
    if (!out || !in || !w || !sv || !workspace || !cos_table || !sin_table) return CGPT_ERR_NULL;
    Dims m;
    CGPT_TRY(check_cfg(cfg, batch, seq, &m));
    const BlockScratch ws = carve(workspace, m);
    const int dt = cfg->dtype;
    const float eps = cfg->rms_epsilon;
    Branches br;
    CGPT_TRY(br.begin(static_cast<cudaStream_t>(stream)));
    CGPT_TRY(br.fork());
    // one stream: the output and down projections run as one product with the residual (diagnosis builds can switch
    // that off with CGPT_B200_MERGE_OUT=0 to compare)
    static const bool merge_out = [] { const char* e = diagnosis_env("CGPT_B200_MERGE_OUT"); return !(e && e[0] == '0'); }();
    const bool merged = !br.two && merge_out;
    void* norm_attn = sv->attention_norm_output != nullptr ? sv->attention_norm_output : ws.norm_f;
    // The attention norm's output is kept only if the caller gave a buffer for it (sv->norm holds the FFN norm's output,
    // as in the reference). One stream: both norms of the block input in one pass over it, before either branch.
    const bool dual = !br.two && dual_norm_enabled();
    if (dual)
        CGPT_TRY(cgpt_rmsnorm_forward_dual(norm_attn, sv->norm, in, w->attention_norm, w->ffn_norm, m.rows, m.d, eps, dt, stream));
    {   // MLP branch on the same block input (parallel residual), on the side stream
        ScratchLane lane(br.lane());
        CGPT_TRY(mlp_forward(in, w, sv, ws, m, dt, eps, !dual, !merged, br.side));
    }
    // attention branch on the caller's stream
    if (!dual) CGPT_TRY(cgpt_rmsnorm_forward(norm_attn, in, w->attention_norm, m.rows, m.d, eps, dt, stream));
    {   // query, key and value projections of the same input as one launch (three in the reference, :496-510)
        void* ys[3] = {sv->query_pre_norm, sv->key_pre_norm, sv->value};
        const void* wts[3] = {w->q_projection, w->k_projection, w->v_projection};
        const size_t outs[3] = {m.qdim, m.kvdim, m.kvdim};
        CGPT_TRY(cgpt_linear_forward_fused(ys, norm_attn, wts, outs, 3, m.rows, m.d, dt, stream));
    }
    {   // per-head QK-norm then RoPE: one fused pass when the shape allows it, else the three separate ops
        int rc = cgpt_qknorm_rope_forward(sv->query, sv->key, sv->query_pre_norm, sv->key_pre_norm, w->q_norm, w->k_norm,
                                          cos_table, sin_table, batch, seq, m.hq, m.hkv, m.hd, cfg->rotary_dim,
                                          position_offset, cfg->max_seq, eps, dt, stream);
        if (rc == CGPT_ERR_UNSUPPORTED) {
            CGPT_TRY(cgpt_rmsnorm_forward(sv->query, sv->query_pre_norm, w->q_norm, m.rows * m.hq, m.hd, eps, dt, stream));
            CGPT_TRY(cgpt_rmsnorm_forward(sv->key, sv->key_pre_norm, w->k_norm, m.rows * m.hkv, m.hd, eps, dt, stream));
            rc = cgpt_rope_forward(sv->query, sv->key, cos_table, sin_table, batch, seq, m.hq, m.hkv, m.hd, cfg->rotary_dim,
                                   position_offset, cfg->max_seq, dt, stream);
        }
        CGPT_TRY(rc);
    }
    CGPT_TRY(cgpt_attention_forward(sv->attention_output, sv->attention_logsumexp, sv->query, sv->key, sv->value, batch,
                                    seq, seq, m.hq, m.hkv, m.hd, 0.0f, 1, position_offset, dt, 0, stream));
    if (merged) {
        // out = in + attention_output Wo^T + activated Wdown^T as ONE product chained along K, the block input added in
        // its epilogue (the reference: two projections and two in-place adds, :541-546 and :580-595)
        const void* xs[2] = {sv->attention_output, sv->activated};
        const void* wts[2] = {w->o_projection, w->down_proj};
        const size_t ins[2] = {m.qdim, m.inter};
        const int rc = cgpt_linear_forward_sum(out, xs, wts, ins, 2, m.rows, m.d, in, dt, stream);
        if (rc != CGPT_ERR_OPTION) return rc;
        // out aliases in and this shape has no adding epilogue: the separate form
        CGPT_TRY(cgpt_linear_forward(ws.ffn_out, sv->activated, w->down_proj, m.rows, m.inter, m.d, dt, stream));
    }
    CGPT_TRY(cgpt_linear_forward(ws.attn_proj, sv->attention_output, w->o_projection, m.rows, m.qdim, m.d, dt, stream));
    CGPT_TRY(br.join());
    return cgpt_add(out, in, ws.attn_proj, ws.ffn_out, m.rows * m.d, dt, stream);
}

extern "C" int cgpt_block_backward(void* grad_in, const void* grad_out, const void* in, const cgpt_block_params* w,
                                   const cgpt_block_params* g, const cgpt_block_saved* sv, void* workspace,
                                   const void* cos_table, const void* sin_table, const cgpt_model_config* cfg,
                                   size_t batch, size_t seq, size_t position_offset, cgpt_stream_t stream) {
    if (!grad_in || !grad_out || !in || !w || !g || !sv || !workspace || !cos_table || !sin_table) return CGPT_ERR_NULL;
    Dims m;
    CGPT_TRY(check_cfg(cfg, batch, seq, &m));
    const BlockScratch ws = carve(workspace, m);
    const int dt = cfg->dtype;
    const float eps = cfg->rms_epsilon;
    Branches br;
    CGPT_TRY(br.begin(static_cast<cudaStream_t>(stream)));
    CGPT_TRY(br.fork());
    const bool dual = !br.two && dual_norm_enabled();
    {   // ---- MLP branch on the side stream; it writes grad_in = grad_out + d(ffn_norm)
        ScratchLane lane(br.lane());
        CGPT_TRY(mlp_backward(grad_in, grad_out, in, w, g, sv, ws, m, dt, eps, !dual, br.side));
    }
    // ---- attention branch (:682-747)
    CGPT_TRY(cgpt_linear_backward(ws.d_attn_out, g->o_projection, nullptr, grad_out, sv->attention_output, w->o_projection,
                                  m.rows, m.qdim, m.d, 0, 0, 0, dt, stream));
    CGPT_TRY(cgpt_attention_backward(ws.dq, ws.dk, ws.dv, ws.d_attn_out, sv->attention_output, sv->attention_logsumexp,
                                     sv->query, sv->key, sv->value, batch, seq, seq, m.hq, m.hkv, m.hd, 0.0f, 1,
                                     position_offset, 0, dt, 0, stream));
    {   // inverse RoPE then QK-norm backward: fused when possible
        int rc = cgpt_qknorm_rope_backward(ws.dq_pre, ws.dk_pre, g->q_norm, g->k_norm, ws.dq, ws.dk, sv->query_pre_norm,
                                           sv->key_pre_norm, w->q_norm, w->k_norm, cos_table, sin_table, batch, seq, m.hq,
                                           m.hkv, m.hd, cfg->rotary_dim, position_offset, cfg->max_seq, eps, dt, stream);
        if (rc == CGPT_ERR_UNSUPPORTED) {
            CGPT_TRY(cgpt_rope_backward(ws.dq, ws.dk, ws.dq, ws.dk, cos_table, sin_table, batch, seq, m.hq, m.hkv, m.hd,
                                        cfg->rotary_dim, position_offset, cfg->max_seq, dt, stream));
            CGPT_TRY(cgpt_rmsnorm_backward(ws.dq_pre, g->q_norm, ws.dq, sv->query_pre_norm, w->q_norm, nullptr, nullptr,
                                           m.rows * m.hq, m.hd, eps, dt, stream));
            rc = cgpt_rmsnorm_backward(ws.dk_pre, g->k_norm, ws.dk, sv->key_pre_norm, w->k_norm, nullptr, nullptr,
                                       m.rows * m.hkv, m.hd, eps, dt, stream);
        }
        CGPT_TRY(rc);
    }
    // the attention-norm output: saved by the forward if the caller provided the buffer, else recomputed as the
    // reference does (:725; its single norm buffer was overwritten by the FFN norm)
    const void* norm_a = sv->attention_norm_output;
    if (norm_a == nullptr) {
        CGPT_TRY(cgpt_rmsnorm_forward(ws.norm_a, in, w->attention_norm, m.rows, m.d, eps, dt, stream));
        norm_a = ws.norm_a;
    }
    {   // d(attention norm output) = dQ Wq + dK Wk + dV Wv in one pass over the buffer (:726-744 runs three
        // GEMMs, the last two accumulating into it)
        const void* dys[3] = {ws.dq_pre, ws.dk_pre, ws.dv};
        const void* wts[3] = {w->q_projection, w->k_projection, w->v_projection};
        const size_t outs[3] = {m.qdim, m.kvdim, m.kvdim};
        CGPT_TRY(cgpt_linear_backward_input_fused(ws.d_attn_norm_in, dys, wts, outs, 3, m.rows, m.d, 0, dt, stream));
    }
    {   // the three weight gradients of the attention input as one launch
        void* dws[3] = {g->q_projection, g->k_projection, g->v_projection};
        const void* dys[3] = {ws.dq_pre, ws.dk_pre, ws.dv};
        const size_t outs[3] = {m.qdim, m.kvdim, m.kvdim};
        CGPT_TRY(cgpt_linear_backward_weight_fused(dws, dys, norm_a, outs, 3, m.rows, m.d, 0, dt, stream));
    }
    if (dual)   // one stream: grad_in = grad_out + d(ffn_norm) + d(attention_norm) in one pass (:678-681, :745-747)
        return cgpt_rmsnorm_backward_dual(grad_in, g->attention_norm, g->ffn_norm, ws.d_attn_norm_in, ws.d_ffn_norm_in, in,
                                          w->attention_norm, w->ffn_norm, grad_out, m.rows, m.d, eps, dt, stream);
    // grad_in += d(attention_norm): needs the MLP branch's grad_in
    CGPT_TRY(br.join());
    return cgpt_rmsnorm_backward(grad_in, g->attention_norm, ws.d_attn_norm_in, in, w->attention_norm, grad_in, nullptr,
                                 m.rows, m.d, eps, dt, stream);
}

extern "C" int cgpt_model_forward(void* logits, const uint32_t* token_ids, const cgpt_model_tensors* w,
                                  const cgpt_model_saved* sv, void* workspace, const void* cos_table,
                                  const void* sin_table, const cgpt_model_config* cfg, size_t batch, size_t seq,
                                  cgpt_stream_t stream) {
    if (!token_ids || !w || !sv || !workspace || !w->layers || !sv->layers || !sv->layer_inputs) return CGPT_ERR_NULL;
    Dims m;
    CGPT_TRY(check_cfg(cfg, batch, seq, &m));
    if (cfg->layers == 0 || cfg->vocab == 0) return CGPT_ERR_SHAPE;
    const int dt = cfg->dtype;
    CGPT_TRY(cgpt_embedding_forward(sv->layer_inputs[0], token_ids, w->token_embedding, m.rows, cfg->vocab, m.d, dt, stream));
    for (std::size_t l = 0; l < cfg->layers; ++l) {
        void* out = l + 1 < cfg->layers ? sv->layer_inputs[l + 1] : sv->hidden;
        CGPT_TRY(cgpt_block_forward(out, sv->layer_inputs[l], &w->layers[l], &sv->layers[l], workspace, cos_table,
                                    sin_table, cfg, batch, seq, 0, stream));
    }
    CGPT_TRY(cgpt_rmsnorm_forward(sv->normalized, sv->hidden, w->final_norm, m.rows, m.d, cfg->rms_epsilon, dt, stream));
    if (logits != nullptr)
        CGPT_TRY(cgpt_linear_forward(logits, sv->normalized, w->lm_head, m.rows, m.d, cfg->vocab, dt, stream));
    return CGPT_OK;
}

extern "C" int cgpt_model_backward_steps(const void* grad_logits, void* grad_normalized, const uint32_t* token_ids,
                                         const cgpt_model_tensors* w, const cgpt_model_tensors* g, const cgpt_model_saved* sv,
                                         void* workspace, const void* cos_table, const void* sin_table,
                                         const cgpt_model_config* cfg, size_t batch, size_t seq, size_t step_begin,
                                         size_t step_end, cgpt_stream_t stream) {
    if (!grad_normalized || !token_ids || !w || !g || !sv || !workspace || !w->layers || !g->layers || !sv->layers ||
        !sv->layer_inputs)
        return CGPT_ERR_NULL;
    Dims m;
    CGPT_TRY(check_cfg(cfg, batch, seq, &m));
    const std::size_t L = cfg->layers;
    if (step_begin > step_end || step_end > L + 2) return CGPT_ERR_SHAPE;
    const BlockScratch ws = carve(workspace, m);
    const int dt = cfg->dtype;
    for (std::size_t step = step_begin; step < step_end; ++step) {
        if (step == 0) {
            if (grad_logits != nullptr) {  // transformer_model.cu:358-361
                CGPT_TRY(cgpt_linear_backward(grad_normalized, g->lm_head, nullptr, grad_logits, sv->normalized, w->lm_head,
                                              m.rows, m.d, cfg->vocab, 0, 0, 0, dt, stream));
            }
            CGPT_TRY(cgpt_rmsnorm_backward(ws.grad_a, g->final_norm, grad_normalized, sv->hidden, w->final_norm, nullptr,
                                           nullptr, m.rows, m.d, cfg->rms_epsilon, dt, stream));
        } else if (step <= L) {
            // the gradient ping-pongs between grad_a and grad_b: step s reads the buffer step s-1 wrote
            const std::size_t l = L - step;
            void* in_grad = (step % 2 == 1) ? ws.grad_a : ws.grad_b;
            void* out_grad = (step % 2 == 1) ? ws.grad_b : ws.grad_a;
            CGPT_TRY(cgpt_block_backward(out_grad, in_grad, sv->layer_inputs[l], &w->layers[l], &g->layers[l], &sv->layers[l],
                                         workspace, cos_table, sin_table, cfg, batch, seq, 0, stream));
        } else {
            // transformer_model.cu:375-380: tied embeddings add the lookup gradient into the LM-head gradient
            const void* last = (L % 2 == 0) ? ws.grad_a : ws.grad_b;
            const bool tied = cfg->tied_embeddings != 0;
            CGPT_TRY(cgpt_embedding_backward(tied ? g->lm_head : g->token_embedding, last, token_ids, m.rows, cfg->vocab, m.d, 1,
                                             tied ? 1 : 0, dt, stream));
        }
    }
    return CGPT_OK;
}

extern "C" int cgpt_model_backward(const void* grad_logits, void* grad_normalized, const uint32_t* token_ids,
                                   const cgpt_model_tensors* w, const cgpt_model_tensors* g, const cgpt_model_saved* sv,
                                   void* workspace, const void* cos_table, const void* sin_table,
                                   const cgpt_model_config* cfg, size_t batch, size_t seq, cgpt_stream_t stream) {
    if (!cfg) return CGPT_ERR_NULL;
    return cgpt_model_backward_steps(grad_logits, grad_normalized, token_ids, w, g, sv, workspace, cos_table, sin_table, cfg, batch,
                                     seq, 0, static_cast<size_t>(cfg->layers) + 2, stream);
}
