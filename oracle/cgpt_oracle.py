"""CPU restatement (numpy, fp32 math) of CGPT's training hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the product path (``cgpt_b200/``) imports this module; it is the
checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py``.

Every function restates one reference function and cites it (paths are relative to the reference
repository). Storage rounding is explicit: ``rnd(x, dtype)`` rounds an fp32 array to the storage dtype
("f16", "bf16", "f32") and returns fp32, exactly where the reference writes a tensor.

Pinning: the restatement is checked in ``tests/test_oracle_pins.py`` against the known-answer vectors of
the reference's own tests (``tests/*_test.cu``) and against outputs of the reference's CPU ops compiled
from its sources (``oracle/_ref``, built by ``oracle/build_ref.py``; fixtures in ``tests/golden``).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


# ------------------------------------------------------------------------------------------ rounding
def rnd(x, dtype: str = "f16"):
    """Round-to-nearest-even to the storage dtype, returned as fp32 (Tensor::copy_from_host /
    __float2half_rn / __float2bfloat16_rn in the reference)."""
    x = np.asarray(x, dtype=F32)
    if dtype == "f32":
        return x
    if dtype == "f16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(F32)
    if dtype == "bf16":
        u = x.view(np.uint32).astype(np.uint64)
        nan = np.isnan(x)
        rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        out = rounded.view(F32).copy()
        out[nan] = np.nan
        return out
    raise ValueError(dtype)


# ------------------------------------------------------------------------------------------- RMSNorm
def rmsnorm_forward(x, w, eps):
    """src/ops/rmsnorm.cu:60,122-125: y = x * rsqrt(mean(x^2)+eps) * w, fp32."""
    x = np.asarray(x, F32); w = np.asarray(w, F32)
    inv = (1.0 / np.sqrt(np.mean(x.astype(np.float64) ** 2, axis=-1, keepdims=True) + eps)).astype(F32)
    return (x * inv * w).astype(F32)


def rmsnorm_backward(dy, x, w, eps):
    """src/ops/backward/rmsnorm_backward.cu:276-293 (dx) and :374-398 (dw).
    c = sum(dy*w*x)/H * inv^3; dx = dy*w*inv - x*c; dw = sum_rows dy*x*inv."""
    dy = np.asarray(dy, np.float64); x = np.asarray(x, np.float64); w = np.asarray(w, np.float64)
    hidden = x.shape[-1]
    inv = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    corr = np.sum(dy * w * x, axis=-1, keepdims=True) / hidden * inv ** 3
    dx = dy * w * inv - x * corr
    dw = np.sum(dy * (x * inv), axis=0)
    return dx.astype(F32), dw.astype(F32)


# ---------------------------------------------------------------------------------------------- RoPE
def rotary_cache(max_seq, rotary_dim, base=10000.0):
    """train/train.cpp:322-333: theta = pos / base^(2i/rotary_dim) in fp32; cos/sin in fp32 (the
    trainer then stores them as fp16)."""
    pos = np.arange(max_seq, dtype=F32)[:, None]
    i = np.arange(rotary_dim // 2, dtype=F32)[None, :]
    theta = (pos / np.power(F32(base), F32(2.0) * i / F32(rotary_dim))).astype(F32)
    return np.cos(theta).astype(F32), np.sin(theta).astype(F32)


def _rope_apply(x, cos, sin, rotary_dim, offset, inverse):
    x = np.asarray(x, F32)
    b, s, h, d = x.shape
    rotary_dim = rotary_dim or d
    out = x.copy()
    c = np.asarray(cos, F32)[offset:offset + s, :][None, :, None, :]
    sn = np.asarray(sin, F32)[offset:offset + s, :][None, :, None, :]
    a = x[..., 0:rotary_dim:2]
    bb = x[..., 1:rotary_dim:2]
    if inverse:   # src/ops/backward/rope_backward.cu:94-105
        out[..., 0:rotary_dim:2] = bb * sn + a * c
        out[..., 1:rotary_dim:2] = -a * sn + bb * c
    else:         # src/ops/rope.cu:133-134
        out[..., 0:rotary_dim:2] = -bb * sn + a * c
        out[..., 1:rotary_dim:2] = a * sn + bb * c
    return out.astype(F32)


def rope_forward(x, cos, sin, rotary_dim=0, position_offset=0):
    return _rope_apply(x, cos, sin, rotary_dim, position_offset, False)


def rope_backward(dy, cos, sin, rotary_dim=0, position_offset=0):
    return _rope_apply(dy, cos, sin, rotary_dim, position_offset, True)


# -------------------------------------------------------------------------------------------- SwiGLU
def swiglu_forward(gate, up):
    """src/ops/swiglu.cu:69-71: g / (1 + exp(-g)) * up."""
    g = np.asarray(gate, np.float64); u = np.asarray(up, np.float64)
    return (g / (1.0 + np.exp(-g)) * u).astype(F32)


def swiglu_backward(dy, gate, up):
    """src/ops/backward/swiglu_backward.cu:61-74: s = sigmoid(g); dgate = dy*up*s*(1+g*(1-s));
    dup = dy*g*s."""
    g = np.asarray(gate, np.float64); u = np.asarray(up, np.float64); d = np.asarray(dy, np.float64)
    s = 1.0 / (1.0 + np.exp(-g))
    return (d * u * (s * (1.0 + g * (1.0 - s)))).astype(F32), (d * (g * s)).astype(F32)


# ----------------------------------------------------------------------------------------- Embedding
def embedding_forward(ids, weight):
    return np.asarray(weight, F32)[np.asarray(ids, np.int64)]


def embedding_backward(dy, ids, vocab, accumulate_into=None, bounds_check=True):
    """src/ops/backward/embedding_backward.cu:39-92: gW[id] += dy[t] for valid ids (fp32 sums here;
    the reference rounds each atomic add to the storage dtype)."""
    dy = np.asarray(dy, F32).reshape(len(ids), -1)
    gw = np.zeros((vocab, dy.shape[1]), np.float64) if accumulate_into is None else np.asarray(accumulate_into, np.float64).copy()
    ids = np.asarray(ids, np.int64)
    ok = ids < vocab
    np.add.at(gw, ids[ok], dy[ok].astype(np.float64))
    return gw.astype(F32)


# -------------------------------------------------------------------------------------------- Linear
def linear_forward(x, w):
    """src/ops/linear.cu: Y = X W^T, fp32 accumulate."""
    return (np.asarray(x, F32) @ np.asarray(w, F32).T).astype(F32)


def linear_backward(dy, x, w):
    """src/ops/backward/linear_backward.cu:135-148,181-200: dX = dY W, dW = dY^T X, db = sum_rows dY."""
    dy = np.asarray(dy, F32).reshape(-1, np.asarray(w).shape[0])
    x2 = np.asarray(x, F32).reshape(dy.shape[0], -1)
    w = np.asarray(w, F32)
    return (dy @ w).astype(F32), (dy.T @ x2).astype(F32), dy.sum(axis=0, dtype=np.float64).astype(F32)


# ----------------------------------------------------------------------------------------- Attention
def _scale(head_dim, attention_scale):
    return F32(attention_scale) if attention_scale and attention_scale > 0 else F32(1.0 / np.sqrt(head_dim))


def attention_forward(q, k, v, causal=True, offset=0, attention_scale=0.0):
    """Causal GQA softmax attention with saved log-sum-exp. q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D].
    Visibility rule k <= offset + q (src/ops/attention.cu:669-690; tests/flash_attention_test.cu:50-99).
    LSE = max + log(sum exp(s - max)) of the scaled scores, natural log (attention.cu:669-690).
    Returns (O [B,Sq,Hq,D], LSE [B,Sq,Hq]) in fp32."""
    q = np.asarray(q, F32); k = np.asarray(k, F32); v = np.asarray(v, F32)
    b, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    ratio = hq // hkv
    scale = _scale(d, attention_scale)
    out = np.zeros_like(q)
    lse = np.zeros((b, sq, hq), F32)
    qpos = np.arange(sq)[:, None] + offset
    kpos = np.arange(sk)[None, :]
    mask = (kpos <= qpos) if causal else np.ones((sq, sk), bool)
    for bi in range(b):
        for h in range(hq):
            kh = h // ratio
            s = (q[bi, :, h, :] @ k[bi, :, kh, :].T) * scale
            s = np.where(mask, s, -np.inf)
            m = s.max(axis=1, keepdims=True)
            p = np.exp(s - m)
            l = p.sum(axis=1, keepdims=True)
            out[bi, :, h, :] = (p / l) @ v[bi, :, kh, :]
            lse[bi, :, h] = (m + np.log(l))[:, 0]
    return out, lse


def attention_backward(do, q, k, v, out=None, lse=None, causal=True, offset=0, attention_scale=0.0,
                       round_p=None):
    """dQ, dK, dV of the attention above (src/ops/backward/attention_backward.cu:1167-1677 and the
    reference's own fp32 check, tests/flash_attention_test.cu:110-174):
      P = exp(scale*QK^T - LSE); delta = rowsum(dO*O); dS = P*(dP - delta), dP = dO V^T;
      dQ = scale*dS K; dK = scale*dS^T Q; dV = P^T dO.
    With out/lse None they are recomputed (flash_gqa_attention_backward without saved statistics).
    round_p="f16" rounds P and scale*dS to fp16 before the second matmuls, as the reference's tensor-core
    path does (attention_backward.cu:1336-1343,1567-1586)."""
    q = np.asarray(q, F32); k = np.asarray(k, F32); v = np.asarray(v, F32); do = np.asarray(do, F32)
    if out is None or lse is None:
        out, lse = attention_forward(q, k, v, causal, offset, attention_scale)
    b, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    ratio = hq // hkv
    scale = _scale(d, attention_scale)
    dq = np.zeros_like(q); dk = np.zeros_like(k); dv = np.zeros_like(v)
    qpos = np.arange(sq)[:, None] + offset
    kpos = np.arange(sk)[None, :]
    mask = (kpos <= qpos) if causal else np.ones((sq, sk), bool)
    for bi in range(b):
        for h in range(hq):
            kh = h // ratio
            s = (q[bi, :, h, :] @ k[bi, :, kh, :].T) * scale
            p = np.where(mask, np.exp(s - lse[bi, :, h][:, None]), F32(0)).astype(F32)
            dp = do[bi, :, h, :] @ v[bi, :, kh, :].T
            delta = np.sum(do[bi, :, h, :] * np.asarray(out, F32)[bi, :, h, :], axis=1, keepdims=True)
            ds = (p * (dp - delta) * scale).astype(F32)
            if round_p:
                p = rnd(p, round_p); ds = rnd(ds, round_p)
            dq[bi, :, h, :] = ds @ k[bi, :, kh, :]
            dk[bi, :, kh, :] += ds.T @ q[bi, :, h, :]
            dv[bi, :, kh, :] += p.T @ do[bi, :, h, :]
    return dq, dk, dv


# ------------------------------------------------------------------------------------- Cross entropy
def cross_entropy(logits, targets, gradient_scale=1.0):
    """src/ops/cross_entropy.cu:134-245: loss = mean over rows of (log sum exp - logit[target]) for
    targets inside the vocabulary; grad = (softmax - onehot)/rows * gradient_scale."""
    z = np.asarray(logits, np.float64)
    rows, vocab = z.shape
    t = np.asarray(targets, np.int64)
    m = z.max(axis=1, keepdims=True)
    e = np.exp(z - m)
    den = e.sum(axis=1, keepdims=True)
    valid = t < vocab
    tl = z[np.arange(rows), np.where(valid, t, 0)]
    row_loss = np.where(valid, np.log(den[:, 0]) + m[:, 0] - tl, 0.0)
    grad = e / den
    grad[np.arange(rows)[valid], t[valid]] -= 1.0
    return F32(row_loss.sum() / rows), (grad / rows * gradient_scale).astype(F32)


def cut_cross_entropy(x, classifier, targets, gradient_scale=1.0):
    """src/ops/cut_cross_entropy.cu:97-160: mean CE of X C^T without storing logits;
    dX = (P C - C[target])/rows, dC = (P - onehot)^T X / rows (times gradient_scale, which the
    reference signature fixes at 1)."""
    x = np.asarray(x, F32); c = np.asarray(classifier, F32)
    loss, g = cross_entropy(x.astype(np.float64) @ c.astype(np.float64).T, targets, gradient_scale)
    g64 = g.astype(np.float64)
    return loss, (g64 @ c).astype(F32), (g64.T @ x).astype(F32)


# --------------------------------------------------------------------------------------------- AdamW
def adamw_step(param_dtype, grads, masters, ms, vs, step, lr, beta1, beta2, eps, wd, loss_scale=1.0,
               max_grad_norm=np.inf, bias_in_float=True):
    """One step of adamw_step_many_async over lists of tensors (src/optim/adamw.cu:74-187, 276-345),
    fp32 arithmetic in the reference's operation order. Returns (params, masters, ms, vs, step, skipped).
    ``bias_in_float`` selects powf on float(step) (the batched device path, adamw.cu:179-180) or the
    double-precision host formula of adamw_step (adamw.cu:414-415)."""
    ls = F32(loss_scale)
    unscaled = [(np.asarray(g, F32) / ls).astype(F32) for g in grads]
    squared = F32(0)
    finite = True
    for u in unscaled:
        if not np.all(np.isfinite(u)):
            finite = False
        squared = F32(squared + np.sum(np.where(np.isfinite(u), u, 0).astype(np.float64) ** 2))
    if not finite or not np.isfinite(squared):
        return ([rnd(m_, param_dtype) for m_ in masters], masters, ms, vs, step, True)
    step = step + 1
    if bias_in_float:
        bc1 = F32(1.0) - np.power(F32(beta1), F32(step), dtype=F32)
        bc2 = F32(1.0) - np.power(F32(beta2), F32(step), dtype=F32)
    else:
        bc1 = F32(1.0 - float(beta1) ** step); bc2 = F32(1.0 - float(beta2) ** step)
    clip = F32(1.0)
    if np.isfinite(max_grad_norm):
        norm = np.sqrt(squared, dtype=F32)
        if norm > F32(max_grad_norm):
            clip = F32(F32(max_grad_norm) / norm)
    b1, b2, lr_, eps_, wd_ = F32(beta1), F32(beta2), F32(lr), F32(eps), F32(wd)
    out_p, out_w, out_m, out_v = [], [], [], []
    for g, w, m_, v_ in zip(grads, masters, ms, vs):
        grad = (np.asarray(g, F32) / ls * clip).astype(F32)
        m1 = (b1 * np.asarray(m_, F32) + (F32(1) - b1) * grad).astype(F32)
        v1 = (b2 * np.asarray(v_, F32) + (F32(1) - b2) * grad * grad).astype(F32)
        normalized = (m1 / bc1 / (np.sqrt(v1 / bc2, dtype=F32) + eps_)).astype(F32)
        w1 = (np.asarray(w, F32) * (F32(1) - lr_ * wd_) - lr_ * normalized).astype(F32)
        out_p.append(rnd(w1, param_dtype)); out_w.append(w1); out_m.append(m1); out_v.append(v1)
    return out_p, out_w, out_m, out_v, step, False


# ------------------------------------------------------------------------------------- Block / model
BLOCK_WEIGHTS = ("attention_norm", "q_projection", "k_projection", "q_norm", "k_norm", "v_projection",
                 "o_projection", "ffn_norm", "gate_proj", "up_proj", "down_proj")


def block_forward(x, w, cfg, cos, sin, store="f16", position_offset=0):
    """transformer_block_forward (src/core/transformer_block.cu:405-611): parallel residual block
    out = x + Attn(RMSNorm_a(x)) + MLP(RMSNorm_f(x)) with per-head QK-RMSNorm before RoPE.
    x: [B*S, d]. cfg: dict(batch, seq, hidden, intermediate, q_heads, kv_heads, head_dim, rotary_dim, eps).
    Every tensor the reference writes is rounded to ``store``. Returns (out, saved activations)."""
    b, s, d = cfg["batch"], cfg["seq"], cfg["hidden"]
    hq, hkv, hd = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]
    eps = cfg["eps"]
    r = lambda a: rnd(a, store)
    sv = {}
    norm_a = r(rmsnorm_forward(x, w["attention_norm"], eps))
    q_pre = r(linear_forward(norm_a, w["q_projection"])).reshape(b, s, hq, hd)
    k_pre = r(linear_forward(norm_a, w["k_projection"])).reshape(b, s, hkv, hd)
    v = r(linear_forward(norm_a, w["v_projection"])).reshape(b, s, hkv, hd)
    qn = r(rmsnorm_forward(q_pre.reshape(-1, hd), w["q_norm"], eps)).reshape(b, s, hq, hd)
    kn = r(rmsnorm_forward(k_pre.reshape(-1, hd), w["k_norm"], eps)).reshape(b, s, hkv, hd)
    q = r(rope_forward(qn, cos, sin, cfg["rotary_dim"], position_offset))
    k = r(rope_forward(kn, cos, sin, cfg["rotary_dim"], position_offset))
    o, lse = attention_forward(q, k, v, True, position_offset)
    o = r(o)
    attn_proj = r(linear_forward(o.reshape(b * s, hq * hd), w["o_projection"]))
    norm_f = r(rmsnorm_forward(x, w["ffn_norm"], eps))
    gate = r(linear_forward(norm_f, w["gate_proj"]))
    up = r(linear_forward(norm_f, w["up_proj"]))
    act = r(swiglu_forward(gate, up))
    ffn = r(linear_forward(act, w["down_proj"]))
    out = r(r(np.asarray(x, F32) + attn_proj) + ffn)   # two fp16 adds, transformer_block.cu:594-595
    sv.update(norm=norm_f, query=q, key=k, value=v, query_pre_norm=q_pre, key_pre_norm=k_pre,
              attention_output=o, attention_logsumexp=lse, gate=gate, up=up, activated=act)
    return out, sv


def block_backward(dout, x, w, sv, cfg, cos, sin, store="f16", position_offset=0, round_intermediates=True):
    """transformer_block_backward (src/core/transformer_block.cu:644-748), same op order. Returns
    (grad_input, dict of parameter gradients). With round_intermediates every tensor the reference
    writes is rounded to ``store``; without it the chain is pure fp32 (ground truth)."""
    b, s, d = cfg["batch"], cfg["seq"], cfg["hidden"]
    hq, hkv, hd = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]
    eps = cfg["eps"]
    r = (lambda a: rnd(a, store)) if round_intermediates else (lambda a: np.asarray(a, F32))
    g = {}
    d_act, g["down_proj"], _ = linear_backward(dout, sv["activated"], w["down_proj"])
    d_act = r(d_act)
    d_gate, d_up = swiglu_backward(d_act, sv["gate"], sv["up"])
    d_gate, d_up = r(d_gate), r(d_up)
    d_norm_f, g["gate_proj"], _ = linear_backward(d_gate, sv["norm"], w["gate_proj"])
    d_norm_f = r(d_norm_f)
    t, g["up_proj"], _ = linear_backward(d_up, sv["norm"], w["up_proj"])
    d_norm_f = r(d_norm_f + t)
    res_f, g["ffn_norm"] = rmsnorm_backward(d_norm_f, x, w["ffn_norm"], eps)
    res_f = r(res_f)
    grad_input = r(np.asarray(dout, F32) + res_f)
    d_o, g["o_projection"], _ = linear_backward(dout, sv["attention_output"].reshape(b * s, hq * hd), w["o_projection"])
    d_o = r(d_o).reshape(b, s, hq, hd)
    dq, dk, dv = attention_backward(d_o, sv["query"], sv["key"], sv["value"], sv["attention_output"],
                                    sv["attention_logsumexp"], True, position_offset)
    dq, dk, dv = r(dq), r(dk), r(dv)
    dq_pre = r(rope_backward(dq, cos, sin, cfg["rotary_dim"], position_offset))
    dk_pre = r(rope_backward(dk, cos, sin, cfg["rotary_dim"], position_offset))
    dqn, g["q_norm"] = rmsnorm_backward(dq_pre.reshape(-1, hd), sv["query_pre_norm"].reshape(-1, hd), w["q_norm"], eps)
    dkn, g["k_norm"] = rmsnorm_backward(dk_pre.reshape(-1, hd), sv["key_pre_norm"].reshape(-1, hd), w["k_norm"], eps)
    dqn = r(dqn).reshape(b * s, hq * hd); dkn = r(dkn).reshape(b * s, hkv * hd)
    norm_a = r(rmsnorm_forward(x, w["attention_norm"], eps))
    d_norm_a, g["q_projection"], _ = linear_backward(dqn, norm_a, w["q_projection"])
    d_norm_a = r(d_norm_a)
    t, g["k_projection"], _ = linear_backward(dkn, norm_a, w["k_projection"])
    d_norm_a = r(d_norm_a + t)
    t, g["v_projection"], _ = linear_backward(dv.reshape(b * s, hkv * hd), norm_a, w["v_projection"])
    d_norm_a = r(d_norm_a + t)
    res_a, g["attention_norm"] = rmsnorm_backward(d_norm_a, x, w["attention_norm"], eps)
    grad_input = r(grad_input + r(res_a))
    g = {k_: r(v_) for k_, v_ in g.items()}
    return grad_input, g


def model_forward(ids, weights, cfg, cos, sin, store="f16"):
    """transformer_model_forward (src/core/transformer_model.cu:170-218) up to the final RMSNorm;
    the LM head + loss are applied by the caller (materialised logits or cut cross-entropy).
    weights: dict(token_embedding, layers=[block dicts], final_norm, lm_head)."""
    r = lambda a: rnd(a, store)
    hidden = embedding_forward(ids.reshape(-1), weights["token_embedding"])
    saved = {"layer_inputs": [], "layers": []}
    for lw in weights["layers"]:
        saved["layer_inputs"].append(hidden)
        hidden, sv = block_forward(hidden, lw, cfg, cos, sin, store)
        saved["layers"].append(sv)
    saved["hidden"] = hidden
    saved["normalized"] = r(rmsnorm_forward(hidden, weights["final_norm"], cfg["eps"]))
    return saved["normalized"], saved


def model_backward(d_normalized, g_lm_head, ids, weights, saved, cfg, cos, sin, store="f16", tied=True,
                   round_intermediates=True):
    """transformer_model_backward (src/core/transformer_model.cu:336-381) from the gradient of the
    final-norm output onwards; ``g_lm_head`` is the LM-head weight gradient already produced by the loss
    layer. Tied embeddings add the lookup gradient into it (transformer_model.cu:375-380)."""
    r = (lambda a: rnd(a, store)) if round_intermediates else (lambda a: np.asarray(a, F32))
    grads = {"layers": [None] * len(weights["layers"])}
    d_hidden, grads["final_norm"] = rmsnorm_backward(d_normalized, saved["hidden"], weights["final_norm"], cfg["eps"])
    d_hidden = r(d_hidden); grads["final_norm"] = r(grads["final_norm"])
    for layer in reversed(range(len(weights["layers"]))):
        d_hidden, grads["layers"][layer] = block_backward(d_hidden, saved["layer_inputs"][layer],
                                                          weights["layers"][layer], saved["layers"][layer], cfg,
                                                          cos, sin, store, 0, round_intermediates)
    vocab = np.asarray(weights["token_embedding"]).shape[0]
    if tied:
        grads["token_embedding"] = r(embedding_backward(d_hidden, ids.reshape(-1), vocab, accumulate_into=g_lm_head))
        grads["lm_head"] = grads["token_embedding"]
    else:
        grads["token_embedding"] = r(embedding_backward(d_hidden, ids.reshape(-1), vocab))
        grads["lm_head"] = r(g_lm_head)
    return grads
