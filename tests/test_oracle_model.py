"""The reference has no value test for block/model backward (only finiteness), so the oracle's restatement of
transformer_block_backward / transformer_model_backward is pinned by central finite differences of its own
forward restatement (fp32 storage), on a very small block. CPU only."""
import numpy as np

from oracle import cgpt_oracle as O


def _setup(seed=0):
    r = np.random.default_rng(seed)
    cfg = dict(batch=1, seq=5, hidden=16, intermediate=24, q_heads=2, kv_heads=1, head_dim=8, rotary_dim=8, eps=1e-5)
    shapes = {"attention_norm": (16,), "q_projection": (16, 16), "k_projection": (8, 16), "q_norm": (8,), "k_norm": (8,),
              "v_projection": (8, 16), "o_projection": (16, 16), "ffn_norm": (16,), "gate_proj": (24, 16), "up_proj": (24, 16),
              "down_proj": (16, 24)}
    w = {n: ((1 + 0.1 * r.standard_normal(s)) if n.endswith("norm") else 0.3 * r.standard_normal(s)).astype(np.float64) for n, s in shapes.items()}
    x = r.standard_normal((5, 16))
    cos, sin = O.rotary_cache(8, 8)
    return r, cfg, w, x, cos, sin


def test_block_backward_matches_finite_differences():
    r, cfg, w, x, cos, sin = _setup()
    probe = r.standard_normal((5, 16))
    f = lambda xx, ww: float(np.sum(O.block_forward(xx, ww, cfg, cos, sin, "f32")[0].astype(np.float64) * probe))
    out, sv = O.block_forward(x, w, cfg, cos, sin, "f32")
    gin, g = O.block_backward(probe, x, w, sv, cfg, cos, sin, "f32", 0, round_intermediates=False)
    eps = 2e-2
    for name in w:
        flat_idx = r.integers(0, w[name].size, 3)
        for fi in flat_idx:
            idx = np.unravel_index(fi, w[name].shape)
            wp = {k: v.copy() for k, v in w.items()}; wm = {k: v.copy() for k, v in w.items()}
            wp[name][idx] += eps; wm[name][idx] -= eps
            num = (f(x, wp) - f(x, wm)) / (2 * eps)
            assert abs(num - g[name][idx]) <= 3e-2 * max(1.0, abs(num)), (name, idx, num, g[name][idx])
    for fi in r.integers(0, x.size, 6):
        idx = np.unravel_index(fi, x.shape)
        xp, xm = x.copy(), x.copy()
        xp[idx] += eps; xm[idx] -= eps
        num = (f(xp, w) - f(xm, w)) / (2 * eps)
        assert abs(num - gin[idx]) <= 3e-2 * max(1.0, abs(num)), (idx, num, gin[idx])


def test_model_loss_gradient_matches_finite_differences():
    r, cfg, w, x, cos, sin = _setup(1)
    vocab = 11
    weights = {"token_embedding": 0.5 * r.standard_normal((vocab, 16)), "layers": [w, {k: v.copy() for k, v in w.items()}],
               "final_norm": np.ones(16)}
    weights["lm_head"] = weights["token_embedding"]
    ids = r.integers(0, vocab, (1, 5)); targets = r.integers(0, vocab, 5)

    def loss_of(ws):
        ws = dict(ws); ws["lm_head"] = ws["token_embedding"]
        normalized, _ = O.model_forward(ids, ws, cfg, cos, sin, "f32")
        return float(O.cut_cross_entropy(normalized, ws["lm_head"], targets)[0])

    normalized, saved = O.model_forward(ids, weights, cfg, cos, sin, "f32")
    loss, d_norm, g_head = O.cut_cross_entropy(normalized, weights["lm_head"], targets)
    grads = O.model_backward(d_norm, g_head, ids, weights, saved, cfg, cos, sin, "f32", tied=True, round_intermediates=False)
    eps = 1e-2
    for fi in r.integers(0, weights["token_embedding"].size, 5):
        idx = np.unravel_index(fi, weights["token_embedding"].shape)
        wp = dict(weights); wm = dict(weights)
        wp["token_embedding"] = weights["token_embedding"].copy(); wm["token_embedding"] = weights["token_embedding"].copy()
        wp["token_embedding"][idx] += eps; wm["token_embedding"][idx] -= eps
        num = (loss_of(wp) - loss_of(wm)) / (2 * eps)
        assert abs(num - grads["token_embedding"][idx]) <= 2e-2 * max(0.05, abs(num)), (idx, num, grads["token_embedding"][idx])
    li, name = 0, "gate_proj"
    for fi in r.integers(0, w[name].size, 4):
        idx = np.unravel_index(fi, w[name].shape)
        def perturbed(delta):
            ws = dict(weights); ws["layers"] = [{k: v.copy() for k, v in l.items()} for l in weights["layers"]]
            ws["layers"][li][name][idx] += delta
            return loss_of(ws)
        num = (perturbed(eps) - perturbed(-eps)) / (2 * eps)
        assert abs(num - grads["layers"][li][name][idx]) <= 2e-2 * max(0.05, abs(num)), (idx, num)
