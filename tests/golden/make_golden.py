"""Generates ``tests/golden/ref_cpu_ops.npz`` from the reference's own CPU operators.

Run where the reference is checked out: ``python oracle/build_ref.py && python tests/golden/make_golden.py``.
Inputs are seeded normals; outputs are what ``oracle/_ref/libcgpt_ref_cpu.so`` (the reference's
``src/ops/cpu/**`` and the CPU branch of ``src/optim/adamw.cu``, compiled unmodified) returns for them.
The fixture travels to machines without the reference; tests compare the numpy oracle and the CUDA
kernels with it.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import ref_cpu as R  # noqa: E402
from oracle.cgpt_oracle import rotary_cache  # noqa: E402


def main() -> None:
    rng = np.random.default_rng(20251125)
    n = lambda *s: rng.standard_normal(s).astype(np.float32)
    out = {}
    for dt in ("f32", "f16"):
        # RMSNorm: odd hidden (7), head_dim-like (64), model-like (256)
        for rows, hidden in ((3, 7), (40, 64), (17, 256)):
            x, dy, w = n(rows, hidden), n(rows, hidden), (1 + 0.02 * n(hidden)).astype(np.float32)
            key = f"rms_{dt}_{rows}x{hidden}"
            out[key + "_x"], out[key + "_dy"], out[key + "_w"] = x, dy, w
            out[key + "_y"] = R.rmsnorm_forward(x, w, 1e-5, dt)
            out[key + "_dx"], out[key + "_dw"] = R.rmsnorm_backward(dy, x, w, 1e-5, dt)
        # RoPE: full and partial rotary dim, non-zero offset
        b, s, hq, hkv, d = 2, 6, 4, 2, 16
        for rotary, off in ((0, 0), (8, 3)):
            r = rotary or d
            cos, sin = rotary_cache(16, r)
            q, k = n(b, s, hq, d), n(b, s, hkv, d)
            key = f"rope_{dt}_r{rotary}_o{off}"
            out[key + "_q"], out[key + "_k"], out[key + "_cos"], out[key + "_sin"] = q, k, cos, sin
            out[key + "_fq"], out[key + "_fk"] = R.rope_forward(q, k, cos, sin, rotary, off, dt)
            out[key + "_bq"], out[key + "_bk"] = R.rope_backward(q, k, cos, sin, rotary, off, dt)
        # SwiGLU
        g, u, dy = 3 * n(9, 40), n(9, 40), n(9, 40)
        key = f"swiglu_{dt}"
        out[key + "_g"], out[key + "_u"], out[key + "_dy"] = g, u, dy
        out[key + "_y"] = R.swiglu_forward(g, u, dt)
        out[key + "_dg"], out[key + "_du"] = R.swiglu_backward(dy, g, u, dt)
        # Linear forward/backward
        x, w, dy = n(12, 24), n(10, 24), n(12, 10)
        key = f"linear_{dt}"
        out[key + "_x"], out[key + "_w"], out[key + "_dy"] = x, w, dy
        out[key + "_y"] = R.linear_forward(x, w, dt)
        out[key + "_dx"], out[key + "_dw"], out[key + "_db"] = R.linear_backward(dy, x, w, dt)
        # Attention: causal GQA, Sq != Sk with offset, explicit scale (shapes of tests/flash_attention_test.cu)
        for name, (bb, sq, sk, h, hk, dd, off, sc) in {"a": (2, 3, 5, 4, 2, 32, 2, 0.23), "b": (1, 9, 9, 4, 2, 16, 0, 0.0),
                                                         "c": (1, 3, 35, 4, 1, 64, 32, 0.0)}.items():
            q, k, v, do = n(bb, sq, h, dd), n(bb, sk, hk, dd), n(bb, sk, hk, dd), n(bb, sq, h, dd)
            key = f"attn_{dt}_{name}"
            out[key + "_q"], out[key + "_k"], out[key + "_v"], out[key + "_do"] = q, k, v, do
            out[key + "_cfg"] = np.array([bb, sq, sk, h, hk, dd, off], np.int64)
            out[key + "_scale"] = np.float32(sc)
            o, lse = R.attention_forward(q, k, v, True, off, sc, dt)
            out[key + "_o"], out[key + "_lse"] = o, lse
            out[key + "_dq"], out[key + "_dk"], out[key + "_dv"] = R.attention_backward(do, q, k, v, o, lse, True, off, sc, dt)
        # Cross entropy with loss scaling, one out-of-vocabulary target
        z, t = 3 * n(6, 11), np.array([0, 10, 5, 3, 11, 2], np.uint32)
        key = f"ce_{dt}"
        out[key + "_z"], out[key + "_t"] = z, t
        loss, grad = R.cross_entropy(z, t, 1024.0, dt)
        out[key + "_loss"], out[key + "_grad"] = np.float32(loss), grad
    # Embedding backward accumulating into an existing table (the reference's CPU overwrite mode is
    # wrong for repeated ids, src/ops/cpu/backward/embedding_backward_cpu.cpp:110, so it is not a fixture)
    ids = np.array([1, 3, 3, 7, 0, 1], np.uint32)
    w, dy = n(8, 12), n(6, 12)
    out["emb_ids"], out["emb_w"], out["emb_dy"] = ids, w, dy
    out["emb_fwd"] = R.embedding_forward(ids, w, "f32")
    out["emb_bwd_acc"] = R.embedding_backward(dy, ids, 8, accumulate_into=w, dtype="f32")
    # AdamW: 3 steps of the single-tensor CPU path with clipping and loss scale
    p, g = n(33), 4 * n(33)
    master, m, v, step = p.copy(), np.zeros(33, np.float32), np.zeros(33, np.float32), 0
    out["adamw_p0"], out["adamw_g"] = p, g
    for it in range(3):
        p, master, m, v, step, ok = R.adamw_step(p, g, master, m, v, step, 3e-4, 0.9, 0.95, 1e-8, 0.1, 4.0, 1.0, "f32")
        assert ok
        out[f"adamw_master{it + 1}"], out[f"adamw_m{it + 1}"], out[f"adamw_v{it + 1}"] = master, m, v
    np.savez_compressed(Path(__file__).with_name("ref_cpu_ops.npz"), **out)
    print("wrote", Path(__file__).with_name("ref_cpu_ops.npz"), len(out), "arrays")


if __name__ == "__main__":
    main()
