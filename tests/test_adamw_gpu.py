"""GPU parity of the fused multi-tensor AdamW (through the C ABI): the reference tests' known answers
(tests/adamw_test.cu:21-91), the committed trajectory of the reference's CPU AdamW, and the numpy
restatement on a many-tensor list. Bar: updates within 1e-6 relative."""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import known_answers as KA
from gpu_util import dev, host
from oracle import cgpt_oracle as O

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "ref_cpu_ops.npz")


@pytest.fixture(scope="module")
def optim():
    from cgpt_b200 import optim as m
    return m


@pytest.mark.parametrize("dt,tol", [("f32", 2e-6), ("f16", 2e-3), ("bf16", 1e-2)])
def test_two_step_known_answer(optim, dt, tol):
    c = KA.ADAMW_TWO_STEPS
    p, g = dev(c["parameter"], dt), dev(c["gradient"], dt)
    st = optim.AdamWState.for_parameter(p)
    o = optim.AdamWOptions(**c["options"])
    assert optim.adamw_step(p, g, st, o)
    np.testing.assert_allclose(host(p), c["after1"], atol=tol)
    np.testing.assert_allclose(host(st.first_moment), c["m1"], atol=tol); np.testing.assert_allclose(host(st.second_moment), c["v1"], atol=tol)
    assert st.step == 1
    assert optim.adamw_step(p, g, st, o)
    np.testing.assert_allclose(host(p), c["after2"], atol=tol)
    assert st.step == 2


def test_clip_and_non_finite_skip(optim):
    c = KA.ADAMW_CLIP
    p, g = dev(c["parameter"]), dev(c["gradient"])
    st = optim.AdamWState.for_parameter(p)
    o = optim.AdamWOptions(**c["options"])
    ws = optim.AdamWWorkspace()
    entry = [optim.AdamWBatchEntry(p, g, st)]
    optim.adamw_step_many_async(entry, o, ws)
    assert optim.adamw_check(ws)
    np.testing.assert_allclose(host(st.master_parameter), c["after"], atol=2e-6)
    before = p.clone()
    g.copy_(torch.tensor([math.inf, 0.0]))
    optim.adamw_step_many_async(entry, o, ws)
    assert not optim.adamw_check(ws)
    assert torch.equal(p, before) and st.step == 1
    assert optim.adamw_check(ws), "the sticky flag is cleared by adamw_check"
    g.copy_(torch.tensor([float("nan"), 0.0]))
    optim.adamw_step_many_async(entry, o, ws)
    assert not optim.adamw_check(ws) and torch.equal(p, before)


def test_validation(optim):
    p, g = dev(np.ones(4)), dev(np.ones(5))
    with pytest.raises(ValueError):
        optim.adamw_step(p, g, optim.AdamWState.for_parameter(p))
    p, g = dev(np.ones(4)), dev(np.ones(4))
    st = optim.AdamWState.for_parameter(p)
    ws = optim.AdamWWorkspace()
    with pytest.raises(ValueError):
        optim.adamw_step_many_async([], optim.AdamWOptions(), ws)
    with pytest.raises(ValueError):
        optim.adamw_step_many_async([optim.AdamWBatchEntry(p, g, st)], optim.AdamWOptions(beta1=1.0), ws)
    optim.adamw_step_many_async([optim.AdamWBatchEntry(p, g, st)], optim.AdamWOptions(), ws)
    with pytest.raises(ValueError):   # a bound workspace rejects a different list (src/optim/adamw.cu:298-305)
        optim.adamw_step_many_async([optim.AdamWBatchEntry(p, g, optim.AdamWState.for_parameter(p))], optim.AdamWOptions(), ws)


def test_reference_cpu_trajectory(optim):
    p, g = dev(GOLD["adamw_p0"]), dev(GOLD["adamw_g"])
    st = optim.AdamWState.for_parameter(p)
    o = optim.AdamWOptions(3e-4, 0.9, 0.95, 1e-8, 0.1, 4.0, 1.0)
    ws = optim.AdamWWorkspace()
    for it in range(3):
        optim.adamw_step_many_async([optim.AdamWBatchEntry(p, g, st)], o, ws)
        assert optim.adamw_check(ws)
        want = GOLD[f"adamw_master{it + 1}"]
        assert np.max(np.abs(host(st.master_parameter) - want) / np.abs(want)) <= 1e-6
        np.testing.assert_allclose(host(st.first_moment), GOLD[f"adamw_m{it + 1}"], rtol=2e-6, atol=1e-9)
        np.testing.assert_allclose(host(st.second_moment), GOLD[f"adamw_v{it + 1}"], rtol=2e-6, atol=1e-12)


@pytest.mark.parametrize("dt,max_norm", [("f16", math.inf), ("f16", 1.0), ("bf16", 1.0), ("f32", 0.5)])
def test_many_tensors_against_oracle(optim, dt, max_norm):
    r = np.random.default_rng(11)
    sizes = [1, 7, 128, 1000, 4096, 4097, 8191, 33000, 100003, 1024 * 256]
    params = [dev(0.02 * r.standard_normal(n), dt) for n in sizes]
    grads = [dev(1024 * 0.01 * r.standard_normal(n), dt) for n in sizes]
    states = [optim.AdamWState.for_parameter(p) for p in params]
    o = optim.AdamWOptions(3e-4, 0.9, 0.95, 1e-8, 0.1, 1024.0, max_norm)
    ws = optim.AdamWWorkspace()
    entries = [optim.AdamWBatchEntry(p, g, s) for p, g, s in zip(params, grads, states)]
    masters = [host(s.master_parameter) for s in states]
    ms = [np.zeros(n, np.float32) for n in sizes]; vs = [np.zeros(n, np.float32) for n in sizes]
    g_np = [host(g) for g in grads]
    step = 0
    for it in range(3):
        optim.adamw_step_many_async(entries, o, ws)
        assert optim.adamw_check(ws)
        ep, masters, ms, vs, step, skipped = O.adamw_step(dt, g_np, masters, ms, vs, step, 3e-4, 0.9, 0.95, 1e-8, 0.1, 1024.0, max_norm)
        assert not skipped and states[0].step == step
        sq, clip = optim.adamw_last_stats(ws)
        want_sq = sum(float(np.sum((g.astype(np.float64) / 1024.0) ** 2)) for g in g_np)
        assert abs(sq - want_sq) <= 1e-5 * want_sq
        for s, w, m, v, p, e in zip(states, masters, ms, vs, params, ep):
            got = host(s.master_parameter)
            # fp32 sums of squares in a different order move the clip factor by ~1e-7 relative
            assert np.max(np.abs(got - w)) <= 1e-6 * np.max(np.abs(w)) + 1e-9
            np.testing.assert_allclose(host(s.first_moment), m, rtol=1e-5, atol=1e-9)
            np.testing.assert_allclose(host(s.second_moment), v, rtol=1e-5, atol=1e-12)
            assert np.max(np.abs(host(p) - O.rnd(got, dt))) == 0.0, "param must be the rounded master"


def test_learning_rate_from_device_scalar_equals_host_value(optim):
    """cgpt_adamw_step_device_lr: the update reads the learning rate from a device scalar when it runs (the form that sits
    inside a captured graph while a schedule changes the rate). Three steps with three rates written to the scalar must
    give bit-identical parameters, master weights and moments to three steps that pass the same rates by value."""
    torch.manual_seed(3)
    sizes = [1000, 4096 * 3 + 5, 257]
    rates = [3e-4, 2.5e-4, 1e-5]
    results = []
    for device_lr in (False, True):
        ps = [(torch.randn(n, device="cuda") * 0.02).half() for n in sizes]
        gs = [torch.randn(n, device="cuda").half() for n in sizes]
        torch.manual_seed(3)      # same tensors in both passes
        sts = [optim.AdamWState.for_parameter(p) for p in ps]
        ws = optim.AdamWWorkspace()
        ent = [optim.AdamWBatchEntry(p, g, s) for p, g, s in zip(ps, gs, sts)]
        scalar = torch.zeros(1, device="cuda")
        for lr in rates:
            o = optim.AdamWOptions(lr if not device_lr else 123.0, 0.9, 0.95, 1e-8, 0.1, 8.0, 1.0)
            if device_lr:
                scalar.fill_(lr)
                optim.adamw_step_many_async(ent, o, ws, learning_rate_device=scalar)
            else:
                optim.adamw_step_many_async(ent, o, ws)
        assert optim.adamw_check(ws) and sts[0].step == 3
        results.append([t.clone() for p, s in zip(ps, sts) for t in (p, s.master_parameter, s.first_moment, s.second_moment)])
    for a, b in zip(*results):
        assert torch.equal(a, b)
    with pytest.raises(Exception):
        optim.adamw_step_many_async(ent, o, ws, learning_rate_device=torch.zeros(2, device="cuda"))
