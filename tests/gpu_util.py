"""Helpers shared by the ``-m gpu`` parity tests."""
import numpy as np
import torch

TORCH = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
# max |a-b| relative to the RMS of the expected tensor (the "fp32 norm-scaled" error of the parity bar)
TOL = {"f32": 2e-5, "f16": 2e-3, "bf16": 1.6e-2}


def dev(a, dt="f32"):
    """numpy -> CUDA tensor of storage dtype `dt` (round to nearest even, like Tensor::copy_from_host)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda").to(TORCH[dt]).contiguous()


def ids_dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int64)).to(torch.int32).to("cuda")


def host(t):
    return t.detach().to(torch.float32).cpu().numpy()


def rounded(t):
    """The values a device tensor actually holds, as fp32 numpy (inputs for the oracle)."""
    return host(t)


def scaled_err(got, want):
    """The harness's norm-scaled error: max_i |a_i - b_i| / (|b_i| + rms(b)). An element may be off by `tol` of its
    own magnitude plus `tol` of the tensor's RMS. A plain max|a-b| / rms(b) would flag correctly rounded outputs of
    heavy-tailed tensors (one fp16 ulp of a 5-sigma element is several 1e-3 of the RMS)."""
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    return float(np.max(np.abs(got - want) / (np.abs(want) + max(rms, 1e-30))))


def max_err(got, want):
    """max |a-b| relative to max |b|: for heavy-tailed tensors (vocabulary-sized gradients, where a few rows carry
    almost all of the norm and the RMS says little about the scale of the entries that matter)."""
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))


def plain_err(got, want):
    """The parity bar's error as it is usually written: max |a-b| / rms(b) (rms(b) = ||b||_2 / sqrt(n))."""
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    return float(np.max(np.abs(got - want)) / max(rms, 1e-30))


# (what, metric used, value, tolerance, plain max|a-b|/rms(b)) of every comparison of the session; tests/conftest.py writes it
# out at the end of a GPU run so that the plain norm-scaled number stands beside the one each assertion used.
REPORT = []


def assert_close(got, want, tol, what="", metric="rms"):
    """metric: "rms" = scaled_err, "max" = max_err, "plain" = plain_err."""
    e = {"rms": scaled_err, "max": max_err, "plain": plain_err}[metric](got, want)
    plain = plain_err(got, want)
    REPORT.append((what, metric, e, tol, plain))
    assert np.all(np.isfinite(np.asarray(got))), f"{what}: non-finite output"
    assert e <= tol, f"{what}: {metric} error {e:.3e} > {tol:.1e} (plain max|a-b|/rms(b) = {plain:.3e})"
