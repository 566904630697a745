"""cgpt_rmsnorm_backward_noalloc, called through the C ABI, must give what cgpt_rmsnorm_backward gives.

The entry point is for embedders that cannot allocate device memory when they call into the library (their
own pool owns the device memory, or their call site may not enter the allocator): its scratch is a fixed
array inside the library, so nothing is allocated, and every call reuses that array. The test therefore
makes two calls in a row per case - the second one finds the first one's partial sums still in the array -
and compares both with the allocating entry point. It is collected last so that a run that stops at the
first failure has already exercised everything else, and it does not depend on anything the other tests
leave behind (it passes alone in a fresh process as well).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import TOL, assert_close, dev, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    from cgpt_b200 import _lib
    return _lib


def _call(fn, dx, dw, dy, x, w, ra, rb, lib):
    p = lambda t: None if t is None else t.data_ptr()
    return fn(p(dx), p(dw), p(dy), p(x), p(w), p(ra), p(rb), x.shape[0], x.shape[1], C.c_float(1e-5), lib.dtype_code(x),
              lib.stream_ptr())


@pytest.mark.parametrize("rows,hidden,dt,residuals", [(4096, 1024, "f16", False), (3000, 4096, "f16", True), (129, 513, "bf16", False),
                                                      (65536, 128, "f16", False), (77, 100, "f32", True), (20000, 8192, "f16", False)])
def test_noalloc_matches_allocating_entry_point(lib, rows, hidden, dt, residuals):
    r = np.random.default_rng(rows + hidden)
    x, dy = dev(r.standard_normal((rows, hidden)), dt), dev(r.standard_normal((rows, hidden)), dt)
    w = dev(1 + 0.02 * r.standard_normal(hidden), dt)
    ra = dev(r.standard_normal((rows, hidden)), dt) if residuals else None
    rb = dev(r.standard_normal((rows, hidden)), dt) if residuals else None
    dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
    lib.check(_call(lib.lib.cgpt_rmsnorm_backward, dx_ref, dw_ref, dy, x, w, ra, rb, lib), "rmsnorm_backward")
    for attempt in range(2):   # the second call reuses the array with the first call's contents in it
        dx, dw = torch.full_like(x, float("nan")), torch.full_like(w, float("nan"))
        lib.check(_call(lib.lib.cgpt_rmsnorm_backward_noalloc, dx, dw, dy, x, w, ra, rb, lib), "rmsnorm_backward_noalloc")
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref), f"dx differs on call {attempt}"
        # dw may be summed over a different number of partial rows (the grid is capped to fit the fixed array)
        assert_close(host(dw), host(dw_ref), TOL[dt] * 2, f"dw on call {attempt}")
    # a different problem in between must not disturb the next one (stale, larger contents in the array)
    x2, dy2, w2 = dev(r.standard_normal((512, 2048)), "f16"), dev(r.standard_normal((512, 2048)), "f16"), dev(np.ones(2048), "f16")
    lib.check(_call(lib.lib.cgpt_rmsnorm_backward_noalloc, torch.empty_like(x2), torch.empty_like(w2), dy2, x2, w2, None, None, lib), "noalloc")
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    lib.check(_call(lib.lib.cgpt_rmsnorm_backward_noalloc, dx, dw, dy, x, w, ra, rb, lib), "rmsnorm_backward_noalloc")
    assert torch.equal(dx, dx_ref)
    assert_close(host(dw), host(dw_ref), TOL[dt] * 2, "dw after an unrelated call")


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch(lib):
    x = dev(np.ones((4, 8200)), "f16"); w = dev(np.ones(8200), "f16")
    rc = _call(lib.lib.cgpt_rmsnorm_backward_noalloc, torch.empty_like(x), torch.empty_like(w), x, x, w, None, None, lib)
    assert rc == 3, "hidden > 8192 must be refused with CGPT_ERR_SHAPE"
    with pytest.raises(ValueError):
        lib.check(rc, "rmsnorm_backward_noalloc")
