"""The allocation-free expert FFN entry point, infmoe_t5ff_run_static.

Some callers of this library cannot allocate device memory at the moment they need the
expert FFN: a TensorRT plugin inside enqueue(), whose engine fixed its memory plan when it was
built, and a serving loop that must not trigger cudaMalloc's device-wide synchronisation.  For
them the library carries its own scratch array.  These tests call the entry point through the C ABI and compare it with
infmoe_t5ff_run (which takes a caller-allocated workspace) on two calls in a row; since both
run the same kernels on the same inputs the outputs must agree to the last bit, which is well
inside the 1e-5 relative-L2 tolerance used for this path elsewhere.

The file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _case(seed, n, D, F):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, D)).astype(np.float32)
    ln = (1 + 0.01 * rng.standard_normal(D)).astype(np.float32)
    wi0 = (rng.standard_normal((F, D)) / np.sqrt(D)).astype(np.float32)
    wi1 = (rng.standard_normal((F, D)) / np.sqrt(D)).astype(np.float32)
    wo = (rng.standard_normal((D, F)) / np.sqrt(F)).astype(np.float32)
    return x, ln, wi0, wi1, wo


def _run_static(g, x, ln, wi0, wi1, wo):
    import torch
    from infmoe_b200 import capi
    n, D = x.shape
    F = wi0.shape[0]
    dx, dl, d0, d1, do = g.dev(x), g.dev(ln), g.dev(wi0), g.dev(wi1), g.dev(wo)
    y = torch.full_like(dx, float("nan"))
    capi.check(capi.lib().infmoe_t5ff_run_static(n, D, F, dl.data_ptr(), d0.data_ptr(), d1.data_ptr(), do.data_ptr(),
                                                 dx.data_ptr(), y.data_ptr(), g.stream()))
    torch.cuda.synchronize()
    return y.cpu().numpy()


def test_static_scratch_matches_workspace_version_twice_in_a_row(oracle):
    import torch
    assert torch.cuda.is_available(), "this test needs a GPU"
    from tests import gpu_util as g
    # first a larger problem, then a smaller one with other data: the second call finds the first
    # call's leftovers in the shared array and must not be affected by them
    for seed, (n, D, F) in enumerate([(200, 256, 512), (37, 128, 384)]):
        x, ln, wi0, wi1, wo = _case(seed, n, D, F)
        got = _run_static(g, x, ln, wi0, wi1, wo)
        want = g.t5ff_run(x, ln, wi0, wi1, wo)
        assert np.isfinite(got).all()
        assert oracle.rel_l2(got, want) <= TOL
        np.testing.assert_array_equal(got, want)
        assert oracle.rel_l2(got, oracle.expert_ffn_f64(x, ln, wi0, wi1, wo)) <= TOL


def test_static_scratch_calls_allocate_nothing():
    """Free device memory is the same before and after the second and third call (the first call may load the
    module and look up the array's address)."""
    import torch
    assert torch.cuda.is_available(), "this test needs a GPU"
    from infmoe_b200 import capi
    from tests import gpu_util as g
    n, D, F = 64, 256, 512
    x, ln, wi0, wi1, wo = _case(7, n, D, F)
    dx, dl, d0, d1, do = g.dev(x), g.dev(ln), g.dev(wi0), g.dev(wi1), g.dev(wo)
    y = torch.empty_like(dx)

    def call():
        capi.check(capi.lib().infmoe_t5ff_run_static(n, D, F, dl.data_ptr(), d0.data_ptr(), d1.data_ptr(),
                                                     do.data_ptr(), dx.data_ptr(), y.data_ptr(), g.stream()))

    call()
    torch.cuda.synchronize()
    for _ in range(2):
        free_before, _total = torch.cuda.mem_get_info()     # cudaMemGetInfo: the driver's view, not torch's cache
        call()
        torch.cuda.synchronize()
        free_after, _total = torch.cuda.mem_get_info()
        assert free_after == free_before, (free_before, free_after)


def test_static_scratch_rejects_sizes_beyond_its_array():
    import torch
    assert torch.cuda.is_available(), "this test needs a GPU"
    from infmoe_b200 import capi
    from tests import gpu_util as g
    need, avail = ctypes.c_size_t(), ctypes.c_size_t()
    capi.check(capi.lib().infmoe_t5ff_static_limit(64, 4096, 10240, ctypes.byref(need), ctypes.byref(avail)))
    assert avail.value == 32 << 20 and need.value > avail.value
    capi.check(capi.lib().infmoe_t5ff_static_limit(256, 512, 1024, ctypes.byref(need), ctypes.byref(avail)))
    assert need.value <= avail.value
    # pointers are never touched when the size check fails, so small dummies are enough
    d = torch.zeros(16, device="cuda")
    rc = capi.lib().infmoe_t5ff_run_static(64, 4096, 10240, d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(),
                                           d.data_ptr(), d.data_ptr(), g.stream())
    assert rc == 6
    assert "built-in array" in capi.last_error()
