"""The allocation-free RMSNorm backward entry point (bmc_rmsnorm_backward_static) against the regular one.

Some embedders of this library cannot let it call cudaMalloc — they have given the whole GPU to their own memory pool,
or they run loops in which the implicit device-wide synchronisation of cudaMalloc/cudaFree is not acceptable. For them the
backend has one entry point whose scratch is a fixed array inside the library. This test calls it through the C ABI twice in a
row (different shapes, so the second call meets the first call's leftovers in the shared scratch) and requires the same
gradients as bmc_rmsnorm_backward and as the CPU oracle, within the tolerances the other kernel tests use; it also checks that a row wider than
the built-in scratch is refused. The file name sorts last so that a run that stops at the first failure has already
executed every other test."""
import ctypes as C

import numpy as np
import pytest

import oracle_check as oc
import portk
from bmcapi import BMC_BF16, BMC_F32, Backend, Ptr, bf16_round

pytestmark = pytest.mark.gpu


def _bind(lib):
    vp, ci = C.c_void_p, C.c_int
    lib.bmc_rmsnorm_backward_static.restype = ci
    lib.bmc_rmsnorm_backward_static.argtypes = [vp, ci, vp, vp, ci, vp, vp, vp, vp, ci, ci, ci, ci]
    lib.bmc_stream.restype = vp
    lib.bmc_stream.argtypes = [vp]


def _one_case(be, rng, dtype, N, C_, accumulate, row0):
    lib = be.lib
    mk = (lambda *s: bf16_round(rng.standard_normal(s).astype(np.float32))) if dtype == BMC_BF16 else (lambda *s: rng.standard_normal(s).astype(np.float32))
    x, go, gx0 = mk(N, C_), mk(N, C_), mk(N, C_)
    w, gw0 = rng.standard_normal(C_).astype(np.float32), rng.standard_normal(C_).astype(np.float32)
    dx, dgo, dw = be.put(x, dtype), be.put(go, dtype), be.put(w)
    out, rstd = be.zeros(N * C_, dtype), be.zeros(N)
    be.ok("rmsnorm_forward", dtype, Ptr(out), Ptr(rstd), Ptr(dx), Ptr(dw), N, C_, 1e-5)
    # existing entry point
    gx_a, gw_a = be.put(gx0, dtype), be.put(gw0)
    be.ok("rmsnorm_backward", dtype, Ptr(gx_a), Ptr(gw_a), accumulate, Ptr(dgo), Ptr(dx), Ptr(dw), Ptr(rstd), N, C_, row0, N)
    # allocation-free entry point, on the same stream
    gx_b, gw_b = be.put(gx0, dtype), be.put(gw0)
    rc = lib.bmc_rmsnorm_backward_static(lib.bmc_stream(be.ctx), dtype, gx_b, gw_b, accumulate, dgo, dx, dw, rstd, N, C_, row0, N)
    assert rc == 0, rc
    assert lib.bmc_sync(be.ctx) == 0
    rel = 1e-5 if dtype == BMC_F32 else 2e-2
    a, b = be.get(gx_a, (N, C_), dtype), be.get(gx_b, (N, C_), dtype)
    assert oc.rel_err(b, a) <= rel
    ga, gb = be.get(gw_a, (C_,)), be.get(gw_b, (C_,))
    assert oc.rel_err(gb, ga) <= rel
    assert np.isfinite(b).all() and np.isfinite(gb).all()
    # and against the CPU oracle, like the regular entry point's own test: gx accumulates, the gain gradient covers rows [row0, N)
    ref_gw = portk.rmsnorm_backward_w(go[row0:], x[row0:]) + (gw0 if accumulate else 0.0)
    assert oc.rel_err(b, portk.rmsnorm_backward_x(go, w, x, gx0)) <= (1e-5 if dtype == BMC_F32 else 2e-2)
    assert oc.rel_err(gb, ref_gw) <= (1e-5 if dtype == BMC_F32 else 2e-2)


def test_static_scratch_entry_point_matches_regular_one_twice_in_a_row(product):
    _bind(product)
    be = Backend(product)
    rng = np.random.default_rng(77)
    try:
        # two calls back to back per dtype; the second is narrower and shorter, so stale partial sums from the first
        # remain in the shared scratch beyond the region it rewrites
        _one_case(be, rng, BMC_F32, 5000, 960, 0, 0)
        _one_case(be, rng, BMC_F32, 70, 576, 1, 35)
        _one_case(be, rng, BMC_BF16, 4096, 1024, 1, 0)
        _one_case(be, rng, BMC_BF16, 33, 128, 0, 0)
    finally:
        be.close()


def test_static_scratch_entry_point_rejects_rows_beyond_its_maximum(product):
    _bind(product)
    be = Backend(product)
    try:
        N, C_ = 8, 2048  # supported by the regular entry point in bf16, wider than the built-in scratch allows
        z = be.zeros(N * C_, BMC_BF16)
        rc = product.bmc_rmsnorm_backward_static(product.bmc_stream(be.ctx), BMC_BF16, z, be.zeros(C_), 0, z, z, be.zeros(C_), be.zeros(N), N, C_, 0, N)
        assert rc == -60  # BMC_ERR_STATIC_TOO_LARGE
        assert product.bmc_sync(be.ctx) == 0
    finally:
        be.close()
