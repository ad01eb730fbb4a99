"""The allocation-free RMSNorm reverse entry point
(launch_rmsnorm_ij_j_reverse_static_r32).

It exists for callers that may not allocate device memory - a plug-in inside a
runtime that owns the whole device through its own pool, or a loop where an
allocation would stall the device - and therefore cannot hand the library the
scratch buffer the regular entry point needs.  The partial sums live in a fixed
8 MiB array inside the library instead.  The test calls it through the C ABI
twice in a row (the array is shared between calls and keeps the previous
call's contents) and compares gx and ggain with the regular entry point.
This file sorts last so that a run stopping at the first failure has already
exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

from util import TOL_RED, assert_close, dev, host, rng_normal, run

pytestmark = pytest.mark.gpu


def call_static(mp, stream, x, gain, gy, eps, gx, gg, alpha, m, n):
    import torch
    torch.cuda.current_stream().synchronize()
    p = lambda t: C.c_void_p(t.data_ptr())
    rc = mp.lib().launch_rmsnorm_ij_j_reverse_static_r32(p(x), p(gain), C.c_void_p(0), p(gy), eps, p(gx), p(gg), alpha,
                                                         m, n, stream.ctx)
    stream.sync()
    return rc


@pytest.mark.parametrize("shape", [(1000, 4096), (301, 1000), (5000, 512), (70, 4099)])
def test_static_scratch_entry_point_matches_the_regular_one_twice(mp, stream, shape):
    import torch
    m, n = shape
    eps = 1e-6
    nbytes = mp.lib().mpRmsnormReverseScratchBytes(m, n, stream.ctx)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    for call, alpha in enumerate((0.0, 1.0)):          # two calls in a row, second one accumulating
        x = dev(rng_normal(10 + call, shape, "r32")); gy = dev(rng_normal(20 + call, shape, "r32"))
        gain = dev(rng_normal(30 + call, n, "r32", scale=0.02, loc=1.0))
        gx0 = rng_normal(40 + call, shape, "r32"); gg0 = rng_normal(50 + call, n, "r32")
        gx_ref, gg_ref = dev(gx0), dev(gg0)
        run(mp, stream, "rmsnorm_ij_j_reverse", "r32", x, gain, None, gy, eps, gx_ref, gg_ref, alpha, scratch, m, n)
        gx, gg = dev(gx0), dev(gg0)
        assert call_static(mp, stream, x, gain, gy, eps, gx, gg, alpha, m, n) == 0
        assert_close(host(gx), host(gx_ref), TOL_RED["r32"], f"static gx call {call} {shape}")
        assert_close(host(gg), host(gg_ref), TOL_RED["r32"], f"static ggain call {call} {shape}")


def test_many_rows_still_fit_because_rows_per_cta_grow(mp, stream):
    import torch
    m, n, eps = 40000, 4096, 1e-6       # 1250 CTAs at 32 rows each would need 20 MB of partials
    x = dev(rng_normal(1, (m, n), "r32")); gy = dev(rng_normal(2, (m, n), "r32"))
    gain = dev(rng_normal(3, n, "r32", scale=0.02, loc=1.0))
    scratch = torch.empty(mp.lib().mpRmsnormReverseScratchBytes(m, n, stream.ctx), dtype=torch.uint8, device="cuda")
    gx_ref = torch.empty_like(x); gg_ref = torch.empty_like(gain)
    run(mp, stream, "rmsnorm_ij_j_reverse", "r32", x, gain, None, gy, eps, gx_ref, gg_ref, 0.0, scratch, m, n)
    gx = torch.empty_like(x); gg = torch.empty_like(gain)
    assert call_static(mp, stream, x, gain, gy, eps, gx, gg, 0.0, m, n) == 0
    assert_close(host(gx), host(gx_ref), TOL_RED["r32"], "static gx, many rows")
    assert_close(host(gg), host(gg_ref), TOL_RED["r32"], "static ggain, many rows")


def test_rows_beyond_the_fixed_scratch_are_rejected(mp, stream):
    import torch
    n = 200000                           # (16 + 1) partial rows of 800 kB exceed 8 MiB
    t = torch.zeros(n, device="cuda")
    rc = call_static(mp, stream, t, t, t, 1e-6, t, t, 0.0, 1, n)
    assert rc == 2                       # MP_STATUS_BAD_ARGUMENT, nothing launched
