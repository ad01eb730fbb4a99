"""GPU parity of softmax / RMSNorm (forward and reverse) against the CPU oracle."""
import ctypes

import numpy as np
import pytest

from util import run, TOL_RED, assert_close, dev, host, narrow, rng_normal, torch_dtype, wide

pytestmark = pytest.mark.gpu

# (m, n): warp-per-row, CTA-per-row in every group size, ragged n (generic path), long rows
SHAPES = [(1, 1), (7, 8), (33, 128), (65, 512), (40, 1024), (19, 2048), (300, 4096), (9, 8192), (5, 16384),
          (11, 50280), (13, 1000), (6, 4099), (3, 40000), (70, 768), (37, 520), (300, 1024)]
DTYPES = ["r16", "r32", "r64"]




@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_softmax_forward_and_reverse(mp, stream, orc, sfx, shape):
    m, n = shape
    x = rng_normal(1, shape, sfx, scale=2.0)
    y = dev(np.full(shape, np.nan, x.dtype))
    run(mp, stream, "softmax_ij_j", sfx, dev(x), y, m, n)
    yref = orc.softmax_ij_j(wide(x))
    assert_close(host(y), narrow(yref, sfx), TOL_RED[sfx], f"softmax fwd {sfx} {shape}")
    # reverse consumes the forward output as stored (rounded to T)
    ys = host(y)
    gy = rng_normal(2, shape, sfx)
    gx = dev(np.full(shape, np.nan, x.dtype))
    run(mp, stream, "softmax_ij_j_reverse", sfx, y, dev(gy), gx, 0.0, m, n)
    assert_close(host(gx), narrow(orc.softmax_ij_j_reverse(wide(ys), wide(gy)), sfx), TOL_RED[sfx], f"softmax rev {sfx} {shape}")
    g0 = rng_normal(3, shape, sfx)
    gx = dev(g0)
    run(mp, stream, "softmax_ij_j_reverse", sfx, y, dev(gy), gx, 1.0, m, n)
    assert_close(host(gx), narrow(orc.softmax_ij_j_reverse(wide(ys), wide(gy), wide(g0).copy(), 1.0), sfx), TOL_RED[sfx],
                 f"softmax rev accumulate {sfx} {shape}")


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("saved_rstd", [True, False])
def test_rmsnorm_forward_and_reverse(mp, stream, orc, sfx, shape, saved_rstd):
    import torch
    m, n = shape
    eps = 1e-6
    x = rng_normal(4, shape, sfx)
    gain = rng_normal(5, n, sfx, scale=0.02, loc=1.0)
    y = dev(np.full(shape, np.nan, x.dtype))
    acc_dt = torch.float64 if sfx == "r64" else torch.float32
    rstd = torch.full((m,), float("nan"), dtype=acc_dt, device="cuda")
    run(mp, stream, "rmsnorm_ij_j", sfx, dev(x), dev(gain), eps, y, rstd if saved_rstd else None, m, n)
    yref, rref = orc.rmsnorm_ij_j(wide(x), wide(gain), eps)
    assert_close(host(y), narrow(yref, sfx), TOL_RED[sfx], f"rmsnorm fwd {sfx} {shape}")
    if saved_rstd:
        assert_close(host(rstd), rref, 1e-5 if sfx != "r64" else 1e-12, "rstd")
    gy = rng_normal(6, shape, sfx)
    nbytes = mp.lib().mpRmsnormReverseScratchBytes(m, n, stream.ctx)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    for alpha in (0.0, 1.0):
        gx0 = rng_normal(7, shape, sfx); gg0 = rng_normal(8, n, sfx)
        gx = dev(gx0 if alpha else np.full(shape, np.nan, x.dtype))
        gg = dev(gg0 if alpha else np.full(n, np.nan, x.dtype))
        run(mp, stream, "rmsnorm_ij_j_reverse", sfx, dev(x), dev(gain), rstd if saved_rstd else None, dev(gy), eps,
            gx, gg, alpha, scratch, m, n)
        rgx, rgg = orc.rmsnorm_ij_j_reverse(wide(x), wide(gain), wide(gy), eps, wide(gx0).copy() if alpha else None,
                                            wide(gg0).copy() if alpha else None, alpha)
        if n == 1 and not alpha:
            # a single column cancels exactly up to eps: compare on the scale of the two terms
            scale = float(np.abs(wide(gy) * wide(gain)).max() * rref.max())
            assert float(np.abs(host(gx).astype(np.float64) - rgx).max()) <= TOL_RED[sfx] * scale
        else:
            assert_close(host(gx), narrow(rgx, sfx), TOL_RED[sfx], f"rmsnorm gx alpha={alpha} {sfx} {shape}")
        assert_close(host(gg), narrow(rgg, sfx), TOL_RED[sfx], f"rmsnorm ggain alpha={alpha} {sfx} {shape}")


@pytest.mark.parametrize("sfx", ["r16", "r32"])
def test_full_size_properties(mp, stream, sfx):
    """[65536, 4096]: size-independent properties instead of a CPU oracle pass -
    softmax rows sum to 1 and are invariant to a per-row shift; RMSNorm output
    with unit gain has unit mean square; reverse-mode row identities."""
    import torch
    m, n = 65536, 4096
    dt = torch_dtype(sfx)
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(m, n, generator=g, device="cuda", dtype=torch.float32).to(dt)
    y = torch.empty_like(x)
    run(mp, stream, "softmax_ij_j", sfx, x, y, m, n)
    sums = y.float().sum(1)
    tol = 2e-3 if sfx == "r16" else 1e-5
    assert float((sums - 1).abs().max()) < tol
    assert bool((y >= 0).all())
    if sfx == "r32":
        shift = torch.randn(m, 1, generator=g, device="cuda") * 3
        y2 = torch.empty_like(x)
        run(mp, stream, "softmax_ij_j", sfx, (x + shift).contiguous(), y2, m, n)
        assert float((y2 - y).abs().max() / y.abs().max()) < 1e-4
    # softmax reverse: rows of gx sum to zero
    gy = torch.randn(m, n, generator=g, device="cuda", dtype=torch.float32).to(dt)
    gx = torch.empty_like(x)
    run(mp, stream, "softmax_ij_j_reverse", sfx, y, gy, gx, 0.0, m, n)
    rs = gx.float().sum(1).abs().max() / gx.float().abs().sum(1).max()
    assert float(rs) < (1e-2 if sfx == "r16" else 1e-5)
    # RMSNorm with gain 1: mean square of every output row is 1 (eps is negligible)
    ones = torch.ones(n, device="cuda", dtype=dt)
    run(mp, stream, "rmsnorm_ij_j", sfx, x, ones, 1e-6, y, None, m, n)
    ms = (y.float() ** 2).mean(1)
    assert float((ms - 1).abs().max()) < (3e-3 if sfx == "r16" else 1e-5)
    # RMSNorm reverse: gx is orthogonal to x in every row when gain = 1
    nbytes = mp.lib().mpRmsnormReverseScratchBytes(m, n, stream.ctx)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    gg = torch.empty(n, device="cuda", dtype=dt)
    run(mp, stream, "rmsnorm_ij_j_reverse", sfx, x, ones, None, gy, 1e-6, gx, gg, 0.0, scratch, m, n)
    dots = (gx.float() * x.float()).sum(1).abs().max() / (gx.float().abs() * x.float().abs()).sum(1).max()
    assert float(dots) < (2e-3 if sfx == "r16" else 1e-4)
    # ggain against a float64 column reduction of the same data (gain = 1)
    rstd = torch.rsqrt((x.double() ** 2).mean(1, keepdim=True) + 1e-6)
    ref = (gy.double() * x.double() * rstd).sum(0)
    err = float((gg.double() - ref).abs().max() / ref.abs().max())
    assert err < (1e-2 if sfx == "r16" else 1e-4)
