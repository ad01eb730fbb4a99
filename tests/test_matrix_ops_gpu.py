"""GPU parity of transpose / reductions / broadcasts against the CPU oracle."""
import numpy as np
import pytest

from util import run, TOL_EW, TOL_RED, assert_close, dev, host, narrow, rng_normal, torch_dtype, wide

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (3, 2), (32, 256), (256, 256), (37, 53), (64, 65), (129, 1000), (1000, 8), (5, 4099)]
DTYPES = ["r16", "r32", "r64"]




@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_permutate_is_bit_exact_and_ignores_fresh_dst(mp, stream, orc, sfx, shape):
    row, col = shape
    s = rng_normal(1, shape, sfx)
    d = dev(np.full((col, row), np.nan, s.dtype))     # fresh output full of NaN: must not leak (alpha = 0)
    run(mp, stream, "permutate_ij_ji", sfx, dev(s), d, 0.0, row, col)
    assert np.array_equal(host(d), s.T)
    d0 = rng_normal(2, (col, row), sfx)
    d = dev(d0)
    run(mp, stream, "permutate_ij_ji", sfx, dev(s), d, 1.0, row, col)
    assert_close(host(d), narrow(orc.permutate_ij_ji(wide(s), wide(d0).copy(), 1.0), sfx), TOL_EW[sfx], "permutate alpha=1")


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", SHAPES + [(4096, 768), (70, 20000)])
def test_reductions(mp, stream, orc, sfx, shape):
    m, n = shape
    s = rng_normal(3, shape, sfx)
    for name, fn, out_len in [("reduce_ij_i", orc.reduce_ij_i, m), ("reduce_ij_j", orc.reduce_ij_j, n)]:
        d = dev(np.full(out_len, np.nan, s.dtype))
        run(mp, stream, name, sfx, dev(s), d, 0.0, m, n)
        assert_close(host(d), narrow(fn(wide(s)), sfx), TOL_RED[sfx], f"{name} alpha=0 {shape}")
        d0 = rng_normal(4, out_len, sfx)
        d = dev(d0)
        run(mp, stream, name, sfx, dev(s), d, 1.0, m, n)
        assert_close(host(d), narrow(fn(wide(s), wide(d0).copy(), 1.0), sfx), TOL_RED[sfx], f"{name} alpha=1 {shape}")


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_broadcasts(mp, stream, orc, sfx, shape):
    m, n = shape
    for name, fn, src_len in [("broadcast_i_ij", orc.broadcast_i_ij, m), ("broadcast_j_ij", orc.broadcast_j_ij, n)]:
        src = rng_normal(5, src_len, sfx)
        d = dev(np.full(shape, np.nan, src.dtype))
        run(mp, stream, name, sfx, dev(src), d, 0.0, m, n)
        assert np.array_equal(host(d), narrow(fn(wide(src), np.empty(shape, wide(src).dtype)), sfx)), name
        d0 = rng_normal(6, shape, sfx)
        d = dev(d0)
        run(mp, stream, name, sfx, dev(src), d, 1.0, m, n)
        assert_close(host(d), narrow(fn(wide(src), wide(d0).copy(), 1.0), sfx), TOL_EW[sfx], f"{name} alpha=1")


def test_reverse_pairs_used_by_the_host_layer(mp, stream, orc):
    # reduce.zig:123-138: reverse of "ij->i" is broadcast_i_ij(g_y, g_x, alpha=1) into a zeroed gradient
    m, n = 48, 100
    gy = rng_normal(7, m, "r32")
    gx = dev(np.zeros((m, n), np.float32))
    run(mp, stream, "broadcast_i_ij", "r32", dev(gy), gx, 1.0, m, n)
    assert np.array_equal(host(gx), np.broadcast_to(gy[:, None], (m, n)))
