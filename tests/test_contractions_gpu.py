"""GPU parity of the einsum contractions (inner_product NN / NT / TN, linear)
against the fp64-accumulating CPU oracle, through the C ABI."""
import numpy as np
import pytest

from util import TOL_RED, assert_close, dev, host, narrow, rng_normal, run, wide

pytestmark = pytest.mark.gpu

# (m, n, k) in the reference's naming: C[m,k] = A[m,n] * B[n,k]
SHAPES = [(3, 2, 2), (32, 256, 256), (128, 64, 128), (129, 72, 200), (256, 384, 512), (100, 1000, 24), (1, 8, 8),
          (300, 40, 264), (64, 2048, 64), (5, 7, 3)]
DTYPES = ["r16", "r32", "r64"]
VARIANTS = [("inner_product_ij_jk_ik", False, False), ("inner_product_ij_kj_ik", False, True),
            ("inner_product_ji_jk_ik", True, False)]


def operands(sfx, m, n, k, ta, tb, seed=0):
    a = rng_normal(seed, (n, m) if ta else (m, n), sfx, scale=1.0)
    b = rng_normal(seed + 1, (k, n) if tb else (n, k), sfx, scale=1.0 / np.sqrt(n))
    return a, b


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("variant", VARIANTS, ids=[v[0][-8:] for v in VARIANTS])
def test_inner_product_variants(mp, stream, orc, sfx, shape, variant):
    name, ta, tb = variant
    m, n, k = shape
    a, b = operands(sfx, m, n, k, ta, tb)
    c = dev(np.full((m, k), np.nan, a.dtype))           # fresh output: beta = 0 must not read it
    run(mp, stream, name, sfx, dev(a), dev(b), 1.0, c, 0.0, m, n, k)
    ref = orc.inner_product(wide(a), wide(b), ta=ta, tb=tb)
    assert_close(host(c), narrow(ref, sfx), TOL_RED[sfx], f"{name} {sfx} {shape}")
    # accumulate form used by the reverse pass: alpha = scale, beta = 1 (inner_product.zig:275-301)
    c0 = rng_normal(7, (m, k), sfx)
    c = dev(c0)
    run(mp, stream, name, sfx, dev(a), dev(b), 0.5, c, 1.0, m, n, k)
    ref = orc.inner_product(wide(a), wide(b), 0.5, wide(c0).copy(), 1.0, ta=ta, tb=tb)
    assert_close(host(c), narrow(ref, sfx), TOL_RED[sfx], f"{name} accumulate {sfx} {shape}")
    assert stream.status() == 0


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", [(32, 256, 256), (129, 72, 200), (5, 7, 3)])
def test_linear_adds_bias_in_the_epilogue(mp, stream, orc, sfx, shape):
    m, n, k = shape
    a, b = operands(sfx, m, n, k, False, False, seed=3)
    bias = rng_normal(9, k, sfx)
    c = dev(np.full((m, k), np.nan, a.dtype))
    run(mp, stream, "linear_ij_jk_ik", sfx, dev(a), dev(b), dev(bias), 1.0, c, 0.0, m, n, k)
    ref = orc.inner_product(wide(a), wide(b), bias=wide(bias))
    assert_close(host(c), narrow(ref, sfx), TOL_RED[sfx], f"linear {sfx} {shape}")


# The residual form "ij,jk,ik->ik": a full [m, k] term added in the epilogue.  Shapes reach the FP-pipe kernel, the
# single-CTA tensor kernel, the CTA-pair kernel (>= 74 tiles of 256 x 256, ragged last column tile) and the split-K fold.
@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", [(5, 7, 3), (129, 72, 200), (300, 40, 264), (2560, 64, 1992), (256, 4096, 512)])
def test_linear_with_a_full_matrix_term(mp, stream, orc, sfx, shape):
    m, n, k = shape
    a, b = operands(sfx, m, n, k, False, False, seed=5)
    r = rng_normal(11, (m, k), sfx)
    c = dev(np.full((m, k), np.nan, a.dtype))
    run(mp, stream, "linear_ij_jk_ik_ik", sfx, dev(a), dev(b), dev(r), 0.5, c, 0.0, m, n, k)
    ref = orc.inner_product(wide(a), wide(b), 0.5) + wide(r)
    assert_close(host(c), narrow(ref, sfx), TOL_RED[sfx], f"linear + matrix {sfx} {shape}")
    # in place on the residual stream: r is also the output
    rc = dev(r.copy())
    run(mp, stream, "linear_ij_jk_ik_ik", sfx, dev(a), dev(b), rc, 0.5, rc, 0.0, m, n, k)
    assert_close(host(rc), narrow(ref, sfx), TOL_RED[sfx], f"linear + matrix in place {sfx} {shape}")
    assert stream.status() == 0


BATCHED = [("inner_product_bij_bjk_bik", False, False), ("inner_product_bij_bkj_bik", False, True),
           ("inner_product_bji_bjk_bik", True, False)]
# (batch, m, n, k): tiles cut at the edges of every batch entry, one entry, odd pitches (FP-pipe kernel), deep n
BATCHED_SHAPES = [(3, 129, 72, 200), (1, 64, 64, 64), (5, 7, 3, 5), (16, 128, 64, 128), (4, 100, 1000, 24), (2, 300, 40, 264),
                  (6, 33, 8, 8)]


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("shape", BATCHED_SHAPES)
@pytest.mark.parametrize("variant", BATCHED, ids=[v[0][-11:] for v in BATCHED])
def test_batched_inner_product_variants(mp, stream, orc, sfx, shape, variant):
    name, ta, tb = variant
    nb, m, n, k = shape
    a = rng_normal(20, (nb, n, m) if ta else (nb, m, n), sfx)
    b = rng_normal(21, (nb, k, n) if tb else (nb, n, k), sfx, scale=1.0 / np.sqrt(n))
    c = dev(np.full((nb, m, k), np.nan, a.dtype))        # beta = 0 must not read the fresh output
    run(mp, stream, name, sfx, dev(a), dev(b), 1.0, c, 0.0, nb, m, n, k)
    ref = orc.inner_product_batched(wide(a), wide(b), ta=ta, tb=tb)
    assert_close(host(c), narrow(ref, sfx), TOL_RED[sfx], f"{name} {sfx} {shape}")
    c0 = rng_normal(22, (nb, m, k), sfx)
    c = dev(c0)
    run(mp, stream, name, sfx, dev(a), dev(b), 0.5, c, 1.0, nb, m, n, k)
    ref = orc.inner_product_batched(wide(a), wide(b), 0.5, wide(c0).copy(), 1.0, ta=ta, tb=tb)
    assert_close(host(c), narrow(ref, sfx), TOL_RED[sfx], f"{name} accumulate {sfx} {shape}")
    assert stream.status() == 0


@pytest.mark.parametrize("sfx", ["r16", "r32"])
def test_batched_entries_equal_the_rank2_contraction(mp, stream, sfx):
    # every batch entry is bit-identical to the rank-2 launcher run on that entry alone (same kernel, same tile walk),
    # at a size the oracle does not reach
    import torch
    nb, m, n, k = 12, 512, 256, 384
    dt = {"r16": torch.float16, "r32": torch.float32}[sfx]
    a = torch.randn(nb, m, n, device="cuda").to(dt); b = (torch.randn(nb, n, k, device="cuda") / 16).to(dt)
    c = torch.empty(nb, m, k, device="cuda", dtype=dt); c1 = torch.empty(m, k, device="cuda", dtype=dt)
    run(mp, stream, "inner_product_bij_bjk_bik", sfx, a, b, 1.0, c, 0.0, nb, m, n, k)
    for q in (0, 5, 11):
        run(mp, stream, "inner_product_ij_jk_ik", sfx, a[q], b[q], 1.0, c1, 0.0, m, n, k)
        assert torch.equal(c[q], c1)


def test_experimental_example_through_the_abi(mp, stream):
    # src/examples/experimental.zig: x = sequence(1,1)[3,2], y = sequence(1,1)[2,2]; z = x.y; reverse with seed 1
    import torch
    x = torch.empty(3, 2, device="cuda"); y = torch.empty(2, 2, device="cuda")
    run(mp, stream, "sequence", "r32", x, 1.0, 1.0, 6)
    run(mp, stream, "sequence", "r32", y, 1.0, 1.0, 4)
    z = torch.empty(3, 2, device="cuda")
    run(mp, stream, "inner_product_ij_jk_ik", "r32", x, y, 1.0, z, 0.0, 3, 2, 2)
    assert z.cpu().tolist() == [[7, 10], [15, 22], [23, 34]]
    gz = torch.empty_like(z); gx = torch.zeros_like(x); gy = torch.zeros_like(y)
    run(mp, stream, "fill", "r32", gz, 1.0, 6)
    run(mp, stream, "inner_product_ij_kj_ik", "r32", gz, y, 1.0, gx, 1.0, 3, 2, 2)   # dx = G . y^T
    run(mp, stream, "inner_product_ji_jk_ik", "r32", x, gz, 1.0, gy, 1.0, 2, 3, 2)   # dy = x^T . G
    assert gx.cpu().tolist() == [[3, 7], [3, 7], [3, 7]]
    assert gy.cpu().tolist() == [[9, 9], [12, 12]]


@pytest.mark.parametrize("sfx", ["r16", "r32"])
def test_large_shape_against_float64_matmul(mp, stream, sfx):
    """A projection-sized contraction (4096 x 768 x 3352): checked against a
    float64 matmul on the GPU instead of the scalar oracle."""
    import torch
    from util import torch_dtype
    m, n, k = 4096, 768, 3352
    g = torch.Generator(device="cuda").manual_seed(0)
    dt = torch_dtype(sfx)
    a = torch.randn(m, n, generator=g, device="cuda").to(dt)
    b = (torch.randn(n, k, generator=g, device="cuda") / n ** 0.5).to(dt)
    c = torch.empty(m, k, device="cuda", dtype=dt)
    run(mp, stream, "inner_product_ij_jk_ik", sfx, a, b, 1.0, c, 0.0, m, n, k)
    ref = a.double() @ b.double()
    err = float((c.double() - ref).abs().max() / ref.abs().max())
    assert err <= TOL_RED[sfx], err
    assert stream.status() == 0
