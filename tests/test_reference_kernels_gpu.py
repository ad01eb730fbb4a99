"""Runs the reference's own kernels (compiled unmodified for sm_100a) on the
GPU and checks, on identical seeded inputs, (1) the CPU oracle against them -
this is what pins the oracle - and (2) this library against them.  Only the
cases where the reference kernel is valid are compared: element counts below
2^27 for accumulate kernels, alpha = 0 for the blend kernels whose alpha = 1
path is wrong or racy (reduce_ij_j, broadcast_i_ij)."""
import numpy as np
import pytest

from util import run, TOL_EW, TOL_RED, assert_close, dev, host, narrow, rng_normal, torch_dtype, wide

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(stream):
    from refkernels import RefLib
    r = RefLib()
    yield r
    r.close()


def ours(mp, stream, name, sfx, *args):
    run(mp, stream, name, sfx, *args)


# r16 reference arithmetic is native half (and half-accumulated in reductions):
# compare it at the r16 tolerance only.
@pytest.mark.parametrize("sfx", ["r16", "r32", "r64"])
@pytest.mark.parametrize("n", [1, 31, 4097, (1 << 20) + 3])
def test_elementwise_reference_vs_oracle_vs_ours(mp, stream, orc, ref, sfx, n):
    a = rng_normal(1, n, sfx); b = rng_normal(2, n, sfx); c = rng_normal(3, n, sfx)
    tol = TOL_EW[sfx]
    cases = [
        ("addition", lambda L, out: L("addition", sfx, dev(a), dev(b), out, n), lambda: orc.addition(wide(a), wide(b)), None),
        ("subtraction", lambda L, out: L("subtraction", sfx, dev(a), dev(b), out, n), lambda: orc.subtraction(wide(a), wide(b)), None),
        ("hadamard", lambda L, out: L("hadamard", sfx, dev(a), dev(b), out, n), lambda: orc.hadamard(wide(a), wide(b)), None),
        ("hadamard_reverse", lambda L, out: L("hadamard_reverse", sfx, dev(a), dev(b), out, n),
         lambda: orc.hadamard_reverse(wide(a), wide(b), wide(c).copy()), c),
        ("negate", lambda L, out: L("negate", sfx, dev(a), out, n), lambda: orc.negate(wide(a)), None),
        ("translate", lambda L, out: L("translate", sfx, dev(a), 0.75, out, n), lambda: orc.translate(wide(a), 0.75), None),
        ("dilate", lambda L, out: L("dilate", sfx, dev(a), 0.75, out, n), lambda: orc.dilate(wide(a), 0.75), None),
        ("dilate_reverse", lambda L, out: L("dilate_reverse", sfx, dev(a), 0.75, out, n),
         lambda: orc.dilate_reverse(wide(a), 0.75, wide(c).copy()), c),
        ("relu", lambda L, out: L("relu", sfx, dev(a), out, n), lambda: orc.relu(wide(a)), None),
        ("relu_reverse", lambda L, out: L("relu_reverse", sfx, dev(a), out, dev(b), n),
         lambda: orc.relu_reverse(wide(a), wide(c).copy(), wide(b)), c),
        ("copy", lambda L, out: L("copy", sfx, dev(a), out, n), lambda: orc.copy(wide(a)), None),
        ("fill", lambda L, out: L("fill", sfx, out, 1.25, n), lambda: orc.fill(np.empty(n, wide(a).dtype), 1.25), None),
    ]
    for name, call, oracle, init in cases:
        start = init if init is not None else np.zeros(n, a.dtype)
        out_ref = dev(start); out_ours = dev(start)
        call(ref.launch, out_ref)
        call(lambda nm, s, *args: ours(mp, stream, nm, s, *args), out_ours)
        want = narrow(oracle(), sfx)
        assert_close(want, host(out_ref), tol, f"oracle vs reference kernel: {name} {sfx} n={n}")
        assert_close(host(out_ours), host(out_ref), tol, f"ours vs reference kernel: {name} {sfx} n={n}")


@pytest.mark.parametrize("sfx", ["r32", "r64"])
def test_sequence_reference_vs_oracle_vs_ours(mp, stream, orc, ref, sfx):
    n = 5000
    npdt = np.float32 if sfx == "r32" else np.float64
    o_ref = dev(np.zeros(n, npdt)); o_ours = dev(np.zeros(n, npdt))
    ref.launch("sequence", sfx, o_ref, 1.0, 0.5, n)
    ours(mp, stream, "sequence", sfx, o_ours, 1.0, 0.5, n)
    want = orc.sequence(np.empty(n, npdt), 1.0, 0.5)
    assert_close(want, host(o_ref), TOL_EW[sfx], "oracle vs reference sequence")
    assert_close(host(o_ours), host(o_ref), TOL_EW[sfx], "ours vs reference sequence")


@pytest.mark.parametrize("sfx", ["r16", "r32", "r64"])
@pytest.mark.parametrize("shape", [(3, 2), (32, 256), (256, 256), (37, 53), (129, 1000)])
def test_rank2_reference_vs_oracle_vs_ours(mp, stream, orc, ref, sfx, shape):
    m, n = shape
    s = rng_normal(4, shape, sfx)
    # transpose, alpha = 0 into a zeroed destination (the reference reads dst: 0*garbage hazard)
    o_ref = dev(np.zeros((n, m), s.dtype)); o_ours = dev(np.zeros((n, m), s.dtype))
    ref.launch("permutate_ij_ji", sfx, dev(s), o_ref, 0.0, m, n)
    ours(mp, stream, "permutate_ij_ji", sfx, dev(s), o_ours, 0.0, m, n)
    assert np.array_equal(host(o_ref), orc.permutate_ij_ji(wide(s)).astype(s.dtype))
    assert np.array_equal(host(o_ours), host(o_ref))
    # row sums (alpha 0 and 1 are both valid in the reference)
    for alpha in (0.0, 1.0):
        d0 = rng_normal(5, m, sfx) if alpha else np.zeros(m, s.dtype)
        o_ref = dev(d0); o_ours = dev(d0)
        ref.launch("reduce_ij_i", sfx, dev(s), o_ref, alpha, m, n)
        ours(mp, stream, "reduce_ij_i", sfx, dev(s), o_ours, alpha, m, n)
        want = narrow(orc.reduce_ij_i(wide(s), wide(d0).copy(), alpha), sfx)
        assert_close(want, host(o_ref), TOL_RED[sfx], f"oracle vs reference reduce_ij_i alpha={alpha}")
        assert_close(host(o_ours), host(o_ref), TOL_RED[sfx], f"ours vs reference reduce_ij_i alpha={alpha}")
    # column sums: reference valid for alpha = 0 and m >= n only
    if m >= n:
        o_ref = dev(np.zeros(n, s.dtype)); o_ours = dev(np.zeros(n, s.dtype))
        ref.launch("reduce_ij_j", sfx, dev(s), o_ref, 0.0, m, n)
        ours(mp, stream, "reduce_ij_j", sfx, dev(s), o_ours, 0.0, m, n)
        assert_close(narrow(orc.reduce_ij_j(wide(s)), sfx), host(o_ref), TOL_RED[sfx], "oracle vs reference reduce_ij_j")
        assert_close(host(o_ours), host(o_ref), TOL_RED[sfx], "ours vs reference reduce_ij_j")
    # broadcasts
    vj = rng_normal(6, n, sfx); vi = rng_normal(7, m, sfx)
    for alpha in (0.0, 1.0):
        d0 = rng_normal(8, shape, sfx) if alpha else np.zeros(shape, s.dtype)
        o_ref = dev(d0); o_ours = dev(d0)
        ref.launch("broadcast_j_ij", sfx, dev(vj), o_ref, alpha, m, n)
        ours(mp, stream, "broadcast_j_ij", sfx, dev(vj), o_ours, alpha, m, n)
        want = narrow(orc.broadcast_j_ij(wide(vj), wide(d0).copy(), alpha), sfx)
        assert_close(want, host(o_ref), TOL_EW[sfx], f"oracle vs reference broadcast_j_ij alpha={alpha}")
        assert_close(host(o_ours), host(o_ref), TOL_EW[sfx], f"ours vs reference broadcast_j_ij alpha={alpha}")
    o_ref = dev(np.zeros(shape, s.dtype)); o_ours = dev(np.zeros(shape, s.dtype))
    ref.launch("broadcast_i_ij", sfx, dev(vi), o_ref, 0.0, m, n)
    ours(mp, stream, "broadcast_i_ij", sfx, dev(vi), o_ours, 0.0, m, n)
    assert np.array_equal(host(o_ref), np.broadcast_to(vi[:, None], shape))
    assert np.array_equal(host(o_ours), host(o_ref))


# The reference's contraction launcher (cuBLAS H/S/Dgemm behind launch_inner_product_ij_jk_ik,
# src/cuda/nvcc_src/inner_product_ij_jk_ik.cu:12-26 and gemm_dispatch.cuh:24,59,95): the oracle's triple loop
# against it, and this library against it.  r16: the reference computes and accumulates in fp16, so it is
# compared at the r16 tolerance; ours is additionally held to the fp64 oracle.
@pytest.mark.parametrize("sfx", ["r16", "r32", "r64"])
@pytest.mark.parametrize("shape", [(32, 256, 256), (128, 128, 128), (37, 53, 29), (256, 768, 512)])
@pytest.mark.parametrize("alpha_beta", [(1.0, 0.0), (0.5, 1.0)])
def test_inner_product_reference_vs_oracle_vs_ours(mp, stream, orc, ref, sfx, shape, alpha_beta):
    m, n, k = shape      # a [m, n], b [n, k], c [m, k] (the reference's argument order)
    alpha, beta = alpha_beta
    a = rng_normal(21, (m, n), sfx); b = rng_normal(22, (n, k), sfx, scale=1.0 / np.sqrt(n))
    c0 = rng_normal(23, (m, k), sfx) if beta else np.zeros((m, k), a.dtype)
    o_ref = dev(c0); o_ours = dev(c0)
    ref.launch("inner_product_ij_jk_ik", sfx, dev(a), dev(b), alpha, o_ref, beta, m, n, k)
    ours(mp, stream, "inner_product_ij_jk_ik", sfx, dev(a), dev(b), alpha, o_ours, beta, m, n, k)
    want = narrow(orc.inner_product(wide(a), wide(b), alpha, wide(c0).copy(), beta), sfx)
    tol = TOL_RED[sfx]
    assert_close(want, host(o_ref), tol, f"oracle vs reference inner_product {sfx} {shape} alpha,beta={alpha_beta}")
    assert_close(host(o_ours), host(o_ref), tol, f"ours vs reference inner_product {sfx} {shape} alpha,beta={alpha_beta}")
    assert_close(host(o_ours), want, tol, f"ours vs oracle inner_product {sfx} {shape} alpha,beta={alpha_beta}")
