"""Fused element-wise chains: code generation (CPU) and GPU parity against the
unfused composition of oracle ops, which is how the reference evaluates the same
expression (one kernel per op, src/ops/*.zig)."""
import ctypes as C
import shutil
import subprocess

import numpy as np
import pytest

from util import TOL_EW, assert_close, dev, host, narrow, rng_uniform, torch_dtype, wide

CHAIN = "selu((a+b)*(c+d))"


def generated_source(mp, expr, key):
    lib = mp.lib()
    p = lib.mpJitGenerateSource(expr.encode(), key)
    if not p:
        return None
    src = C.string_at(p).decode()
    lib.mpJitFreeSource(p)
    return src


def test_generated_source_compiles_for_sm_100a(mp, tmp_path):
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not on PATH")
    for key in (0, 1, 2):
        src = generated_source(mp, CHAIN, key)
        assert src and "mp_jit_fwd_vec" in src and "mp_jit_rev_vec" in src
        f = tmp_path / f"chain_{key}.cu"
        f.write_text(src)
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-cubin", "-o",
                        str(tmp_path / f"chain_{key}.cubin"), str(f)], check=True, capture_output=True)


def test_leaf_order_and_parse_errors(mp):
    src = generated_source(mp, "x*y + relu(-x) - 2.5*z", 1)
    assert src is not None and "const T* l2" in src and "const T* l3" not in src   # x, y, z
    assert generated_source(mp, "a +* b", 1) is None
    assert generated_source(mp, "tanh(a)", 1) is None
    assert generated_source(mp, "(a+b", 1) is None
    assert generated_source(mp, "3.0", 1) is None    # no tensor operand


def oracle_chain(orc, a, b, c, d):
    """e = selu((a+b)*(c+d)) and its reverse as the reference's op layer composes
    it: addition, addition, hadamard, selu; reverse = selu_reverse,
    hadamard_reverse x2, in-place addition x4 (addition.zig:60-82, hadamard.zig:58-80)."""
    s1 = orc.addition(a, b); s2 = orc.addition(c, d)
    p = orc.hadamard(s1, s2)
    return s1, s2, p, orc.selu(p)


def oracle_chain_reverse(orc, a, b, c, d, ge):
    s1, s2, p, e = oracle_chain(orc, a, b, c, d)
    gp = orc.selu_reverse(p, np.zeros_like(p), ge)
    gs1 = orc.hadamard_reverse(gp, s2, np.zeros_like(p))
    gs2 = orc.hadamard_reverse(gp, s1, np.zeros_like(p))
    ga = orc.addition(gs1, np.zeros_like(p)); gb = orc.addition(gs1, np.zeros_like(p))
    gc = orc.addition(gs2, np.zeros_like(p)); gd = orc.addition(gs2, np.zeros_like(p))
    return ga, gb, gc, gd


@pytest.mark.gpu
@pytest.mark.parametrize("sfx", ["r16", "r32", "r64"])
@pytest.mark.parametrize("n", [1, 31, 4097, (1 << 20) + 3])
def test_fused_chain_forward_and_reverse(mp, stream, orc, sfx, n):
    import torch
    leaves = [rng_uniform(s, n, sfx) for s in range(4)]
    chain = mp.FusedChain(CHAIN, torch_dtype(sfx))
    assert chain.leaves == ["a", "b", "c", "d"]
    dl = [dev(x) for x in leaves]
    out = dev(np.full(n, np.nan, leaves[0].dtype))
    torch.cuda.current_stream().synchronize()
    chain.forward(dl, out, n, stream); stream.sync()
    ref = oracle_chain(orc, *[wide(x) for x in leaves])[3]
    assert_close(host(out), narrow(ref, sfx), TOL_EW[sfx], f"fused forward {sfx} n={n}")
    # reverse with an explicit upstream gradient, fresh (NaN) outputs, alpha = 0
    ge = rng_uniform(9, n, sfx)
    grads = [dev(np.full(n, np.nan, leaves[0].dtype)) for _ in range(4)]
    dge = dev(ge)
    torch.cuda.current_stream().synchronize()
    chain.reverse(dl, dge, grads, 0.0, n, stream); stream.sync()
    refs = oracle_chain_reverse(orc, *[wide(x) for x in leaves], wide(ge))
    for g, r, nm in zip(grads, refs, "abcd"):
        assert_close(host(g), narrow(r, sfx), TOL_EW[sfx] * 4, f"fused reverse g_{nm} {sfx} n={n}")
    # implicit ones seed (sum loss) accumulated into existing gradients (alpha = 1), one leaf skipped
    g0 = [rng_uniform(20 + i, n, sfx) for i in range(4)]
    grads = [dev(x) for x in g0]
    torch.cuda.current_stream().synchronize()
    chain.reverse(dl, None, [grads[0], None, grads[2], grads[3]], 1.0, n, stream); stream.sync()
    refs = oracle_chain_reverse(orc, *[wide(x) for x in leaves], np.ones(n, wide(ge).dtype))
    for i in (0, 2, 3):
        assert_close(host(grads[i]), narrow(refs[i] + wide(g0[i]), sfx), TOL_EW[sfx] * 4, f"fused reverse accumulate {i}")
    assert np.array_equal(host(grads[1]), g0[1])
    chain.close()


@pytest.mark.gpu
def test_fused_chain_at_full_size_matches_the_unfused_launchers(mp, stream):
    """2^28 elements per tensor: the fused kernels against the library's own
    unfused launch sequence (the composition the oracle pins at small sizes)."""
    import torch
    from util import run
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(0)
    a, b, c, d = (torch.rand(n, generator=g, device="cuda") * 2 - 1 for _ in range(4))
    chain = mp.FusedChain(CHAIN, torch.float32)
    e = torch.empty(n, device="cuda")
    torch.cuda.current_stream().synchronize()
    chain.forward([a, b, c, d], e, n, stream); stream.sync()
    s1 = torch.empty(n, device="cuda"); s2 = torch.empty(n, device="cuda"); p = torch.empty(n, device="cuda")
    run(mp, stream, "addition", "r32", a, b, s1, n)
    run(mp, stream, "addition", "r32", c, d, s2, n)
    run(mp, stream, "hadamard", "r32", s1, s2, p, n)
    e2 = torch.empty(n, device="cuda")
    run(mp, stream, "selu", "r32", p, e2, n)
    assert float((e - e2).abs().max()) <= 1e-5 * float(e2.abs().max())
    del e2
    ga, gb, gc, gd = (torch.empty(n, device="cuda") for _ in range(4))
    torch.cuda.current_stream().synchronize()
    chain.reverse([a, b, c, d], None, [ga, gb, gc, gd], 0.0, n, stream); stream.sync()
    gp = torch.zeros(n, device="cuda"); ones = torch.ones(n, device="cuda")
    run(mp, stream, "selu_reverse", "r32", p, gp, ones, n)
    del ones
    ref_a = gp * s2
    assert float((ga - ref_a).abs().max()) <= 4e-5 * float(ref_a.abs().max())
    assert torch.equal(ga, gb) and torch.equal(gc, gd)
    ref_c = gp * s1
    assert float((gc - ref_c).abs().max()) <= 4e-5 * float(ref_c.abs().max())
    chain.close()
