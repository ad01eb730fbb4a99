"""Oracle checks at the sizes the benchmark configurations name.  The units of
these operators are independent (rows, elements, (batch, head) sequences), so a
sample of units is compared with the CPU oracle exactly as a small case would
be, while the kernels run on the full-size tensors."""
import math

import numpy as np
import pytest

from util import TOL_EW, TOL_RED, assert_close, host, narrow

pytestmark = pytest.mark.gpu


def sample_rows(m, seed):
    r = np.random.default_rng(seed)
    return np.unique(np.concatenate([np.arange(0, 2048), np.arange(m - 2048, m), r.integers(0, m, 4096)]))


@pytest.mark.parametrize("sfx", ["r32", "r16"])
def test_row_reductions_at_65536_by_4096(mp, stream, orc, sfx):
    """configs[1]: softmax and RMSNorm forward + reverse over X[65536, 4096]; rows {0..2047, last 2048, 4096 random}
    against the oracle, and the gain gradient of the whole matrix against a float64 sum."""
    import torch
    m, n, eps = 65536, 4096, 1e-6
    dt = torch.float32 if sfx == "r32" else torch.float16
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(m, n, generator=g, device="cuda").to(dt); gy = torch.randn(m, n, generator=g, device="cuda").to(dt)
    gain = (1 + 0.02 * torch.randn(n, generator=g, device="cuda")).to(dt)
    y = torch.empty_like(x); gx = torch.empty_like(x); yn = torch.empty_like(x); gxn = torch.empty_like(x); gg = torch.empty_like(gain)
    scratch = torch.empty(mp.lib().mpRmsnormReverseScratchBytes(m, n, stream.ctx), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    mp.launch("softmax_ij_j", dt, x, y, m, n, stream)
    mp.launch("softmax_ij_j_reverse", dt, y, gy, gx, 0.0, m, n, stream)
    mp.launch("rmsnorm_ij_j", dt, x, gain, eps, yn, None, m, n, stream)
    mp.launch("rmsnorm_ij_j_reverse", dt, x, gain, None, gy, eps, gxn, gg, 0.0, scratch, m, n, stream)
    stream.sync()
    assert stream.status() == 0
    rows = torch.from_numpy(sample_rows(m, 5)).cuda()
    f64 = lambda t: np.ascontiguousarray(host(t[rows]).astype(np.float64))
    xs, gys, ys = f64(x), f64(gy), f64(y)
    gain64 = host(gain).astype(np.float64)
    tol = TOL_RED[sfx]
    assert_close(host(y[rows]), narrow(orc.softmax_ij_j(xs), sfx), tol, f"softmax {sfx}")
    assert_close(host(gx[rows]), narrow(orc.softmax_ij_j_reverse(ys, gys), sfx), tol, f"softmax reverse {sfx}")
    assert_close(host(yn[rows]), narrow(orc.rmsnorm_ij_j(xs, gain64, eps)[0], sfx), tol, f"rmsnorm {sfx}")
    rgx, _ = orc.rmsnorm_ij_j_reverse(xs, gain64, gys, eps)
    assert_close(host(gxn[rows]), narrow(rgx, sfx), tol, f"rmsnorm reverse gx {sfx}")
    # full-matrix gain gradient: sum_i gy_ij x_ij rstd_i in float64 on the device (torch used as a calculator only)
    x64, gy64 = x.double(), gy.double()
    rstd = torch.rsqrt((x64 * x64).mean(dim=1, keepdim=True) + eps)
    want = (gy64 * x64 * rstd).sum(dim=0)
    assert_close(host(gg), narrow(host(want), sfx), tol, f"rmsnorm reverse ggain {sfx}")


def test_fused_chain_at_2p28(mp, stream, orc):
    """configs[2]: e = selu((a+b)*(c+d)) and its reverse over 2^28 r32 elements; three index ranges against the
    oracle's unfused composition, forward at 1e-5 and every leaf gradient at 1e-5."""
    import torch
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(0)
    leaves = [torch.rand(n, generator=g, device="cuda") * 2 - 1 for _ in range(4)]
    ge = torch.randn(n, generator=g, device="cuda")
    out = torch.empty(n, device="cuda"); grads = [torch.empty(n, device="cuda") for _ in range(4)]
    chain = mp.FusedChain("selu((a+b)*(c+d))", torch.float32)
    torch.cuda.synchronize()
    chain.forward(leaves, out, n, stream)
    chain.reverse(leaves, ge, grads, 0.0, n, stream)
    stream.sync()
    assert stream.status() == 0
    for lo in (0, (1 << 27) - 70001, n - (1 << 17)):
        hi = lo + (1 << 17)
        a, b, c, d = [np.ascontiguousarray(host(t[lo:hi])) for t in leaves]
        gs = np.ascontiguousarray(host(ge[lo:hi]))
        t1 = orc.addition(a, b); t2 = orc.addition(c, d); t3 = orc.hadamard(t1, t2)
        assert_close(host(out[lo:hi]), orc.selu(t3), TOL_EW["r32"], f"chain forward [{lo}, {hi})")
        g3 = np.zeros_like(t3); orc.selu_reverse(t3, g3, gs)
        g1 = np.zeros_like(t3); g2 = np.zeros_like(t3)
        orc.hadamard_reverse(g3, t2, g1); orc.hadamard_reverse(g3, t1, g2)
        for i, want in enumerate((g1, g1, g2, g2)):
            assert_close(host(grads[i][lo:hi]), want, TOL_EW["r32"], f"chain reverse leaf {i} [{lo}, {hi})")
    chain.close()


def test_ssd_scan_batch8_seqlen8192(mp, stream, orc):
    """configs[3]: batch 8, seqlen 8192, 32 heads, headdim 64, d_state 128, chunk 256.  y, gx and gdt of two
    (batch, head) pairs against the float64 sequential recurrence of exactly those sequences; gB / gC (summed over
    the 32 heads) and gA need every head, so batch 5 alone is run through the oracle for them."""
    import torch
    nb, L, H, P, N, G, Q = 8, 8192, 32, 64, 128, 1, 256
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(nb, L, H, P, generator=g, device="cuda").half()
    Bm = torch.randn(nb, L, G, N, generator=g, device="cuda").half(); Cm = torch.randn(nb, L, G, N, generator=g, device="cuda").half()
    dtv = torch.nn.functional.softplus(torch.randn(nb, L, H, generator=g, device="cuda") - 4)
    Av = -torch.exp(torch.rand(H, generator=g, device="cuda") * math.log(16))
    gy = torch.randn(nb, L, H, P, generator=g, device="cuda").half()
    y = torch.empty_like(x); gx = torch.empty_like(x); gdt = torch.empty_like(dtv); gA = torch.empty_like(Av)
    gB = torch.empty_like(Bm); gC = torch.empty_like(Cm)
    dims = (nb, L, H, P, N, G, Q)
    lib = mp.lib()
    scr = torch.empty(max(lib.mpSsdScanScratchBytes(*dims, 0), lib.mpSsdScanScratchBytes(*dims, 1)), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    mp.launch("ssd_scan", torch.float16, x, dtv, Av, Bm, Cm, y, scr, *dims, stream)
    mp.launch("ssd_scan_reverse", torch.float16, x, dtv, Av, Bm, Cm, gy, gx, gdt, gA, gB, gC, scr, *dims, stream)
    stream.sync()
    assert stream.status() == 0
    f64 = lambda t: np.ascontiguousarray(host(t).astype(np.float64))
    for b, h in ((0, 0), (7, 31)):
        xs, gys = f64(x[b:b + 1, :, h:h + 1]), f64(gy[b:b + 1, :, h:h + 1])
        dts, As = f64(dtv[b:b + 1, :, h:h + 1]), f64(Av[h:h + 1])
        Bs, Cs = f64(Bm[b:b + 1]), f64(Cm[b:b + 1])
        ry = orc.ssd_forward(xs, dts, As, Bs, Cs)
        assert_close(host(y[b:b + 1, :, h:h + 1]), ry.astype(np.float16), 1e-2, f"y ({b}, {h})")
        rgx, rgdt, _, _, _ = orc.ssd_reverse(xs, dts, As, Bs, Cs, gys)
        assert_close(host(gx[b:b + 1, :, h:h + 1]), rgx.astype(np.float16), 1e-2, f"gx ({b}, {h})")
        assert_close(host(gdt[b:b + 1, :, h:h + 1]), rgdt, 1e-2, f"gdt ({b}, {h})")
    b = 5
    _, _, rgA_b, rgB, rgC = orc.ssd_reverse(f64(x[b:b + 1]), f64(dtv[b:b + 1]), f64(Av), f64(Bm[b:b + 1]), f64(Cm[b:b + 1]), f64(gy[b:b + 1]))
    assert_close(host(gB[b:b + 1]), rgB.astype(np.float16), 1e-2, "gB batch 5")
    assert_close(host(gC[b:b + 1]), rgC.astype(np.float16), 1e-2, "gC batch 5")
    # gA sums over the batch: the same launcher on batch 5 alone must reproduce the oracle's single-batch value
    gA1 = torch.empty_like(Av); gx1 = torch.empty_like(x[b:b + 1]); gdt1 = torch.empty_like(dtv[b:b + 1])
    gB1 = torch.empty_like(Bm[b:b + 1]); gC1 = torch.empty_like(Cm[b:b + 1])
    d1 = (1, L, H, P, N, G, Q)
    mp.launch("ssd_scan_reverse", torch.float16, x[b:b + 1].contiguous(), dtv[b:b + 1].contiguous(), Av, Bm[b:b + 1].contiguous(),
              Cm[b:b + 1].contiguous(), gy[b:b + 1].contiguous(), gx1, gdt1, gA1, gB1, gC1, scr, *d1, stream)
    stream.sync()
    assert_close(host(gA1), rgA_b, 1e-2, "gA batch 5")


@pytest.mark.parametrize("sfx", ["r16", "r32"])
@pytest.mark.parametrize("shape", [(16384, 768, 3352, "nn"), (16384, 1536, 768, "nn"), (16384, 768, 50280, "nt"),
                                   (768, 16384, 3352, "tn"), (1536, 16384, 768, "tn")])
def test_lm_projection_shapes_on_sampled_rows(mp, stream, orc, sfx, shape):
    """The projection shapes of the configs[4] model and the two weight-gradient contractions: sampled output rows
    against the oracle's double-accumulated triple loop."""
    import torch
    m, k, n, form = shape       # C[m, n], inner size k
    dt = torch.float32 if sfx == "r32" else torch.float16
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randn((k, m) if form == "tn" else (m, k), generator=g, device="cuda").to(dt)
    b = (torch.randn((n, k) if form == "nt" else (k, n), generator=g, device="cuda") / math.sqrt(k)).to(dt)
    c = torch.empty(m, n, device="cuda", dtype=dt)
    name = {"nn": "inner_product_ij_jk_ik", "nt": "inner_product_ij_kj_ik", "tn": "inner_product_ji_jk_ik"}[form]
    torch.cuda.synchronize()
    mp.launch(name, dt, a, b, 1.0, c, 0.0, m, k, n, stream)
    stream.sync()
    assert stream.status() == 0
    # 256 sampled rows; 32 where a row of the oracle's triple loop costs more than 5 M multiply-adds
    q = 64 if k * n <= 5_000_000 else 8
    rows = np.unique(np.concatenate([np.arange(0, q), np.arange(m - q, m), np.random.default_rng(1).integers(0, m, 2 * q)]))
    ridx = torch.from_numpy(rows).cuda()
    w64 = lambda t: np.ascontiguousarray(host(t).astype(np.float64) if sfx == "r16" else host(t))
    a_rows = w64(a[:, ridx].t().contiguous() if form == "tn" else a[ridx])
    want = orc.inner_product(a_rows, w64(b), tb=(form == "nt"))
    assert_close(host(c[ridx]), narrow(want, sfx), TOL_RED[sfx], f"{name} {sfx} {shape}")
