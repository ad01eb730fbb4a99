"""GPU parity of the Mamba-2 SSD chunked scan (forward and reverse, r16 storage,
fp32 accumulation) against the sequential-recurrence CPU oracle in float64.
Inputs follow the benchmark configuration's distributions: x, B, C ~ N(0,1) in
r16, dt = softplus(N(-4,1)), A = -exp(U(log 1, log 16))."""
import numpy as np
import pytest

from util import assert_close, dev, host

pytestmark = pytest.mark.gpu

TOL = 1e-2   # r16 storage


def make_inputs(seed, nb, L, H, P, N, G):
    r = np.random.default_rng(seed)
    x = r.standard_normal((nb, L, H, P)).astype(np.float16)
    Bm = r.standard_normal((nb, L, G, N)).astype(np.float16)
    Cm = r.standard_normal((nb, L, G, N)).astype(np.float16)
    dt = np.log1p(np.exp(r.standard_normal((nb, L, H)) - 4.0)).astype(np.float32)
    A = (-np.exp(r.uniform(0.0, np.log(16.0), H))).astype(np.float32)
    gy = r.standard_normal((nb, L, H, P)).astype(np.float16)
    return x, dt, A, Bm, Cm, gy


def scratch_for(mp, dims, reverse):
    import torch
    n = mp.lib().mpSsdScanScratchBytes(*dims, 1 if reverse else 0)
    return torch.empty(n, dtype=torch.uint8, device="cuda")


CASES = [  # (batch, seqlen, heads, headdim, dstate, groups, chunk)
    (2, 512, 4, 64, 128, 1, 256),
    (1, 768, 4, 64, 128, 2, 256),
    (2, 256, 2, 64, 128, 1, 128),
    (1, 512, 2, 128, 128, 1, 256),
    # more sequences than SMs (and than half of them, the reverse's share per walk): the chunk walk gives every CTA the
    # same number of chunks, so sequences are cut between CTAs and their state crosses through global memory
    (10, 384, 16, 64, 128, 1, 128),
    (5, 640, 20, 64, 128, 2, 128),
]


@pytest.mark.parametrize("dims", CASES)
def test_ssd_forward(mp, stream, orc, dims):
    import torch
    nb, L, H, P, N, G, Q = dims
    x, dt, A, Bm, Cm, _ = make_inputs(0, nb, L, H, P, N, G)
    y = dev(np.full(x.shape, np.nan, np.float16))
    scratch = scratch_for(mp, dims, False)
    args = [dev(a) for a in (x, dt, A, Bm, Cm)]
    torch.cuda.current_stream().synchronize()
    mp.launch("ssd_scan", torch.float16, *args, y, scratch, nb, L, H, P, N, G, Q, stream)
    stream.sync()
    assert stream.status() == 0
    f64 = lambda a: np.ascontiguousarray(a.astype(np.float64))
    ref = orc.ssd_forward(f64(x), f64(dt), f64(A), f64(Bm), f64(Cm))
    assert_close(host(y), ref.astype(np.float16), TOL, f"ssd forward {dims}")


@pytest.mark.parametrize("dims", CASES)
def test_ssd_reverse(mp, stream, orc, dims):
    import torch
    nb, L, H, P, N, G, Q = dims
    x, dt, A, Bm, Cm, gy = make_inputs(1, nb, L, H, P, N, G)
    gx = dev(np.full(x.shape, np.nan, np.float16)); gdt = dev(np.full(dt.shape, np.nan, np.float32))
    gA = dev(np.full(A.shape, np.nan, np.float32)); gB = dev(np.full(Bm.shape, np.nan, np.float16))
    gC = dev(np.full(Cm.shape, np.nan, np.float16))
    scratch = scratch_for(mp, dims, True)
    args = [dev(a) for a in (x, dt, A, Bm, Cm, gy)]
    torch.cuda.current_stream().synchronize()
    mp.launch("ssd_scan_reverse", torch.float16, *args, gx, gdt, gA, gB, gC, scratch, nb, L, H, P, N, G, Q, stream)
    stream.sync()
    assert stream.status() == 0
    f64 = lambda a: np.ascontiguousarray(a.astype(np.float64))
    rgx, rgdt, rgA, rgB, rgC = orc.ssd_reverse(f64(x), f64(dt), f64(A), f64(Bm), f64(Cm), f64(gy))
    assert_close(host(gx), rgx.astype(np.float16), TOL, f"gx {dims}")
    assert_close(host(gC), rgC.astype(np.float16), TOL, f"gC {dims}")
    assert_close(host(gB), rgB.astype(np.float16), TOL, f"gB {dims}")
    assert_close(host(gdt), rgdt, TOL, f"gdt {dims}")
    assert_close(host(gA), rgA, TOL, f"gA {dims}")


def test_full_length_against_the_sequential_path(mp, stream):
    """Benchmark-length sequences (seqlen 8192 = 32 chunks, 32 heads, one batch): the chunked tensor-core path
    against the sequential-recurrence kernels of the same library, forward and every gradient."""
    import os
    import torch
    dims = (1, 8192, 32, 64, 128, 1, 256)
    nb, L, H, P, N, G, Q = dims
    x, dt, A, Bm, Cm, gy = make_inputs(11, nb, L, H, P, N, G)
    args = [dev(a) for a in (x, dt, A, Bm, Cm)]
    dgy = dev(gy)
    lib = mp.lib()
    out = {}
    for path in ("tensor", "sequential"):
        if path == "sequential":
            os.environ["MP_SSD_FORCE_GENERIC"] = "1"
        try:
            n = max(lib.mpSsdScanScratchBytes(*dims, 0), lib.mpSsdScanScratchBytes(*dims, 1))
            scr = torch.empty(n, dtype=torch.uint8, device="cuda")
            y = dev(np.full(x.shape, np.nan, np.float16))
            gx = dev(np.full(x.shape, np.nan, np.float16)); gdt = dev(np.full(dt.shape, np.nan, np.float32))
            gA = dev(np.full(A.shape, np.nan, np.float32)); gB = dev(np.full(Bm.shape, np.nan, np.float16)); gC = dev(np.full(Cm.shape, np.nan, np.float16))
            torch.cuda.current_stream().synchronize()
            mp.launch("ssd_scan", torch.float16, *args, y, scr, *dims, stream)
            mp.launch("ssd_scan_reverse", torch.float16, *args, dgy, gx, gdt, gA, gB, gC, scr, *dims, stream)
            stream.sync()
            assert stream.status() == 0
            out[path] = [host(t).astype(np.float64) for t in (y, gx, gdt, gA, gB, gC)]
        finally:
            os.environ.pop("MP_SSD_FORCE_GENERIC", None)
    for got, want, name in zip(out["tensor"], out["sequential"], ("y", "gx", "gdt", "gA", "gB", "gC")):
        assert_close(got, want, 1e-2, f"full-length {name}")


@pytest.mark.parametrize("dims", [(2, 512, 4, 64, 128, 1, 256), (10, 384, 16, 64, 128, 1, 128), (1, 512, 2, 128, 128, 1, 256)])
def test_scan_from_raw_step_sizes_is_the_three_launches_in_one(mp, stream, dims):
    """launch_ssd_scan_raw (softplus of the raw step sizes and -exp(A_log) inside the scan) against launch_softplus_bias +
    launch_neg_exp + launch_ssd_scan on the same inputs: dt, A and y bit for bit (the last shape takes the composed path)."""
    import torch
    nb, L, H, P, N, G, Q = dims
    x, _, _, Bm, Cm, _ = make_inputs(5, nb, L, H, P, N, G)
    r = np.random.default_rng(6)
    pitch = H + 8
    raw = (r.standard_normal((nb * L, pitch)) - 4.0).astype(np.float16)
    bias = (0.5 * r.standard_normal(H)).astype(np.float32)
    A_log = np.log(r.uniform(1.0, 16.0, H)).astype(np.float32)
    dx, dB, dC, draw, dbias, dAlog = (dev(a) for a in (x, Bm, Cm, raw, bias, A_log))
    scratch = scratch_for(mp, dims, False)
    dt1 = dev(np.full((nb, L, H), np.nan, np.float32)); A1 = dev(np.full(H, np.nan, np.float32)); y1 = dev(np.full(x.shape, np.nan, np.float16))
    dt2 = dev(np.full((nb, L, H), np.nan, np.float32)); A2 = dev(np.full(H, np.nan, np.float32)); y2 = dev(np.full(x.shape, np.nan, np.float16))
    torch.cuda.current_stream().synchronize()
    mp.launch("softplus_bias", torch.float16, draw, pitch, dbias, dt1, nb * L, H, stream)
    mp.launch("neg_exp", torch.float32, dAlog, A1, H, stream)
    mp.launch("ssd_scan", torch.float16, dx, dt1, A1, dB, dC, y1, scratch, *dims, stream)
    mp.launch("ssd_scan_raw", torch.float16, dx, draw, pitch, dbias, dAlog, dB, dC, y2, dt2, A2, scratch, *dims, stream)
    stream.sync()
    assert stream.status() == 0
    assert np.array_equal(host(dt1), host(dt2))
    assert np.array_equal(host(A1), host(A2))
    assert np.array_equal(host(y1), host(y2))
    assert np.isfinite(host(y2).astype(np.float32)).all()


@pytest.mark.parametrize("dims", [(2, 512, 4, 64, 128, 1, 256), (10, 384, 16, 64, 128, 1, 128), (1, 512, 2, 128, 128, 1, 256)])
def test_reverse_with_the_raw_side_gradients_is_the_three_launches_in_one(mp, stream, dims):
    """launch_ssd_scan_reverse_raw against launch_ssd_scan_reverse + launch_softplus_bias_reverse + launch_hadamard_reverse:
    gx, gdt, gA, gB, gC and the raw step sizes' gradient bit for bit, the accumulated dt_bias / A_log gradients to 1e-5."""
    import torch
    nb, L, H, P, N, G, Q = dims
    x, _, _, Bm, Cm, gy = make_inputs(7, nb, L, H, P, N, G)
    r = np.random.default_rng(8)
    pitch = H + 8
    raw = (r.standard_normal((nb * L, pitch)) - 4.0).astype(np.float16)
    bias = (0.5 * r.standard_normal(H)).astype(np.float32)
    A_log = np.log(r.uniform(1.0, 16.0, H)).astype(np.float32)
    dx, dB, dC, dgy, draw, dbias, dAlog = (dev(a) for a in (x, Bm, Cm, gy, raw, bias, A_log))
    dt = dev(np.zeros((nb, L, H), np.float32)); A = dev(np.zeros(H, np.float32))
    torch.cuda.current_stream().synchronize()
    mp.launch("softplus_bias", torch.float16, draw, pitch, dbias, dt, nb * L, H, stream)
    mp.launch("neg_exp", torch.float32, dAlog, A, H, stream)
    scratch = scratch_for(mp, dims, True)
    gb0 = r.standard_normal(H).astype(np.float32); gl0 = r.standard_normal(H).astype(np.float32)
    outs = []
    for fused in (False, True):
        gx = dev(np.full(x.shape, np.nan, np.float16)); gdt = dev(np.full((nb, L, H), np.nan, np.float32)); gA = dev(np.full(H, np.nan, np.float32))
        gB = dev(np.full(Bm.shape, np.nan, np.float16)); gC = dev(np.full(Cm.shape, np.nan, np.float16))
        graw = dev(np.full((nb * L, pitch), 2, np.float16)); gbias = dev(gb0.copy()); glog = dev(gl0.copy())
        torch.cuda.current_stream().synchronize()
        if fused:
            mp.launch("ssd_scan_reverse_raw", torch.float16, dx, dt, A, dB, dC, dgy, draw, pitch, dbias, gx, gdt, gA, graw, pitch, gbias, glog,
                      gB, gC, scratch, *dims, stream)
        else:
            mp.launch("ssd_scan_reverse", torch.float16, dx, dt, A, dB, dC, dgy, gx, gdt, gA, gB, gC, scratch, *dims, stream)
            mp.launch("softplus_bias_reverse", torch.float16, draw, pitch, dbias, gdt, graw, pitch, gbias, nb * L, H, stream)
            mp.launch("hadamard_reverse", torch.float32, gA, A, glog, H, stream)
        stream.sync()
        assert stream.status() == 0
        outs.append([host(t) for t in (gx, gdt, gA, gB, gC, graw, gbias, glog)])
    for a, b, name in zip(outs[0][:6], outs[1][:6], ("gx", "gdt", "gA", "gB", "gC", "graw")):
        assert np.array_equal(a, b), name
    assert np.all(outs[1][5][:, H:] == 2)
    for a, b, name in zip(outs[0][6:], outs[1][6:], ("gdt_bias", "gA_log")):
        assert_close(b, a.astype(np.float64), 1e-5, name)
