"""Sequential-recurrence SSD path (r32, r64, and r16 shapes outside the tensor-core path) against the float64
oracle: forward and every gradient, odd sizes included (headdim not a power of two, ragged last block,
several groups)."""
import numpy as np
import pytest

from util import NP_OF, assert_close, dev, host, run

pytestmark = pytest.mark.gpu

CASES = [  # (batch, seqlen, heads, headdim, dstate, groups)
    (2, 70, 4, 8, 16, 2),
    (1, 130, 3, 5, 7, 1),
    (1, 64, 2, 64, 128, 1),
    (2, 33, 2, 24, 40, 2),
]
TOL = {"r16": 1e-2, "r32": 1e-4, "r64": 1e-10}
KEY = {"r16": 0, "r32": 1, "r64": 2}


def make(seed, nb, L, H, P, N, G, sfx):
    r = np.random.default_rng(seed)
    st = NP_OF[sfx]
    acc = np.float64 if sfx == "r64" else np.float32
    x = r.standard_normal((nb, L, H, P)).astype(st)
    Bm = r.standard_normal((nb, L, G, N)).astype(st)
    Cm = r.standard_normal((nb, L, G, N)).astype(st)
    dt = np.log1p(np.exp(r.standard_normal((nb, L, H)) - 2.0)).astype(acc)
    A = (-np.exp(r.uniform(0.0, np.log(8.0), H))).astype(acc)
    gy = r.standard_normal((nb, L, H, P)).astype(st)
    return x, dt, A, Bm, Cm, gy


@pytest.mark.parametrize("sfx", ["r16", "r32", "r64"])
@pytest.mark.parametrize("dims", CASES)
def test_generic_scan_forward_and_reverse(mp, stream, orc, sfx, dims):
    import torch
    nb, L, H, P, N, G = dims
    x, dt, A, Bm, Cm, gy = make(3, *dims, sfx)
    chunk = 64   # r16: (L % chunk != 0 or N != 128 or P not in (64, 128)) selects the sequential path
    if sfx == "r16" and (N == 128 and P in (64, 128) and L % chunk == 0):
        chunk = 48   # force the sequential path for the one shape the tensor cores could take
    w = [a.astype(np.float64) for a in (x, dt, A, Bm, Cm, gy)]
    ref_y = orc.ssd_forward(*w[:5])
    ref = orc.ssd_reverse(*w)
    acc = np.float64 if sfx == "r64" else np.float32
    y = dev(np.full(x.shape, np.nan, NP_OF[sfx]))
    lib = mp.lib()
    nfwd = lib.mpSsdScanScratchBytes(nb, L, H, P, N, G, chunk, 0) if sfx == "r16" else lib.mpSsdScanGenericScratchBytes(KEY[sfx], nb, L, H, P, N, G, 0)
    nrev = lib.mpSsdScanScratchBytes(nb, L, H, P, N, G, chunk, 1) if sfx == "r16" else lib.mpSsdScanGenericScratchBytes(KEY[sfx], nb, L, H, P, N, G, 1)
    scr = torch.empty(max(nfwd, nrev), dtype=torch.uint8, device="cuda")
    args = [dev(a) for a in (x, dt, A, Bm, Cm)]
    run(mp, stream, "ssd_scan", sfx, *args, y, scr, nb, L, H, P, N, G, chunk)
    assert stream.status() == 0
    assert_close(host(y), ref_y, TOL[sfx], f"generic ssd forward {dims} {sfx}")
    gx = dev(np.full(x.shape, np.nan, NP_OF[sfx])); gdt = dev(np.full(dt.shape, np.nan, acc)); gA = dev(np.full(A.shape, np.nan, acc))
    gB = dev(np.full(Bm.shape, np.nan, NP_OF[sfx])); gC = dev(np.full(Cm.shape, np.nan, NP_OF[sfx]))
    run(mp, stream, "ssd_scan_reverse", sfx, *args, dev(gy), gx, gdt, gA, gB, gC, scr, nb, L, H, P, N, G, chunk)
    assert stream.status() == 0
    for got, want, name in zip((gx, gdt, gA, gB, gC), ref, ("gx", "gdt", "gA", "gB", "gC")):
        assert_close(host(got), want, TOL[sfx], f"generic ssd {name} {dims} {sfx}")
