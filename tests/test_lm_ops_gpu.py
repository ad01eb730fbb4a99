"""GPU parity of the operators around the scan in a language-model step
(embedding, causal conv + SiLU, softplus, skip + gate, cross-entropy, precision
conversion) against the float64 numpy oracle, through the C ABI."""
import numpy as np
import pytest

from util import NP_OF, assert_close, dev, host, run

pytestmark = pytest.mark.gpu

DTYPES = ["r16", "r32", "r64"]
TOL = {"r16": 1e-2, "r32": 1e-5, "r64": 1e-12}
ACC = {"r16": np.float32, "r32": np.float32, "r64": np.float64}


def draw(rng, shape, sfx, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(NP_OF[sfx])


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("n,dim,vocab", [(37, 64, 50), (5, 7, 3), (0, 8, 4)])
def test_embedding(mp, stream, orc, sfx, n, dim, vocab):
    rng = np.random.default_rng(0)
    table = draw(rng, (vocab, dim), sfx)
    ids = rng.integers(-1, vocab + 1, size=n).astype(np.int32)   # includes out-of-range ids
    out = dev(np.full((n, dim), 7, NP_OF[sfx]))
    run(mp, stream, "embedding", sfx, dev(table), dev(ids), out, n, dim, vocab)
    assert np.array_equal(host(out).astype(np.float64), orc.embedding(table.astype(np.float64), ids))
    gy = draw(rng, (n, dim), sfx)
    gt0 = rng.standard_normal((vocab, dim)).astype(ACC[sfx])
    gt = dev(gt0.copy())
    run(mp, stream, "embedding_reverse", sfx, dev(ids), dev(gy), gt, n, dim, vocab)
    ref = gt0.astype(np.float64) + orc.embedding_reverse(ids, gy, vocab)
    assert_close(host(gt), ref, 1e-5 if sfx != "r64" else 1e-12, "embedding reverse")


CONV_CASES = [(2, 300, 64, 4, 96), (1, 17, 24, 3, 24), (3, 128, 8, 2, 40), (1, 5, 7, 4, 7)]


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("nb,L,Cn,W,pitch", CONV_CASES)
def test_causal_conv1d_silu(mp, stream, orc, sfx, nb, L, Cn, W, pitch):
    rng = np.random.default_rng(1)
    xfull = draw(rng, (nb, L, pitch), sfx)
    off = pitch - Cn   # the convolved channels are the last Cn columns of a wider row
    w = draw(rng, (Cn, W), sfx, 0.5)
    bias = draw(rng, (Cn,), sfx, 0.1)
    x = xfull[:, :, off:]
    dx = dev(xfull)
    y = dev(np.zeros((nb, L, Cn), NP_OF[sfx]))
    esz = xfull.itemsize
    run(mp, stream, "causal_conv1d_silu", sfx, dx.data_ptr() + off * esz, pitch, dev(w), dev(bias), y, Cn, nb, L, Cn, W)
    ref = orc.causal_conv1d_silu(x.astype(np.float64), w.astype(np.float64), bias.astype(np.float64))
    assert_close(host(y), ref, TOL[sfx], "conv forward")
    gy = draw(rng, (nb, L, Cn), sfx)
    gxfull = dev(np.full((nb, L, pitch), 3, NP_OF[sfx]))
    gw0 = rng.standard_normal((Cn, W)).astype(ACC[sfx])
    gb0 = rng.standard_normal((Cn,)).astype(ACC[sfx])
    gw, gb = dev(gw0.copy()), dev(gb0.copy())
    run(mp, stream, "causal_conv1d_silu_reverse", sfx, dx.data_ptr() + off * esz, pitch, dev(w), dev(bias), dev(gy), Cn,
        gxfull.data_ptr() + off * esz, pitch, gw, gb, nb, L, Cn, W)
    rgx, rgw, rgb = orc.causal_conv1d_silu_reverse(x.astype(np.float64), w.astype(np.float64), bias.astype(np.float64), gy.astype(np.float64))
    got = host(gxfull)
    assert_close(got[:, :, off:], rgx, TOL[sfx], "conv gx")
    assert np.all(got[:, :, :off] == 3), "columns outside the slice were written"
    ptol = 1e-4 if sfx != "r64" else 1e-11
    assert_close(host(gw), gw0.astype(np.float64) + rgw, ptol, "conv gw")
    assert_close(host(gb), gb0.astype(np.float64) + rgb, ptol, "conv gbias")


# (batch, len, segment widths, taps, pitch of the wide input row): tile-aligned segments, segments ending inside a
# 64-channel tile, widths that rule out 16-byte accesses (one launch per segment)
SEG_CASES = [(2, 200, (128, 64, 64), 4, 320), (1, 70, (72, 8, 40), 4, 136), (2, 33, (24, 16), 3, 40), (1, 9, (5, 3, 7), 2, 20)]


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("nb,L,widths,W,pitch", SEG_CASES)
def test_causal_conv1d_silu_segments(mp, stream, orc, sfx, nb, L, widths, W, pitch):
    import ctypes as C
    rng = np.random.default_rng(11)
    Cn = sum(widths)
    off = pitch - Cn
    xfull = draw(rng, (nb, L, pitch), sfx)
    w = draw(rng, (Cn, W), sfx, 0.5)
    bias = draw(rng, (Cn,), sfx, 0.1)
    x = xfull[:, :, off:]
    dx, dw, db = dev(xfull), dev(w), dev(bias)
    esz = xfull.itemsize
    ys = [dev(np.full((nb, L, cw), np.nan, NP_OF[sfx])) for cw in widths]
    ptrs = (C.c_void_p * len(widths))(*[t.data_ptr() for t in ys])
    cw = (C.c_ulong * len(widths))(*widths)
    run(mp, stream, "causal_conv1d_silu_segments", sfx, dx.data_ptr() + off * esz, pitch, dw, db, ptrs, cw, cw, len(widths), nb, L, W)
    ref = orc.causal_conv1d_silu(x.astype(np.float64), w.astype(np.float64), bias.astype(np.float64))
    c0 = 0
    for t, cwid in zip(ys, widths):
        assert_close(host(t), ref[:, :, c0:c0 + cwid], TOL[sfx], f"segment forward at channel {c0}")
        # the same segment through the plain launcher: identical bits
        single = dev(np.zeros((nb, L, cwid), NP_OF[sfx]))
        run(mp, stream, "causal_conv1d_silu", sfx, dx.data_ptr() + (off + c0) * esz, pitch, dw.data_ptr() + c0 * W * esz,
            db.data_ptr() + c0 * esz, single, cwid, nb, L, cwid, W)
        assert np.array_equal(host(t), host(single))
        c0 += cwid
    gys_np = [draw(rng, (nb, L, cwid), sfx) for cwid in widths]
    gys = [dev(g) for g in gys_np]
    gptrs = (C.c_void_p * len(widths))(*[t.data_ptr() for t in gys])
    gxfull = dev(np.full((nb, L, pitch), 3, NP_OF[sfx]))
    gw0 = rng.standard_normal((Cn, W)).astype(ACC[sfx]); gb0 = rng.standard_normal((Cn,)).astype(ACC[sfx])
    gw, gb = dev(gw0.copy()), dev(gb0.copy())
    run(mp, stream, "causal_conv1d_silu_segments_reverse", sfx, dx.data_ptr() + off * esz, pitch, dw, db, gptrs, cw, cw, len(widths),
        gxfull.data_ptr() + off * esz, pitch, gw, gb, nb, L, W)
    gy = np.concatenate(gys_np, axis=2)
    rgx, rgw, rgb = orc.causal_conv1d_silu_reverse(x.astype(np.float64), w.astype(np.float64), bias.astype(np.float64), gy.astype(np.float64))
    got = host(gxfull)
    assert_close(got[:, :, off:], rgx, TOL[sfx], "segments gx")
    assert np.all(got[:, :, :off] == 3), "columns outside the slice were written"
    ptol = 1e-4 if sfx != "r64" else 1e-11
    assert_close(host(gw), gw0.astype(np.float64) + rgw, ptol, "segments gw")
    assert_close(host(gb), gb0.astype(np.float64) + rgb, ptol, "segments gbias")


# The reverse with a scaled skip term on the first segment (the scan's D skip in a Mamba-2 block): against the oracle
# fed with gys[0] + D[channel / group] * skip.  Tiled r16 path (group = one 64-channel tile, and a group that spans
# tiles), a segment that ends inside a tile, and the dense fallback of the other dtypes.
@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("nb,L,widths,W,pitch,group", [(2, 200, (128, 64, 64), 4, 320, 64), (1, 70, (96, 8, 40), 4, 160, 32),
                                                       (2, 33, (32, 16), 3, 56, 16), (1, 130, (256, 64), 4, 320, 128)])
def test_causal_conv1d_silu_segments_reverse_with_a_skip_term(mp, stream, orc, sfx, nb, L, widths, W, pitch, group):
    import ctypes as C
    rng = np.random.default_rng(17)
    Cn = sum(widths)
    off = pitch - Cn
    xfull = draw(rng, (nb, L, pitch), sfx)
    w = draw(rng, (Cn, W), sfx, 0.5)
    bias = draw(rng, (Cn,), sfx, 0.1)
    x = xfull[:, :, off:]
    dx, dw, db = dev(xfull), dev(w), dev(bias)
    esz = xfull.itemsize
    cw = (C.c_ulong * len(widths))(*widths)
    gys_np = [draw(rng, (nb, L, cwid), sfx) for cwid in widths]
    skip_np = draw(rng, (nb, L, widths[0]), sfx)
    scale = rng.standard_normal(widths[0] // group).astype(ACC[sfx])
    gys = [dev(g) for g in gys_np]
    dskip, dscale = dev(skip_np), dev(scale)
    gptrs = (C.c_void_p * len(widths))(*[t.data_ptr() for t in gys])
    sptrs = (C.c_void_p * len(widths))(*([dskip.data_ptr()] + [None] * (len(widths) - 1)))
    spitch = (C.c_ulong * len(widths))(*([widths[0]] + [0] * (len(widths) - 1)))
    scales = (C.c_void_p * len(widths))(*([dscale.data_ptr()] + [None] * (len(widths) - 1)))
    gxfull = dev(np.full((nb, L, pitch), 3, NP_OF[sfx]))
    gw0 = rng.standard_normal((Cn, W)).astype(ACC[sfx]); gb0 = rng.standard_normal((Cn,)).astype(ACC[sfx])
    gw, gb = dev(gw0.copy()), dev(gb0.copy())
    run(mp, stream, "causal_conv1d_silu_segments_reverse_skip", sfx, dx.data_ptr() + off * esz, pitch, dw, db, gptrs, cw, cw, len(widths),
        sptrs, spitch, scales, group, gxfull.data_ptr() + off * esz, pitch, gw, gb, nb, L, W)
    f64 = lambda a: a.astype(np.float64)
    gy = np.concatenate([f64(g) for g in gys_np], axis=2)
    gy[:, :, :widths[0]] += np.repeat(f64(scale), group) * f64(skip_np)
    rgx, rgw, rgb = orc.causal_conv1d_silu_reverse(f64(x), f64(w), f64(bias), gy)
    got = host(gxfull)
    assert_close(got[:, :, off:], rgx, TOL[sfx], "skip segments gx")
    assert np.all(got[:, :, :off] == 3), "columns outside the slice were written"
    ptol = 1e-4 if sfx != "r64" else 1e-11
    assert_close(host(gw), f64(gw0) + rgw, ptol, "skip segments gw")
    assert_close(host(gb), f64(gb0) + rgb, ptol, "skip segments gbias")
    assert stream.status() == 0


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("rows,H,pitch", [(1000, 24, 40), (3, 5, 5), (70, 300, 304), (50, 256, 256), (4099, 32, 32)])
def test_softplus_bias(mp, stream, orc, sfx, rows, H, pitch):
    rng = np.random.default_rng(2)
    rawfull = draw(rng, (rows, pitch), sfx, 3.0)
    off = pitch - H
    bias = rng.standard_normal(H).astype(ACC[sfx])
    d = dev(rawfull)
    out = dev(np.zeros((rows, H), ACC[sfx]))
    esz = rawfull.itemsize
    run(mp, stream, "softplus_bias", sfx, d.data_ptr() + off * esz, pitch, dev(bias), out, rows, H)
    raw = rawfull[:, off:].astype(np.float64)
    assert_close(host(out), orc.softplus_bias(raw, bias), 1e-5 if sfx != "r64" else 1e-12, "softplus")
    gdt = rng.standard_normal((rows, H)).astype(ACC[sfx])
    graw = dev(np.zeros((rows, pitch), NP_OF[sfx]))
    gb0 = rng.standard_normal(H).astype(ACC[sfx])
    gb = dev(gb0.copy())
    run(mp, stream, "softplus_bias_reverse", sfx, d.data_ptr() + off * esz, pitch, dev(bias), dev(gdt), graw.data_ptr() + off * esz, pitch, gb, rows, H)
    rg, rgb = orc.softplus_bias_reverse(raw, bias, gdt)
    assert_close(host(graw)[:, off:], rg, TOL[sfx], "softplus graw")
    assert_close(host(gb), gb0.astype(np.float64) + rgb, 1e-4 if sfx != "r64" else 1e-11, "softplus gbias")


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("rows,H,P,pitch", [(257, 4, 64, 300), (3, 2, 5, 10)])
def test_ssd_gate(mp, stream, orc, sfx, rows, H, P, pitch):
    rng = np.random.default_rng(3)
    width = H * P
    y, x, gu = (draw(rng, (rows, width), sfx) for _ in range(3))
    zfull = draw(rng, (rows, pitch), sfx)
    D = rng.standard_normal(H).astype(ACC[sfx])
    z = zfull[:, :width].astype(np.float64)
    u = dev(np.zeros((rows, width), NP_OF[sfx]))
    dz = dev(zfull)
    run(mp, stream, "ssd_gate", sfx, dev(y), dev(x), dev(D), dz, pitch, u, rows, H, P)
    assert_close(host(u), orc.ssd_gate(y.astype(np.float64), x.astype(np.float64), D, z, H, P), TOL[sfx], "gate")
    gy = dev(np.zeros((rows, width), NP_OF[sfx]))
    gz = dev(np.full((rows, pitch), 2, NP_OF[sfx]))
    gD0 = rng.standard_normal(H).astype(ACC[sfx])
    gD = dev(gD0.copy())
    run(mp, stream, "ssd_gate_reverse", sfx, dev(y), dev(x), dev(D), dz, pitch, dev(gu), gy, gz, pitch, gD, rows, H, P)
    rgy, rgz, rgD = orc.ssd_gate_reverse(y.astype(np.float64), x.astype(np.float64), D, z, gu.astype(np.float64), H, P)
    assert_close(host(gy), rgy, TOL[sfx], "gate gy")
    assert_close(host(gz)[:, :width], rgz, TOL[sfx], "gate gz")
    assert np.all(host(gz)[:, width:] == 2)
    assert_close(host(gD), gD0.astype(np.float64) + rgD, 1e-2 if sfx == "r16" else (1e-4 if sfx == "r32" else 1e-11), "gate gD")
    gx0 = draw(rng, (rows, width), sfx)
    gx = dev(gx0.copy())
    run(mp, stream, "head_scale_accumulate", sfx, dev(D), gy, gx, rows, H, P)
    ref = gx0.astype(np.float64) + np.repeat(D.astype(np.float64), P) * host(gy).astype(np.float64)
    assert_close(host(gx), ref, TOL[sfx], "skip accumulate")


# Gate and RMSNorm in one kernel: against the oracle's gate followed by its RMSNorm (and the reverses in the opposite
# order).  Shapes: a row that fits the register plan of every dtype, a scalar ragged one, the language model's
# [*, 24 x 64] inside a 3352-wide projection output, and a vectorised width outside the register plan.
@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("rows,H,P,pitch", [(257, 4, 64, 300), (3, 2, 5, 10), (70, 24, 64, 3352), (33, 3, 40, 128)])
def test_ssd_gate_rmsnorm(mp, stream, orc, sfx, rows, H, P, pitch):
    rng = np.random.default_rng(13)
    width = H * P
    eps = 1e-5
    y, x, gout = (draw(rng, (rows, width), sfx) for _ in range(3))
    zfull = draw(rng, (rows, pitch), sfx)
    D = rng.standard_normal(H).astype(ACC[sfx])
    gain = (1.0 + 0.1 * rng.standard_normal(width)).astype(NP_OF[sfx])
    f64 = lambda a: a.astype(np.float64)
    z = f64(zfull[:, :width])
    u = orc.ssd_gate(f64(y), f64(x), D, z, H, P)
    want, want_rstd = orc.rmsnorm_ij_j(u, f64(gain), eps)
    out = dev(np.zeros((rows, width), NP_OF[sfx]))
    rstd = dev(np.zeros(rows, ACC[sfx]))
    dz = dev(zfull)
    run(mp, stream, "ssd_gate_rmsnorm", sfx, dev(y), dev(x), dev(D), dz, pitch, dev(gain), eps, out, rstd, rows, H, P)
    assert_close(host(out), want, TOL[sfx], "gated norm")
    assert_close(host(rstd), want_rstd, 1e-5 if sfx != "r64" else 1e-12, "gated norm rstd")
    # reverse, with the oracle's rstd so that both sides start from the same numbers
    gu, want_ggain = orc.rmsnorm_ij_j_reverse(u, f64(gain), f64(gout), eps)
    rgy, rgz, rgD = orc.ssd_gate_reverse(f64(y), f64(x), D, z, gu, H, P)
    gy = dev(np.zeros((rows, width), NP_OF[sfx]))
    gz = dev(np.full((rows, pitch), 2, NP_OF[sfx]))
    gD0 = rng.standard_normal(H).astype(ACC[sfx])
    gD = dev(gD0.copy())
    gg0 = draw(rng, width, sfx)
    nbytes = mp.lib().mpSsdGateRmsnormReverseScratchBytes(rows, H, P, stream.ctx)
    scratch = dev(np.zeros(max(1, nbytes // 8), np.float64))
    for alpha in (0.0, 1.0):
        ggain = dev(gg0.copy())
        gD = dev(gD0.copy())
        run(mp, stream, "ssd_gate_rmsnorm_reverse", sfx, dev(y), dev(x), dev(D), dz, pitch, dev(gain), dev(want_rstd.astype(ACC[sfx])),
            dev(gout), gy, gz, pitch, gD, ggain, alpha, scratch, rows, H, P)
        assert_close(host(gy), rgy, TOL[sfx], "gated norm gy")
        assert_close(host(gz)[:, :width], rgz, TOL[sfx], "gated norm gz")
        assert np.all(host(gz)[:, width:] == 2)
        assert_close(host(gD), f64(gD0) + rgD, 1e-2 if sfx == "r16" else (1e-4 if sfx == "r32" else 1e-11), "gated norm gD")
        assert_close(host(ggain), alpha * f64(gg0) + want_ggain, 1e-2 if sfx == "r16" else (1e-4 if sfx == "r32" else 1e-11), "gated norm ggain")


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("m,n", [(64, 50280), (7, 1024), (3, 37), (2, 120000)])
def test_cross_entropy(mp, stream, orc, sfx, m, n):
    rng = np.random.default_rng(4)
    logits = draw(rng, (m, n), sfx, 3.0)
    targets = rng.integers(0, n, size=m).astype(np.int32)
    targets[0] = -1   # ignored row
    scale = 0.37
    loss = dev(np.zeros(m, ACC[sfx]))
    d = dev(logits.copy())
    run(mp, stream, "cross_entropy", sfx, d, dev(targets), scale, loss, d, m, n)   # gradient in place
    rl, rg = orc.cross_entropy(logits, targets, scale)
    assert_close(host(loss), rl, 1e-5 if sfx != "r64" else 1e-12, "cross-entropy loss")
    assert_close(host(d), rg, TOL[sfx], "cross-entropy gradient")


def test_neg_exp_and_convert(mp, stream):
    import torch
    rng = np.random.default_rng(5)
    a = rng.standard_normal(1000).astype(np.float32)
    out = dev(np.zeros(1000, np.float32))
    run(mp, stream, "neg_exp", "r32", dev(a), out, 1000)
    assert_close(host(out), -np.exp(a.astype(np.float64)), 1e-5, "neg_exp")
    for n in (4096, 1001):
        h = rng.standard_normal(n).astype(np.float16)
        f0 = rng.standard_normal(n).astype(np.float32)
        f = dev(f0.copy())
        torch.cuda.current_stream().synchronize()
        mp.lib().launch_convert_r16_r32(dev(h).data_ptr(), f.data_ptr(), 0.5, n, stream.ctx)
        stream.sync()
        assert_close(host(f), h.astype(np.float64) + 0.5 * f0, 1e-6, "convert r16->r32")
        back = dev(np.zeros(n, np.float16))
        torch.cuda.current_stream().synchronize()
        mp.lib().launch_convert_r32_r16(dev(f0).data_ptr(), back.data_ptr(), n, stream.ctx)
        stream.sync()
        assert np.array_equal(host(back), f0.astype(np.float16))
