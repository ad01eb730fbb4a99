"""Kernels against the committed golden vectors (tests/golden/golden.npz), through the C ABI."""
from pathlib import Path

import numpy as np
import pytest

from util import assert_close, dev, host, run

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).resolve().parent / "golden" / "golden.npz")


@pytest.mark.parametrize("sfx,tol", [("r32", 1e-5), ("r64", 1e-11)])
def test_row_ops_against_golden(mp, stream, sfx, tol):
    dt = np.float32 if sfx == "r32" else np.float64
    x, gy, gain = (dev(G[k].astype(dt)) for k in ("row_x", "row_gy", "row_gain"))
    m, n = G["row_x"].shape
    y = dev(np.zeros((m, n), dt)); gx = dev(np.zeros((m, n), dt))
    run(mp, stream, "softmax_ij_j", sfx, x, y, m, n)
    assert_close(host(y), G["softmax_y"], tol, "softmax")
    run(mp, stream, "softmax_ij_j_reverse", sfx, y, gy, gx, 0.0, m, n)
    assert_close(host(gx), G["softmax_gx"], 10 * tol, "softmax reverse")
    yn = dev(np.zeros((m, n), dt)); rstd = dev(np.zeros(m, dt)); gg = dev(np.zeros(n, dt))
    run(mp, stream, "rmsnorm_ij_j", sfx, x, gain, 1e-6, yn, rstd, m, n)
    assert_close(host(yn), G["rmsnorm_y"], tol, "rmsnorm")
    import torch
    scratch = torch.empty(mp.lib().mpRmsnormReverseScratchBytes(m, n, stream.ctx), dtype=torch.uint8, device="cuda")
    run(mp, stream, "rmsnorm_ij_j_reverse", sfx, x, gain, rstd, gy, 1e-6, gx, gg, 0.0, scratch, m, n)
    assert_close(host(gx), G["rmsnorm_gx"], 10 * tol, "rmsnorm gx")
    assert_close(host(gg), G["rmsnorm_ggain"], 10 * tol, "rmsnorm ggain")


def test_flat_ops_against_golden(mp, stream):
    a = dev(G["ew_a"].astype(np.float32)); out = dev(np.zeros(64, np.float32))
    run(mp, stream, "selu", "r32", a, out, 64)
    assert_close(host(out), G["selu"], 1e-5, "selu")
    w = dev(G["adam_w0"].astype(np.float32)); g = dev(G["adam_g"].astype(np.float32))
    m = dev(np.zeros(32, np.float32)); v = dev(np.zeros(32, np.float32))
    run(mp, stream, "adam", "r32", w, g, m, v, 3e-4, 0.9, 0.95, 1e-8, 1.0, 1, 32)
    assert_close(host(w), G["adam_w1"], 1e-6, "adam w")
    assert_close(host(m), G["adam_m1"], 1e-6, "adam m")
    assert_close(host(v), G["adam_v1"], 1e-6, "adam v")
    A = dev(G["mm_a"].astype(np.float32)); B = dev(G["mm_b"].astype(np.float32)); C = dev(np.zeros((5, 4), np.float32))
    run(mp, stream, "inner_product_ij_jk_ik", "r32", A, B, 1.0, C, 0.0, 5, 7, 4)
    assert_close(host(C), G["mm_c"], 1e-4, "inner product")
    lg = dev(G["ce_logits"].astype(np.float32)); tg = dev(G["ce_targets"]); loss = dev(np.zeros(5, np.float32))
    run(mp, stream, "cross_entropy", "r32", lg, tg, 0.25, loss, lg, 5, 33)
    assert_close(host(loss), G["ce_loss"], 1e-5, "cross-entropy loss")
    assert_close(host(lg), G["ce_glogits"], 1e-5, "cross-entropy gradient")


def test_rank3_ops_against_golden(mp, stream):
    import ctypes as C
    x = dev(G["perm_x"].astype(np.float32)); out = dev(np.zeros((5, 3, 4), np.float32))
    run(mp, stream, "permutate", "r32", x, out, 0.0, (C.c_ulong * 3)(3, 4, 5), (C.c_ulong * 3)(1, 2, 0), 3)
    assert np.array_equal(host(out), G["perm_kij"].astype(np.float32))
    a = dev(G["bmm_a"].astype(np.float32)); b = dev(G["bmm_b"].astype(np.float32)); c = dev(np.zeros((3, 5, 4), np.float32))
    run(mp, stream, "inner_product_bij_bjk_bik", "r32", a, b, 1.0, c, 0.0, 3, 5, 7, 4)
    assert_close(host(c), G["bmm_c"], 1e-4, "batched inner product")
    w = dev(G["mom_w0"].astype(np.float32)); g = dev(G["mom_g"].astype(np.float32)); m = dev(G["mom_m0"].astype(np.float32))
    run(mp, stream, "momentum", "r32", w, g, m, 0.1, 0.9, -0.5, 0.5, 32)
    assert_close(host(w), G["mom_w1"], 1e-6, "momentum w")
    assert_close(host(m), G["mom_m1"], 1e-6, "momentum m")
