"""Writes tests/golden/golden.npz: inputs and float64-oracle outputs of a few operators at fixed seeds.

The reference has no golden vectors for these operators (its examples print, they do not assert), so the
fixtures pin THIS repository's oracle: `tests/test_golden.py` checks the C / numpy oracle against them on
every CPU run (a change of the oracle's arithmetic shows up as a diff of this file) and the GPU tests check
the kernels against the same arrays.  Regenerate with `python tests/golden/make_golden.py` after a
deliberate change of a definition and commit the new file together with the reason.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def build() -> dict:
    from oracle import pyoracle as orc
    r = np.random.default_rng(20240607)
    g = {}
    x = r.standard_normal((6, 40)); gy = r.standard_normal((6, 40)); gain = 1 + 0.02 * r.standard_normal(40)
    g["row_x"], g["row_gy"], g["row_gain"] = x, gy, gain
    y = orc.softmax_ij_j(x.copy())
    g["softmax_y"] = y
    g["softmax_gx"] = orc.softmax_ij_j_reverse(y.copy(), gy.copy())
    yn, rstd = orc.rmsnorm_ij_j(x.copy(), gain.copy(), 1e-6)
    g["rmsnorm_y"], g["rmsnorm_rstd"] = yn, rstd
    gx, gg = orc.rmsnorm_ij_j_reverse(x.copy(), gain.copy(), gy.copy(), 1e-6)
    g["rmsnorm_gx"], g["rmsnorm_ggain"] = gx, gg
    a = r.uniform(-2, 2, 64)
    g["ew_a"] = a
    g["selu"] = orc.selu(a.copy())
    w = r.standard_normal(32); gr = r.standard_normal(32); m = np.zeros(32); v = np.zeros(32)
    g["adam_w0"], g["adam_g"] = w.copy(), gr.copy()
    w1, m1, v1 = orc.adam(w.copy(), gr.copy(), m, v, 3e-4, 0.9, 0.95, 1e-8, 1.0, 1)
    g["adam_w1"], g["adam_m1"], g["adam_v1"] = w1, m1, v1
    A = r.standard_normal((5, 7)); B = r.standard_normal((7, 4))
    g["mm_a"], g["mm_b"] = A, B
    g["mm_c"] = orc.inner_product(A.copy(), B.copy())
    logits = 3 * r.standard_normal((5, 33)); tg = r.integers(0, 33, 5).astype(np.int32)
    g["ce_logits"], g["ce_targets"] = logits, tg
    loss, gl = orc.cross_entropy(logits, tg, 0.25)
    g["ce_loss"], g["ce_glogits"] = loss, gl
    # SSD: batch 1, seqlen 8, heads 2, headdim 3, dstate 4, one group (sequential recurrence)
    xs = r.standard_normal((1, 8, 2, 3)); Bm = r.standard_normal((1, 8, 1, 4)); Cm = r.standard_normal((1, 8, 1, 4))
    dt = np.log1p(np.exp(r.standard_normal((1, 8, 2)) - 1.0)); Ah = -np.exp(r.uniform(0, 1, 2))
    g["ssd_x"], g["ssd_B"], g["ssd_C"], g["ssd_dt"], g["ssd_A"] = xs, Bm, Cm, dt, Ah
    g["ssd_y"] = orc.ssd_forward(xs.copy(), dt.copy(), Ah.copy(), Bm.copy(), Cm.copy())
    # rank-3 operators (appended, so the arrays above keep their values)
    px = r.standard_normal((3, 4, 5))
    g["perm_x"] = px
    g["perm_kij"] = orc.permutate(px.copy(), [1, 2, 0])            # "ijk->kij"
    ba = r.standard_normal((3, 5, 7)); bb = r.standard_normal((3, 7, 4))
    g["bmm_a"], g["bmm_b"] = ba, bb
    g["bmm_c"] = orc.inner_product_batched(ba.copy(), bb.copy())
    mw = r.standard_normal(32); mg = r.standard_normal(32); mm = r.standard_normal(32)
    g["mom_w0"], g["mom_g"], g["mom_m0"] = mw, mg, mm
    g["mom_w1"], g["mom_m1"] = orc.momentum(mw.copy(), mg.copy(), mm.copy(), 0.1, 0.9, -0.5, 0.5)
    return g


if __name__ == "__main__":
    out = Path(__file__).resolve().parent / "golden.npz"
    np.savez_compressed(out, **build())
    print("wrote", out, out.stat().st_size, "bytes")
