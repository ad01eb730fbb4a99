"""The oracle against the committed golden vectors (tests/golden/golden.npz, written by
tests/golden/make_golden.py).  CPU only: a mismatch means the oracle's arithmetic changed."""
import sys
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden" / "golden.npz"


def test_oracle_reproduces_golden_vectors():
    sys.path.insert(0, str(GOLDEN.parent))
    import make_golden
    want = np.load(GOLDEN)
    got = make_golden.build()
    assert sorted(want.files) == sorted(got.keys())
    for k in want.files:
        np.testing.assert_allclose(np.asarray(got[k], dtype=np.float64), want[k].astype(np.float64), rtol=1e-12, atol=1e-14,
                                   err_msg=f"golden vector {k}")


def test_golden_known_answers():
    g = np.load(GOLDEN)
    # closed-form checks that do not go through the oracle at all
    x = g["row_x"]
    e = np.exp(x - x.max(axis=1, keepdims=True))
    np.testing.assert_allclose(g["softmax_y"], e / e.sum(axis=1, keepdims=True), rtol=1e-12)
    np.testing.assert_allclose(g["mm_c"], g["mm_a"] @ g["mm_b"], rtol=1e-12)
    a = g["ew_a"]
    lam, al = 1.0507009873554805, 1.6732632423543772
    np.testing.assert_allclose(g["selu"], lam * np.where(a > 0, a, al * (np.exp(a) - 1)), rtol=1e-12)
    # SSD recurrence written out directly
    xs, Bm, Cm, dt, A = g["ssd_x"], g["ssd_B"], g["ssd_C"], g["ssd_dt"], g["ssd_A"]
    y = np.zeros_like(xs)
    for h in range(2):
        S = np.zeros((4, 3))
        for t in range(8):
            S = np.exp(dt[0, t, h] * A[h]) * S + dt[0, t, h] * np.outer(Bm[0, t, 0], xs[0, t, h])
            y[0, t, h] = Cm[0, t, 0] @ S
    np.testing.assert_allclose(g["ssd_y"], y, rtol=1e-10, atol=1e-12)
    # "ijk->kij": out[k, i, j] = x[i, j, k]
    np.testing.assert_array_equal(g["perm_kij"], np.transpose(g["perm_x"], (2, 0, 1)))
    np.testing.assert_allclose(g["bmm_c"], np.einsum("bij,bjk->bik", g["bmm_a"], g["bmm_b"]), rtol=1e-12)
    m1 = 0.9 * g["mom_m0"] + np.clip(g["mom_g"], -0.5, 0.5)
    np.testing.assert_allclose(g["mom_m1"], m1, rtol=1e-14)
    np.testing.assert_allclose(g["mom_w1"], g["mom_w0"] - 0.1 * m1, rtol=1e-14)
