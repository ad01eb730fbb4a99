"""Rank-1 losses (mse, bce) and the momentum step against the float64 numpy oracle."""
import numpy as np
import pytest

from util import NP_OF, assert_close, dev, host, run

pytestmark = pytest.mark.gpu
ACC = {"r16": np.float32, "r32": np.float32, "r64": np.float64}
TOL = {"r16": 1e-2, "r32": 1e-5, "r64": 1e-12}


@pytest.mark.parametrize("sfx", ["r16", "r32", "r64"])
@pytest.mark.parametrize("n", [1, 4097, 100003])
def test_losses(mp, stream, orc, sfx, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(NP_OF[sfx]); t = rng.standard_normal(n).astype(NP_OF[sfx])
    scratch = dev(np.zeros(n // 4096 + 2, ACC[sfx])); redux = dev(np.zeros(1, ACC[sfx])); grad = dev(np.zeros(n, NP_OF[sfx]))
    run(mp, stream, "mse_loss_i_i", sfx, dev(x), grad, dev(t), scratch, redux, n)
    loss, g = orc.mse_loss(x, t)
    assert abs(float(host(redux)[0]) - loss) <= (1e-5 if sfx != "r64" else 1e-12) * max(1.0, abs(loss))
    assert_close(host(grad), g, TOL[sfx], "mse gradient")
    p = rng.uniform(0.01, 0.99, n).astype(NP_OF[sfx]); y = (rng.uniform(0, 1, n) > 0.5).astype(NP_OF[sfx])
    run(mp, stream, "bce_loss_i_i", sfx, dev(p), grad, dev(y), scratch, redux, n)
    loss, g = orc.bce_loss(p, y)
    assert abs(float(host(redux)[0]) - loss) <= (1e-5 if sfx != "r64" else 1e-12) * max(1.0, abs(loss))
    assert_close(host(grad), g, TOL[sfx], "bce gradient")


@pytest.mark.parametrize("sfx", ["r16", "r32", "r64"])
@pytest.mark.parametrize("n", [5, 8192, 100003])
def test_momentum(mp, stream, orc, sfx, n):
    rng = np.random.default_rng(n + 1)
    w = rng.standard_normal(n).astype(NP_OF[sfx]); g = rng.standard_normal(n).astype(NP_OF[sfx]); m = (0.1 * rng.standard_normal(n)).astype(NP_OF[sfx])
    dw, dm = dev(w.copy()), dev(m.copy())
    run(mp, stream, "momentum", sfx, dw, dev(g), dm, 0.01, 0.9, -0.5, 0.5, n)
    rw, rm = orc.momentum(w, g, m, 0.01, 0.9, -0.5, 0.5)
    assert_close(host(dw), rw, TOL[sfx], "momentum w")
    assert_close(host(dm), rm, TOL[sfx], "momentum m")
