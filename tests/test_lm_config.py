"""Host-side checks of the Mamba-2 LM composition that need no GPU: parameter inventory of the benchmark
configuration, flat-buffer layout, initialisation ranges."""
import math

import numpy as np

from metaphor_b200.mamba_lm import ALIGN, LMConfig, init_weights


def test_benchmark_configuration_has_the_expected_size():
    cfg = LMConfig()
    assert (cfg.d_inner, cfg.heads, cfg.conv_dim, cfg.d_in_proj) == (1536, 24, 1792, 3352)
    assert cfg.n_params() == 128_983_488
    names = [n for n, _ in cfg.param_shapes()]
    assert names[0] == "embedding" and names[-1] == "normf_w" and len(names) == 2 + 9 * cfg.n_layer


def test_flat_layout_is_aligned_and_disjoint():
    cfg = LMConfig(d_model=256, n_layer=2, vocab=1000)
    off, spans = 0, []
    for name, shape in cfg.param_shapes():
        n = math.prod(shape)
        assert off % ALIGN == 0
        spans.append((off, off + n))
        off += (n + ALIGN - 1) // ALIGN * ALIGN
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    # every row pitch the contractions see is a multiple of 16 bytes in r16
    assert (cfg.d_in_proj * 2) % 16 == 0 and (cfg.d_model * 2) % 16 == 0 and (cfg.d_inner * 2) % 16 == 0


def test_initial_weights():
    cfg = LMConfig(d_model=256, n_layer=1, vocab=512)
    w = init_weights(cfg, seed=0)
    assert set(w) == {n for n, _ in cfg.param_shapes()}
    dt = np.log1p(np.exp(w["layers.0.dt_bias"].astype(np.float64)))      # softplus(dt_bias)
    assert np.all(dt > 0.9e-3) and np.all(dt < 1.1e-1)
    A = -np.exp(w["layers.0.A_log"].astype(np.float64))
    assert np.all(A <= -1.0 + 1e-6) and np.all(A >= -16.0 - 1e-4)
    assert np.all(w["layers.0.norm_w"] == 1) and np.all(w["layers.0.conv_b"] == 0)
    assert abs(float(w["embedding"].std()) - 0.02) < 2e-3
    w2 = init_weights(cfg, seed=0)
    assert all(np.array_equal(w[k], w2[k]) for k in w)
