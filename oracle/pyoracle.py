"""numpy front end of the C oracle (``oracle/liboracle.so``).

TEST INFRASTRUCTURE: imported only by tests/, the smoke check and the
benchmark's CPU-baseline / reference legs.  Arrays are float32 or float64
numpy arrays (r16 inputs are widened to float64 by the caller and the result
rounded back, which is what "fp64 oracle rounded to r16" means in the tests).
In-place arguments (accumulators) are modified and also returned.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None


def build() -> Path:
    """Compile liboracle.so with gcc if it is missing or stale."""
    so = HERE / "liboracle.so"
    srcs = [HERE / "oracle.c", HERE / "oracle_body.inc"]
    if not so.exists() or so.stat().st_mtime < max(s.stat().st_mtime for s in srcs):
        subprocess.run(["make", "-C", str(HERE), "liboracle.so"], check=True, capture_output=True)
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(str(build()))
    return _LIB


def _sfx(a: np.ndarray) -> str:
    if a.dtype == np.float32:
        return "f32"
    if a.dtype == np.float64:
        return "f64"
    raise TypeError(f"oracle works on float32/float64 arrays, got {a.dtype}")


def _p(a):
    if a is None:
        return C.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def _call(name, like, *args):
    fn = getattr(lib(), f"{name}_{_sfx(like)}")
    fn.restype = None
    conv = []
    for a in args:
        if isinstance(a, np.ndarray) or a is None:
            conv.append(_p(a))
        elif isinstance(a, float):
            conv.append(C.c_double(a))
        elif isinstance(a, (int, np.integer)):
            conv.append(C.c_size_t(int(a)))
        else:
            raise TypeError(type(a))
    fn(*conv)


# ---- flat element-wise -----------------------------------------------------
def addition(a, b):
    c = np.empty_like(a); _call("orc_addition", a, a, b, c, a.size); return c


def subtraction(a, b):
    c = np.empty_like(a); _call("orc_subtraction", a, a, b, c, a.size); return c


def hadamard(a, b):
    c = np.empty_like(a); _call("orc_hadamard", a, a, b, c, a.size); return c


def hadamard_reverse(a, b, c):
    _call("orc_hadamard_reverse", a, a, b, c, a.size); return c


def negate(a):
    b = np.empty_like(a); _call("orc_negate", a, a, b, a.size); return b


def translate(a, value):
    c = np.empty_like(a); _call("orc_translate", a, a, float(value), c, a.size); return c


def dilate(a, value):
    c = np.empty_like(a); _call("orc_dilate", a, a, float(value), c, a.size); return c


def dilate_reverse(a, value, b):
    _call("orc_dilate_reverse", a, a, float(value), b, a.size); return b


def relu(a):
    b = np.empty_like(a); _call("orc_relu", a, a, b, a.size); return b


def relu_reverse(a, ga, gb):
    _call("orc_relu_reverse", a, a, ga, gb, a.size); return ga


def stepwise(a):
    b = np.empty_like(a); _call("orc_stepwise", a, a, b, a.size); return b


def fill(a, value):
    _call("orc_fill", a, a, float(value), a.size); return a


def sequence(a, init, step):
    _call("orc_sequence", a, a, float(init), float(step), a.size); return a


def copy(a):
    b = np.empty_like(a); _call("orc_copy", a, a, b, a.size); return b


def selu(a):
    b = np.empty_like(a); _call("orc_selu", a, a, b, a.size); return b


def selu_reverse(a, ga, gb):
    _call("orc_selu_reverse", a, a, ga, gb, a.size); return ga


def sgd(w, g, rate, lo=-np.inf, hi=np.inf):
    _call("orc_sgd", w, w, g, float(rate), float(lo), float(hi), w.size); return w


def adam(w, g, m, v, lr, b1, b2, eps, grad_scale, step):
    _call("orc_adam", w, w, g, m, v, float(lr), float(b1), float(b2), float(eps), float(grad_scale), int(step), w.size)
    return w, m, v


# ---- rank-2 ------------------------------------------------------------------
def permutate_ij_ji(src, dst=None, alpha=0.0):
    row, col = src.shape
    if dst is None:
        dst = np.zeros((col, row), dtype=src.dtype)
    _call("orc_permutate_ij_ji", src, src, dst, float(alpha), row, col); return dst


def permutate(src, perm, dst=None, alpha=0.0):
    """dst = permute(src) + alpha*dst; perm[i] = output position of source dimension i."""
    perm = [int(q) for q in perm]
    out_shape = [0] * src.ndim
    for i, q in enumerate(perm):
        out_shape[q] = src.shape[i]
    if dst is None:
        dst = np.zeros(out_shape, dtype=src.dtype)
    assert list(dst.shape) == out_shape
    sizes = (C.c_size_t * src.ndim)(*src.shape)
    pm = (C.c_size_t * src.ndim)(*perm)
    fn = getattr(lib(), f"orc_permutate_{_sfx(src)}")
    fn.restype = None
    fn(_p(src), _p(dst), C.c_double(alpha), sizes, pm, C.c_size_t(src.ndim))
    return dst


def reduce_ij_i(src, dst=None, alpha=0.0):
    m, n = src.shape
    if dst is None:
        dst = np.zeros(m, dtype=src.dtype)
    _call("orc_reduce_ij_i", src, src, dst, float(alpha), m, n); return dst


def reduce_ij_j(src, dst=None, alpha=0.0):
    m, n = src.shape
    if dst is None:
        dst = np.zeros(n, dtype=src.dtype)
    _call("orc_reduce_ij_j", src, src, dst, float(alpha), m, n); return dst


def broadcast_i_ij(src, dst, alpha=0.0):
    m, n = dst.shape
    _call("orc_broadcast_i_ij", src, src, dst, float(alpha), m, n); return dst


def broadcast_j_ij(src, dst, alpha=0.0):
    m, n = dst.shape
    _call("orc_broadcast_j_ij", src, src, dst, float(alpha), m, n); return dst


def inner_product(a, b, alpha=1.0, c=None, beta=0.0, ta=False, tb=False, bias=None):
    """C = alpha*op(A)*op(B) + bias + beta*C (row-major); see orc_inner_product."""
    m = a.shape[1] if ta else a.shape[0]
    n = a.shape[0] if ta else a.shape[1]
    k = b.shape[0] if tb else b.shape[1]
    assert (b.shape[1] if tb else b.shape[0]) == n
    if c is None:
        c = np.zeros((m, k), dtype=a.dtype)
    fn = getattr(lib(), f"orc_inner_product_{_sfx(a)}")
    fn.restype = None
    fn(_p(a), _p(b), _p(bias), C.c_double(alpha), _p(c), C.c_double(beta),
       C.c_size_t(m), C.c_size_t(n), C.c_size_t(k), C.c_int(int(ta)), C.c_int(int(tb)))
    return c


def inner_product_batched(a, b, alpha=1.0, c=None, beta=0.0, ta=False, tb=False):
    """One rank-2 contraction (orc_inner_product) per leading batch entry."""
    outs = []
    for q in range(a.shape[0]):
        cq = None if c is None else np.ascontiguousarray(c[q])
        outs.append(inner_product(np.ascontiguousarray(a[q]), np.ascontiguousarray(b[q]), alpha, cq, beta, ta=ta, tb=tb))
    return np.stack(outs) if outs else np.zeros((0,) + ((a.shape[2] if ta else a.shape[1]), (b.shape[1] if tb else b.shape[2])), a.dtype)


# ---- row-wise ----------------------------------------------------------------
def softmax_ij_j(x):
    y = np.empty_like(x); _call("orc_softmax_ij_j", x, x, y, x.shape[0], x.shape[1]); return y


def softmax_ij_j_reverse(y, gy, gx=None, alpha=0.0):
    if gx is None:
        gx = np.zeros_like(y)
    _call("orc_softmax_ij_j_reverse", y, y, gy, gx, float(alpha), y.shape[0], y.shape[1]); return gx


def rmsnorm_ij_j(x, gain, eps):
    y = np.empty_like(x)
    rstd = np.empty(x.shape[0], dtype=x.dtype)
    _call("orc_rmsnorm_ij_j", x, x, gain, float(eps), y, rstd, x.shape[0], x.shape[1])
    return y, rstd


def rmsnorm_ij_j_reverse(x, gain, gy, eps, gx=None, ggain=None, alpha=0.0):
    if gx is None:
        gx = np.zeros_like(x)
    if ggain is None:
        ggain = np.zeros_like(gain)
    _call("orc_rmsnorm_ij_j_reverse", x, x, gain, gy, float(eps), gx, ggain, float(alpha), x.shape[0], x.shape[1])
    return gx, ggain


# ---- SSD scan (float64 only) ---------------------------------------------------
def ssd_forward(x, dt, A, Bm, Cm):
    nb, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    y = np.empty_like(x)
    fn = lib().orc_ssd_forward_f64
    fn.restype = None
    fn(_p(x), _p(dt), _p(A), _p(Bm), _p(Cm), _p(y), *(C.c_size_t(v) for v in (nb, L, H, P, N, G)))
    return y


def ssd_reverse(x, dt, A, Bm, Cm, gy):
    nb, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    gx = np.empty_like(x); gdt = np.empty_like(dt); gA = np.empty_like(A)
    gB = np.empty_like(Bm); gC = np.empty_like(Cm)
    fn = lib().orc_ssd_reverse_f64
    fn.restype = None
    fn(_p(x), _p(dt), _p(A), _p(Bm), _p(Cm), _p(gy), _p(gx), _p(gdt), _p(gA), _p(gB), _p(gC),
       *(C.c_size_t(v) for v in (nb, L, H, P, N, G)))
    return gx, gdt, gA, gB, gC


# ---------------------------------------------------------------------------
# Operators around the scan in a language-model step (numpy float64, written
# from the definitions in include/mp_kernels.h; no reference file exists).
# ---------------------------------------------------------------------------
def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def embedding(table, ids):
    out = np.zeros((len(ids), table.shape[1]), dtype=np.float64)
    ok = (ids >= 0) & (ids < table.shape[0])
    out[ok] = table[ids[ok]]
    return out


def embedding_reverse(ids, gy, vocab):
    g = np.zeros((vocab, gy.shape[1]), dtype=np.float64)
    ok = (ids >= 0) & (ids < vocab)
    np.add.at(g, ids[ok], gy[ok].astype(np.float64))
    return g


def _conv_pre(x, w, bias):
    nb, L, Cn = x.shape
    W = w.shape[1]
    xp = np.concatenate([np.zeros((nb, W - 1, Cn)), x.astype(np.float64)], axis=1)
    pre = np.zeros((nb, L, Cn)) + (0.0 if bias is None else bias.astype(np.float64))
    for k in range(W):
        pre += w[:, k].astype(np.float64) * xp[:, k:k + L, :]
    return pre, xp


def causal_conv1d_silu(x, w, bias):
    pre, _ = _conv_pre(x, w, bias)
    return pre * _sigmoid(pre)


def causal_conv1d_silu_reverse(x, w, bias, gy):
    nb, L, Cn = x.shape
    W = w.shape[1]
    pre, xp = _conv_pre(x, w, bias)
    s = _sigmoid(pre)
    dpre = gy.astype(np.float64) * s * (1.0 + pre * (1.0 - s))
    dpad = np.concatenate([dpre, np.zeros((nb, W - 1, Cn))], axis=1)
    gx = np.zeros((nb, L, Cn))
    gw = np.zeros((Cn, W))
    for k in range(W):
        gx += w[:, k].astype(np.float64) * dpad[:, W - 1 - k:W - 1 - k + L, :]
        gw[:, k] = np.sum(dpre * xp[:, k:k + L, :], axis=(0, 1))
    return gx, gw, dpre.sum(axis=(0, 1))


def softplus_bias(raw, bias):
    v = raw.astype(np.float64) + bias.astype(np.float64)
    return np.where(v > 20.0, v, np.log1p(np.exp(np.minimum(v, 20.0))))


def softplus_bias_reverse(raw, bias, gdt):
    g = gdt.astype(np.float64) * _sigmoid(raw.astype(np.float64) + bias.astype(np.float64))
    return g, g.sum(axis=0)


def ssd_gate(y, x, D, z, heads, headdim):
    d = np.repeat(D.astype(np.float64), headdim)
    return (y + d * x) * z * _sigmoid(z)


def ssd_gate_reverse(y, x, D, z, gu, heads, headdim):
    d = np.repeat(D.astype(np.float64), headdim)
    s = _sigmoid(z)
    gy = gu * z * s
    gz = gu * (y + d * x) * (s + z * s * (1.0 - s))
    gD = (gy * x).reshape(-1, heads, headdim).sum(axis=(0, 2))
    return gy, gz, gD


def cross_entropy(logits, targets, scale):
    x = logits.astype(np.float64)
    m, n = x.shape
    mx = x.max(axis=1, keepdims=True)
    e = np.exp(x - mx)
    s = e.sum(axis=1, keepdims=True)
    valid = (targets >= 0) & (targets < n)
    tg = np.where(valid, targets, 0)
    loss = np.where(valid, np.log(s[:, 0]) + mx[:, 0] - x[np.arange(m), tg], 0.0)
    g = e / s
    g[np.arange(m), tg] -= 1.0
    g = np.where(valid[:, None], g * scale, 0.0)
    return loss, g


def mse_loss(x, t):
    d = x.astype(np.float64) - t.astype(np.float64)
    return float(np.mean(d * d)), 2.0 * d / d.size


def bce_loss(p, t):
    p64, t64 = p.astype(np.float64), t.astype(np.float64)
    pc = np.clip(p64, 1e-12, 1 - 1e-12)
    return float(-np.mean(t64 * np.log(pc) + (1 - t64) * np.log(1 - pc))), (p64 - t64) / p64.size


def momentum(w, g, m, rate, alpha, lo=-np.inf, hi=np.inf):
    m2 = alpha * m.astype(np.float64) + np.clip(g.astype(np.float64), lo, hi)
    return w.astype(np.float64) - rate * m2, m2
