"""Shared helpers of the parity tests: error metric, dtype tables, uploads."""
import numpy as np

# tolerances of the north star: r32 element-wise 1e-5, r32 reductions / scans /
# contractions 1e-4, r16 1e-2 (against the fp64 oracle rounded to r16)
TOL_EW = {"r16": 1e-2, "r32": 1e-5, "r64": 1e-12}
TOL_RED = {"r16": 1e-2, "r32": 1e-4, "r64": 1e-10}
NP_OF = {"r16": np.float16, "r32": np.float32, "r64": np.float64}


def torch_dtype(sfx):
    import torch
    return {"r16": torch.float16, "r32": torch.float32, "r64": torch.float64}[sfx]


def wide(a: np.ndarray) -> np.ndarray:
    """Array in the precision the oracle runs in for this dtype."""
    return np.ascontiguousarray(a.astype(np.float64) if a.dtype == np.float16 else a)


def narrow(a: np.ndarray, sfx: str) -> np.ndarray:
    return a.astype(NP_OF[sfx])


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max|got-ref| / max(max|ref|, tiny), in float64."""
    g = np.asarray(got, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    if g.size == 0:
        return 0.0
    denom = max(float(np.max(np.abs(r))), 1e-30)
    return float(np.max(np.abs(g - r))) / denom


def assert_close(got, ref, tol, what=""):
    g = np.asarray(got, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    assert g.shape == r.shape, (what, g.shape, r.shape)
    assert np.all(np.isfinite(g)) or not np.all(np.isfinite(r)), f"{what}: non-finite output"
    e = rel_err(g, r)
    assert e <= tol, f"{what}: rel err {e:.3e} > {tol:.1e}"
    if g.size:
        mx = float(np.max(np.abs(r)))
        bad = np.abs(g - r) > tol * (np.abs(r) + mx) + 1e-300
        assert not bad.any(), f"{what}: {int(bad.sum())} elements outside tol*(|ref|+max|ref|)"


def dev(a: np.ndarray):
    """Upload a numpy array (float16/32/64) as a CUDA tensor."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t) -> np.ndarray:
    return t.detach().cpu().numpy()


def rng_normal(seed, shape, sfx, scale=1.0, loc=0.0):
    r = np.random.default_rng(seed)
    return (r.standard_normal(shape) * scale + loc).astype(np.float32).astype(NP_OF[sfx])


def rng_uniform(seed, shape, sfx, lo=-1.0, hi=1.0):
    r = np.random.default_rng(seed)
    return r.uniform(lo, hi, shape).astype(np.float32).astype(NP_OF[sfx])


def run(mp, stream, name, sfx, *args):
    """Launch through the C ABI on the library's stream and wait for it.  The
    stream is non-blocking, so work torch queued on its own stream (uploads,
    random fills) is drained first."""
    import torch
    torch.cuda.current_stream().synchronize()
    mp.launch(name, torch_dtype(sfx), *args, stream)
    stream.sync()
