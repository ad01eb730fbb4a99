"""Benchmark cases shared by `bench.py` (the `per_config` block of its JSON line)
and by `bench.py --profile-case` (ncu captures and single-kernel timings).

Every case is a small object with
    once()   one launch of the kernel (or launcher) through the C ABI
    work     algorithmic work of one launch: {"bytes": B} and / or {"flops": F}
    bound    "hbm" | "tensor" | "both" | "latency"
Timing is `time_case`: CUDA events on the library's stream around every single
launch, the L2 flushed (256 MiB fill) before each one unless the inputs exceed
the L2 by themselves.

Baselines next to each case (reported, not optimised):
    cpu_*    the scalar C oracle (oracle/liboracle.so) on a bounded sample
    ref_*    the reference's own CUDA kernels (oracle/_ref/libref_kernels.so,
             built unmodified by oracle/build_ref.py) where the reference has one
"""
from __future__ import annotations

import ctypes as C
import json
import math
import os
import statistics
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent

L2_BYTES = 126 * 1024 * 1024
EPS = 1e-6


def peaks():
    """(hbm GB/s, bf16 TFLOP/s burst, bf16 TFLOP/s sustained, 'measured' | 'fallback')."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, 1400.0, "fallback"


class Flusher:
    """Writes a buffer twice the size of the L2 on the given stream, then reads it once (row sums): the write evicts the
    timed kernel's inputs, the read pass leaves the L2 full of CLEAN lines.  Without the read pass the timed kernel
    also pays for writing back up to 126 MB of the flush's dirty lines, which for a 30 us kernel is most of its time."""

    def __init__(self, mp, stream):
        import torch
        self.mp, self.stream = mp, stream
        self.rows, self.cols = 4096, 2 * L2_BYTES // 4 // 4096
        self.buf = torch.empty(self.rows * self.cols, dtype=torch.float32, device="cuda")
        self.sums = torch.empty(self.rows, dtype=torch.float32, device="cuda")

    def __call__(self):
        import torch
        self.mp.launch("fill", torch.float32, self.buf, 0.0, self.buf.numel(), self.stream)
        self.mp.launch("reduce_ij_i", torch.float32, self.buf, self.sums, 0.0, self.rows, self.cols, self.stream)


def time_case(once, stream, iters=10, warmup=3, flush=None):
    """Mean and minimum device time (ms) of `once()`, one CUDA-event pair per launch."""
    import torch
    ts = stream.torch_stream()
    for _ in range(warmup):
        once()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in evs:
        if flush is not None:
            flush()
        a.record(ts)
        once()
        b.record(ts)
    stream.sync()
    if stream.status() != 0:
        raise SystemExit("a kernel reported a non-zero status word")
    t = [a.elapsed_time(b) for a, b in evs]
    return statistics.mean(t), min(t)


def rate_record(ms, work, bound, tensor_peak=None):
    """Achieved rate and roofline fraction of one launch that took `ms`."""
    hbm, burst, sustained, kind = peaks()
    tensor_peak = tensor_peak if tensor_peak is not None else burst
    out = {"us": round(ms * 1e3, 2), "bound": bound, "peak_kind": kind}
    t_roof = 0.0
    if "bytes" in work:
        out["GB/s"] = round(work["bytes"] / (ms * 1e-3) / 1e9, 1)
        out["algorithmic_bytes"] = work["bytes"]
        t_roof = max(t_roof, work["bytes"] / (hbm * 1e9))
    if "flops" in work:
        out["TFLOP/s"] = round(work["flops"] / (ms * 1e-3) / 1e12, 1)
        out["algorithmic_flops"] = work["flops"]
        t_roof = max(t_roof, work["flops"] / (tensor_peak * 1e12))
    if bound == "hbm":
        out["achieved"], out["peak"], out["unit"] = out["GB/s"], hbm, "GB/s"
        out["frac"] = round(out["GB/s"] / hbm, 4)
    elif bound == "tensor":
        out["achieved"], out["peak"], out["unit"] = out["TFLOP/s"], tensor_peak, "TFLOP/s"
        out["frac"] = round(out["TFLOP/s"] / tensor_peak, 4)
    elif bound == "both":      # roofline time = the slower of the HBM and the tensor-pipe time
        out["roofline_us"] = round(t_roof * 1e6, 2)
        out["frac"] = round(t_roof / (ms * 1e-3), 4)
        out["peak"] = {"hbm_GB/s": hbm, "tensor_TFLOP/s": tensor_peak}
    return out


class Case:
    def __init__(self, once, work, bound, note="", tensor_peak=None, big=False, keep=()):
        self.once, self.work, self.bound, self.note = once, work, bound, note
        self.tensor_peak = tensor_peak
        self.big = big            # inputs exceed the L2: no flush needed
        self.keep = keep          # tensors that must stay alive

    def measure(self, stream, flush, iters=10):
        ms, _ = time_case(self.once, stream, iters=iters, flush=None if self.big else flush)
        return rate_record(ms, self.work, self.bound, self.tensor_peak)


# ----------------------------------------------------------------------------
# case builders (seeded synthetic inputs with the shapes and distributions of the configs)
# ----------------------------------------------------------------------------
def _gen(seed=0):
    import torch
    return torch.Generator(device="cuda").manual_seed(seed)


def _dt(sfx):
    import torch
    return {"r16": torch.float16, "r32": torch.float32, "r64": torch.float64}[sfx]


def rows_case(mp, s, op, sfx, m, n):
    """softmax_fwd | softmax_rev | rmsnorm_fwd | rmsnorm_rev over [m, n] (configs[1])."""
    import torch
    g, dt = _gen(1), _dt(sfx)
    size = torch.empty(0, dtype=dt).element_size()
    x = torch.randn(m, n, generator=g, device="cuda").to(dt); gy = torch.randn(m, n, generator=g, device="cuda").to(dt)
    y = torch.empty_like(x); gx = torch.empty_like(x)
    gain = (1 + 0.02 * torch.randn(n, generator=g, device="cuda")).to(dt); gg = torch.empty_like(gain)
    scratch = torch.empty(mp.lib().mpRmsnormReverseScratchBytes(m, n, s.ctx), dtype=torch.uint8, device="cuda")
    mn = m * n * size
    if op == "softmax_fwd":
        once = lambda: mp.launch("softmax_ij_j", dt, x, y, m, n, s); nb = 2 * mn
    elif op == "softmax_rev":
        mp.launch("softmax_ij_j", dt, x, y, m, n, s)
        once = lambda: mp.launch("softmax_ij_j_reverse", dt, y, gy, gx, 0.0, m, n, s); nb = 3 * mn
    elif op == "rmsnorm_fwd":
        once = lambda: mp.launch("rmsnorm_ij_j", dt, x, gain, EPS, y, None, m, n, s); nb = 2 * mn + n * size
    elif op == "rmsnorm_rev":
        once = lambda: mp.launch("rmsnorm_ij_j_reverse", dt, x, gain, None, gy, EPS, gx, gg, 0.0, scratch, m, n, s)
        nb = 3 * mn + 2 * n * size
    else:
        raise SystemExit(f"unknown row op {op}")
    return Case(once, {"bytes": nb}, "hbm", big=mn > L2_BYTES, keep=(x, gy, y, gx, gain, gg, scratch))


CHAIN_EXPR = "selu((a+b)*(c+d))"


def chain_case(mp, s, op, sfx, n, seed_ones=False):
    """chain_fwd | chain_rev: e = selu((a+b)*(c+d)) and its reverse over n elements (configs[2])."""
    import torch
    g, dt = _gen(0), _dt(sfx)
    size = torch.empty(0, dtype=dt).element_size()
    leaves = [(torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dt) for _ in range(4)]
    chain = mp.FusedChain(CHAIN_EXPR, dt)
    if op == "chain_fwd":
        out = torch.empty_like(leaves[0])
        return Case(lambda: chain.forward(leaves, out, n, s), {"bytes": 5 * n * size}, "hbm", big=n * size > L2_BYTES,
                    keep=(leaves, out, chain))
    grads = [torch.empty_like(leaves[0]) for _ in range(4)]
    ge = None if seed_ones else torch.randn(n, generator=g, device="cuda").to(dt)
    nb = (8 if seed_ones else 9) * n * size
    return Case(lambda: chain.reverse(leaves, ge, grads, 0.0, n, s), {"bytes": nb}, "hbm", big=n * size > L2_BYTES,
                keep=(leaves, grads, ge, chain))


SSD_SHAPE = dict(H=32, P=64, NS=128, G=1, Q=256)


def ssd_flops(nb, L, H, P, NS, G, Q, reverse):
    """Algorithmic flops of the chunked scan (scores counted once per group)."""
    chunks = nb * L // Q
    if not reverse:
        return 2 * Q * Q * NS * chunks * G + (2 * Q * Q * P + 4 * Q * NS * P) * chunks * H
    return (4 * Q * Q * P + 8 * Q * NS * P) * chunks * H + 4 * Q * Q * NS * chunks * G


def ssd_bytes(nb, L, H, P, NS, G, reverse):
    x = nb * L * H * P * 2; bc = nb * L * G * NS * 2; dt = nb * L * H * 4
    if not reverse:
        return 2 * x + 2 * bc + dt                      # read x, B, C, dt; write y
    return (2 * x + 2 * bc + dt) + (x + 2 * bc + dt)    # read x, gy, B, C, dt; write gx, gB, gC, gdt (gA negligible)


def ssd_inputs(nb, L, H, P, NS, G, seed=0):
    import torch
    g = _gen(seed)
    x = torch.randn(nb, L, H, P, generator=g, device="cuda").half()
    Bm = torch.randn(nb, L, G, NS, generator=g, device="cuda").half()
    Cm = torch.randn(nb, L, G, NS, generator=g, device="cuda").half()
    dtv = torch.nn.functional.softplus(torch.randn(nb, L, H, generator=g, device="cuda") - 4)
    Av = -torch.exp(torch.rand(H, generator=g, device="cuda") * math.log(16))
    gy = torch.randn(nb, L, H, P, generator=g, device="cuda").half()
    return x, dtv, Av, Bm, Cm, gy


def ssd_case(mp, s, op, nb, L, H=32, P=64, NS=128, G=1, Q=256):
    """ssd_fwd | ssd_rev at [nb, L, H, P], d_state NS, G groups, chunk Q (configs[3] = 8, 8192, 32, 64, 128, 1, 256)."""
    import torch
    x, dtv, Av, Bm, Cm, gy = ssd_inputs(nb, L, H, P, NS, G)
    dims = (nb, L, H, P, NS, G, Q)
    rev = op == "ssd_rev"
    scr = torch.empty(mp.lib().mpSsdScanScratchBytes(*dims, 1 if rev else 0), dtype=torch.uint8, device="cuda")
    work = {"flops": ssd_flops(nb, L, H, P, NS, G, Q, rev), "bytes": ssd_bytes(nb, L, H, P, NS, G, rev)}
    if rev:
        gx = torch.empty_like(x); gdt = torch.empty_like(dtv); gA = torch.empty_like(Av)
        gB = torch.empty_like(Bm); gC = torch.empty_like(Cm)
        once = lambda: mp.launch("ssd_scan_reverse", torch.float16, x, dtv, Av, Bm, Cm, gy, gx, gdt, gA, gB, gC, scr, *dims, s)
        keep = (x, dtv, Av, Bm, Cm, gy, gx, gdt, gA, gB, gC, scr)
    else:
        y = torch.empty_like(x)
        once = lambda: mp.launch("ssd_scan", torch.float16, x, dtv, Av, Bm, Cm, y, scr, *dims, s)
        keep = (x, dtv, Av, Bm, Cm, y, scr)
    c = Case(once, work, "both", big=work["bytes"] > L2_BYTES, keep=keep)
    c.scratch_bytes = scr.numel()
    return c


def gemm_case(mp, s, sfx, m, n, k, form="nn"):
    """C[m,n] = A·B with inner size k; form nn: A[m,k] B[k,n]; nt: A[m,k] B[n,k]; tn: A[k,m] B[k,n]."""
    import torch
    g, dt = _gen(0), _dt(sfx)
    sc = 1.0 / math.sqrt(k)
    a = torch.randn((k, m) if form == "tn" else (m, k), generator=g, device="cuda").to(dt)
    b = (torch.randn((n, k) if form == "nt" else (k, n), generator=g, device="cuda") * sc).to(dt)
    c = torch.empty(m, n, device="cuda", dtype=dt)
    name = {"nn": "inner_product_ij_jk_ik", "nt": "inner_product_ij_kj_ik", "tn": "inner_product_ji_jk_ik"}[form]
    once = lambda: mp.launch(name, dt, a, b, 1.0, c, 0.0, m, k, n, s)
    _, burst, sustained, _ = peaks()
    # r32 runs three tf32 MMAs per product on a pipe with half the 16-bit rate: useful ceiling = peak / 2 / 3
    tp = burst if sfx == "r16" else burst / 6.0
    nbytes = (a.numel() + b.numel() + c.numel()) * a.element_size()
    return Case(once, {"flops": 2.0 * m * n * k}, "tensor", tensor_peak=tp, big=nbytes > 2 * L2_BYTES, keep=(a, b, c))


def bmm_case(mp, s, sfx, nb, n):
    import torch
    g, dt = _gen(0), _dt(sfx)
    a = torch.randn(nb, n, n, generator=g, device="cuda").to(dt); b = (torch.randn(nb, n, n, generator=g, device="cuda") / 32).to(dt)
    c = torch.empty(nb, n, n, device="cuda", dtype=dt)
    once = lambda: mp.launch("inner_product_bij_bjk_bik", dt, a, b, 1.0, c, 0.0, nb, n, n, n, s)
    _, burst, _, _ = peaks()
    return Case(once, {"flops": 2.0 * nb * n * n * n}, "tensor", tensor_peak=burst if sfx == "r16" else burst / 6.0,
                big=3 * a.numel() * a.element_size() > 2 * L2_BYTES, keep=(a, b, c))


def conv_case(mp, s, op, sfx, nb, L):
    """conv_fwd | conv_rev | conv_rev_skip: the segmented causal convolution over the 1792 [x | B | C] columns of a Mamba-2 block."""
    import torch
    g, dt = _gen(0), _dt(sfx)
    widths, dip, di, W = (1536, 128, 128), 3352, 1536, 4
    Cn = sum(widths)
    zx = torch.randn(nb * L, dip, generator=g, device="cuda").to(dt); gzx = torch.empty_like(zx)
    w = torch.randn(Cn, W, generator=g, device="cuda").to(dt); bias = torch.randn(Cn, generator=g, device="cuda").to(dt)
    outs = [torch.randn(nb * L, cw, generator=g, device="cuda").to(dt) for cw in widths]
    gw = torch.zeros(Cn, W, device="cuda"); gb = torch.zeros(Cn, device="cuda")
    ptrs = (C.c_void_p * 3)(*[t.data_ptr() for t in outs]); cw = (C.c_ulong * 3)(*widths)
    esz = zx.element_size()
    if op == "conv_fwd":
        once = lambda: mp.launch("causal_conv1d_silu_segments", dt, zx.data_ptr() + di * esz, dip, w, bias, ptrs, cw, cw, 3, nb, L, W, s)
        nbytes = 2 * nb * L * Cn * esz
    elif op == "conv_rev_skip":   # with the scan's D skip (scale per 64-channel head) joining the x segment's upstream gradient
        skip = torch.randn(nb * L, widths[0], generator=g, device="cuda").to(dt)
        D = torch.randn(widths[0] // 64, generator=g, device="cuda")
        sp = (C.c_void_p * 3)(skip.data_ptr(), None, None); spitch = (C.c_ulong * 3)(widths[0], 0, 0)
        sc = (C.c_void_p * 3)(D.data_ptr(), None, None)
        once = lambda: mp.launch("causal_conv1d_silu_segments_reverse_skip", dt, zx.data_ptr() + di * esz, dip, w, bias, ptrs, cw, cw, 3,
                                 sp, spitch, sc, 64, gzx.data_ptr() + di * esz, dip, gw, gb, nb, L, W, s)
        nbytes = (3 * Cn + widths[0]) * nb * L * esz
        outs = outs + [skip, D, sp, spitch, sc]
    else:
        once = lambda: mp.launch("causal_conv1d_silu_segments_reverse", dt, zx.data_ptr() + di * esz, dip, w, bias, ptrs, cw, cw, 3,
                                 gzx.data_ptr() + di * esz, dip, gw, gb, nb, L, W, s)
        nbytes = 3 * nb * L * Cn * esz
    return Case(once, {"bytes": nbytes}, "hbm", big=nbytes > 2 * L2_BYTES, keep=(zx, gzx, w, bias, outs, gw, gb, ptrs, cw))


def gated_norm_case(mp, s, op, sfx, rows, H=24, P=64):
    """gated_norm_fwd | gated_norm_rev: skip + gate + RMSNorm in one kernel on [rows, H x P] with z inside a wider
    projection output; gate_unfused_fwd | gate_unfused_rev: the same work as ssd_gate + rmsnorm (two launches each way)."""
    import torch
    g, dt = _gen(0), _dt(sfx)
    width, dip = H * P, 2 * H * P + 2 * 128 + H
    dip += (-dip) % 8
    rn = lambda *shape: torch.randn(*shape, generator=g, device="cuda").to(dt)
    y, x, gout, zx, gain = rn(rows, width), rn(rows, width), rn(rows, width), rn(rows, dip), rn(width)
    out, gy, gzx, u, gu = (torch.empty_like(t) for t in (y, y, zx, y, y))
    ggain = torch.empty_like(gain)
    D = torch.randn(H, generator=g, device="cuda"); gD = torch.zeros(H, device="cuda")
    rstd = torch.rand(rows, generator=g, device="cuda") + 0.5
    nscr = max(mp.lib().mpSsdGateRmsnormReverseScratchBytes(rows, H, P, s.ctx), mp.lib().mpRmsnormReverseScratchBytes(rows, width, s.ctx))
    scratch = torch.empty(max(nscr, 16), dtype=torch.uint8, device="cuda")
    esz = y.element_size()
    if op == "gated_norm_fwd":
        once = lambda: mp.launch("ssd_gate_rmsnorm", dt, y, x, D, zx, dip, gain, 1e-5, out, rstd, rows, H, P, s)
        nbytes = 4 * rows * width * esz
    elif op == "gated_norm_rev":
        once = lambda: mp.launch("ssd_gate_rmsnorm_reverse", dt, y, x, D, zx, dip, gain, rstd, gout, gy, gzx, dip, gD, ggain, 0.0, scratch,
                                 rows, H, P, s)
        nbytes = 6 * rows * width * esz
    elif op == "gate_unfused_fwd":
        def once():
            mp.launch("ssd_gate", dt, y, x, D, zx, dip, u, rows, H, P, s)
            mp.launch("rmsnorm_ij_j", dt, u, gain, 1e-5, out, rstd, rows, width, s)
        nbytes = 4 * rows * width * esz    # algorithmic bytes of the fused operator; the two launches move 6 tensors
    else:
        def once():
            mp.launch("rmsnorm_ij_j_reverse", dt, u, gain, rstd, gout, 1e-5, gu, ggain, 0.0, scratch, rows, width, s)
            mp.launch("ssd_gate_reverse", dt, y, x, D, zx, dip, gu, gy, gzx, dip, gD, rows, H, P, s)
        nbytes = 6 * rows * width * esz
    return Case(once, {"bytes": nbytes}, "hbm", big=nbytes > 2 * L2_BYTES,
                keep=(y, x, gout, zx, gain, out, gy, gzx, u, gu, ggain, D, gD, rstd, scratch))


def permute_case(mp, s, op, sfx, nb, L):
    import torch
    g, dt = _gen(0), _dt(sfx)
    shape = (nb, L, 32, 128)
    perm = (0, 2, 1, 3) if op == "permute_heads" else (3, 2, 1, 0)
    x = torch.randn(shape, generator=g, device="cuda").to(dt); y = torch.empty_like(x)
    sizes = (C.c_ulong * 4)(*shape); pm = (C.c_ulong * 4)(*perm)
    once = lambda: mp.launch("permutate", dt, x, y, 0.0, sizes, pm, 4, s)
    nbytes = 2 * x.numel() * x.element_size()
    return Case(once, {"bytes": nbytes}, "hbm", big=nbytes > 2 * L2_BYTES, keep=(x, y, sizes, pm))


def transpose_case(mp, s, sfx, m, n):
    import torch
    g, dt = _gen(0), _dt(sfx)
    x = torch.randn(m, n, generator=g, device="cuda").to(dt); y = torch.empty(n, m, device="cuda", dtype=dt)
    once = lambda: mp.launch("permutate_ij_ji", dt, x, y, 0.0, m, n, s)
    nbytes = 2 * x.numel() * x.element_size()
    return Case(once, {"bytes": nbytes}, "hbm", big=nbytes > 2 * L2_BYTES, keep=(x, y))


def adam_case(mp, s, n):
    import torch
    g = _gen(0)
    w = torch.randn(n, generator=g, device="cuda"); gr = torch.randn(n, generator=g, device="cuda")
    m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    once = lambda: mp.launch("adam", torch.float32, w, gr, m, v, 3e-4, 0.9, 0.95, 1e-8, 1.0, 1, n, s)
    return Case(once, {"bytes": 28 * n}, "hbm", big=True, keep=(w, gr, m, v))


def build_case(mp, s, spec: str) -> Case:
    """OP:DTYPE:SIZES...  (the grammar of `bench.py --profile-case`)."""
    parts = spec.split(":")
    op, sfx = parts[0], parts[1]
    nums = [int(p) for p in parts[2:] if p.isdigit()]
    tail = [p for p in parts[2:] if not p.isdigit()]
    if op in ("softmax_fwd", "softmax_rev", "rmsnorm_fwd", "rmsnorm_rev"):
        return rows_case(mp, s, op, sfx, nums[0], nums[1] if len(nums) > 1 else 4096)
    if op in ("chain_fwd", "chain_rev"):
        return chain_case(mp, s, op, sfx, nums[0], seed_ones="ones" in tail)
    if op in ("ssd_fwd", "ssd_rev"):
        kw = dict(zip(("H", "P", "NS", "G", "Q"), nums[2:]))
        return ssd_case(mp, s, op, nums[0], nums[1], **kw)
    if op == "gemm":
        if len(nums) == 2:
            return gemm_case(mp, s, sfx, nums[0], nums[1], nums[1])
        return gemm_case(mp, s, sfx, nums[0], nums[1], nums[2], tail[0] if tail else "nn")
    if op == "bmm":
        return bmm_case(mp, s, sfx, nums[0], nums[1])
    if op in ("conv_fwd", "conv_rev", "conv_rev_skip"):
        return conv_case(mp, s, op, sfx, nums[0], nums[1])
    if op in ("gated_norm_fwd", "gated_norm_rev", "gate_unfused_fwd", "gate_unfused_rev"):
        return gated_norm_case(mp, s, op, sfx, nums[0], *nums[1:3])
    if op in ("permute_heads", "permute_reverse"):
        return permute_case(mp, s, op, sfx, nums[0], nums[1])
    if op == "transpose":
        return transpose_case(mp, s, sfx, nums[0], nums[1])
    if op == "adam":
        return adam_case(mp, s, nums[0])
    raise SystemExit(f"unknown profile case {op}")


# ----------------------------------------------------------------------------
# reference-CUDA baseline (oracle/_ref/libref_kernels.so)
# ----------------------------------------------------------------------------
class RefCuda:
    """The reference's own kernels, timed on their own stream with CUDA events."""

    def __init__(self):
        from oracle.refkernels import RefLib
        self.ref = RefLib()
        self.ts = self.ref.torch_stream()

    def launch(self, name, sfx, *args):
        conv = [C.c_void_p(a.data_ptr()) if hasattr(a, "data_ptr") else a for a in args]
        getattr(self.ref.lib, f"launch_{name}_{sfx}")(*conv, self.ref.ctx)

    def time(self, once, iters=5, warmup=2, flush_buf=None):
        import torch
        torch.cuda.synchronize()
        for _ in range(warmup):
            once()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for a, b in evs:
            if flush_buf is not None:
                self.launch("fill", "r32", flush_buf, C.c_double(0.0), C.c_ulong(flush_buf.numel()))
            a.record(self.ts)
            once()
            b.record(self.ts)
        self.ref.lib.mpStreamSynchronize(self.ref.ctx)
        return statistics.mean(a.elapsed_time(b) for a, b in evs)

    def close(self):
        self.ref.close()


def ref_cuda_or_none():
    try:
        return RefCuda()
    except Exception as e:       # the shared object was not built (no reference checkout at build time)
        return str(e)


# ----------------------------------------------------------------------------
# per-config measurements
# ----------------------------------------------------------------------------
D, UL = C.c_double, C.c_ulong


def _threads():
    return os.cpu_count() or 1


def _pool_time(work, chunks, threads):
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as pool:
        list(pool.map(work, chunks))
    return time.perf_counter() - t0


def config_rows(mp, s, flush, m=65536, n=4096, cpu_rows=8192):
    """configs[1]: softmax and RMSNorm forward + reverse over X[65536, 4096], r32 and r16."""
    import numpy as np
    import torch
    from oracle import pyoracle as orc
    out = {"workload": f"softmax + RMSNorm (eps 1e-6) forward+reverse over X[{m},{n}], r32 and r16, gradients overwritten",
           "kernels": {}}
    tot_ms = tot_b = 0.0
    for sfx in ("r32", "r16"):
        for op in ("softmax_fwd", "softmax_rev", "rmsnorm_fwd", "rmsnorm_rev"):
            c = rows_case(mp, s, op, sfx, m, n)
            r = c.measure(s, flush)
            out["kernels"][f"{op}_{sfx}"] = r
            tot_ms += r["us"] * 1e-3; tot_b += c.work["bytes"]
            del c
            torch.cuda.empty_cache()
    hbm = peaks()[0]
    out["achieved"] = round(tot_b / (tot_ms * 1e-3) / 1e9, 1); out["unit"] = "GB/s"; out["peak"] = hbm
    out["frac"] = round(out["achieved"] / hbm, 4)
    # CPU oracle on the first cpu_rows rows
    threads = _threads()
    r = np.random.default_rng(0)
    x = r.standard_normal((cpu_rows, n)).astype(np.float32); gy = r.standard_normal((cpu_rows, n)).astype(np.float32)
    gain = (1 + 0.02 * r.standard_normal(n)).astype(np.float32)
    bounds = [(cpu_rows * i // threads, cpu_rows * (i + 1) // threads) for i in range(threads)]

    def work(b):
        xs, gs = x[b[0]:b[1]], gy[b[0]:b[1]]
        y = orc.softmax_ij_j(xs); orc.softmax_ij_j_reverse(y, gs)
        orc.rmsnorm_ij_j(xs, gain, EPS); orc.rmsnorm_ij_j_reverse(xs, gain, gs, EPS)
    orc.lib()
    dt = _pool_time(work, bounds, threads)
    nb = 10 * cpu_rows * n * 4     # 2 + 3 + 2 + 3 passes of r32
    out["cpu_baseline"] = {"value": round(nb / dt / 1e9, 2), "unit": "GB/s", "cores": threads, "kind": "port",
                           "sample": f"first {cpu_rows} rows, the four r32 kernels once, scalar C oracle, {dt:.2f} s"}
    out["ref_cuda"] = "no reference kernel (the reference has neither softmax nor RMSNorm)"
    return out


def config_chain(mp, s, flush, n=1 << 28, cpu_n=1 << 24, ref=None):
    """configs[2]: e = selu((a+b)*(c+d)) and its reverse over four r32 tensors of 2^28 elements."""
    import numpy as np
    import torch
    from oracle import pyoracle as orc
    out = {"workload": f"fused chain e = {CHAIN_EXPR} forward and reverse, four r32 leaves of {n} elements ~U(-1,1)"}
    c = chain_case(mp, s, "chain_fwd", "r32", n)
    out["forward"] = c.measure(s, flush, iters=5)
    leaves = c.keep[0]
    # reference CUDA: the unfused forward it can express (two additions and a hadamard; it has no SELU kernel)
    if isinstance(ref, RefCuda):
        t1 = torch.empty_like(leaves[0]); t2 = torch.empty_like(leaves[0]); t3 = torch.empty_like(leaves[0])

        def ref_fwd():
            ref.launch("addition", "r32", leaves[0], leaves[1], t1, UL(n))
            ref.launch("addition", "r32", leaves[2], leaves[3], t2, UL(n))
            ref.launch("hadamard", "r32", t1, t2, t3, UL(n))
        ms = ref.time(ref_fwd, iters=3)
        out["ref_cuda"] = {"forward_us": round(ms * 1e3, 1), "kernels": "launch_addition_r32 x2 + launch_hadamard_r32 (no SELU kernel in the reference)",
                           "GB/s_of_fused_algorithmic_bytes": round(5 * n * 4 / (ms * 1e-3) / 1e9, 1),
                           "unfused_bytes_moved": 9 * n * 4,
                           "reverse": "reference accumulate kernels are invalid at this size (32-bit thread index wraps for N >= 2^27); timed at 2^26 below"}
        del t1, t2, t3
    else:
        out["ref_cuda"] = f"unavailable: {ref}"
    del c, leaves
    torch.cuda.empty_cache()
    c = chain_case(mp, s, "chain_rev", "r32", n)
    out["reverse"] = c.measure(s, flush, iters=5)
    del c
    torch.cuda.empty_cache()
    c = chain_case(mp, s, "chain_rev", "r32", n, seed_ones=True)
    out["reverse_ones_seed"] = c.measure(s, flush, iters=5)
    del c
    torch.cuda.empty_cache()
    if isinstance(ref, RefCuda):
        # the (a+b)*(c+d) part of the reverse with the reference's kernels at 2^26 (valid there):
        # g_t1 += g*t2, g_t2 += g*t1 (hadamard_reverse), then g_a += g_t1 ... as in-place additions
        n2 = 1 << 26
        g = _gen(5)
        t1 = torch.rand(n2, generator=g, device="cuda"); t2 = torch.rand(n2, generator=g, device="cuda"); gg = torch.randn(n2, generator=g, device="cuda")
        g1 = torch.zeros(n2, device="cuda"); g2 = torch.zeros(n2, device="cuda")
        ga = [torch.zeros(n2, device="cuda") for _ in range(4)]

        def ref_rev():
            ref.launch("hadamard_reverse", "r32", gg, t2, g1, UL(n2))
            ref.launch("hadamard_reverse", "r32", gg, t1, g2, UL(n2))
            ref.launch("addition", "r32", g1, ga[0], ga[0], UL(n2)); ref.launch("addition", "r32", g1, ga[1], ga[1], UL(n2))
            ref.launch("addition", "r32", g2, ga[2], ga[2], UL(n2)); ref.launch("addition", "r32", g2, ga[3], ga[3], UL(n2))
        ms = ref.time(ref_rev, iters=3)
        cr = chain_case(mp, s, "chain_rev", "r32", n2)
        ours = cr.measure(s, flush, iters=5)
        out["ref_cuda"]["reverse_2p26"] = {"ref_us": round(ms * 1e3, 1), "ours_us": ours["us"],
                                           "kernels": "launch_hadamard_reverse_r32 x2 + in-place launch_addition_r32 x4 (SELU reverse missing in the reference)"}
        del cr, t1, t2, gg, g1, g2, ga
        torch.cuda.empty_cache()
    # CPU oracle, forward + reverse on cpu_n elements
    threads = _threads()
    r = np.random.default_rng(0)
    a, b, cc, d = [r.uniform(-1, 1, cpu_n).astype(np.float32) for _ in range(4)]
    ge = r.standard_normal(cpu_n).astype(np.float32)
    bounds = [(cpu_n * i // threads, cpu_n * (i + 1) // threads) for i in range(threads)]

    def work(bd):
        sl = slice(bd[0], bd[1])
        t1 = orc.addition(a[sl], b[sl]); t2 = orc.addition(cc[sl], d[sl]); t3 = orc.hadamard(t1, t2); orc.selu(t3)
        g3 = np.zeros_like(t3); orc.selu_reverse(t3, g3, np.ascontiguousarray(ge[sl]))
        g1 = np.zeros_like(t3); g2 = np.zeros_like(t3)
        orc.hadamard_reverse(g3, t2, g1); orc.hadamard_reverse(g3, t1, g2)
    orc.lib()
    dt = _pool_time(work, bounds, threads)
    out["cpu_baseline"] = {"value": round((5 + 9) * cpu_n * 4 / dt / 1e9, 2), "unit": "GB/s (fused algorithmic bytes, forward + reverse)",
                           "cores": threads, "kind": "port",
                           "sample": f"first {cpu_n} elements, unfused scalar C oracle ops, {dt:.2f} s"}
    return out


def config_ssd(mp, s, flush, nb=8, L=8192, cpu_pairs=2, cpu_len=2048):
    """configs[3]: Mamba-2 SSD chunked scan forward + reverse, batch 8, seqlen 8192, 32 heads, headdim 64, d_state 128."""
    import numpy as np
    import torch
    from oracle import pyoracle as orc
    sh = SSD_SHAPE
    out = {"workload": f"SSD scan forward and reverse, batch {nb}, seqlen {L}, heads {sh['H']}, headdim {sh['P']}, d_state {sh['NS']}, "
                       f"ngroups {sh['G']}, chunk {sh['Q']}; x, B, C r16, dt and A r32, fp32 accumulation"}
    _, burst, sustained, _ = peaks()
    for op, key in (("ssd_fwd", "forward"), ("ssd_rev", "reverse")):
        c = ssd_case(mp, s, op, nb, L)
        c.tensor_peak = sustained
        r = c.measure(s, flush, iters=8)
        r["scratch_bytes"] = c.scratch_bytes
        r["tensor_peak_kind"] = "sustained bf16 (fp16 runs on the same pipe)"
        out[key] = r
        del c
        torch.cuda.empty_cache()
    # CPU oracle: sequential recurrence (float64) on cpu_pairs (batch, head) pairs of cpu_len steps
    threads = min(_threads(), cpu_pairs)
    r = np.random.default_rng(0)
    H1 = 1
    xs = [r.standard_normal((1, cpu_len, H1, sh["P"])) for _ in range(cpu_pairs)]
    Bs = [r.standard_normal((1, cpu_len, 1, sh["NS"])) for _ in range(cpu_pairs)]
    Cs = [r.standard_normal((1, cpu_len, 1, sh["NS"])) for _ in range(cpu_pairs)]
    dts = [np.log1p(np.exp(r.standard_normal((1, cpu_len, H1)) - 4)) for _ in range(cpu_pairs)]
    As = [-np.exp(r.uniform(0, math.log(16), H1)) for _ in range(cpu_pairs)]
    gys = [r.standard_normal((1, cpu_len, H1, sh["P"])) for _ in range(cpu_pairs)]
    orc.lib()

    def work(i):
        orc.ssd_forward(xs[i], dts[i], As[i], Bs[i], Cs[i])
        orc.ssd_reverse(xs[i], dts[i], As[i], Bs[i], Cs[i], gys[i])
    dt = _pool_time(work, list(range(cpu_pairs)), threads)
    steps = cpu_pairs * cpu_len
    full_steps = nb * L * sh["H"]
    out["cpu_baseline"] = {"value": round(steps / dt, 1), "unit": "(batch, head) time steps/s, forward + reverse", "cores": threads, "kind": "port",
                           "sample": f"{cpu_pairs} (batch, head) sequences of {cpu_len} steps, sequential float64 recurrence and its adjoint, {dt:.2f} s; "
                                     f"the full config is {full_steps} steps",
                           "extrapolated_full_config_s": round(full_steps / (steps / dt), 1)}
    out["ref_cuda"] = "no reference kernel"
    return out


LM_EINSUMS = [
    # (label, form, m, n, k): forward projections and the two reverse contractions of each
    ("in_proj [16384,768]x[768,3352]", "nn", 16384, 3352, 768),
    ("out_proj [16384,1536]x[1536,768]", "nn", 16384, 768, 1536),
    ("lm_head [16384,768]x[50280,768]^T", "nt", 16384, 50280, 768),
    ("in_proj dX [16384,3352]x[768,3352]^T", "nt", 16384, 768, 3352),
    ("in_proj dW [16384,768]^Tx[16384,3352]", "tn", 768, 3352, 16384),
    ("out_proj dX [16384,768]x[1536,768]^T", "nt", 16384, 1536, 768),
    ("out_proj dW [16384,1536]^Tx[16384,768]", "tn", 1536, 768, 16384),
    ("lm_head dX [16384,50280]x[50280,768]", "nn", 16384, 768, 50280),
    ("lm_head dW [16384,50280]^Tx[16384,768]", "tn", 50280, 768, 16384),
]


def config_einsum(mp, s, flush, ref=None, cpu_rows=64):
    """The contraction shapes of the configs[4] model (projection, LM head, and their reverse contractions), r16 and r32."""
    import numpy as np
    import torch
    from oracle import pyoracle as orc
    out = {"workload": "contractions of the Mamba-2 LM step at 16384 tokens: forward projections and both reverse contractions, r16 and r32",
           "r32_note": "r32 runs 3 tf32 MMAs per product (error ~1e-5); its ceiling is the 16-bit peak / 2 / 3", "shapes": {}}
    flush_buf = flush.buf
    for label, form, m, n, k in LM_EINSUMS:
        rec = {}
        for sfx in ("r16", "r32"):
            c = gemm_case(mp, s, sfx, m, n, k, form)
            rec[sfx] = c.measure(s, flush, iters=6)
            if isinstance(ref, RefCuda):
                a, b, cc = c.keep
                if form == "nn":
                    once = lambda: ref.launch("inner_product_ij_jk_ik", sfx, a, b, D(1.0), cc, D(0.0), UL(m), UL(k), UL(n))
                    kern = f"launch_inner_product_ij_jk_ik_{sfx} (cuBLAS {'Hgemm' if sfx == 'r16' else 'Sgemm'})"
                else:
                    # the reference has no transposed contraction: it transposes into scratch first (inner_product.zig:275-330)
                    src = b if form == "nt" else a
                    tmp = torch.empty(src.shape[1], src.shape[0], device="cuda", dtype=src.dtype)
                    if form == "nt":
                        def once():
                            ref.launch("permutate_ij_ji", sfx, b, tmp, D(0.0), UL(n), UL(k))
                            ref.launch("inner_product_ij_jk_ik", sfx, a, tmp, D(1.0), cc, D(0.0), UL(m), UL(k), UL(n))
                    else:
                        def once():
                            ref.launch("permutate_ij_ji", sfx, a, tmp, D(0.0), UL(k), UL(m))
                            ref.launch("inner_product_ij_jk_ik", sfx, tmp, b, D(1.0), cc, D(0.0), UL(m), UL(k), UL(n))
                    kern = f"launch_permutate_ij_ji_{sfx} + launch_inner_product_ij_jk_ik_{sfx}"
                ms = ref.time(once, iters=4, flush_buf=flush_buf)
                rec[sfx]["ref_cuda"] = {"us": round(ms * 1e3, 1), "TFLOP/s": round(2.0 * m * n * k / (ms * 1e-3) / 1e12, 1), "kernels": kern}
            else:
                rec[sfx]["ref_cuda"] = f"unavailable: {ref}"
            del c
            torch.cuda.empty_cache()
        out["shapes"][label] = rec
    # CPU oracle: cpu_rows rows of the first projection (fp64-accumulated triple loop)
    threads = _threads()
    m, n, k = cpu_rows * threads, 3352, 768
    r = np.random.default_rng(0)
    a = r.standard_normal((m, k)).astype(np.float32); b = (r.standard_normal((k, n)) / math.sqrt(k)).astype(np.float32)
    bounds = [(cpu_rows * i, cpu_rows * (i + 1)) for i in range(threads)]
    orc.lib()
    dt = _pool_time(lambda bd: orc.inner_product(a[bd[0]:bd[1]], b), bounds, threads)
    out["cpu_baseline"] = {"value": round(2.0 * m * n * k / dt / 1e9, 2), "unit": "GFLOP/s", "cores": threads, "kind": "port",
                           "sample": f"{m} rows of [16384,768]x[768,3352] r32, scalar triple loop with double accumulation, {dt:.2f} s"}
    return out


def config_feed_forward(mp, s, ref=None):
    """configs[0]: README feed-forward block y = selu(linear(x, A, b)), sum-loss reverse(.free), one SGD step (r32 [32,256]x[256,256])."""
    import numpy as np
    import torch
    from oracle import pyoracle as orc
    host = C.CDLL(str(ROOT / "metaphor_b200" / "lib" / "libmp_host.so"))
    host.mpHostFeedForwardBench.restype = C.c_int
    host.mpHostFeedForwardBench.argtypes = [C.c_int, C.POINTER(C.c_double)]
    res = (C.c_double * 8)()
    rc = host.mpHostFeedForwardBench(2000, res)
    if rc != 0:
        raise SystemExit("feed-forward block bench failed")
    out = {"workload": "y = selu(linear(x[32,256], A[256,256], b[256])) r32; reverse(.free) of the sum loss; SGD lr 1e-2; through the C++ mirror of the host graph layer",
           "bound": "launch latency (12.6 MFLOP and 0.63 MB per step)",
           "forward_us": round(res[0], 2), "forward_reverse_sgd_us": round(res[1], 2),
           "forward_launches": int(res[2]), "step_launches": int(res[3]),
           "timing": "host wall clock per step over 2000 steps; every step ends with the stream synchronisation of the .free walk"}
    m, n, k = 32, 256, 256
    if isinstance(ref, RefCuda):
        g = _gen(0)
        x = torch.randn(m, n, generator=g, device="cuda"); A = torch.randn(n, k, generator=g, device="cuda") / 16; b = torch.zeros(k, device="cuda")
        y = torch.empty(m, k, device="cuda"); G = torch.ones(m, k, device="cuda")
        At = torch.empty(k, n, device="cuda"); xt = torch.empty(n, m, device="cuda")
        gx = torch.zeros(m, n, device="cuda"); gA = torch.zeros(n, k, device="cuda"); gb = torch.zeros(k, device="cuda")

        def fwd():
            ref.launch("inner_product_ij_jk_ik", "r32", x, A, D(1.0), y, D(0.0), UL(m), UL(n), UL(k))
            ref.launch("broadcast_j_ij", "r32", b, y, D(1.0), UL(m), UL(k))

        def rev():
            ref.launch("permutate_ij_ji", "r32", A, At, D(0.0), UL(n), UL(k))
            ref.launch("inner_product_ij_jk_ik", "r32", G, At, D(1.0), gx, D(1.0), UL(m), UL(k), UL(n))
            ref.launch("permutate_ij_ji", "r32", x, xt, D(0.0), UL(m), UL(n))
            ref.launch("inner_product_ij_jk_ik", "r32", xt, G, D(1.0), gA, D(1.0), UL(n), UL(m), UL(k))
            ref.launch("reduce_ij_j", "r32", G, gb, D(0.0), UL(m), UL(k))

        def both():
            fwd(); rev()
        f_ms = ref.time(lambda: [fwd() for _ in range(100)], iters=3) / 100
        a_ms = ref.time(lambda: [both() for _ in range(100)], iters=3) / 100
        out["ref_cuda"] = {"forward_device_us": round(f_ms * 1e3, 2), "forward_reverse_device_us": round(a_ms * 1e3, 2),
                           "kernels": "forward: launch_inner_product_ij_jk_ik_r32 (cuBLAS Sgemm) + launch_broadcast_j_ij_r32; reverse: 2 x "
                                      "(launch_permutate_ij_ji_r32 + Sgemm, beta 1) + launch_reduce_ij_j_r32; the reference has no SELU and no SGD kernel, "
                                      "so those two parts of the step are missing from this figure",
                           "launches": "2 forward, 7 forward + reverse"}
    else:
        out["ref_cuda"] = f"unavailable: {ref}"
    # CPU oracle of the whole step, one thread
    r = np.random.default_rng(0)
    x = r.standard_normal((m, n)).astype(np.float32); A = (r.standard_normal((n, k)) / 16).astype(np.float32); b = np.zeros(k, np.float32)
    orc.lib()
    reps = 50
    t0 = time.perf_counter()
    for _ in range(reps):
        lin = orc.inner_product(x, A, bias=b); orc.selu(lin)
        gl = np.zeros_like(lin); orc.selu_reverse(lin, gl, np.ones_like(lin))
        gx = orc.inner_product(gl, A, tb=True); gA = orc.inner_product(x, gl, ta=True); gb = orc.reduce_ij_j(gl)
        orc.sgd(A.copy(), gA, 1e-2); orc.sgd(b.copy(), gb, 1e-2)
    dt = (time.perf_counter() - t0) / reps
    out["cpu_baseline"] = {"value": round(dt * 1e6, 1), "unit": "us per forward + reverse + SGD step", "cores": 1, "kind": "port",
                           "sample": f"the full block, scalar C oracle, mean of {reps} steps"}
    return out
