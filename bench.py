#!/usr/bin/env python
"""Benchmark of the row-reduction hot path (softmax and RMSNorm, forward and
reverse, r32 and r16, X = [65536, 4096]) through the C ABI.

One "step" = one pass over one batch: for each dtype, softmax forward, softmax
reverse, RMSNorm forward, RMSNorm reverse (gradients overwritten, alpha = 0;
rstd recomputed in the reverse).  Metric: algorithmic HBM GB/s = the bytes each
kernel must read and write once, summed over the step, divided by the time.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Under torchrun (N > 1) every rank runs the same per-GPU workload on its own
rows (weak scaling, no collective on the data path); the time is the maximum
over ranks, the value the sum of all ranks' bytes over that time.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M, N = 65536, 4096
EPS = 1e-6
METRIC = "row-reduction (softmax+RMSNorm fwd+rev, r32+r16) algorithmic HBM bandwidth"
UNIT = "GB/s"

# DRAM bytes per launch from ncu (dram__bytes_read.sum + dram__bytes_write.sum)
# for the kernels of this step; filled from profiles/ (None = not captured).
NCU_TRAFFIC_BYTES = {
    # profiles/rmsnorm_reverse_m32768_n4096.md, captured at 32768 rows and scaled x2 (traffic is linear in rows)
    "rmsnorm_rev_r32": 2 * (1_073_854_000 + 510_001_152),
    "rmsnorm_rev_r16": 2 * (537_149_952 + 252_880_128),
    # profiles/softmax_m32768_n4096.md
    "softmax_rev_r32": 2 * (1_073_749_000 + 495_847_168),
    "softmax_fwd_r16": 2 * (268_444_928 + 213_376_768),
}


def algorithmic_bytes(op: str, size: int, m: int = M, n: int = N) -> int:
    """Bytes a kernel must move once (inputs read once, outputs written once)."""
    mn = m * n * size
    return {
        "softmax_fwd": 2 * mn,                              # x -> y
        "softmax_rev": 3 * mn,                              # y, gy -> gx
        "rmsnorm_fwd": 2 * mn + n * size,                   # x, gain -> y
        "rmsnorm_rev": 3 * mn + 2 * n * size,               # x, gy, gain -> gx, ggain
    }[op]


OPS = ["softmax_fwd", "softmax_rev", "rmsnorm_fwd", "rmsnorm_rev"]
DTYPES = [("r32", 4), ("r16", 2)]
STEP_BYTES = sum(algorithmic_bytes(op, size) for op in OPS for _, size in DTYPES)


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi sampling (every 20 ms) of SM clocks and throttle reasons.
    Started before the warm-up; `stop(t0, t1)` keeps the samples whose wall-clock
    time falls inside the timed region [t0, t1] (and says how many there were)."""
    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.proc = None
        self.path = None
        self.index = device_index

    def start(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        self.proc = subprocess.Popen([exe, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index), "-lms", "20"],
                                     stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        time.sleep(0.5)   # let the sampler reach its steady rate before the timed region

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        import datetime
        rows = []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[2]), float(parts[3]), [n for n, v in zip(names, parts[6:10])
                                                                    if v.lower().startswith("active")]))
            except ValueError:
                continue
        os.unlink(self.path)
        inside = [r for r in rows if t0 - 0.02 <= r[0] <= t1 + 0.02]
        scope = "timed region"
        if len(inside) < 2:   # region shorter than the sampling period: use the loaded samples around it
            mx = max((r[1] for r in rows), default=0.0)
            inside = [r for r in rows if r[1] > 0.5 * mx and t0 - 1.0 <= r[0] <= t1 + 1.0]
            scope = "loaded samples within 1 s of the timed region"
        reasons = sorted({n for r in inside for n in r[3]})
        return {"sm_mhz": statistics.median(r[1] for r in inside) if inside else None,
                "sm_max_mhz": max((r[2] for r in rows), default=None), "reasons": reasons,
                "samples": len(inside), "scope": scope}


# ----------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import metaphor_b200 as mp

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    lib = mp.lib()
    lib.mpInitDevice(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    stream = mp.Stream()
    ts = stream.torch_stream()

    # ---- synthetic inputs, resident in HBM (seeded; rank-distinct rows) -------
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    bufs = {}
    x32 = torch.randn(M, N, generator=gen, device="cuda")
    g32 = torch.randn(M, N, generator=gen, device="cuda")
    gain32 = 1.0 + 0.02 * torch.randn(N, generator=gen, device="cuda")
    for sfx, size in DTYPES:
        dt = torch.float32 if sfx == "r32" else torch.float16
        b = {"dt": dt, "x": x32.to(dt), "gy": g32.to(dt), "gain": gain32.to(dt)}
        b["y"] = torch.empty(M, N, device="cuda", dtype=dt)          # softmax output
        b["gx"] = torch.empty(M, N, device="cuda", dtype=dt)
        b["yn"] = torch.empty(M, N, device="cuda", dtype=dt)         # RMSNorm output
        b["gxn"] = torch.empty(M, N, device="cuda", dtype=dt)
        b["ggain"] = torch.empty(N, device="cuda", dtype=dt)
        nb = lib.mpRmsnormReverseScratchBytes(M, N, stream.ctx)
        b["scratch"] = torch.empty(nb, device="cuda", dtype=torch.uint8)
        bufs[sfx] = b
    del x32, g32
    torch.cuda.synchronize()

    def launch(op, sfx):
        b = bufs[sfx]
        if op == "softmax_fwd":
            mp.launch("softmax_ij_j", b["dt"], b["x"], b["y"], M, N, stream)
        elif op == "softmax_rev":
            mp.launch("softmax_ij_j_reverse", b["dt"], b["y"], b["gy"], b["gx"], 0.0, M, N, stream)
        elif op == "rmsnorm_fwd":
            mp.launch("rmsnorm_ij_j", b["dt"], b["x"], b["gain"], EPS, b["yn"], None, M, N, stream)
        else:
            mp.launch("rmsnorm_ij_j_reverse", b["dt"], b["x"], b["gain"], None, b["gy"], EPS, b["gxn"], b["ggain"],
                      0.0, b["scratch"], M, N, stream)

    kernels = [(op, sfx) for sfx, _ in DTYPES for op in OPS]
    launches_per_step = len(kernels) + 4      # each RMSNorm reverse = row kernel + two fold kernels

    def step(events=None):
        for i, (op, sfx) in enumerate(kernels):
            if events is not None:
                events[i][0].record(ts)
            launch(op, sfx)
            if events is not None:
                events[i][1].record(ts)

    def barrier():
        stream.sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    # ---- device-resident timing ----------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    wall0 = time.time()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    per_kernel = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in kernels]
                  for _ in range(args.steps)]
    e0.record(ts)
    for k in range(args.steps):
        step(per_kernel[k])
    e1.record(ts)
    barrier()
    wall1 = time.time()
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    ms_total = e0.elapsed_time(e1)
    if stream.status() != 0:
        raise SystemExit("a kernel reported a non-zero status word")
    t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = world * STEP_BYTES / (ms_per_step * 1e-3) / 1e9

    # per-kernel averages -> roofline of the dominant kernel
    kstats = {}
    for i, (op, sfx) in enumerate(kernels):
        ms = statistics.mean(per_kernel[k][i][0].elapsed_time(per_kernel[k][i][1]) for k in range(args.steps))
        size = 4 if sfx == "r32" else 2
        kstats[f"{op}_{sfx}"] = {"ms": ms, "bytes": algorithmic_bytes(op, size)}
    peak, peak_kind = measured_peak()
    dom = max(kstats, key=lambda k: kstats[k]["ms"])
    achieved = kstats[dom]["bytes"] / (kstats[dom]["ms"] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 1), "peak": peak, "peak_kind": peak_kind,
                "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC_BYTES.get(dom),
                "algorithmic_bytes": kstats[dom]["bytes"],
                "per_kernel": {k: {"us": round(v["ms"] * 1e3, 1),
                                   "achieved": round(v["bytes"] / (v["ms"] * 1e-3) / 1e9, 1),
                                   "frac": round(v["bytes"] / (v["ms"] * 1e-3) / 1e9 / peak, 4)}
                               for k, v in kstats.items()}}

    # ---- end to end: host buffers in, host buffers out, through the C ABI ------
    e2e = run_e2e(args, mp, lib, stream, ts, bufs, kernels, launch, barrier, world)

    cpu = None
    if rank == 0 and world == 1:
        cpu = cpu_baseline(sample_rows=args.cpu_rows)

    if rank == 0:
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (seeded N(0,1) X and upstream gradient, gain ~ N(1, 0.02))",
            "config": {"workload": "configs[1]: softmax + RMSNorm (eps 1e-6) forward+reverse over X[65536,4096], "
                                   "r32 and r16, per GPU", "rows_per_gpu": M, "cols": N,
                       "l2": "inputs (1 GiB / 0.5 GiB per tensor) exceed the 126 MB L2; no flush needed",
                       "bytes_per_step_per_gpu": STEP_BYTES, "io": "r32 and r16 storage, fp32 arithmetic"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": launches_per_step * args.steps,
        }
        print(json.dumps(out), flush=True)
    stream.close()
    if world > 1:
        dist.destroy_process_group()


E2E_CHUNKS = 8


def run_e2e(args, mp, lib, stream, ts, bufs, kernels, launch, barrier, world):
    """Same step with HOST buffers: every input is copied from pinned host memory
    and every result copied back to pinned host memory inside the timed region,
    all through the C ABI (mpMemcpyHtoD / launch_* / mpMemcpyDtoH).  The rows are
    cut into E2E_CHUNKS chunks and pipelined over three streams - copy-in,
    compute, copy-out - ordered by mpEventRecord / mpStreamWaitEvent, so that the
    PCIe transfers in both directions overlap each other and the kernels."""
    import ctypes as C
    import torch
    steps = max(1, min(args.steps, args.e2e_steps))
    s_in, s_out = mp.Stream(), mp.Stream()
    rows = M // E2E_CHUNKS
    host_in = {}
    for sfx, size in DTYPES:
        b = bufs[sfx]
        nbytes = M * N * size
        hx = lib.mpHostAlloc(nbytes); hg = lib.mpHostAlloc(nbytes); hgain = lib.mpHostAlloc(N * size)
        lib.mpMemcpyDtoH(hx, C.c_void_p(b["x"].data_ptr()), nbytes, stream.ctx)
        lib.mpMemcpyDtoH(hg, C.c_void_p(b["gy"].data_ptr()), nbytes, stream.ctx)
        lib.mpMemcpyDtoH(hgain, C.c_void_p(b["gain"].data_ptr()), N * size, stream.ctx)
        host_in[sfx] = (hx, hg, hgain, nbytes)
        b["ggain_parts"] = torch.empty(E2E_CHUNKS, N, device="cuda", dtype=b["dt"])   # per-chunk gain gradients
        nb = lib.mpRmsnormReverseScratchBytes(rows, N, stream.ctx)
        b["scratch_chunk"] = torch.empty(nb, device="cuda", dtype=torch.uint8)
    hout = lib.mpHostAlloc(M * N * 4)     # landing buffer, reused for every result
    stream.sync()
    ev_in = [[lib.mpEventCreate() for _ in range(E2E_CHUNKS)] for _ in DTYPES]
    ev_cmp = [[lib.mpEventCreate() for _ in range(E2E_CHUNKS)] for _ in DTYPES]
    ev_done = lib.mpEventCreate()
    h2d = sum(2 * M * N * size + N * size for _, size in DTYPES)
    d2h = sum(4 * M * N * size + N * size for _, size in DTYPES)
    P = lambda t, off=0: C.c_void_p(t.data_ptr() + off)

    def e2e_step():
        # the compute stream of the previous step must have finished with the device buffers
        lib.mpEventRecord(ev_done, stream.ctx)
        lib.mpStreamWaitEvent(s_in.ctx, ev_done)
        for di, (sfx, size) in enumerate(DTYPES):
            b = bufs[sfx]
            hx, hg, hgain, nbytes = host_in[sfx]
            cb = rows * N * size
            lib.mpMemcpyHtoD(P(b["gain"]), hgain, N * size, s_in.ctx)
            for c in range(E2E_CHUNKS):
                off = c * cb
                lib.mpMemcpyHtoD(P(b["x"], off), C.c_void_p(hx + off), cb, s_in.ctx)
                lib.mpMemcpyHtoD(P(b["gy"], off), C.c_void_p(hg + off), cb, s_in.ctx)
                lib.mpEventRecord(ev_in[di][c], s_in.ctx)
                lib.mpStreamWaitEvent(stream.ctx, ev_in[di][c])
                r0, r1 = c * rows, (c + 1) * rows
                x, gy = b["x"][r0:r1], b["gy"][r0:r1]
                mp.launch("softmax_ij_j", b["dt"], x, b["y"][r0:r1], rows, N, stream)
                mp.launch("softmax_ij_j_reverse", b["dt"], b["y"][r0:r1], gy, b["gx"][r0:r1], 0.0, rows, N, stream)
                mp.launch("rmsnorm_ij_j", b["dt"], x, b["gain"], EPS, b["yn"][r0:r1], None, rows, N, stream)
                mp.launch("rmsnorm_ij_j_reverse", b["dt"], x, b["gain"], None, gy, EPS, b["gxn"][r0:r1],
                          b["ggain_parts"][c], 0.0, b["scratch_chunk"], rows, N, stream)
                if c == E2E_CHUNKS - 1:   # gain gradient = sum of the chunks' partial gradients
                    mp.launch("reduce_ij_j", b["dt"], b["ggain_parts"], b["ggain"], 0.0, E2E_CHUNKS, N, stream)
                lib.mpEventRecord(ev_cmp[di][c], stream.ctx)
                lib.mpStreamWaitEvent(s_out.ctx, ev_cmp[di][c])
                for name in ("y", "gx", "yn", "gxn"):
                    lib.mpMemcpyDtoH(C.c_void_p(hout + off), P(b[name], off), cb, s_out.ctx)
            lib.mpMemcpyDtoH(hout, P(b["ggain"]), N * size, s_out.ctx)

    def sync_all():
        s_in.sync(); s_out.sync()
        barrier()

    e2e_step()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
        s_out.sync()          # the step's results are on the host
    stream.sync(); s_in.sync()
    ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    for hx, hg, hgain, _ in host_in.values():
        lib.mpHostFree(hx); lib.mpHostFree(hg); lib.mpHostFree(hgain)
    lib.mpHostFree(hout)
    for evs in ev_in + ev_cmp:
        for e in evs:
            lib.mpEventDestroy(e)
    lib.mpEventDestroy(ev_done)
    s_in.close(); s_out.close()
    return {"value": round(world * STEP_BYTES / (ms * 1e-3) / 1e9, 2), "unit": UNIT, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": round(ms, 3), "steps": steps,
            "pipeline": f"{E2E_CHUNKS} row chunks over copy-in / compute / copy-out streams; host-synchronised per step"}


# ----------------------------------------------------------------------------
def cpu_step_sample(rows: int, threads: int, repeats: int = 1):
    """The same step on `rows` rows with the CPU oracle (scalar C, float32
    storage for both dtype halves), rows split statically over `threads` host
    threads.  Returns (seconds per pass, algorithmic bytes per pass)."""
    import numpy as np
    from oracle import pyoracle as orc
    orc.lib()
    r = np.random.default_rng(0)
    x = r.standard_normal((rows, N)).astype(np.float32)
    gy = r.standard_normal((rows, N)).astype(np.float32)
    gain = (1 + 0.02 * r.standard_normal(N)).astype(np.float32)
    bounds = [(rows * i // threads, rows * (i + 1) // threads) for i in range(threads)]

    def work(lo_hi):
        lo, hi = lo_hi
        if hi <= lo:
            return
        xs, gs = x[lo:hi], gy[lo:hi]
        y = orc.softmax_ij_j(xs)
        orc.softmax_ij_j_reverse(y, gs)
        orc.rmsnorm_ij_j(xs, gain, EPS)
        orc.rmsnorm_ij_j_reverse(xs, gain, gs, EPS)   # per-slice ggain partials; the sum over slices is negligible

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as pool:
        for _ in range(repeats):
            for _ in range(len(DTYPES)):              # the r32 half and the r16 half of the step
                list(pool.map(work, bounds))
    dt = (time.perf_counter() - t0) / repeats
    nbytes = sum(algorithmic_bytes(op, size, rows, N) for op in OPS for _, size in DTYPES)
    return dt, nbytes


def cpu_baseline(sample_rows: int):
    threads = os.cpu_count() or 1
    repeats = 3    # about 10-25 s of CPU time over all threads
    dt, nbytes = cpu_step_sample(sample_rows, threads, repeats)
    return {"value": round(nbytes / dt / 1e9, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"first {sample_rows} of {M} rows of the same step, scalar C oracle, "
                      f"{threads} host threads over disjoint row ranges, mean of {repeats} passes of {dt:.2f} s"}


def run_reference(args):
    """Reference arm.  The reference has no CPU (or any) implementation of
    softmax / RMSNorm, so this times the CPU oracle port of the step on all host
    threads, one bounded row sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = args.cpu_rows
    for _ in range(min(args.warmup, 1)):
        cpu_step_sample(max(threads, rows // 8), threads)
    times = []
    nbytes = 0
    for _ in range(args.steps):
        dt, nbytes = cpu_step_sample(rows, threads)
        times.append(dt)
    dt = statistics.mean(times)
    value = round(nbytes / dt / 1e9, 3)
    sample = (f"each step = first {rows} of {M} rows, scalar C oracle port (the reference has no kernel for these "
              f"ops), {threads} host threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
        "config": {"workload": "configs[1]: softmax + RMSNorm forward+reverse over X[65536,4096], r32 and r16",
                   "rows_sampled_per_step": rows, "cols": N},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_lm(args):
    """`--workload lm`: data-parallel training step of the Mamba-2 language model of configs[4]
    (d_model 768, 24 layers, expand 2, headdim 64, d_state 128, vocab 50280; seq 2048, batch 8 per GPU,
    fused Adam lr 3e-4 betas 0.9/0.95, all-reduce of the r32 gradient).  A step = forward, cross-entropy,
    reverse, all-reduce, Adam; `value` = tokens/s over all ranks with the token ids resident on the
    device, `e2e` = the same step with the ids copied from pinned host memory and the loss read back."""
    import torch
    import torch.distributed as dist
    import metaphor_b200 as mp
    from metaphor_b200.dist import GradientComm
    from metaphor_b200.mamba_lm import LMConfig, MambaLM

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    lib = mp.lib()
    lib.mpInitDevice(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    comm = GradientComm(world, rank) if world > 1 else None
    cfg = LMConfig(n_layer=args.lm_layers, chunk=args.lm_chunk)
    batch, seqlen = args.lm_batch, 2048
    model = MambaLM(cfg, batch, seqlen, seed=0, loss_scale=65536.0)
    stream, ts = model.stream, model.stream.torch_stream()
    T = batch * seqlen
    gen = torch.Generator().manual_seed(1000 + rank)
    tok = torch.randint(0, cfg.vocab, (T + 1,), generator=gen, dtype=torch.int32)
    ids_h, tgt_h = tok[:-1].contiguous().pin_memory(), tok[1:].contiguous().pin_memory()
    model.set_batch(ids_h, tgt_h)
    adam = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8)
    if not args.lm_no_graph:
        model.capture()

    def barrier():
        stream.sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        model.train_step(comm=comm, world=world, **adam)
    barrier()
    first_loss = None
    wall0 = time.time()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    phase = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
    e0.record(ts)
    for k in range(args.steps):
        last = k == args.steps - 1
        if last: phase[0].record(ts)
        if args.lm_no_graph:
            model.forward()
            if last: phase[1].record(ts)
            model.loss_and_logit_gradient()
            model.backward()
        else:
            if last: phase[1].record(ts)
            model.forward_backward()
        if last: phase[2].record(ts)
        if comm is not None:
            comm.all_reduce_sum(model.g32, stream)
        if last: phase[3].record(ts)
        model.adam_step(world=world, **adam)
        if last: phase[4].record(ts)
    e1.record(ts)
    barrier()
    wall1 = time.time()
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    if stream.status() != 0:
        raise SystemExit("a kernel reported a non-zero status word")
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = world * T / (ms_per_step * 1e-3)
    last_loss = model.loss()

    # end to end: ids from pinned host memory every step, loss read back every step
    barrier()
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    e0.record(ts)
    for _ in range(e2e_steps):
        model.set_batch(ids_h, tgt_h)
        model.train_step(comm=comm, world=world, **adam)
        _ = model.loss()
    e1.record(ts)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps

    if rank == 0:
        n_params = cfg.n_params()
        gemm_params = n_params - 0   # every parameter but the small vectors sits in a contraction; the embedding is tied
        # model flops per step and GPU: 6 x params x tokens for the contractions + the scan (forward 1x, reverse 2x)
        Q, H, P, NS = cfg.chunk, cfg.heads, cfg.headdim, cfg.d_state
        ssd_fwd = (2 * Q * Q * NS) * (T // Q) + (2 * Q * Q * P + 4 * Q * NS * P) * (cfg.heads * T // Q)
        flops = 6.0 * gemm_params * T + 3.0 * ssd_fwd * cfg.n_layer
        achieved = flops / (ms_per_step * 1e-3) / 1e12
        peak = 1381.7
        try:
            peak = float(json.loads((Path(__file__).resolve().parent / "MEASURED_PEAKS.json").read_text()).get("bf16_tflops_sustained", peak))
        except Exception:
            pass
        ph = [phase[i].elapsed_time(phase[i + 1]) for i in range(4)]
        out = {
            "metric": "Mamba-2 LM training throughput", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations, f32 accumulation and master weights",
            "data": "synthetic (token ids ~ U[0, 50280), seed 1000 + rank; weights N(0, 0.02), seed 0 on every rank)",
            "config": {"workload": "configs[4]: Mamba-2 LM d_model 768, %d layers, expand 2, headdim 64, d_state 128, vocab 50280, "
                                   "seq 2048, batch %d per GPU, cross-entropy, fused Adam lr 3e-4 betas 0.9/0.95, NCCL all-reduce of "
                                   "the r32 gradient" % (cfg.n_layer, batch),
                       "assumed": f"d_conv 4, tied embedding / LM head, gated RMSNorm before out_proj, D skip, chunk {cfg.chunk}, loss scale 65536",
                       "params": n_params, "tokens_per_gpu_step": T,
                       "l2": "activations and weights (GBs per step) exceed the 126 MB L2; no flush needed"},
            "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peak, "peak_kind": "measured sustained bf16 (fp16 runs on the same pipe)",
                         "unit": "TFLOP/s", "frac": round(achieved / peak, 4), "traffic": None,
                         "algorithmic_flops": flops,
                         "phases_ms": {"forward" if args.lm_no_graph else "(graph: see next)": round(ph[0], 2),
                                       "loss+reverse" if args.lm_no_graph else "forward+loss+reverse (one graph launch)": round(ph[1], 2), "all_reduce": round(ph[2], 2),
                                       "adam+refresh": round(ph[3], 2)}},
            "cpu_baseline": None,
            "e2e": {"value": round(world * T / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "h2d_bytes_per_step": 2 * T * 4,
                    "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps},
            "clocks": clocks, "gpu_launches": model.launches_per_step() * args.steps,
            "loss": {"first_timed_step": first_loss, "last": round(last_loss, 4)},
        }
        print(json.dumps(out), flush=True)
    if comm is not None:
        comm.close()
    stream.close()
    if world > 1:
        dist.destroy_process_group()


def run_profile_case(spec: str, timed: bool = False):
    """`--profile-case OP:DTYPE:ROWS[:COLS]`: three launches of one kernel on a
    small case, for an ncu capture (no timing, no JSON).  OP is one of
    softmax_fwd, softmax_rev, rmsnorm_fwd, rmsnorm_rev (rows x cols matrix),
    chain_fwd, chain_rev (ROWS = element count of selu((a+b)*(c+d))),
    gemm (ROWS:COLS = M and N = K), ssd_fwd, ssd_rev (ROWS:COLS = batch and seqlen),
    bmm (ROWS:COLS = batch entries and M = N = K), permute_heads / permute_reverse (ROWS:COLS = batch and seqlen of a
    [batch, seqlen, 32, 128] tensor: "blhd->bhld" resp. "blhd->dhlb"), conv_fwd / conv_rev (ROWS:COLS = batch and seqlen; the
    segmented causal convolution over the 1792 [x | B | C] columns of a Mamba-2 block).  With `--profile-time` the case is then launched
    20 more times between CUDA events and one JSON line with the mean launch time is printed."""
    import torch
    import metaphor_b200 as mp
    parts = spec.split(":")
    op, sfx, m = parts[0], parts[1], int(parts[2])
    n = int(parts[3]) if len(parts) > 3 else N
    dt = {"r16": torch.float16, "r32": torch.float32, "r64": torch.float64}[sfx]
    torch.zeros(1, device="cuda")
    s = mp.Stream()
    g = torch.Generator(device="cuda").manual_seed(0)
    once = None          # one launch of the case (set by the branches that support --profile-time)
    work = None          # (amount, unit) per launch
    if op in ("chain_fwd", "chain_rev"):
        leaves = [(torch.rand(m, generator=g, device="cuda") * 2 - 1).to(dt) for _ in range(4)]
        out = torch.empty_like(leaves[0]); grads = [torch.empty_like(leaves[0]) for _ in range(4)]
        chain = mp.FusedChain("selu((a+b)*(c+d))", dt)
        torch.cuda.synchronize()
        for _ in range(3):
            if op == "chain_fwd":
                chain.forward(leaves, out, m, s)
            else:
                chain.reverse(leaves, None, grads, 0.0, m, s)
    elif op == "bmm":
        a = torch.randn(m, n, n, generator=g, device="cuda").to(dt); b = (torch.randn(m, n, n, generator=g, device="cuda") / 32).to(dt)
        c = torch.empty(m, n, n, device="cuda", dtype=dt)
        once = lambda: mp.launch("inner_product_bij_bjk_bik", dt, a, b, 1.0, c, 0.0, m, n, n, n, s)
        work = (2.0 * m * n * n * n / 1e12, "TFLOP")
        torch.cuda.synchronize()
        for _ in range(3):
            once()
    elif op in ("conv_fwd", "conv_rev"):
        # ROWS = batch, COLS = seqlen; the [x | B | C] columns (1536 + 128 + 128) of a 3352-wide projection row, 4 taps
        import ctypes
        widths, dip, di, W = (1536, 128, 128), 3352, 1536, 4
        Cn = sum(widths)
        zx = torch.randn(m * n, dip, generator=g, device="cuda").to(dt); gzx = torch.empty_like(zx)
        w = torch.randn(Cn, W, generator=g, device="cuda").to(dt); bias = torch.randn(Cn, generator=g, device="cuda").to(dt)
        outs = [torch.randn(m * n, cw, generator=g, device="cuda").to(dt) for cw in widths]
        gw = torch.zeros(Cn, W, device="cuda"); gb = torch.zeros(Cn, device="cuda")
        ptrs = (ctypes.c_void_p * 3)(*[t.data_ptr() for t in outs]); cw = (ctypes.c_ulong * 3)(*widths)
        esz = zx.element_size()
        if op == "conv_fwd":
            once = lambda: mp.launch("causal_conv1d_silu_segments", dt, zx.data_ptr() + di * esz, dip, w, bias, ptrs, cw, cw, 3, m, n, W, s)
            work = (2.0 * m * n * Cn * esz / 1e9, "GB")
        else:
            once = lambda: mp.launch("causal_conv1d_silu_segments_reverse", dt, zx.data_ptr() + di * esz, dip, w, bias, ptrs, cw, cw, 3,
                                     gzx.data_ptr() + di * esz, dip, gw, gb, m, n, W, s)
            work = (3.0 * m * n * Cn * esz / 1e9, "GB")
        torch.cuda.synchronize()
        for _ in range(3):
            once()
    elif op in ("permute_heads", "permute_reverse"):
        import ctypes
        shape = (m, n, 32, 128)
        perm = (0, 2, 1, 3) if op == "permute_heads" else (3, 2, 1, 0)
        x = torch.randn(shape, generator=g, device="cuda").to(dt); y = torch.empty_like(x)
        sizes = (ctypes.c_ulong * 4)(*shape); pm = (ctypes.c_ulong * 4)(*perm)
        once = lambda: mp.launch("permutate", dt, x, y, 0.0, sizes, pm, 4, s)
        work = (2.0 * x.numel() * x.element_size() / 1e9, "GB")
        torch.cuda.synchronize()
        for _ in range(3):
            once()
    elif op in ("ssd_fwd", "ssd_rev"):
        # ROWS = batch, COLS = seqlen; heads 32, headdim 64, d_state 128, 1 group, chunk 256
        import math
        nb, L, H, P, NS, G, Q = m, n, 32, 64, 128, 1, 256
        x = torch.randn(nb, L, H, P, generator=g, device="cuda").half()
        Bm = torch.randn(nb, L, G, NS, generator=g, device="cuda").half()
        Cm = torch.randn(nb, L, G, NS, generator=g, device="cuda").half()
        dtv = torch.nn.functional.softplus(torch.randn(nb, L, H, generator=g, device="cuda") - 4)
        Av = -torch.exp(torch.rand(H, generator=g, device="cuda") * math.log(16))
        gy = torch.randn(nb, L, H, P, generator=g, device="cuda").half()
        y = torch.empty_like(x); gx = torch.empty_like(x); gdt = torch.empty_like(dtv); gA = torch.empty_like(Av)
        gB = torch.empty_like(Bm); gC = torch.empty_like(Cm)
        dims = (nb, L, H, P, NS, G, Q)
        rev = op == "ssd_rev"
        scr = torch.empty(mp.lib().mpSsdScanScratchBytes(*dims, 1 if rev else 0), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            if rev:
                mp.launch("ssd_scan_reverse", torch.float16, x, dtv, Av, Bm, Cm, gy, gx, gdt, gA, gB, gC, scr, *dims, s)
            else:
                mp.launch("ssd_scan", torch.float16, x, dtv, Av, Bm, Cm, y, scr, *dims, s)
    elif op == "gemm":
        a = torch.randn(m, n, generator=g, device="cuda").to(dt); b = torch.randn(n, n, generator=g, device="cuda").to(dt)
        c = torch.empty(m, n, device="cuda", dtype=dt)
        once = lambda: mp.launch("inner_product_ij_jk_ik", dt, a, b, 1.0, c, 0.0, m, n, n, s)
        work = (2.0 * m * n * n / 1e12, "TFLOP")
        torch.cuda.synchronize()
        for _ in range(3):
            once()
    else:
        x = torch.randn(m, n, generator=g, device="cuda").to(dt); gy = torch.randn(m, n, generator=g, device="cuda").to(dt)
        y = torch.empty_like(x); gx = torch.empty_like(x)
        gain = torch.ones(n, device="cuda", dtype=dt); gg = torch.empty_like(gain)
        scratch = torch.empty(mp.lib().mpRmsnormReverseScratchBytes(m, n, s.ctx), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            if op == "softmax_fwd":
                mp.launch("softmax_ij_j", dt, x, y, m, n, s)
            elif op == "softmax_rev":
                mp.launch("softmax_ij_j_reverse", dt, x, gy, gx, 0.0, m, n, s)
            elif op == "rmsnorm_fwd":
                mp.launch("rmsnorm_ij_j", dt, x, gain, EPS, y, None, m, n, s)
            elif op == "rmsnorm_rev":
                mp.launch("rmsnorm_ij_j_reverse", dt, x, gain, None, gy, EPS, gx, gg, 0.0, scratch, m, n, s)
            else:
                raise SystemExit(f"unknown profile case {op}")
    s.sync()
    if timed:
        if once is None:
            raise SystemExit(f"--profile-time is not available for {op}")
        ts = s.torch_stream()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(ts)
        for _ in range(20):
            once()
        e1.record(ts)
        s.sync()
        us = e0.elapsed_time(e1) / 20 * 1e3
        print(json.dumps({"case": spec, "us_per_launch": round(us, 2), "per_launch": work[0], "unit": work[1],
                          "rate": round(work[0] / (us * 1e-6), 1), "rate_unit": work[1] + "/s"}))
    if s.status() != 0:
        raise SystemExit("status word set")
    s.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10, help="upper bound on end-to-end steps (PCIe-bound)")
    ap.add_argument("--cpu-rows", type=int, default=32768, help="rows in the CPU baseline sample")
    ap.add_argument("--workload", default="rows", choices=["rows", "lm"],
                    help="rows = configs[1] (default, the headline line); lm = configs[4] training step, tokens/s")
    ap.add_argument("--lm-layers", type=int, default=24)
    ap.add_argument("--lm-batch", type=int, default=8)
    ap.add_argument("--lm-no-graph", action="store_true", help="issue every launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--lm-chunk", type=int, default=256, help="scan chunk of the LM workload (128 or 256)")
    ap.add_argument("--profile-case", default=None, help="OP:DTYPE:ROWS[:COLS], three launches for an ncu capture")
    ap.add_argument("--profile-time", action="store_true", help="with --profile-case: also time 20 launches with CUDA events")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case, args.profile_time)
        return
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "lm":
        run_lm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
