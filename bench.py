#!/usr/bin/env python
"""Benchmark of the device layer behind mp.ops / mp.optm.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (default): the data-parallel training step of the Mamba-2 language
model of configs[4] - forward, cross-entropy, reverse, NCCL all-reduce of the r32
gradient (N > 1), fused Adam - in tokens/s over all ranks.  One process per GPU
(torchrun for N > 1), weak scaling: every rank runs batch 8 x seq 2048 of its
own token stream.  At N = 1 the same JSON line carries `per_config`: the other
four configs (README feed-forward block, row reductions, fused chain, SSD scan)
and the contraction shapes of the model, each with its roofline fraction, a
CPU-oracle baseline and, where the reference has kernels for it, the
reference's own CUDA kernels timed in the same run (`ref_cuda`).

`--impl reference` times the float64 CPU oracle of the same training step
(oracle/lm_oracle.py, full model width, a short batch; tokens/s is
size-normalised): the reference has no CPU implementation and no kernels for
most of this step, so the oracle port is the reference arm.

`--workload rows` runs configs[1] alone (the former default line);
`--profile-case OP:DTYPE:SIZES [--profile-time]` launches a single case three
times for an ncu capture and optionally times it (see bench_cases.build_case).
"""
from __future__ import annotations

import argparse
import json
import math
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
def run_rows(args, standalone=True):
    """configs[1] alone: the record printed by `--workload rows`, and the C2 entry of `per_config`."""
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
    if world > 1 and standalone:
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
    out = None

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
            "ref_cuda": "no reference kernel (the reference has neither softmax nor RMSNorm)",
        }
        if standalone:
            emit(json.dumps(out), flush=True)
    del bufs
    torch.cuda.empty_cache()
    stream.close()
    if world > 1 and standalone:
        dist.destroy_process_group()
    return out if rank == 0 else None


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


def run_reference_rows(args):
    """Reference arm of `--workload rows`.  The reference has no CPU (or any) implementation of
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
    emit(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
        "config": {"workload": "configs[1]: softmax + RMSNorm forward+reverse over X[65536,4096], r32 and r16",
                   "rows_sampled_per_step": rows, "cols": N},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ----------------------------------------------------------------------------
# configs[4]: the data-parallel Mamba-2 LM training step (the headline)
# ----------------------------------------------------------------------------
LM_METRIC = "Mamba-2 LM training throughput (data-parallel step: forward, cross-entropy, reverse, gradient all-reduce, fused Adam)"
LM_SEQ = 2048
ADAM = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8)
ORACLE_BATCH, ORACLE_SEQ = 1, 64     # the CPU oracle's sample of the step: full model width, 64 tokens


def lm_workload_text(n_layer, batch):
    return ("configs[4]: Mamba-2 LM d_model 768, %d layers, expand 2, headdim 64, d_state 128, ngroups 1, RMSNorm, vocab 50280, "
            "seq 2048, batch %d per GPU, cross-entropy, fused Adam lr 3e-4 betas 0.9/0.95, NCCL all-reduce of the r32 gradient"
            % (n_layer, batch))


# launcher -> DRAM bytes of one call from ncu (dram__bytes_read.sum + dram__bytes_write.sum over the launcher's tensor-core
# kernels: both chunk walks and the group-gradient kernel; the prefix-sum and scalar-gradient kernels were not captured),
# taken at batch 4 x seqlen 4096 x 32 heads (profiles/ssd_walk_and_group_gradients_b4_l4096_h32.md).  Every CTA walks one
# (batch, head) sequence, so traffic grows in proportion to batch x seqlen x heads and is scaled to the step's shape.
# A launcher that is not listed reports traffic null.
LM_NCU_TRAFFIC = {
    "ssd_scan_raw_r16": {"bytes": 81.9e6 + 29.9e6, "units": 4 * 4096 * 32},
    "ssd_scan_reverse_r16": {"bytes": 247.2e6 + 194.5e6 + 286.7e6, "units": 4 * 4096 * 32},
    "ssd_scan_reverse_raw_r16": {"bytes": 247.2e6 + 194.5e6 + 286.7e6, "units": 4 * 4096 * 32},   # the same three kernels
    "ssd_scan_r16": {"bytes": 81.9e6 + 29.9e6, "units": 4 * 4096 * 32},
}


def lm_ncu_traffic(label, cfg, batch, seqlen):
    rec = LM_NCU_TRAFFIC.get(label)
    if rec is None:
        return None
    return int(rec["bytes"] * (batch * seqlen * cfg.heads) / rec["units"])


def lm_launcher_work(label, cfg, batch, seqlen):
    """Algorithmic work of ONE call of a launcher of the step: ({"flops": F} | {"bytes": B}, bound)."""
    import re
    from bench_cases import ssd_bytes, ssd_flops
    T = batch * seqlen
    dims = (batch, seqlen, cfg.heads, cfg.headdim, cfg.d_state, cfg.ngroups)
    if label.startswith("ssd_scan_reverse"):
        return {"flops": ssd_flops(*dims, cfg.chunk, True), "bytes": ssd_bytes(*dims, True)}, "both"
    if label.startswith("ssd_scan"):
        return {"flops": ssd_flops(*dims, cfg.chunk, False), "bytes": ssd_bytes(*dims, False)}, "both"
    m = re.match(r"(?:inner_product|linear)_\w+\[(\d+)x(\d+)x(\d+)\]", label)
    if m:
        a, b, c = (int(v) for v in m.groups())
        return {"flops": 2.0 * a * b * c}, "tensor"
    if label.startswith("cross_entropy"):
        return {"bytes": 2 * T * cfg.vocab * 2}, "hbm"
    return None, None


def lm_oracle_sample(steps, warmup, threads=None):
    """The float64 CPU oracle of the training step (oracle/lm_oracle.py: sequential-recurrence scan, torch autograd,
    Adam) at the full model width on ORACLE_BATCH x ORACLE_SEQ tokens.  Returns (seconds per step, tokens per step,
    threads, first loss)."""
    import numpy as np
    import torch
    from metaphor_b200.mamba_lm import LMConfig, init_weights
    from oracle import lm_oracle
    threads = threads or (os.cpu_count() or 1)
    torch.set_num_threads(threads)
    cfg = LMConfig()
    w = {k: torch.from_numpy(v).double().requires_grad_() for k, v in init_weights(cfg, 0).items()}
    m = {k: torch.zeros_like(v) for k, v in w.items()}
    v2 = {k: torch.zeros_like(v) for k, v in w.items()}
    T = ORACLE_BATCH * ORACLE_SEQ
    tok = torch.from_numpy(np.random.default_rng(1000).integers(0, cfg.vocab, T + 1))
    ids, tgt = tok[:-1], tok[1:]
    times, first = [], None
    for k in range(warmup + steps):
        t0 = time.perf_counter()
        loss = lm_oracle.forward_loss(cfg, w, ids, tgt, ORACLE_BATCH, ORACLE_SEQ)
        loss.backward()
        with torch.no_grad():
            b1, b2, step = ADAM["beta1"], ADAM["beta2"], k + 1
            for name, p in w.items():
                g = p.grad
                m[name].mul_(b1).add_(g, alpha=1 - b1)
                v2[name].mul_(b2).addcmul_(g, g, value=1 - b2)
                p.addcdiv_(m[name] / (1 - b1 ** step), (v2[name] / (1 - b2 ** step)).sqrt_().add_(ADAM["eps"]), value=-ADAM["lr"])
                p.grad = None
        dt = time.perf_counter() - t0
        if first is None:
            first = float(loss.detach())
        if k >= warmup:
            times.append(dt)
    return statistics.mean(times), T, threads, first


def run_reference_lm(args):
    """Reference arm of the headline: the CPU oracle of the same training step on the box's host cores."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps = max(1, min(args.steps, 8))          # ~2-4 s per step: bounded so that the arm ends within minutes
    warmup = 1 if args.warmup > 0 else 0
    dt, T, threads, first = lm_oracle_sample(steps, warmup)
    value = round(T / dt, 2)
    sample = (f"each step = the full-width model (24 layers, vocab 50280) on {ORACLE_BATCH} x {ORACLE_SEQ} tokens instead of 8 x 2048 "
              f"(tokens/s is size-normalised), float64 oracle port: sequential-recurrence scan, torch autograd, Adam; {threads} host threads; "
              f"{steps} timed steps (of the {args.steps} asked for) after {warmup} warm-up; the reference itself has no CPU code and no kernels for most of this step")
    emit(json.dumps({
        "impl": "reference", "metric": LM_METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": round(dt * 1e3, 1), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64", "data": "synthetic (token ids ~ U[0, 50280), seed 1000; weights N(0, 0.02), seed 0)",
        "config": {"workload": lm_workload_text(24, 8), "tokens_sampled_per_step": T},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "loss": {"first_step": round(first, 4)},
    }), flush=True)


def run_lm(args):
    """The headline line.  A step = forward, cross-entropy, reverse, all-reduce, Adam; `value` = tokens/s over all
    ranks with the token ids resident on the device, `e2e` = the same step with the ids copied from pinned host
    memory and the loss read back every step."""
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
    batch, seqlen = args.lm_batch, LM_SEQ
    model = MambaLM(cfg, batch, seqlen, seed=0, loss_scale=65536.0, overlap=not args.lm_no_overlap)
    stream, ts = model.stream, model.stream.torch_stream()
    T = batch * seqlen
    gen = torch.Generator().manual_seed(1000 + rank)
    tok = torch.randint(0, cfg.vocab, (T + 1,), generator=gen, dtype=torch.int32)
    ids_h, tgt_h = tok[:-1].contiguous().pin_memory(), tok[1:].contiguous().pin_memory()
    model.set_batch(ids_h, tgt_h)
    if not args.lm_no_graph:
        model.capture(comm=comm, world=world, **ADAM)
    losses = torch.zeros(args.steps + 1, dtype=torch.float32, device="cuda")   # summed loss of every timed step

    def barrier():
        stream.sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        model.train_step(comm=comm, world=world, **ADAM)
    barrier()
    wall0 = time.time()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record(ts)
    for k in range(args.steps):
        model.train_step(comm=comm, world=world, **ADAM)
        # the step's summed loss, kept on the device (one 4-byte copy kernel; read after the timed region)
        lib.launch_copy_r32(model.loss_sum.data_ptr(), losses.data_ptr() + 4 * k, 1, stream.ctx)
    e1.record(ts)
    barrier()
    wall1 = time.time()
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    if stream.status() != 0:
        raise SystemExit("a kernel reported a non-zero status word")
    ms_per_step = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    value = world * T / (ms_per_step * 1e-3)
    loss_host = (losses.cpu() / T).tolist()

    # every rank must hold the same weights after the same number of all-reduced steps
    wsum = torch.zeros(1, dtype=torch.float32, device="cuda")
    mp.launch("reduce_ij_i", torch.float32, model.w32, wsum, 0.0, 1, model.n_flat, stream)
    stream.sync()
    sums = [torch.zeros_like(wsum) for _ in range(world)]
    if world > 1:
        dist.all_gather(sums, wsum)
    else:
        sums = [wsum]
    checksums = [float(x.item()) for x in sums]

    # end to end: ids from pinned host memory every step, loss read back every step
    barrier()
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    e0.record(ts)
    for _ in range(e2e_steps):
        model.set_batch(ids_h, tgt_h)
        model.train_step(comm=comm, world=world, **ADAM)
        _ = model.loss()
    e1.record(ts)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps

    # one more step issued launcher by launcher with an event pair around each: the share of every launcher
    prof = model.profile_step(comm=comm, world=world, **ADAM)
    barrier()
    graph_kernels = model.launches_per_step(world) or None
    n_params = cfg.n_params()

    out = None
    if rank == 0:
        from bench_cases import peaks, rate_record
        hbm, burst, sustained, peak_kind = peaks()
        Q, H, P, NS = cfg.chunk, cfg.heads, cfg.headdim, cfg.d_state
        ssd_fwd = (2 * Q * Q * NS) * (T // Q) + (2 * Q * Q * P + 4 * Q * NS * P) * (cfg.heads * T // Q)
        flops = 6.0 * n_params * T + 3.0 * ssd_fwd * cfg.n_layer
        total_prof = sum(r["ms"] for r in prof.values())
        top = sorted(prof.items(), key=lambda kv: -kv[1]["ms"])
        dom, dom_rec = top[0]
        work, bound = lm_launcher_work(dom, cfg, batch, seqlen)
        per_call_ms = dom_rec["ms"] / dom_rec["calls"]
        roofline = {"kernel": dom, "calls_per_step": dom_rec["calls"], "share_of_step": round(dom_rec["ms"] / total_prof, 4),
                    "us_per_call": round(per_call_ms * 1e3, 1), "traffic": lm_ncu_traffic(dom, cfg, batch, seqlen),
                    "timing": "CUDA events around every call of the launcher in one step issued without graph replay, same process, right after the timed region"}
        if work is not None:
            rr = rate_record(per_call_ms, work, bound, tensor_peak=sustained)
            if bound == "hbm":
                roofline.update({"bound": "hbm", "achieved": rr["GB/s"], "peak": hbm, "unit": "GB/s", "frac": rr["frac"]})
            else:
                roofline.update({"bound": "tensor", "achieved": rr["TFLOP/s"], "peak": sustained, "unit": "TFLOP/s",
                                 "frac": round(rr["TFLOP/s"] / sustained, 4)})
                if bound == "both":
                    roofline["note"] = ("the scan sits at the ridge: roofline time = max(HBM, tensor) = %.1f us, fraction of that %.4f"
                                        % (rr["roofline_us"], rr["frac"]))
            roofline["peak_kind"] = peak_kind + (" sustained bf16 (fp16 runs on the same pipe)" if bound != "hbm" else " copy bandwidth")
            roofline.update({k: v for k, v in rr.items() if k.startswith("algorithmic")})
        roofline["step_model_flops"] = {"achieved_TFLOP/s": round(flops / (ms_per_step * 1e-3) / 1e12, 1), "flops": flops,
                                        "frac_of_sustained_peak": round(flops / (ms_per_step * 1e-3) / 1e12 / sustained, 4)}
        roofline["launchers_ms"] = {k: {"ms": round(v["ms"], 3), "calls": v["calls"]} for k, v in top}
        out = {
            "metric": LM_METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations / f32 accumulate, master weights and optimizer state",
            "data": "synthetic (token ids ~ U[0, 50280), seed 1000 + rank; weights N(0, 0.02), seed 0 on every rank)",
            "config": {"workload": lm_workload_text(cfg.n_layer, batch),
                       "assumed": f"d_conv 4, tied embedding / LM head, gated RMSNorm before out_proj, D skip, scan chunk argument {cfg.chunk}, static loss scale 65536",
                       "params": n_params, "tokens_per_gpu_step": T, "graph_replay": not args.lm_no_graph,
                       "all_reduce": ("none (one rank)" if world == 1 else model.all_reduce_description()),
                       "l2": "activations and weights (GBs per step) exceed the 126 MB L2; no flush needed"},
            "roofline": roofline, "cpu_baseline": None,
            "e2e": {"value": round(world * T / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "h2d_bytes_per_step": 2 * T * 4,
                    "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps,
                    "path": "MambaLM.set_batch (mpMemcpyHtoD from pinned memory) + train_step + loss() (mpMemcpyDtoH + stream sync) every step"},
            "clocks": clocks,
            "gpu_launches": ((graph_kernels or 0) + 1) * args.steps,
            "gpu_launches_per_step": {"kernels of this library": graph_kernels,
                                      "how": "kernel nodes of the %d captured graphs (forward, loss, reverse, cut at the update buckets) + the live launches of the bucket updates "
                                             "(mixed-precision Adam; gradient folding before an all-reduce)%s + one 4-byte copy of the step's loss"
                                             % (len(model.buckets), "; NCCL's all-reduce kernels are not counted" if world > 1 else "")},
            "loss": {"first_timed_step": round(loss_host[0], 4), "last_timed_step": round(loss_host[args.steps - 1], 4),
                     "expected_at_init": round(math.log(cfg.vocab), 4),
                     "note": "one fixed random batch per rank is repeated, so the loss falls as the model memorises it"},
            "weights_checksum": {"per_rank": checksums, "all_equal": len(set(checksums)) == 1,
                                 "meaning": "sum of the r32 master weights after the last step; equal on all ranks only if every step's gradient was all-reduced"},
        }
    if comm is not None:
        comm.close()
    model.release()
    del model
    torch.cuda.empty_cache()
    if rank == 0:
        if world == 1 and not args.no_per_config:
            out["cpu_baseline"] = lm_cpu_baseline()
            out["per_config"] = run_per_config(args, mp)
        else:
            out["per_config"] = "skipped (--no-per-config)" if world == 1 else "reported at N = 1 only (rank 0 of a single-GPU run)"
        emit(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def lm_cpu_baseline():
    dt, T, threads, first = lm_oracle_sample(steps=2, warmup=1)
    return {"value": round(T / dt, 2), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"full-width model on {ORACLE_BATCH} x {ORACLE_SEQ} tokens (tokens/s is size-normalised), float64 oracle: sequential-recurrence scan, "
                      f"torch autograd, Adam; mean of 2 steps of {dt:.2f} s after 1 warm-up", "first_loss": round(first, 4)}


def run_per_config(args, mp):
    """The other four configs and the contraction shapes, one after another on a fresh stream."""
    import torch
    import bench_cases as bc
    out = {}
    s = mp.Stream()
    flush = bc.Flusher(mp, s)
    ref = bc.ref_cuda_or_none()
    try:
        out["C1_feed_forward_block"] = bc.config_feed_forward(mp, s, ref)
        rows_args = argparse.Namespace(**vars(args)); rows_args.steps = 5; rows_args.warmup = 3; rows_args.e2e_steps = 2; rows_args.cpu_rows = 16384
        out["C2_row_reductions"] = run_rows(rows_args, standalone=False)
        torch.cuda.empty_cache()
        out["C3_fused_chain"] = bc.config_chain(mp, s, flush, ref=ref)
        torch.cuda.empty_cache()
        out["C4_ssd_scan"] = bc.config_ssd(mp, s, flush)
        torch.cuda.empty_cache()
        out["einsum_lm_shapes"] = bc.config_einsum(mp, s, flush, ref=ref)
    finally:
        if isinstance(ref, bc.RefCuda):
            ref.close()
        s.close()
    return out


def run_profile_case(spec: str, timed: bool = False):
    """`--profile-case OP:DTYPE:SIZES`: three launches of one case on a small size, for an ncu capture; with
    `--profile-time` the case is then timed (CUDA events, L2 flushed between launches when the inputs fit it) and one
    JSON line is printed.  Grammar: bench_cases.build_case."""
    import torch
    import metaphor_b200 as mp
    import bench_cases as bc
    torch.zeros(1, device="cuda")
    s = mp.Stream()
    case = bc.build_case(mp, s, spec)
    torch.cuda.synchronize()
    for _ in range(3):
        case.once()
    s.sync()
    if timed:
        rec = case.measure(s, bc.Flusher(mp, s), iters=20)
        rec["case"] = spec
        emit(json.dumps(rec))
    if s.status() != 0:
        raise SystemExit("status word set")
    s.close()


_RESULT_FD = None


def own_stdout():
    """Libraries loaded by the run (NCCL with NCCL_DEBUG set, torchrun's children) write to file descriptor 1; the result
    line must be the only thing on it.  From here on descriptor 1 is a copy of stderr and `emit` writes to the old one."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line, flush=True):
    if _RESULT_FD is None:
        sys.stdout.write(line + "\n"); sys.stdout.flush()
    else:
        os.write(_RESULT_FD, (line + "\n").encode())


def main():
    own_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10, help="upper bound on end-to-end steps")
    ap.add_argument("--cpu-rows", type=int, default=32768, help="rows in the CPU baseline sample of --workload rows")
    ap.add_argument("--workload", default="lm", choices=["lm", "rows"],
                    help="lm = configs[4] training step, tokens/s (default, the headline line); rows = configs[1] alone")
    ap.add_argument("--no-per-config", action="store_true", help="skip the per_config block (and the CPU baseline) of the headline line")
    ap.add_argument("--lm-layers", type=int, default=24)
    ap.add_argument("--lm-batch", type=int, default=8)
    ap.add_argument("--lm-no-graph", action="store_true", help="issue every launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--lm-no-overlap", action="store_true", help="run the bucket updates (all-reduce, Adam) on the main stream instead of a second one")
    ap.add_argument("--lm-chunk", type=int, default=256, help="scan chunk of the LM workload (128 or 256)")
    ap.add_argument("--profile-case", default=None, help="OP:DTYPE:SIZES, three launches for an ncu capture")
    ap.add_argument("--profile-time", action="store_true", help="with --profile-case: also time 20 launches with CUDA events")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case, args.profile_time)
        return
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        (run_reference_lm if args.workload == "lm" else run_reference_rows)(args)
    elif args.workload == "lm":
        run_lm(args)
    else:
        run_rows(args)


if __name__ == "__main__":
    main()
