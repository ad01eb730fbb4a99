"""Worker run as `python -m torch.distributed.run ... tests/dist_worker.py MODE`.

MODE cpu: gloo ranks exercise the host logic of the data-parallel path - row
sharding, the unique-id exchange, "sum of shard gradients = full-batch
gradient", optimizer step with grad_scale = 1/world - with the CPU oracle doing
the arithmetic.  MODE gpu: the same step with the library's kernels and its
NCCL all-reduce (mpAllReduceSum).  MODE fail_init / leave: failure detection
among CPU ranks - a rank whose communicator creation fails (host fail point),
and a rank that leaves between two steps; the survivors must notice on the host
(status codes, heartbeat, bounded collective) and never hang.  Exit code 0 = all
checks passed."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from metaphor_b200.dist import exchange_unique_id, shard_range  # noqa: E402

M, N, EPS = 96, 256, 1e-6


def inputs():
    r = np.random.default_rng(0)
    x = r.standard_normal((M, N)).astype(np.float32)
    gy = r.standard_normal((M, N)).astype(np.float32)
    gain = (1 + 0.02 * r.standard_normal(N)).astype(np.float32)
    return x, gy, gain


def failure_modes(mode, rank, world):
    import datetime
    import metaphor_b200 as mp
    from metaphor_b200.dist import ERROR, TIMEOUT, CommFailure, GradientComm, Heartbeat
    lib = mp.lib()
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20))
    store = dist.distributed_c10d._get_default_store()
    if mode == "fail_init":
        # rank 1's communicator creation fails; every rank learns of it before any collective is started
        if rank == 1:
            lib.mpSetFailPoint(b"mpCommInit", 1)
        try:
            comm = GradientComm(world, rank, host_fake=True)
            mine = 0
        except CommFailure as e:
            assert e.status == ERROR and rank == 1
            comm, mine = None, e.status
        status = torch.tensor([mine], dtype=torch.int32)
        gathered = [torch.zeros_like(status) for _ in range(world)]
        dist.all_gather(gathered, status)
        failed = [r for r, t in enumerate(gathered) if int(t) != 0]
        assert failed == [1], failed
        # the fail point is spent: a second attempt on rank 1 succeeds (the recovery path rebuilds the communicator)
        if rank == 1:
            comm = GradientComm(world, rank, host_fake=True)
        t = torch.full((8,), float(rank + 1))
        comm.all_reduce_sum(t)
        assert float(t[0]) == world * (world + 1) / 2
        # bad handles and arguments are reported, not dereferenced
        import ctypes as C
        assert lib.mpAllReduceSumStatus(None, None, 0, 1, mp.abi.StreamContext()) == 4
        out = C.c_void_p(0)
        assert lib.mpCommInitStatus(None, 2, 5, C.byref(out)) == 5
        lib.mpSetFailPoint(b"mpAllReduceSum", 1)
        try:
            comm.all_reduce_sum(torch.zeros(4))
            raise AssertionError("the fail point did not fire")
        except CommFailure as e:
            assert e.status == ERROR
        lib.mpSetFailPoint(None, 0)
        comm.close()
        dist.barrier()
    else:
        # two steps; rank 1 leaves after the first, with nothing in flight
        comm = GradientComm(world, rank, host_fake=True, timeout_s=2.0)
        hb = Heartbeat(store, world, rank, timeout_s=1.5)
        hb.post(1)
        assert hb.missing(1) == []
        t = torch.full((1024,), float(rank + 1))
        comm.all_reduce_sum(t)
        assert float(t[0]) == world * (world + 1) / 2
        if rank == 1:
            comm.close()
            print(f"rank {rank}/{world} ok", flush=True)
            os._exit(0)                              # gone without a word, between steps
        hb.post(2)
        gone = hb.missing(2)                         # noticed on the host before the next launch
        assert gone == [1], gone
        # and a collective started anyway ends with a status within the time-out instead of hanging
        import time
        t0 = time.monotonic()
        try:
            comm.all_reduce_sum(torch.ones(1024))
            raise AssertionError("the collective towards a rank that left did not fail")
        except CommFailure as e:
            assert e.status in (ERROR, TIMEOUT)
        assert time.monotonic() - t0 < 10.0
        comm.close()
    print(f"rank {rank}/{world} ok", flush=True)
    os._exit(0)      # no collective shutdown: a peer may be gone


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if mode in ("fail_init", "leave"):
        return failure_modes(mode, rank, world)
    from oracle import pyoracle as orc
    x, gy, gain = inputs()
    lo, hi = shard_range(M, world, rank)
    full_gx, full_gg = orc.rmsnorm_ij_j_reverse(x, gain, gy, EPS)
    w_ref = gain.copy(); m_ref = np.zeros(N, np.float32); v_ref = np.zeros(N, np.float32)
    orc.adam(w_ref, (full_gg / world).astype(np.float32), m_ref, v_ref, 3e-4, 0.9, 0.95, 1e-8, 1.0, 1)

    if mode == "cpu":
        dist.init_process_group("gloo")
        uid = exchange_unique_id(lambda: bytes(range(128)), world, rank)
        assert uid == bytes(range(128)), "unique id did not reach every rank"
        gx, gg = orc.rmsnorm_ij_j_reverse(x[lo:hi], gain, gy[lo:hi], EPS)
        assert np.allclose(gx, full_gx[lo:hi], rtol=0, atol=1e-6)
        t = torch.from_numpy(gg.copy())
        dist.all_reduce(t)                                   # sum of the shards' partial gradients
        assert np.allclose(t.numpy(), full_gg, rtol=1e-5, atol=1e-5)
        w = gain.copy(); m = np.zeros(N, np.float32); v = np.zeros(N, np.float32)
        orc.adam(w, t.numpy(), m, v, 3e-4, 0.9, 0.95, 1e-8, 1.0 / world, 1)   # mean folded into the step
        assert np.allclose(w, w_ref, rtol=1e-6, atol=1e-7)
    else:
        import metaphor_b200 as mp
        from metaphor_b200.dist import GradientComm
        torch.cuda.set_device(local)
        mp.lib().mpInitDevice(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        s = mp.Stream()
        comm = GradientComm(world, rank)
        # plain all-reduce check on three dtypes
        for dt, tol in ((torch.float32, 0), (torch.float64, 0), (torch.float16, 1e-3)):
            t = torch.full((1000003,), float(rank + 1), device="cuda", dtype=dt)
            torch.cuda.synchronize()
            comm.all_reduce_sum(t, s); s.sync()
            want = world * (world + 1) / 2
            assert float((t.double() - want).abs().max()) <= tol * want, (dt, float(t[0]))
        # sharded RMSNorm reverse -> all-reduce of the gain gradient -> Adam with grad_scale = 1/world
        rows = hi - lo
        dx = torch.from_numpy(x[lo:hi]).cuda(); dgy = torch.from_numpy(gy[lo:hi]).cuda(); dgain = torch.from_numpy(gain).cuda()
        gx = torch.empty_like(dx); gg = torch.empty_like(dgain)
        scratch = torch.empty(mp.lib().mpRmsnormReverseScratchBytes(rows, N, s.ctx), dtype=torch.uint8, device="cuda")
        w = dgain.clone(); mm = torch.zeros_like(w); vv = torch.zeros_like(w)
        torch.cuda.synchronize()
        mp.launch("rmsnorm_ij_j_reverse", torch.float32, dx, dgain, None, dgy, EPS, gx, gg, 0.0, scratch, rows, N, s)
        comm.all_reduce_sum(gg, s)
        mp.launch("adam", torch.float32, w, gg, mm, vv, 3e-4, 0.9, 0.95, 1e-8, 1.0 / world, 1, N, s)
        s.sync()
        assert s.status() == 0
        assert np.allclose(gx.cpu().numpy(), full_gx[lo:hi], rtol=0, atol=1e-4)
        assert np.allclose(gg.cpu().numpy(), full_gg, rtol=1e-4, atol=1e-4)
        assert np.allclose(w.cpu().numpy(), w_ref, rtol=1e-5, atol=1e-6)
        comm.close(); s.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}/{world} ok", flush=True)


if __name__ == "__main__":
    main()
