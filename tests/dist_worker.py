"""Worker run as `python -m torch.distributed.run ... tests/dist_worker.py MODE`.

MODE cpu: gloo ranks exercise the host logic of the data-parallel path - row
sharding, the unique-id exchange, "sum of shard gradients = full-batch
gradient", optimizer step with grad_scale = 1/world - with the CPU oracle doing
the arithmetic.  MODE gpu: the same step with the library's kernels and its
NCCL all-reduce (mpAllReduceSum).  Exit code 0 = all checks passed."""
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


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
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
