"""Host-side helpers for the data-parallel path: how work is split over ranks
and how the NCCL communicator of the C ABI (include/mp_comm.h) is bootstrapped
from a torch.distributed process group (any backend: the 128-byte unique id
travels through a broadcast of a CPU tensor or through the store)."""
from __future__ import annotations

import ctypes as C


def shard_range(n: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous slice [lo, hi) of n units owned by `rank`: the first n % world
    ranks get one extra unit, no unit is dropped or duplicated."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def exchange_unique_id(make_id, world: int, rank: int) -> bytes:
    """Rank 0 creates the id with `make_id()` (bytes of length 128); every rank
    returns it.  Uses the default torch.distributed group."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return make_id()
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = torch.frombuffer(bytearray(make_id()), dtype=torch.uint8).clone()
    backend = dist.get_backend()
    if backend == "nccl":
        dev = buf.cuda()
        dist.broadcast(dev, src=0)
        buf = dev.cpu()
    else:
        dist.broadcast(buf, src=0)
    return bytes(buf.numpy().tobytes())


class GradientComm:
    """The library's own communicator (mpCommInit) for a process that already
    belongs to a torch.distributed group."""

    def __init__(self, world: int, rank: int):
        from .runtime import lib
        self._lib = lib()
        self.world, self.rank = world, rank

        def make_id() -> bytes:
            raw = C.create_string_buffer(128)
            self._lib.mpCommGetUniqueId(raw)
            return raw.raw

        uid = exchange_unique_id(make_id, world, rank)
        self.handle = self._lib.mpCommInit(C.c_char_p(uid), world, rank)

    def all_reduce_sum(self, tensor, stream):
        from .runtime import suffix_of
        key = {"r16": 0, "r32": 1, "r64": 2}[suffix_of(tensor.dtype)]
        self._lib.mpAllReduceSum(self.handle, C.c_void_p(tensor.data_ptr()), tensor.numel(), key, stream.ctx)

    def close(self):
        if self.handle:
            self._lib.mpCommDestroy(self.handle)
            self.handle = None
