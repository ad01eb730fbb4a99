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


OK, ERROR, TIMEOUT = 0, 2, 3     # MP_COMM_* of include/mp_comm.h


class CommFailure(RuntimeError):
    def __init__(self, what: str, status: int):
        super().__init__(f"{what}: status {status}")
        self.status = status


class GradientComm:
    """The library's own communicator (mpCommInit) for a process that already
    belongs to a torch.distributed group.

    Failure handling is host-side: creation and every collective go through the
    status-returning entry points and raise CommFailure instead of ending the
    process; `poll` waits for a stream with a time-out while NCCL's asynchronous
    error state is checked; `abort` gives a stuck communicator up.

    host_fake=True (tests among CPU ranks): the handle is a one-rank communicator
    (so the C entry points, their handle checks and fail points are exercised) and
    the sum travels through the process group with a time-out - a host-memory
    stand-in with the same interface, for recovery logic that must not need a GPU."""

    def __init__(self, world: int, rank: int, host_fake: bool = False, timeout_s: float = 2.0):
        from .runtime import lib
        self._lib = lib()
        self.world, self.rank, self.host_fake, self.timeout_s = world, rank, host_fake, timeout_s

        def make_id() -> bytes:
            raw = C.create_string_buffer(128)
            self._lib.mpCommGetUniqueId(raw)
            return raw.raw

        handle = C.c_void_p(0)
        if host_fake:
            rc = self._lib.mpCommInitStatus(None, 1, 0, C.byref(handle))
        else:
            uid = exchange_unique_id(make_id, world, rank)
            rc = self._lib.mpCommInitStatus(C.c_char_p(uid), world, rank, C.byref(handle))
        if rc != OK:
            raise CommFailure(f"mpCommInit on rank {rank}", rc)
        self.handle = handle.value

    def all_reduce_sum(self, tensor, stream=None):
        from .runtime import suffix_of
        if self.host_fake:
            rc = self._lib.mpAllReduceSumStatus(self.handle, None, 0, 1, stream.ctx if stream is not None else _null_ctx())
            if rc != OK:
                raise CommFailure("mpAllReduceSum", rc)
            return self._host_sum(tensor)
        key = {"r16": 0, "r32": 1, "r64": 2}[suffix_of(tensor.dtype)]
        rc = self._lib.mpAllReduceSumStatus(self.handle, C.c_void_p(tensor.data_ptr()), tensor.numel(), key, stream.ctx)
        if rc != OK:
            raise CommFailure("mpAllReduceSum", rc)

    def _host_sum(self, tensor):
        import datetime
        import torch.distributed as dist
        try:
            work = dist.all_reduce(tensor, async_op=True)
            if not work.wait(timeout=datetime.timedelta(seconds=self.timeout_s)):
                raise CommFailure("host all-reduce", TIMEOUT)
        except CommFailure:
            raise
        except Exception as e:      # a peer that left closes its connections: the process group reports it here
            raise CommFailure(f"host all-reduce ({type(e).__name__})", ERROR)

    def poll(self, stream, timeout_ms: int = 1000) -> int:
        """MP_COMM_OK once everything queued on `stream` has finished; ERROR / TIMEOUT otherwise (never blocks longer)."""
        return int(self._lib.mpCommPoll(self.handle, stream.ctx, timeout_ms))

    def abort(self):
        if self.handle:
            self._lib.mpCommAbort(self.handle)
            self.handle = None

    def close(self):
        if self.handle:
            self._lib.mpCommDestroy(self.handle)
            self.handle = None


def _null_ctx():
    from .abi import StreamContext
    return StreamContext()


class Heartbeat:
    """Liveness of the ranks, through the process group's key-value store: every rank posts the step it is about
    to start; `missing(step)` names the ranks that have not posted it within the time-out.  Checked on the host
    before a step's first launch, so that no collective is started towards a rank that has left."""

    def __init__(self, store, world: int, rank: int, timeout_s: float = 2.0):
        self.store, self.world, self.rank, self.timeout_s = store, world, rank, timeout_s

    def post(self, step: int):
        self.store.set(f"mp_alive/{self.rank}", str(step))

    def missing(self, step: int):
        import time
        deadline = time.monotonic() + self.timeout_s
        waiting = set(range(self.world)) - {self.rank}
        while waiting and time.monotonic() < deadline:
            for r in list(waiting):
                try:
                    if self.store.check([f"mp_alive/{r}"]) and int(self.store.get(f"mp_alive/{r}").decode()) >= step:
                        waiting.discard(r)
                except Exception:
                    pass
            if waiting:
                time.sleep(0.02)
        return sorted(waiting)
