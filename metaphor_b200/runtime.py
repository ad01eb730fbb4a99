"""Small helpers over the C ABI for tests and benchmarks (torch is used for
device memory only; every computation goes through ``launch_*``)."""
from __future__ import annotations

import ctypes as C
import functools

from . import abi


@functools.lru_cache(maxsize=None)
def lib() -> C.CDLL:
    """The loaded shared library (raises ImportError when it is not built)."""
    return abi.load()


def suffix_of(dtype) -> str:
    """Dtype-key suffix in the order of the reference's scalar.zig Tag enum."""
    import torch
    return {torch.float16: "r16", torch.float32: "r32", torch.float64: "r64"}[dtype]


def _arg(a):
    # torch tensors are passed as raw device pointers
    if hasattr(a, "data_ptr"):
        return C.c_void_p(a.data_ptr())
    if a is None:
        return C.c_void_p(0)
    return a


class Stream:
    """A StreamContext obtained from mpInitStream (own stream) or mpWrapStream
    (``wrap`` = an existing ``cudaStream_t`` value, e.g. torch's current stream)."""

    def __init__(self, wrap: int | None = None):
        self._lib = lib()
        if wrap is None:
            self.ctx = self._lib.mpInitStream()
        else:
            self.ctx = self._lib.mpWrapStream(C.c_void_p(wrap))
        self._open = True

    @property
    def handle(self) -> int:
        return self.ctx.cuda_stream.ptr or 0

    def torch_stream(self):
        import torch
        return torch.cuda.ExternalStream(self.handle)

    def sync(self):
        self._lib.mpStreamSynchronize(self.ctx)

    def status(self) -> int:
        return int(self._lib.mpGetStatus(self.ctx))

    def close(self):
        if self._open:
            self._lib.mpDeinitStream(self.ctx)
            self._open = False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def launch(name: str, dtype, *args):
    """Call ``launch_<name>_<suffix>(*args)``; tensors become device pointers.
    The last argument must be a Stream or a StreamContext."""
    fn = getattr(lib(), f"launch_{name}_{suffix_of(dtype)}")
    conv = [_arg(a) for a in args[:-1]]
    ctx = args[-1].ctx if isinstance(args[-1], Stream) else args[-1]
    fn(*conv, ctx)


class FusedChain:
    """A JIT-compiled element-wise expression (include/mp_jit.h)."""

    def __init__(self, expr: str, dtype):
        self._lib = lib()
        self.dtype = dtype
        key = {"r16": 0, "r32": 1, "r64": 2}[suffix_of(dtype)]
        self.handle = self._lib.mpJitCompile(expr.encode(), key)
        if not self.handle:
            raise ValueError(f"cannot compile expression {expr!r}")
        n = self._lib.mpJitNumLeaves(self.handle)
        self.leaves = [self._lib.mpJitLeafName(self.handle, i).decode() for i in range(n)]

    def _ptrs(self, tensors):
        arr = (C.c_void_p * len(tensors))(*[(t.data_ptr() if t is not None else 0) for t in tensors])
        return arr

    def forward(self, leaves, out, n, stream):
        assert len(leaves) == len(self.leaves)
        self._lib.mpJitForward(self.handle, self._ptrs(leaves), C.c_void_p(out.data_ptr()), n, stream.ctx)

    def reverse(self, leaves, g_out, g_leaves, alpha, n, stream):
        assert len(leaves) == len(self.leaves) == len(g_leaves)
        self._lib.mpJitReverse(self.handle, self._ptrs(leaves), C.c_void_p(g_out.data_ptr() if g_out is not None else 0),
                               self._ptrs(g_leaves), float(alpha), n, stream.ctx)

    def close(self):
        if self.handle:
            self._lib.mpJitRelease(self.handle)
            self.handle = None
