"""Loader for the reference's own CUDA kernels (oracle/_ref/libref_kernels.so,
built unmodified from the reference checkout by oracle/build_ref.py).  Test
infrastructure: used as a checker and as a timed baseline, never by the product."""
import ctypes as C
from pathlib import Path

from metaphor_b200.abi import LAUNCHERS, StreamContext, SUFFIXES

REF_SO = Path(__file__).resolve().parent / "_ref" / "libref_kernels.so"

# the 20 launchers that exist in the reference (src/cuda/kernel_decls.h)
REF_LAUNCHERS = ["reduce_ij_i", "reduce_ij_j", "broadcast_i_ij", "dilate_reverse", "subtraction", "relu_reverse",
                 "dilate", "translate", "permutate_ij_ji", "negate", "hadamard_reverse", "inner_product_ij_jk_ik",
                 "hadamard", "fill", "relu", "addition", "broadcast_j_ij", "copy", "sequence", "stepwise"]


class RefLib:
    def __init__(self):
        if not REF_SO.exists():
            raise FileNotFoundError(f"{REF_SO} missing: run `python oracle/build_ref.py` where the reference is mounted")
        self.lib = C.CDLL(str(REF_SO))
        for name in REF_LAUNCHERS:
            for s in SUFFIXES:
                fn = getattr(self.lib, f"launch_{name}_{s}")
                fn.restype = None
                fn.argtypes = LAUNCHERS[name]
        self.lib.mpInitStream.restype = StreamContext
        self.lib.mpInitStream.argtypes = []
        self.lib.mpStreamSynchronize.argtypes = [StreamContext]
        self.lib.mpDeinitStream.argtypes = [StreamContext]
        # the caller must have made a CUDA context current (torch does); the
        # reference's mpInitStream creates the stream and its cuBLAS handle
        self.ctx = self.lib.mpInitStream()

    def launch(self, name, sfx, *args):
        import torch
        torch.cuda.current_stream().synchronize()
        conv = [C.c_void_p(a.data_ptr()) if hasattr(a, "data_ptr") else a for a in args]
        getattr(self.lib, f"launch_{name}_{sfx}")(*conv, self.ctx)
        self.lib.mpStreamSynchronize(self.ctx)

    def torch_stream(self):
        import torch
        return torch.cuda.ExternalStream(self.ctx.cuda_stream.ptr)

    def close(self):
        self.lib.mpDeinitStream(self.ctx)
