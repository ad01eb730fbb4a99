"""ctypes binding of the C ABI declared in ``include/*.h``.

This module is plumbing for tests and benchmarks: it loads the in-tree
``lib/libmp_kernels.so`` and attaches argument types to every exported entry
point.  There is no fallback: if the shared library has not been built the
import fails with an instruction to build it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libmp_kernels.so"


class PaddedPtr(C.Structure):
    _fields_ = [("ptr", C.c_void_p)]


class StreamContext(C.Structure):
    """Mirror of ``StreamContext`` in include/mp_types.h (two pointers, by value)."""
    _fields_ = [("cuda_stream", PaddedPtr), ("blas_handle", PaddedPtr)]


P, D, L, U32, CTX = C.c_void_p, C.c_double, C.c_ulong, C.c_uint32, StreamContext

# name -> argument types (without the dtype suffix); every entry exists as
# launch_<name>_{r16,r32,r64}.  Order of arguments = include/mp_kernels.h.
LAUNCHERS = {
    "reduce_ij_i": [P, P, D, L, L, CTX],
    "reduce_ij_j": [P, P, D, L, L, CTX],
    "broadcast_i_ij": [P, P, D, L, L, CTX],
    "broadcast_j_ij": [P, P, D, L, L, CTX],
    "dilate_reverse": [P, D, P, L, CTX],
    "subtraction": [P, P, P, L, CTX],
    "relu_reverse": [P, P, P, L, CTX],
    "dilate": [P, D, P, L, CTX],
    "translate": [P, D, P, L, CTX],
    "permutate_ij_ji": [P, P, D, L, L, CTX],
    "negate": [P, P, L, CTX],
    "hadamard_reverse": [P, P, P, L, CTX],
    "inner_product_ij_jk_ik": [P, P, D, P, D, L, L, L, CTX],
    "hadamard": [P, P, P, L, CTX],
    "fill": [P, D, L, CTX],
    "relu": [P, P, L, CTX],
    "addition": [P, P, P, L, CTX],
    "copy": [P, P, L, CTX],
    "sequence": [P, D, D, L, CTX],
    "stepwise": [P, P, L, CTX],
    # additive
    "selu": [P, P, L, CTX],
    "selu_reverse": [P, P, P, L, CTX],
    "softmax_ij_j": [P, P, L, L, CTX],
    "softmax_ij_j_reverse": [P, P, P, D, L, L, CTX],
    "rmsnorm_ij_j": [P, P, D, P, P, L, L, CTX],
    "rmsnorm_ij_j_reverse": [P, P, P, P, D, P, P, D, P, L, L, CTX],
    "sgd": [P, P, D, D, D, L, CTX],
    "adam": [P, P, P, P, D, D, D, D, D, L, L, CTX],
    "inner_product_ij_kj_ik": [P, P, D, P, D, L, L, L, CTX],
    "inner_product_ji_jk_ik": [P, P, D, P, D, L, L, L, CTX],
    "linear_ij_jk_ik": [P, P, P, D, P, D, L, L, L, CTX],
    "linear_ij_jk_ik_ik": [P, P, P, D, P, D, L, L, L, CTX],
    "ssd_scan": [P, P, P, P, P, P, P, L, L, L, L, L, L, L, CTX],
    "ssd_scan_reverse": [P, P, P, P, P, P, P, P, P, P, P, P, L, L, L, L, L, L, L, CTX],
    "ssd_scan_raw": [P, P, L, P, P, P, P, P, P, P, P, L, L, L, L, L, L, L, CTX],
    "ssd_scan_reverse_raw": [P, P, P, P, P, P, P, L, P, P, P, P, P, L, P, P, P, P, P, L, L, L, L, L, L, L, CTX],
    # operators around the scan in a language-model step
    "embedding": [P, P, P, L, L, L, CTX],
    "embedding_reverse": [P, P, P, L, L, L, CTX],
    "causal_conv1d_silu": [P, L, P, P, P, L, L, L, L, L, CTX],
    "causal_conv1d_silu_reverse": [P, L, P, P, P, L, P, L, P, P, L, L, L, L, CTX],
    "causal_conv1d_silu_segments": [P, L, P, P, P, P, P, L, L, L, L, CTX],
    "causal_conv1d_silu_segments_reverse": [P, L, P, P, P, P, P, L, P, L, P, P, L, L, L, CTX],
    "causal_conv1d_silu_segments_reverse_skip": [P, L, P, P, P, P, P, L, P, P, P, L, P, L, P, P, L, L, L, CTX],
    "softplus_bias": [P, L, P, P, L, L, CTX],
    "softplus_bias_reverse": [P, L, P, P, P, L, P, L, L, CTX],
    "ssd_gate": [P, P, P, P, L, P, L, L, L, CTX],
    "ssd_gate_reverse": [P, P, P, P, L, P, P, P, L, P, L, L, L, CTX],
    "ssd_gate_rmsnorm": [P, P, P, P, L, P, D, P, P, L, L, L, CTX],
    "ssd_gate_rmsnorm_reverse": [P, P, P, P, L, P, P, P, P, P, L, P, P, D, P, L, L, L, CTX],
    "head_scale_accumulate": [P, P, P, L, L, L, CTX],
    "cross_entropy": [P, P, D, P, P, L, L, CTX],
    "neg_exp": [P, P, L, CTX],
    "mse_loss_i_i": [P, P, P, P, P, L, CTX],
    "bce_loss_i_i": [P, P, P, P, P, L, CTX],
    "momentum": [P, P, P, D, D, D, D, L, CTX],
    # beyond rank 2: sizes / perm are host arrays of len_t
    "permutate": [P, P, D, P, P, L, CTX],
    "inner_product_bij_bjk_bik": [P, P, D, P, D, L, L, L, L, CTX],
    "inner_product_bij_bkj_bik": [P, P, D, P, D, L, L, L, L, CTX],
    "inner_product_bji_bjk_bik": [P, P, D, P, D, L, L, L, L, CTX],
}

# name -> (restype, argtypes)
UTILS = {
    "mpInitDevice": (None, [U32]),
    "mpMemAlloc": (P, [L, CTX]),
    "mpMemcpyHtoD": (None, [P, P, L, CTX]),
    "mpMemcpyDtoH": (None, [P, P, L, CTX]),
    "mpMemFree": (None, [P, CTX]),
    "mpDeviceSynchronize": (None, []),
    "mpStreamSynchronize": (None, [CTX]),
    "mpInitStream": (CTX, []),
    "mpDeinitStream": (None, [CTX]),
    "mpCheckLastError": (None, []),
    "mpDeviceTotalMemory": (L, [U32]),
    "mpWrapStream": (CTX, [P]),
    "mpGetStatus": (U32, [CTX]),
    "mpSetWaitLimit": (None, [CTX, L]),
    "mpSelfTestWaitTimeout": (None, [CTX]),
    "mpSsdWalkPartition": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]),
    "mpWorkspaceBytes": (L, [CTX]),
    "mpDeviceSmCount": (U32, [CTX]),
    "mpHostAlloc": (P, [L]),
    "mpHostFree": (None, [P]),
    "mpEventCreate": (P, []),
    "mpEventDestroy": (None, [P]),
    "mpEventRecord": (None, [P, CTX]),
    "mpStreamWaitEvent": (None, [CTX, P]),
    "mpGraphBeginCapture": (None, [CTX]),
    "mpGraphEndCapture": (P, [CTX]),
    "mpGraphLaunch": (None, [P, CTX]),
    "mpGraphDestroy": (None, [P]),
    "mpGraphKernelNodes": (L, [P]),
    "mpRmsnormReverseScratchBytes": (L, [L, L, CTX]),
    "mpSsdGateRmsnormReverseScratchBytes": (L, [L, L, L, CTX]),
    "mpSsdScanScratchBytes": (L, [L, L, L, L, L, L, L, U32]),
    "mpSsdScanGenericScratchBytes": (L, [U32, L, L, L, L, L, L, U32]),
    "launch_rmsnorm_ij_j_reverse_static_r32": (C.c_int, [P, P, P, P, D, P, P, D, L, L, CTX]),
    "launch_convert_r16_r32": (None, [P, P, D, L, CTX]),
    "launch_convert_r32_r16": (None, [P, P, L, CTX]),
    "launch_adam_tick": (None, [P, D, D, CTX]),
    "launch_adam_mixed_r32": (None, [P, P, P, P, P, P, D, D, D, D, D, P, L, CTX]),
    # include/mp_comm.h
    "mpCommGetUniqueId": (None, [P]),
    "mpCommInit": (P, [P, U32, U32]),
    "mpCommDestroy": (None, [P]),
    "mpCommWorldSize": (U32, [P]),
    "mpAllReduceSum": (None, [P, P, L, U32, CTX]),
    "mpCommInitStatus": (C.c_int32, [P, U32, U32, C.POINTER(C.c_void_p)]),
    "mpAllReduceSumStatus": (C.c_int32, [P, P, L, U32, CTX]),
    "mpCommPoll": (C.c_int32, [P, CTX, U32]),
    "mpCommAbort": (None, [P]),
    "mpSetFailPoint": (None, [C.c_char_p, C.c_int32]),
    # include/mp_jit.h
    "mpJitCompile": (P, [C.c_char_p, U32]),
    "mpJitRelease": (None, [P]),
    "mpJitNumLeaves": (U32, [P]),
    "mpJitLeafName": (C.c_char_p, [P, U32]),
    "mpJitForward": (None, [P, C.POINTER(C.c_void_p), P, L, CTX]),
    "mpJitReverse": (None, [P, C.POINTER(C.c_void_p), P, C.POINTER(C.c_void_p), D, L, CTX]),
    "mpJitGenerateSource": (P, [C.c_char_p, U32]),
    "mpJitFreeSource": (None, [P]),
}

SUFFIXES = ("r16", "r32", "r64")


def load(path: Path | None = None) -> C.CDLL:
    path = Path(path) if path is not None else LIB_PATH
    if not path.exists():
        raise ImportError(
            f"{path} is missing: the CUDA library has not been built. "
            "Run `python -m metaphor_b200.build` (needs nvcc); there is no CPU fallback.")
    lib = C.CDLL(str(path))
    for name, args in LAUNCHERS.items():
        for sfx in SUFFIXES:
            fn = getattr(lib, f"launch_{name}_{sfx}", None)
            if fn is None:
                continue  # reported by the symbol test, not at import
            fn.restype = None
            fn.argtypes = args
    for name, (res, args) in UTILS.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.restype = res
        fn.argtypes = args
    return lib
