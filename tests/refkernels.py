"""The loader of the reference's own CUDA kernels lives beside the recipe that builds them (oracle/refkernels.py)."""
from oracle.refkernels import REF_LAUNCHERS, REF_SO, RefLib  # noqa: F401
