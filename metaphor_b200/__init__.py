"""B200-native device layer behind Metaphor's ``mp.ops`` / ``mp.optm``.

The product is the C-ABI shared library built from ``csrc/`` (declared in
``include/*.h``).  This package only loads it and offers a thin helper for
tests and benchmarks; importing it without the built library raises.
"""
from .abi import StreamContext, LAUNCHERS, UTILS, SUFFIXES, LIB_PATH, load
from .runtime import Stream, FusedChain, lib, suffix_of, launch

__all__ = ["StreamContext", "LAUNCHERS", "UTILS", "SUFFIXES", "LIB_PATH", "load",
           "Stream", "FusedChain", "lib", "suffix_of", "launch"]
