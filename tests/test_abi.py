"""CPU checks of the drop-in boundary: the library loads without a GPU, exports
every symbol include/*.h declares, and the headers are valid C."""
import ctypes
import re
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
INC = ROOT / "include"

# the 20 launchers of the reference's generated header (src/cuda/kernel_decls.h:11-436)
REFERENCE_LAUNCHERS = [
    "reduce_ij_i", "reduce_ij_j", "broadcast_i_ij", "dilate_reverse", "subtraction", "relu_reverse", "dilate",
    "translate", "permutate_ij_ji", "negate", "hadamard_reverse", "inner_product_ij_jk_ik", "hadamard", "fill",
    "relu", "addition", "broadcast_j_ij", "copy", "sequence", "stepwise"]
# the 11 utilities of src/cuda/device_utils.h:12-22
REFERENCE_UTILS = ["mpInitDevice", "mpMemAlloc", "mpMemcpyHtoD", "mpMemcpyDtoH", "mpMemFree", "mpDeviceSynchronize",
                   "mpStreamSynchronize", "mpInitStream", "mpDeinitStream", "mpCheckLastError", "mpDeviceTotalMemory"]


def declared_symbols():
    names = []
    for h in sorted(INC.glob("*.h")):
        text = h.read_text()
        for m in re.finditer(r"^MP_DECL3\((\w+),", text, re.M):
            names += [f"launch_{m.group(1)}_{s}" for s in ("r16", "r32", "r64")]
        for m in re.finditer(r"^MP_EXTERN_C\s+[\w\s\*]+?\b(\w+)\s*\(", text, re.M):
            names.append(m.group(1))
    return names


def test_library_loads_without_gpu_and_exports_every_declared_symbol(mp):
    lib = mp.lib()
    names = declared_symbols()
    assert len(names) >= 60 + 11
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_reference_symbol_set_is_declared():
    names = set(declared_symbols())
    for l in REFERENCE_LAUNCHERS:
        for s in ("r16", "r32", "r64"):
            assert f"launch_{l}_{s}" in names
    for u in REFERENCE_UTILS:
        assert u in names


def test_binding_table_matches_headers(mp):
    names = set(declared_symbols())
    bound = {f"launch_{n}_{s}" for n in mp.LAUNCHERS for s in mp.SUFFIXES} | set(mp.UTILS)
    assert bound == names, (sorted(bound - names), sorted(names - bound))


def test_stream_context_layout(mp):
    # two pointers by value, 16 bytes (reference kernel_header.h:10-17)
    assert ctypes.sizeof(mp.StreamContext) == 16
    assert mp.StreamContext.cuda_stream.offset == 0 and mp.StreamContext.blas_handle.offset == 8


def test_headers_are_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "mp_types.h"\n#include "mp_device_utils.h"\n#include "mp_kernels.h"\n'
                   "int main(void){ StreamContext c; c.cuda_stream.ptr = 0; (void)c;"
                   " return (int)sizeof(SortPair_r16) - (int)sizeof(SortPair_r16); }\n")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(INC), "-c", str(src), "-o", str(tmp_path / "t.o")],
                   check=True)


def test_reference_artefact_names_exist(mp):
    # build.zig:125-146 links src/lib/mp_kernels.a and libdev_utils.so
    libdir = Path(mp.LIB_PATH).parent
    assert (libdir / "mp_kernels.a").exists() and (libdir / "libdev_utils.so").exists()
