"""Build the sm_100a device library in-tree with nvcc.

Outputs (all under ``metaphor_b200/lib/``, git-ignored, shipped as built files):

* ``libmp_kernels.so`` - every launcher plus the ``mp*`` utilities; this is
  what the Python binding and the tests load.
* ``mp_kernels.a`` and ``libdev_utils.so`` - the same objects under the
  artefact names the reference's build.zig links (build.zig:125-146), so a Zig
  build can link this library in place of its own.

Run ``python -m metaphor_b200.build`` (add ``--force`` to rebuild everything).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "lib" / "obj"
LIB = ROOT / "lib"
INCLUDE = ROOT.parent / "include"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                           "--expt-relaxed-constexpr", "-I", str(INCLUDE)]
UTIL_SOURCES = {"device_utils.cu"}


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def _compile(src: Path, force: bool, hdr_mtime: float) -> Path:
    obj = OBJ / (src.stem + ".o")
    if (not force and obj.exists() and obj.stat().st_mtime > src.stat().st_mtime
            and obj.stat().st_mtime > hdr_mtime):
        return obj
    cmd = [NVCC] + NVCC_FLAGS + ["-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if res.stderr.strip():
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = True) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    hdr_mtime = _headers_mtime()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, hdr_mtime), sources))
    so = LIB / "libmp_kernels.so"
    newest = max(o.stat().st_mtime for o in objs)
    if force or not so.exists() or so.stat().st_mtime < newest:
        # cudart is linked statically (nvcc default); the driver API and NVRTC/NCCL
        # are resolved at run time, so the library loads on a machine without a GPU.
        subprocess.run([NVCC] + ARCH_FLAGS + ["-shared", "-o", str(so)] + [str(o) for o in objs] + ["-ldl"],
                       check=True)
        kernel_objs = [str(o) for o, s in zip(objs, sources) if s.name not in UTIL_SOURCES]
        util_objs = [str(o) for o, s in zip(objs, sources) if s.name in UTIL_SOURCES]
        archive = LIB / "mp_kernels.a"
        if archive.exists():
            archive.unlink()
        subprocess.run(["ar", "-rcs", str(archive)] + kernel_objs, check=True)
        subprocess.run([NVCC] + ARCH_FLAGS + ["-shared", "-o", str(LIB / "libdev_utils.so")] + util_objs + ["-ldl"],
                       check=True)
        if verbose:
            print(f"built {so}")
    build_host()
    return so


def build_host() -> Path:
    """C++ mirror of the reference's Zig host layer (host/metaphor.{hpp,cpp}) ->
    lib/libmp_host.so, linked against libmp_kernels.so in the same directory."""
    src = ROOT / "host" / "metaphor.cpp"
    hdr = ROOT / "host" / "metaphor.hpp"
    out = LIB / "libmp_host.so"
    newest = max(src.stat().st_mtime, hdr.stat().st_mtime, (LIB / "libmp_kernels.so").stat().st_mtime)
    if not out.exists() or out.stat().st_mtime < newest:
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-o", str(out), str(src),
                        "-L" + str(LIB), "-lmp_kernels", "-Wl,-rpath,$ORIGIN"], check=True)
    return out


if __name__ == "__main__":
    build(force="--force" in sys.argv)
