"""Compile the reference's own CUDA kernels, unmodified, into oracle/_ref/.

TEST INFRASTRUCTURE.  The result (``oracle/_ref/libref_kernels.so``) is used
only by the GPU parity tests and by the benchmark's baseline legs, as the
checker - never by the product path.

The recipe follows the reference's build (file_gen.zig:226-238 and
script_compiler.zig:150-176): every ``src/cuda/nvcc_src/*.cu`` is emitted three
times with the token ``Scalar`` replaced by ``r16``, ``r32`` and ``r64``, and
compiled with ``nvcc -O3 -std=c++20 --expt-relaxed-constexpr`` for the target
architecture (sm_100a here instead of config.json's sm_89), together with
``device_utils.cu``.  Sources are read where they lie under the reference
checkout; the substituted text exists only in a temporary directory that is
deleted afterwards.  Nothing but the shared object is written into the repo.

Usage: ``python oracle/build_ref.py [--reference <checkout>]`` (default: the directory named by the
environment variable MP_REFERENCE_DIR, else a sibling checkout ``../reference``)
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_HOME = Path(NVCC).resolve().parent.parent


DEFAULT_REFERENCE = Path(os.environ.get("MP_REFERENCE_DIR", str(Path(__file__).resolve().parents[2] / "reference")))


def build(reference: Path = DEFAULT_REFERENCE, verbose: bool = True) -> Path | None:
    src_cuda = reference / "src" / "cuda"
    if not src_cuda.is_dir():
        if verbose:
            print(f"reference checkout not found at {reference}; keeping any prebuilt {OUT}")
        return None
    OUT.mkdir(exist_ok=True)
    so = OUT / "libref_kernels.so"
    sources = sorted((src_cuda / "nvcc_src").glob("*.cu"))
    newest = max(p.stat().st_mtime for p in list(sources) + list(src_cuda.glob("*.h")) + list(src_cuda.glob("*.cu*")))
    if so.exists() and so.stat().st_mtime > newest:
        return so
    with tempfile.TemporaryDirectory(prefix="mp_ref_build_") as tmp:
        tmp = Path(tmp)
        cuda_dir = tmp / "src" / "cuda"
        trg = cuda_dir / "nvcc_trg"
        trg.mkdir(parents=True)
        # headers are used in place through symlinks (kernel_header.h includes
        # ../../deps/cuda/include/*, which the README asks the user to symlink)
        for h in list(src_cuda.glob("*.h")) + list(src_cuda.glob("*.cuh")) + [src_cuda / "device_utils.cu"]:
            (cuda_dir / h.name).symlink_to(h)
        (tmp / "deps").mkdir()
        (tmp / "deps" / "cuda").symlink_to(CUDA_HOME)
        units = []
        for src in sources:
            text = src.read_text()
            gen = "\n".join(text.replace("Scalar", r) for r in ("r16", "r32", "r64"))
            out = trg / src.name
            out.write_text(gen)
            units.append(out)
        units.append(cuda_dir / "device_utils.cu")
        flags = ["-O3", "-std=c++20", "--expt-relaxed-constexpr", "--gpu-architecture=sm_100a",
                 "-Xcompiler", "-fPIC", "-w"]

        def cc(u: Path) -> Path:
            obj = tmp / (u.stem + ".o")
            subprocess.run([NVCC, "-c", str(u), "-o", str(obj)] + flags, check=True)
            return obj

        with cf.ThreadPoolExecutor(max_workers=8) as pool:
            objs = list(pool.map(cc, units))
        lib64 = CUDA_HOME / "lib64"
        subprocess.run([NVCC, "-shared", "-o", str(so)] + [str(o) for o in objs] +
                       ["-L" + str(lib64), "-L" + str(lib64 / "stubs"), "-lcublas", "-lcuda",
                        "-Xlinker", "-Bsymbolic", "-Xlinker", "-rpath=" + str(lib64)], check=True)
    if verbose:
        print(f"built {so}")
    return so


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=str(DEFAULT_REFERENCE))
    args = ap.parse_args()
    sys.exit(0 if build(Path(args.reference)) else 1)
