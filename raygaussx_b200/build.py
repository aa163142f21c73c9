"""In-tree build of librgx.so (the CUDA kernels and the C ABI) for sm_100a.

    python -m raygaussx_b200.build [--force]

nvcc cross-compiles without a GPU.  The library is written next to this file so
that it is found by ``raygaussx_b200._lib`` without any install step.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "librgx.so")
SOURCES = ["api.cu", "build.cu", "color.cu", "march.cu", "march_lists.cu", "binning.cu", "static_forward.cu", "knn.cu", "peaks.cu"]
HEADERS = ["rgx_internal.cuh", "device_math.cuh", "march_common.cuh", os.path.join("..", "..", "include", "rgx.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False, extra=(), out=None):
    """Compile every .cu of the package into librgx.so (or ``out``).  Returns the library path.
    ``extra`` and ``$RGX_NVCC_FLAGS`` are added to the compiler's flags (tuning macros)."""
    extra = tuple(extra) + tuple(os.environ.get("RGX_NVCC_FLAGS", "").split())
    lib = out or LIB
    if not force and out is None and not needs_build():
        return LIB
    objs = []
    objdir = os.path.join(HERE, "build") if out is None else os.path.join(os.path.dirname(os.path.abspath(out)), "obj_" + os.path.basename(out))
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stdout.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [_nvcc(), "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(cmd, check=True)
    return lib


if __name__ == "__main__":
    out_arg = [a.split("=", 1)[1] for a in sys.argv if a.startswith("--out=")]
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, out=out_arg[0] if out_arg else None))
