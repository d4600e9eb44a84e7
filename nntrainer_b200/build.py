"""Builds nntrainer_b200/libnntr_cuda.so from csrc/*.cu with nvcc for sm_100a.

The library links the static CUDA runtime and nothing else, so it loads next to
any framework. Run as ``python -m nntrainer_b200.build`` or through
``__graft_entry__.build()``; nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnntr_cuda.so")
HOST_CXX = "/usr/bin/g++"  # the image's $CXX points at a toolchain without libgomp/specs

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v", "-cudart", "static",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(HERE, "..", "include", "nntr_cuda.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link if any source is newer than the library. Several processes may call this at once (one rank per
    GPU, test workers): an exclusive file lock lets one of them build while the others wait and then find it done."""
    if not force and not stale():
        return LIB
    import fcntl
    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not stale():
            return LIB
        return _build_locked(verbose)


def _build_locked(verbose: bool) -> str:
    objs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    ccbin = ["-ccbin", HOST_CXX] if os.path.exists(HOST_CXX) else []
    for src in sources():
        obj = os.path.join(HERE, "build", os.path.basename(src)[:-3] + ".o")
        cmd = ["nvcc", *ccbin, *NVCC_FLAGS, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        with open(obj + ".ptxas.txt", "w") as f:
            f.write(r.stdout + r.stderr)
        objs.append(obj)
    cmd = ["nvcc", *ccbin, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
           "-o", LIB, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
