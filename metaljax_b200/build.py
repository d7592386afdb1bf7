"""Builds libqmm.so (hand-written CUDA for sm_100a + the C ABI) in-tree with nvcc.

    python -m metaljax_b200.build [--force] [--verbose]

The shared object lands next to this file so that it travels with the source tree;
nothing is installed into site-packages and no JIT cache is involved.
"""

from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libqmm.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libqmm.so cannot be built")


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    deps += glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return LIB
    objs = []
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [_nvcc(), *[f for f in NVCC_FLAGS if f != "-shared"], "-c", src, "-o", obj]
        cmd[1:1] = os.environ.get("QMM_NVCC_EXTRA", "").split()      # e.g. -DQMM_GEMV_TRACING=1
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, pr in procs:
        out = pr.communicate()[0].decode()
        if pr.returncode != 0 or verbose:
            sys.stdout.write(out)
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the output above")
    tmp = LIB + ".tmp"
    subprocess.check_call([_nvcc(), "-shared", "-o", tmp, *objs,
                           "-gencode", "arch=compute_100a,code=sm_100a"])
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
