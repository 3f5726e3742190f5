"""Ahead-of-time build of the native library (sm_100a only, in-tree).

`python -m yirage_b200.build` compiles every csrc/*.cu into yirage_b200/libypk.so with nvcc:
the host side of the C ABI (ypk_abi.cu) and one translation unit per kernel variant
(megakernel_decode.cu, megakernel_decode_tp.cu, megakernel_wide.cu, megakernel_moe.cu), each
of which includes the task runners (runners.cuh) and so owns its copies of them; relocatable
device code linked at the end.  There is no per-model JIT: shapes travel in the task table at
run time, unlike the reference which runs nvcc for every graph
(python/yirage/persistent_kernel.py:1138-1318).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libypk.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-rdc=true", "--threads", "0",
    # every runner is called from a kernel of 288 threads (one CTA per SM): 168 registers per
    # thread is what such a kernel can have, and a callee may not use more than its caller
    "-maxrregcount", "168",
    "-Xcompiler", "-fPIC", "-shared",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "ypk.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compile libypk.so if it is missing or older than its sources."""
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    cmd = [nvcc] + NVCC_FLAGS + ["-o", LIB] + sources() + ["-lcudart"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libypk.so")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(LIB)
