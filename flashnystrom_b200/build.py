"""Build the C-ABI CUDA library in-tree with nvcc for sm_100a.

    python -m flashnystrom_b200.build            # build if sources are newer than the .so
    python -m flashnystrom_b200.build --force

The result is flashnystrom_b200/lib/libflashnystrom_b200.so; nothing is installed elsewhere.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, os.environ.get("FNB_LIB_NAME", "libflashnystrom_b200.so"))
SOURCES = ["fnb_api.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
]
if os.environ.get("FNB_PTXAS_VERBOSE"):      # registers, spills, shared memory per kernel
    NVCC_FLAGS += ["-Xptxas", "-v"]
NVCC_FLAGS += os.environ.get("FNB_EXTRA_NVCC_FLAGS", "").split()   # e.g. -DFNB_NS_TRACE for a profiling build


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build flashnystrom_b200")
    return exe


def _stale():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(PKG), "include", "flashnystrom_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc()] + NVCC_FLAGS + [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB_PATH]
    if verbose:
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose or os.environ.get("FNB_PTXAS_VERBOSE"):
        print(res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
