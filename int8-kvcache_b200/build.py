"""Build the native library (lib/libkvq_b200.so) with nvcc for sm_100a.

    python int8-kvcache_b200/build.py [--force] [--verbose]

The library is plain CUDA C++ behind a C ABI (include/kvq_b200.h): no PyTorch headers, static cudart.
nvcc cross-compiles without a GPU, so this runs on any machine with the CUDA 12.8+ toolkit.
"""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libkvq_b200.so")
SOURCES = ["kvq_api.cu", "kvq_quant.cu", "kvq_decode.cu", "kvq_prefill.cu", "kvq_calib.cu", "kvq_gather.cu"]
HEADERS = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".inl"))) + [
    os.path.join(os.path.dirname(HERE), "include", "kvq_b200.h")]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler",
         "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-cudart", "static"]


def nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the native library needs the CUDA toolkit to build")
    return exe


def up_to_date():
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS + [os.path.abspath(__file__)]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, verbose=False):
    """Compile if the library is missing or older than its sources. Returns the library path."""
    if not force and up_to_date():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc(), *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB, *[os.path.join(CSRC, s) for s in SOURCES]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("nvcc failed building libkvq_b200.so")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(args.force, args.verbose))
