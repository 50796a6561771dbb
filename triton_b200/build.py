"""Build the in-tree shared library `triton_b200/libtriton_b200.so` with nvcc for sm_100a.

    python -m triton_b200.build [--force] [--verbose] [--trace]

Each .cu under csrc/ is compiled to an object next to the library (stale objects are
rebuilt when the source or a header is newer) and linked with the static CUDA runtime;
the driver API is reached through cudaGetDriverEntryPoint, so the library loads on a
machine without a GPU driver (it then reports B200_ERR_DEVICE from every compute call).
"""
import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libtriton_b200.so")
OBJ = os.path.join(PKG, "csrc", "_obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the library has to be built where the CUDA toolkit is installed")
    return exe


def _newest_header():
    t = os.path.getmtime(os.path.join(ROOT, "include", "triton_b200.h"))
    for f in os.listdir(CSRC):
        if f.endswith((".h", ".cuh")):
            t = max(t, os.path.getmtime(os.path.join(CSRC, f)))
    return t


def build(force=False, verbose=False, trace=False):
    """trace=True builds the instrumented variant (-DB200_TRACE) next to the production library, as
    libtriton_b200_trace.so with its own object directory; see triton_b200/trace.py."""
    nvcc = _nvcc()
    OBJ = os.path.join(PKG, "csrc", "_obj_trace" if trace else "_obj")
    LIB = os.path.join(PKG, "libtriton_b200_trace.so" if trace else "libtriton_b200.so")
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr_t = _newest_header()
    jobs = []
    for s in srcs:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_t):
            cmd = [nvcc, *NVCC_FLAGS, *(["-DB200_TRACE"] if trace else []), "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in srcs]
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--trace", action="store_true", help="build the instrumented variant libtriton_b200_trace.so")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.trace))
