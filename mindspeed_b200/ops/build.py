"""Builds the in-tree native libraries with nvcc / g++ (no torch headers needed).

  libmsb200_kernels.so   every .cu under csrc/kernels and csrc/runtime (sm_100a only)
  libmsb200_host.so      host-side C++ (allocator, flop counter, adaptive-cp algorithms, ...)

Objects are cached under csrc/build/ keyed by a hash of the source and the headers.
Run as ``python -m mindspeed_b200.ops.build``.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import hashlib
import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
BUILD = os.path.join(CSRC, "build")
KERNEL_LIB = os.path.join(CSRC, "libmsb200_kernels.so")
HOST_LIB = os.path.join(CSRC, "libmsb200_host.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
              "-I" + os.path.join(CSRC, "include")]
NVCC_FLAGS += os.environ.get("MSB200_NVCC_EXTRA", "").split()     # extra flags for experiments (part of the object hash)
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-fstack-protector-strong", "-D_FORTIFY_SOURCE=2",
             "-I" + os.path.join(CSRC, "include"), "-pthread"]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _hash(path: str, headers) -> str:
    h = hashlib.sha256()
    for p in [path] + sorted(headers):
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()[:16]


def _compile(src: str, headers, verbose: bool) -> str:
    os.makedirs(BUILD, exist_ok=True)
    tag = _hash(src, headers)
    obj = os.path.join(BUILD, f"{os.path.basename(src)}.{tag}.o")
    if os.path.exists(obj):
        return obj
    if src.endswith(".cu"):
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    else:
        cmd = ["g++"] + CXX_FLAGS + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    # drop stale objects of the same source
    for old in glob.glob(os.path.join(BUILD, f"{os.path.basename(src)}.*.o")):
        if old != obj:
            os.remove(old)
    return obj


def build(verbose: bool = False, jobs: int = 0) -> None:
    headers = glob.glob(os.path.join(CSRC, "include", "*"))
    cu = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")) + glob.glob(os.path.join(CSRC, "runtime", "*.cu")))
    cpp = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    jobs = jobs or min(8, os.cpu_count() or 4)
    with cf.ThreadPoolExecutor(jobs) as ex:
        cu_objs = list(ex.map(lambda s: _compile(s, headers, verbose), cu))
        cpp_objs = list(ex.map(lambda s: _compile(s, headers, verbose), cpp))

    def link(out, objs, extra):
        if not objs:
            return
        newest = max(os.path.getmtime(o) for o in objs)
        if os.path.exists(out) and os.path.getmtime(out) >= newest:
            return
        tmp = out + ".tmp"
        cmd = [_nvcc(), "-shared", "-o", tmp] + objs + extra
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, out)

    # static cudart (nvcc default): shares the primary context with torch's runtime; no libcuda link dependency
    link(KERNEL_LIB, cu_objs, [])
    link(HOST_LIB, cpp_objs, ["-lpthread"])


if __name__ == "__main__":
    build(verbose="-v" in sys.argv)
    print("built", KERNEL_LIB, os.path.exists(KERNEL_LIB), HOST_LIB, os.path.exists(HOST_LIB))
