"""Builds the native libraries of this package, in-tree.

  warp34_b200/lib/libwarp34_b200.so   CUDA kernels + C ABI (include/warp34_b200.h), sm_100a only
  warp34_b200/lib/libwarp34_host.so   C++ page manager + C ABI (include/warp34_host.h), no CUDA

`python -m warp34_b200.build` rebuilds what is stale.  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", INCLUDE]
# The append unit is built like the reference's kernels (-use_fast_math): rsqrtf() and '/'
# must lower to the same approximate instructions for the packed bytes to be identical.
CUDA_UNITS = [
    ("tq4_append.cu", ["-use_fast_math"]),
    ("tq4_attention.cu", []),
    ("abi_misc.cu", []),
]
HOST_UNITS = ["page_pool.cpp", "prefix_cache.cpp"]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _headers():
    out = []
    for d in (CSRC, INCLUDE):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                out.append(os.path.join(d, f))
    return out


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("native build failed: " + os.path.basename(cmd[-1]))


def build_cuda(force=False, extra_defines=(), out_name="libwarp34_b200.so", verbose=False):
    os.makedirs(LIB, exist_ok=True)
    objdir = os.path.join(LIB, "obj" + ("_" + out_name if extra_defines else ""))
    os.makedirs(objdir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    hdrs = _headers()
    objs = []
    for src, flags in CUDA_UNITS:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + hdrs):
            cmd = [nvcc] + ARCH + COMMON + flags + list(extra_defines)
            if verbose:
                cmd += ["-Xptxas", "-v"]
            _run(cmd + ["-c", s, "-o", o])
        objs.append(o)
    target = os.path.join(LIB, out_name)
    if force or _stale(target, objs):
        _run([nvcc, "-shared", "-o", target] + objs + ["-lcudart"])
    return target


def build_host(force=False):
    os.makedirs(LIB, exist_ok=True)
    target = os.path.join(LIB, "libwarp34_host.so")
    srcs = [os.path.join(CSRC, "host", s) for s in HOST_UNITS]
    if force or _stale(target, srcs + _headers()):
        _run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall",
              "-I", INCLUDE, "-o", target] + srcs)
    return target


def build_bounds(force=False):
    """The bounds-checked build of the kernel library (-DW34_BOUNDS): same sources, every block-table
    index, page id and write slot range-checked, violations recorded instead of trapping."""
    return build_cuda(force, extra_defines=("-DW34_BOUNDS",), out_name="libwarp34_b200_bounds.so")


def build_all(force=False):
    """Everything, the regular and the bounds-checked kernel library side by side (nvcc is the long pole)."""
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=3) as pool:
        jobs = [pool.submit(build_cuda, force), pool.submit(build_host, force), pool.submit(build_bounds, force)]
        return tuple(j.result() for j in jobs)


if __name__ == "__main__":
    if "--bounds" in sys.argv:
        print("built", build_bounds(force="--force" in sys.argv))
    else:
        for t in build_all(force="--force" in sys.argv):
            print("built", t)
