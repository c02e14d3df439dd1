"""Compile the CUDA sources of this package for sm_100a, in-tree.

``python -m cuda_llm_b200.build`` (or ``build()``) writes ``lib/libb2ops.so``: the
kernels plus the C ABI declared in include/b2ops.h.  nvcc cross-compiles without a
GPU.  The flags follow the reference's build where they are observable behaviour:
C++17 and per-thread default streams (reference CMakeLists.txt:5-9).
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libb2ops.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--default-stream", "per-thread", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
]


# sources whose kernels launch other kernels from the device (the sampler's rarely needed whole-row route is launched
# by the kernel that finds out whether it is needed): relocatable device code, linked against the device runtime
RDC_SOURCES = {"sampler_fallback.cu"}


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def build(force: bool = False, verbose: bool = False) -> str:
    """Build lib/libb2ops.so when it is missing or older than a source; returns its path.
    Every .cu file becomes an object of its own (compiled in parallel, and only when it or a header is newer
    than the object), then the objects are linked."""
    import concurrent.futures as cf
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        [os.path.join(ROOT, "include", "b2ops.h")]
    if not force and _newer(LIB, sources() + headers):
        return LIB
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]

    def compile_one(src):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        if not force and _newer(obj, [src] + headers):
            return obj, ""
        cmd = [nvcc] + compile_flags + (["-Xptxas", "-v"] if verbose else []) + \
            (["-rdc=true"] if os.path.basename(src) in RDC_SOURCES else []) + \
            ["-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", src, "-o", obj]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed on " + src + ":\n" + proc.stdout + proc.stderr)
        return obj, proc.stderr

    with cf.ThreadPoolExecutor(max(1, min(8, os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, sources()))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    proc = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] +
                          [obj for obj, _ in results] + ["-lcudadevrt"], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc (link) failed:\n" + proc.stdout + proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))


SHIM_DIR = os.path.join(CSRC, "llm")
SHIM_LIB = os.path.join(LIB_DIR, "libb2llm.so")


def shim_sources():
    return sorted(glob.glob(os.path.join(SHIM_DIR, "*.cu")) + glob.glob(os.path.join(SHIM_DIR, "*.cpp")))


def build_shim(force: bool = False) -> str:
    """Build lib/libb2llm.so: the C++ functions with the reference's own signatures
    (namespace llm, headers under include/llm/), linked against libb2ops.so.
    Returns the path, or "" when the sources are not present."""
    srcs = shim_sources()
    if not srcs:
        return ""
    build(force=False)
    deps = srcs + glob.glob(os.path.join(ROOT, "include", "llm", "*.h")) + [LIB]
    if not force and _newer(SHIM_LIB, deps):
        return SHIM_LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = [f if f != "-fPIC,-fvisibility=hidden" else "-fPIC" for f in NVCC_FLAGS]   # llm:: symbols stay visible
    cmd = [nvcc] + flags + ["-x", "cu", "-I", os.path.join(ROOT, "include"), "-o", SHIM_LIB] + srcs + \
        ["-L", LIB_DIR, "-lb2ops", "-Xlinker", "-rpath,$ORIGIN"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc (shim) failed:\n" + proc.stdout + proc.stderr)
    return SHIM_LIB
