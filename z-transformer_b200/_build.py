"""Compiles the CUDA library in-tree for sm_100a (nvcc cross-compiles without a GPU)."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libztattn.so")
HOST_LIB_PATH = os.path.join(HERE, "libzthost.so")
HARNESS_PATH = os.path.join(HERE, "zt_attn_harness")
# the negative-control build: the same sources with defect switches compiled into the kernels (-DZT_DEFECTS)
DEFECTS_LIB_PATH = os.path.join(HERE, "libztattn_defects.so")
DEFECTS_HARNESS_PATH = os.path.join(HERE, "zt_attn_harness_defects")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-shared"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _sources() -> list[str]:
    out = [os.path.join(HERE, "..", "include", "zt_attn.h")]
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".hpp", ".cpp", ".h"))]
    return out


def build_library(force: bool = False, verbose: bool = False) -> str:
    """nvcc -> libztattn.so (kernels + C ABI), libzthost.so (C++ host mirror + its C shim, when its
    source exists) and the zt_attn_harness program."""
    srcs = _sources()
    if force or _stale(LIB_PATH, srcs):
        cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, os.path.join(CSRC, "zt_attn.cu"), "-lcuda"]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        subprocess.check_call(cmd)
    host_src = os.path.join(CSRC, "host", "zt_host.cpp")
    if os.path.exists(host_src) and (force or _stale(HOST_LIB_PATH, srcs)):
        cmd = [_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-shared",
               "-o", HOST_LIB_PATH, host_src, "-L" + HERE, "-lztattn",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        subprocess.check_call(cmd)
    harness_src = os.path.join(CSRC, "zt_harness.cpp")
    if os.path.exists(harness_src) and (force or _stale(HARNESS_PATH, srcs)):
        # the twin-directory harness: a host program over the C ABI (csrc/zt_harness.cpp)
        cmd = [_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-Wall", "-o", HARNESS_PATH, harness_src,
               "-L" + HERE, "-lztattn", "-ldl", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        subprocess.check_call(cmd)
    if os.path.exists(harness_src) and (force or _stale(DEFECTS_HARNESS_PATH, srcs)):
        # the library once more with the in-kernel defect switches, and the harness linked against THAT one;
        # nothing else ever loads it
        subprocess.check_call([_nvcc(), *NVCC_FLAGS, "-DZT_DEFECTS", "-o", DEFECTS_LIB_PATH,
                               os.path.join(CSRC, "zt_attn.cu"), "-lcuda"])
        subprocess.check_call([_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-Wall", "-o", DEFECTS_HARNESS_PATH,
                               harness_src, "-L" + HERE, "-lztattn_defects", "-ldl", "-Xlinker", "-rpath", "-Xlinker",
                               "$ORIGIN"])
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
