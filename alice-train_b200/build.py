"""Builds libalice_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python alice-train_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU.  The shared object lands next to this file so that it
travels with the source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libalice_b200.so")
SOURCES = ["api.cu", "quantize.cu", "act_quant.cu", "norm_act.cu", "lm_head.cu", "matvec.cu", "matvec_mma.cu", "matvec_tma.cu", "gemm_simt.cu", "gemm_tc.cu", "gemm_tc2.cu", "dp_allreduce.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "alice_b200.h"),
                                                                os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    common = [nvcc, "-std=c++17", "-O3", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-ccbin", "/usr/bin/g++"]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", os.path.join(CSRC, src), "-o", obj],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-shared", *ARCH, "-o", OUT, *objs, "-ccbin", "/usr/bin/g++",
                           "-cudart", "static"])
    return OUT


def build_cpp_test() -> str:
    """Compiles tests/cpp/host_mirror_test.cpp (the C++ host mirror's own test) with g++ against the library."""
    src = os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp")
    hdr = os.path.join(HERE, "cpp", "alice_train.hpp")
    exe = os.path.join(ROOT, "tests", "cpp", "_build", "host_mirror_test")
    os.makedirs(os.path.dirname(exe), exist_ok=True)
    deps = [src, hdr, os.path.join(ROOT, "include", "alice_b200.h"), OUT]
    if os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
        return exe
    subprocess.check_call(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
                           "-I", os.path.join(HERE, "cpp"), src, "-o", exe, "-L", HERE, "-lalice_b200",
                           "-Wl,-rpath," + HERE, "-Wl,-rpath,$ORIGIN/../../../alice-train_b200"])
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
