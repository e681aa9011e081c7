"""Builds libtempest_b200.so, the C-ABI shared library, in-tree with nvcc for sm_100a.

    python tempest.jl_b200/csrc/build.py [--force] [--verbose]

The library links the CUDA runtime statically and nothing else, so it loads
from Julia (`ccall`), C or Python (`ctypes`) without torch.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.dirname(HERE)
LIB = os.path.join(PACKAGE, "libtempest_b200.so")
SOURCES = ["abi.cu", "rowreduce.cu", "gemm.cu", "pointwise.cu", "attention_fwd.cu", "attention_bwd.cu", "attention_simt.cu", "deltanet.cu", "generic.cu", "rowgen.cu", "dp.cu", "scan.cu", "route.cu", "products.cu"]
HEADERS = ["common.cuh", "sm100.cuh", "attention_simt.cuh", "generic.cuh", os.path.join("..", "..", "include", "tempest_b200.h")]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def nvcc():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    raise RuntimeError("nvcc not found")


def stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(HERE, h) for h in HEADERS] + [os.path.abspath(__file__)]
    objects = []
    procs = []
    for src in SOURCES:
        path = os.path.join(HERE, src)
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objects.append(obj)
        if force or stale(obj, [path] + headers):
            cmd = [nvcc()] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}\n")
    if failed:
        raise RuntimeError("build of libtempest_b200.so failed")
    if force or procs or stale(LIB, objects):
        cmd = [nvcc(), "-shared", "-o", LIB] + objects + ["-cudart", "static", "-ldl", "-gencode", "arch=compute_100a,code=sm_100a"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
