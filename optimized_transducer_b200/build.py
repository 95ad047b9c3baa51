"""Builds ``libot_b200.so`` (the sm_100a kernels + the C ABI) in-tree with nvcc.

Usage: ``python -m optimized_transducer_b200.build [-v]``.  The library links
the CUDA runtime statically and has no dependency on torch or Python.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libot_b200.so")
SOURCES = ["api.cu", "prep.cu", "logprob.cu", "lattice.cu", "gradient.cu", "noalloc.cu", "pack.cu",
           "exchange.cu", "fused_linear.cu"]
HEADERS = [os.path.join(CSRC, "ot_common.cuh"),
           os.path.join(HERE, os.pardir, "include", "ot_b200.h")]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path():
    cand = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.isfile(cand):
        raise RuntimeError("nvcc not found; it is needed to build libot_b200.so")
    return cand


def up_to_date():
    if not os.path.isfile(LIB):
        return False
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, verbose=False):
    """Compiles every kernel for sm_100a; returns the path of the library."""
    if not force and up_to_date():
        return LIB
    nvcc = nvcc_path()
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src[:-3] + ".o")
        cmd = [nvcc, *ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
               "-ccbin", "g++", "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(out)
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    link = [nvcc, *ARCH, "-shared", "-ccbin", "g++", "-o", LIB, *objs]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
