"""Compiles the reference's own CPU implementation into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  Two extension modules are produced, both from the
reference's sources where they lie (nothing is copied into this repository):

* ``_optimized_transducer``: the unmodified reference extension
  (csrc/cpu.cc, csrc/transducer-loss.cc, python/csrc/optimized_transducer.cc).
  It is the parity target and the timed CPU baseline.
* ``_ot_ref_stages``: ``ref_stage_shim.cc``, which includes csrc/cpu.cc and
  binds its file-static log-prob / alpha / beta stages.

The reference's Python layer (python/optimized_transducer/transducer_loss.py)
is installed next to them, as ``_ref/python/transducer_loss.py``, the way a
``pip install --target`` of the reference would place it: the benchmark's
reference arm runs the reference's own ``transducer_loss`` + ``backward`` on top
of its own extension.

``build_cuda()`` additionally compiles the reference's own CUDA implementation
(csrc/cuda.cu, csrc/kernels.cu, unmodified, with the reference's nvcc options,
csrc/CMakeLists.txt:16) for sm_100 into ``_ref/_optimized_transducer_cuda``.
Those sources include two headers of the third-party ``moderngpu`` library, which
the reference downloads at configure time (cmake/moderngpu.cmake:24-25) and which
is not available offline; ``oracle/mgpu_stub`` restates the one function and the
one base class they use (row splits -> row ids: index bookkeeping, no
arithmetic).  This build is only used to TIME the reference's kernels on the
same GPU (``bench.py --impl reference-cuda``); parity is pinned on the CPU build.

The reference tree is the one ``$OT_REFERENCE_ROOT`` names, else a checkout
called ``reference`` beside this repository; where neither exists nothing is
built and outputs that already exist are used.  Outputs are git-ignored; they
only need torch and g++ to build.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def reference_root():
    """``$OT_REFERENCE_ROOT``, else the directory ``reference`` beside this repository."""
    env = os.environ.get("OT_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def available():
    root = reference_root()
    return os.path.isfile(os.path.join(root, "optimized_transducer", "csrc", "cpu.cc"))


def build(verbose=False):
    """Builds both modules and installs the reference's Python layer; returns the
    output directory, or None when no reference tree is found."""
    if not available():
        return None
    # An inherited $CXX may name a compiler wrapper that cannot link; use g++.
    os.environ["CXX"] = "g++"
    os.environ["CC"] = "gcc"
    from torch.utils.cpp_extension import load

    root = reference_root()
    src = os.path.join(root, "optimized_transducer")
    for name, sources in (
        ("_optimized_transducer", [
            os.path.join(src, "csrc", "cpu.cc"),
            os.path.join(src, "csrc", "transducer-loss.cc"),
            os.path.join(src, "python", "csrc", "optimized_transducer.cc"),
        ]),
        ("_ot_ref_stages", [os.path.join(HERE, "ref_stage_shim.cc")]),
    ):
        bdir = os.path.join(OUT, name)
        os.makedirs(bdir, exist_ok=True)
        load(name=name, sources=sources, extra_include_paths=[root],
             extra_cflags=["-O2"], build_directory=bdir, verbose=verbose,
             is_python_module=False)
    pydir = os.path.join(OUT, "python")
    os.makedirs(pydir, exist_ok=True)
    shutil.copyfile(os.path.join(src, "python", "optimized_transducer", "transducer_loss.py"),
                    os.path.join(pydir, "transducer_loss.py"))
    return OUT


def build_cuda(verbose=False):
    """Cross-compiles the reference's CUDA extension for sm_100 (needs nvcc, not a
    GPU); returns the path of the module's directory, or None without a reference tree."""
    if not available():
        return None
    os.environ["CXX"] = "g++"
    os.environ["CC"] = "gcc"
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    from torch.utils.cpp_extension import load

    root = reference_root()
    src = os.path.join(root, "optimized_transducer")
    bdir = os.path.join(OUT, "_optimized_transducer_cuda")
    os.makedirs(bdir, exist_ok=True)
    load(name="_optimized_transducer",
         sources=[os.path.join(src, "csrc", "cpu.cc"), os.path.join(src, "csrc", "transducer-loss.cc"),
                  os.path.join(src, "csrc", "cuda.cu"), os.path.join(src, "csrc", "kernels.cu"),
                  os.path.join(src, "python", "csrc", "optimized_transducer.cc")],
         extra_include_paths=[root, os.path.join(HERE, "mgpu_stub")],
         extra_cflags=["-O2", "-DOT_WITH_CUDA"],
         extra_cuda_cflags=["-O3", "-DOT_WITH_CUDA", "-lineinfo", "--expt-extended-lambda",
                            "-use_fast_math", "-Xptxas=-w"],
         with_cuda=True, build_directory=bdir, verbose=verbose, is_python_module=False)
    return bdir


if __name__ == "__main__":
    if "--cuda" in sys.argv:
        print("reference CUDA build:", build_cuda(verbose="-v" in sys.argv))
        sys.exit(0)
    out = build(verbose="-v" in sys.argv)
    print("reference CPU build:", out if out else f"no reference tree at {reference_root()}; set OT_REFERENCE_ROOT")
