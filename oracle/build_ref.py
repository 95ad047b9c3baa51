"""Compiles the reference's own CPU implementation into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  Two extension modules are produced, both from the
reference's sources where they lie (nothing is copied into this repository):

* ``_optimized_transducer``: the unmodified reference extension
  (csrc/cpu.cc, csrc/transducer-loss.cc, python/csrc/optimized_transducer.cc).
  It is the parity target and the timed CPU baseline.
* ``_ot_ref_stages``: ``ref_stage_shim.cc``, which includes csrc/cpu.cc and
  binds its file-static log-prob / alpha / beta stages.

The reference's CUDA sources are not built: they need the third-party
``moderngpu`` headers, which the reference downloads at configure time.

The location of the reference tree is taken from ``$OT_REFERENCE_ROOT``.
Outputs are git-ignored; they only need torch and g++ to build.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_ROOT = os.path.join(os.sep, "root", "reference")


def reference_root():
    return os.environ.get("OT_REFERENCE_ROOT", DEFAULT_ROOT)


def available():
    root = reference_root()
    return os.path.isfile(os.path.join(root, "optimized_transducer", "csrc", "cpu.cc"))


def build(verbose=False):
    """Builds both modules; returns the output directory, or None when the
    reference tree is not present on this machine."""
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
    return OUT


if __name__ == "__main__":
    out = build(verbose="-v" in sys.argv)
    print("reference CPU build:", out if out else "reference tree not found")
