"""The C-ABI library loads and exports every symbol ``include/ot_b200.h`` declares;
argument checks that need no GPU return the documented status codes."""
import ctypes
import os
import re

import pytest

from optimized_transducer_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ot_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ot_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_abi_version():
    assert _lib.load().ot_b200_abi_version() == _lib.ABI_VERSION


@pytest.mark.parametrize("flags", [0, _lib.FROM_LOG_SOFTMAX, _lib.FP64, _lib.FP64 | _lib.FROM_LOG_SOFTMAX])
def test_workspace_layout_is_aligned_and_ordered(flags):
    n, rows, max_u = 7, 12345, 20
    lay = _lib.workspace_layout(n, rows, max_u, flags)
    es = 8 if flags & _lib.FP64 else 4
    offs = [lay.status_off, lay.split_off, lay.cell_split_off, lay.den_off, lay.lp_off,
            lay.alpha_off, lay.beta_off, lay.coef_off, lay.scores_beta_off, lay.total_bytes]
    assert all(o % 256 == 0 for o in offs)
    assert offs == sorted(offs) and lay.status_off == 0
    # room for every diagonal-major block: rows + sum U*(U+1) + one pad entry each
    assert lay.max_cells >= rows + n * max_u * (max_u + 1) + n
    assert lay.lp_off - lay.den_off >= (0 if flags & _lib.FROM_LOG_SOFTMAX else rows * es)
    assert lay.alpha_off - lay.lp_off >= 2 * lay.max_cells * es
    assert lay.beta_off - lay.alpha_off >= lay.max_cells * es
    total = ctypes.c_uint64()
    assert _lib.load().ot_b200_workspace_bytes(n, rows, max_u, flags, ctypes.byref(total)) == _lib.OK
    assert total.value == lay.total_bytes
    mod = _lib.workspace_layout(n, rows, max_u, flags | _lib.ONE_SYM_PER_FRAME)
    assert mod.max_cells == rows + n  # row-major blocks, one pad entry each


def test_argument_errors_without_touching_a_gpu():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(1 << 16)
    ws = (ctypes.addressof(buf) + 255) & ~255
    one = ctypes.c_void_p(ws)
    # N <= 0
    rc = lib.ot_b200_forward(one, one, one, one, 0, 10, 5, 1, 0, 0, one, 1 << 15, one, None, 1.0, None)
    assert rc == _lib.ERR_ARGUMENT and "N must be positive" in _lib.last_error()
    # blank out of range: the reference's wording (transducer-loss.cc:58-60)
    rc = lib.ot_b200_forward(one, one, one, one, 1, 10, 5, 1, 5, 0, one, 1 << 15, one, None, 1.0, None)
    assert rc == _lib.ERR_ARGUMENT and "Expect 0 <= blank < logits.size(1)" in _lib.last_error()
    # workspace too small / missing / misaligned
    rc = lib.ot_b200_forward(one, one, one, one, 1, 10, 5, 1, 0, 0, one, 16, one, None, 1.0, None)
    assert rc == _lib.ERR_WORKSPACE
    rc = lib.ot_b200_forward(one, one, one, one, 1, 10, 5, 1, 0, 0, None, 1 << 15, one, None, 1.0, None)
    assert rc == _lib.ERR_WORKSPACE
    rc = lib.ot_b200_forward(one, one, one, one, 1, 10, 5, 1, 0, 0, ctypes.c_void_p(ws + 8), 1 << 15, one, None, 1.0, None)
    assert rc == _lib.ERR_WORKSPACE
    # unknown flag bits
    rc = lib.ot_b200_forward(one, one, one, one, 1, 10, 5, 1, 0, 1 << 20, one, 1 << 15, one, None, 1.0, None)
    assert rc == _lib.ERR_ARGUMENT
    # NULL logits
    rc = lib.ot_b200_forward(None, one, one, one, 1, 10, 5, 1, 0, 0, one, 1 << 15, one, None, 1.0, None)
    assert rc == _lib.ERR_ARGUMENT
    # log-softmax gradient must not alias its input (cuda.cu:444 allocates a new tensor)
    rc = lib.ot_b200_backward(one, one, 1, 10, 5, 1, 0, _lib.FROM_LOG_SOFTMAX, one, 1 << 15, None, 1.0, None)
    assert rc == _lib.ERR_ARGUMENT
    with pytest.raises(RuntimeError):
        _lib.check(rc)


def test_exchange_table_size_and_argument_checks():
    """Host-side part of the peer-memory exchange: 16 bytes per (slot, rank)."""
    lib = _lib.load()
    n = ctypes.c_uint64(0)
    assert lib.ot_b200_exchange_bytes(8, 256, ctypes.byref(n)) == _lib.OK and n.value == 8 * 256 * 16
    assert lib.ot_b200_exchange_bytes(33, 256, ctypes.byref(n)) == _lib.ERR_ARGUMENT
    assert lib.ot_b200_exchange_publish(None, 0, None, 2, 0, 256, 0, None) == _lib.ERR_ARGUMENT
    assert lib.ot_b200_exchange_gather(None, 2, 256, 0, None, 0, 1.0, None, 1000, None) == _lib.ERR_ARGUMENT


def test_reference_side_adapter_compiles_against_the_header():
    """``include/examples/reference_adapter.cc`` is the function a maintainer of the
    reference would put in place of ot::ComputeTransducerLossCuda (it is also the
    snippet shown in INTEGRATION.md).  It must stay valid C++ against the current
    ``ot_b200.h`` and torch headers: syntax-checked here (no linking, no GPU)."""
    import shutil
    import subprocess
    import sysconfig
    from torch.utils.cpp_extension import include_paths
    if shutil.which("g++") is None:
        pytest.skip("g++ not available")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    if not os.path.isfile(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("CUDA headers not available")
    inc = include_paths() + [sysconfig.get_paths()["include"], cuda_inc, os.path.join(ROOT, "include")]
    src = os.path.join(ROOT, "include", "examples", "reference_adapter.cc")
    cmd = ["g++", "-fsyntax-only", "-std=c++17"] + [f"-I{p}" for p in inc] + [src]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-2000:]
    # and the snippet in INTEGRATION.md is that function
    body = open(src).read().split("namespace ot {", 1)[1].rsplit("}  // namespace ot", 1)[0].strip()
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    assert body in doc
