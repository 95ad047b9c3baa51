"""ctypes binding of ``libot_b200.so`` (declared in ``include/ot_b200.h``).

There is no fallback: if the library is missing or does not load, importing
the loss raises, and so does calling it without a CUDA device.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libot_b200.so")

ABI_VERSION = 3

# ot_b200_status
OK, ERR_ARGUMENT, ERR_CUDA, ERR_WORKSPACE, ERR_INPUT = range(5)

# flags
FROM_LOG_SOFTMAX = 1
ONE_SYM_PER_FRAME = 2
FP64 = 4
CHECK_INPUTS = 8
FAST_MATH = 16
SCALE_PER_UTTERANCE = 32
SHARE_SMS = 64
BF16 = 128
FP16 = 256
TRACE = 512
REPORT_ERRORS = 1024
LINEAR_DOMAIN = 2048

# Every symbol include/ot_b200.h declares.
EXPORTS = (
    "ot_b200_abi_version",
    "ot_b200_last_error",
    "ot_b200_workspace_layout_query",
    "ot_b200_workspace_bytes",
    "ot_b200_forward",
    "ot_b200_backward",
    "ot_b200_loss_and_gradient",
    "ot_b200_loss_and_gradient_groups",
    "ot_b200_scale_gradient",
    "ot_b200_forward_linear",
    "ot_b200_backward_linear",
    "ot_b200_compute_transducer_loss",
    "ot_b200_poll_errors",
    "ot_b200_read_input_status",
    "ot_b200_scores_noalloc",
    "ot_b200_pack_workspace_bytes",
    "ot_b200_pack_joiner_input",
    "ot_b200_pack_joiner_input_backward",
    "ot_b200_pack_padded",
    "ot_b200_unpack_to_padded",
    "ot_b200_exchange_bytes",
    "ot_b200_exchange_allreduce",
    "ot_b200_exchange_wait",
    "ot_b200_exchange_publish",
    "ot_b200_exchange_gather",
)


class WorkspaceLayout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in (
        "total_bytes", "status_off", "split_off", "cell_split_off", "den_off", "lp_off",
        "alpha_off", "beta_off", "coef_off", "scores_beta_off", "max_cells")]


_lib = None


def load():
    """Loads the library once and declares the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with "
            "`python -m optimized_transducer_b200.build` (needs nvcc). "
            "There is no CPU or PyTorch fallback for the transducer loss.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64, u32, u64 = (ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64,
                              ctypes.c_uint32, ctypes.c_uint64)
    lib.ot_b200_abi_version.restype = ctypes.c_int
    lib.ot_b200_abi_version.argtypes = []
    lib.ot_b200_last_error.restype = ctypes.c_char_p
    lib.ot_b200_last_error.argtypes = []
    lib.ot_b200_workspace_layout_query.restype = ctypes.c_int
    lib.ot_b200_workspace_layout_query.argtypes = [i32, i64, i32, u32, ctypes.POINTER(WorkspaceLayout)]
    lib.ot_b200_workspace_bytes.restype = ctypes.c_int
    lib.ot_b200_workspace_bytes.argtypes = [i32, i64, i32, u32, ctypes.POINTER(u64)]
    lib.ot_b200_forward.restype = ctypes.c_int
    lib.ot_b200_forward.argtypes = [vp, vp, vp, vp, i32, i64, i32, i32, i32, u32, vp, u64, vp, vp,
                                    ctypes.c_double, vp]
    lib.ot_b200_backward.restype = ctypes.c_int
    lib.ot_b200_backward.argtypes = [vp, vp, i32, i64, i32, i32, i32, u32, vp, u64, vp, ctypes.c_double, vp]
    lib.ot_b200_loss_and_gradient.restype = ctypes.c_int
    lib.ot_b200_loss_and_gradient.argtypes = [vp, vp, vp, vp, vp, i32, i64, i32, i32, i32, u32, vp, u64, vp, vp,
                                              ctypes.c_double, ctypes.c_double, vp]
    lib.ot_b200_loss_and_gradient_groups.restype = ctypes.c_int
    lib.ot_b200_loss_and_gradient_groups.argtypes = [vp, vp, vp, vp, vp, i32, i64, i32, i32, i32, u32, vp, u64,
                                                     vp, vp, ctypes.c_double, ctypes.c_double,
                                                     ctypes.POINTER(i64), i32, vp]
    lib.ot_b200_forward_linear.restype = ctypes.c_int
    lib.ot_b200_forward_linear.argtypes = [vp, vp, vp, vp, vp, vp, i32, i64, i32, i32, i32, i32, u32, vp, u64,
                                           vp, vp, ctypes.c_double, vp]
    lib.ot_b200_backward_linear.restype = ctypes.c_int
    lib.ot_b200_backward_linear.argtypes = [vp, vp, vp, i32, i64, i32, i32, i32, i32, u32, vp, u64, vp, vp,
                                            ctypes.c_double, vp]
    lib.ot_b200_scale_gradient.restype = ctypes.c_int
    lib.ot_b200_scale_gradient.argtypes = [vp, i64, vp, u32, vp]
    lib.ot_b200_compute_transducer_loss.restype = ctypes.c_int
    lib.ot_b200_compute_transducer_loss.argtypes = [vp, vp, vp, vp, vp, i32, i64, i32, i32, i32, u32, vp, u64, vp, vp]
    lib.ot_b200_poll_errors.restype = ctypes.c_int
    lib.ot_b200_poll_errors.argtypes = [ctypes.POINTER(i32), ctypes.POINTER(i32), ctypes.POINTER(i32), vp, i32]
    lib.ot_b200_read_input_status.restype = ctypes.c_int
    lib.ot_b200_read_input_status.argtypes = [vp, u64, ctypes.POINTER(i32), ctypes.POINTER(i32), vp]
    lib.ot_b200_scores_noalloc.restype = ctypes.c_int
    lib.ot_b200_scores_noalloc.argtypes = [vp, vp, vp, vp, i32, i64, i32, i32, i32, vp, vp]
    lib.ot_b200_pack_workspace_bytes.restype = ctypes.c_int
    lib.ot_b200_pack_workspace_bytes.argtypes = [i32, ctypes.POINTER(u64)]
    lib.ot_b200_pack_joiner_input.restype = ctypes.c_int
    lib.ot_b200_pack_joiner_input.argtypes = [vp, vp, vp, vp, i32, i64, i32, i32, i32, u32, vp, vp, vp]
    lib.ot_b200_pack_joiner_input_backward.restype = ctypes.c_int
    lib.ot_b200_pack_joiner_input_backward.argtypes = [vp, vp, vp, i32, i64, i32, i32, i32, u32, vp, vp, vp, vp]
    for name in ("ot_b200_pack_padded", "ot_b200_unpack_to_padded"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [vp, vp, vp, i32, i64, i32, i32, i32, u32, vp, vp, vp]
    lib.ot_b200_exchange_bytes.restype = ctypes.c_int
    lib.ot_b200_exchange_bytes.argtypes = [i32, i32, ctypes.POINTER(u64)]
    lib.ot_b200_exchange_allreduce.restype = ctypes.c_int
    lib.ot_b200_exchange_allreduce.argtypes = [vp, vp, u32, vp, vp, i32, i32, i32, u64, ctypes.c_double, vp, u64, vp]
    lib.ot_b200_exchange_wait.restype = ctypes.c_int
    lib.ot_b200_exchange_wait.argtypes = [vp]
    lib.ot_b200_exchange_publish.restype = ctypes.c_int
    lib.ot_b200_exchange_publish.argtypes = [vp, u32, vp, i32, i32, i32, u64, vp]
    lib.ot_b200_exchange_gather.restype = ctypes.c_int
    lib.ot_b200_exchange_gather.argtypes = [vp, i32, i32, u64, vp, u32, ctypes.c_double, vp, u64, vp]
    if lib.ot_b200_abi_version() != ABI_VERSION:
        raise ImportError("libot_b200.so was built from a different ABI version; rebuild it")
    _lib = lib
    return lib


def last_error():
    return load().ot_b200_last_error().decode("utf-8", "replace")


def check(rc):
    """Raises the Python exception that matches a non-OK status."""
    if rc == OK:
        return
    msg = last_error()
    if rc in (ERR_ARGUMENT, ERR_INPUT, ERR_WORKSPACE, ERR_CUDA):
        raise RuntimeError(msg)
    raise RuntimeError(f"libot_b200 returned status {rc}: {msg}")


def workspace_layout(n, rows, max_u, flags):
    out = WorkspaceLayout()
    check(load().ot_b200_workspace_layout_query(int(n), int(rows), int(max_u), int(flags),
                                                ctypes.byref(out)))
    return out
