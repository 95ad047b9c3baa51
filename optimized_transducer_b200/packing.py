"""Callers' side of the packed layout (what sits right before the loss).

The reference expects the joiner to work on packed 2-D tensors and leaves the
packing to the user (reference README.md:131-204): a Python loop of slices, a
broadcast add per utterance and ``torch.cat``.  Here every step is one CUDA
kernel of ``libot_b200.so``, differentiable through ``torch.autograd``:

* :func:`pack_joiner_input`: ``(N,T,D)`` encoder + ``(N,U+1,D)`` decoder output
  -> packed ``(rows, D)`` joiner input (README.md:165-177);
* :func:`pack_padded` / :func:`unpack_to_padded`: a padded
  ``(N, maxT, maxU+1, V)`` tensor <-> packed ``(rows, V)``;
* :func:`rnnt_loss`: a ``torchaudio.functional.rnnt_loss``-shaped entry point
  on padded logits (pack, packed loss, gradients scattered back).

``rows = sum_b T_b * (U_b + 1)`` must be known on the host to size the result;
pass it if you have it, otherwise it is read from the lengths (one
device-to-host copy, as the reference's own loop does N times).

Lengths that do not fit the tensors (``T_b > maxT``, ``U_b + 1 > maxU+1``, a sum
that is not ``rows``) are found on the device.  The kernels then do not follow
them and fill their outputs with NaN (zero for :func:`unpack_to_padded`), and
the failure reaches the caller the way the loss's input errors do
(``OT_CHECKS``, see ``transducer_loss.py``): raised by the next call into the
library (default), by the call itself (``OT_CHECKS=2``), or not at all (``0``).
float32, float64, bfloat16 and float16 are accepted; 16-bit data is added and
summed in float32 and rounded once.
"""
import ctypes

import torch

from . import _lib
from .transducer_loss import _CHECK_FLAG, _DTYPE_FLAG, _check_mode, _on_device, transducer_loss

__all__ = ["pack_joiner_input", "pack_padded", "unpack_to_padded", "rnnt_loss", "packed_rows"]


def packed_rows(logit_lengths, target_lengths):
    """sum_b T_b * (U_b + 1) as a Python int (synchronises if the lengths are on a GPU)."""
    return int((logit_lengths.to(torch.int64) * (target_lengths.to(torch.int64) + 1)).sum().item())


def _check(x, logit_lengths, target_lengths, ndim, who):
    if not x.is_cuda:
        raise RuntimeError(f"{who}: CUDA tensors only (sm_100a kernels, no CPU path)")
    if x.dtype not in _DTYPE_FLAG:
        raise RuntimeError(f"{who}: expected float32, float64, bfloat16 or float16, got {x.dtype}")
    if x.dim() != ndim or not x.is_contiguous():
        raise RuntimeError(f"{who}: expected a contiguous {ndim}-D tensor")
    for name, t in (("logit_lengths", logit_lengths), ("target_lengths", target_lengths)):
        if t.dtype != torch.int32 or t.dim() != 1 or not t.is_contiguous() or t.device != x.device:
            raise RuntimeError(f"{who}: {name} must be a contiguous 1-D int32 tensor on {x.device}")
    if logit_lengths.numel() != target_lengths.numel() or logit_lengths.numel() != x.size(0):
        raise RuntimeError(f"{who}: lengths must have one entry per batch element")


def _workspace(n, device):
    size = ctypes.c_uint64()
    _lib.check(_lib.load().ot_b200_pack_workspace_bytes(int(n), ctypes.byref(size)))
    return torch.empty(int(size.value), dtype=torch.uint8, device=device)


def _flags(x):
    mode = _check_mode()
    return _DTYPE_FLAG[x.dtype] | (_CHECK_FLAG["deferred"] if mode == "deferred" else 0)


def _stream(x):
    return ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)


def _finish(rc, ws, n, who):
    """Raises for a failed call; with strict checks also for lengths the device
    found inconsistent (reads the status word of the workspace: one synchronisation)."""
    _lib.check(rc)
    if _check_mode() == "strict":
        code = int(ws[(n + 1) * 8:(n + 1) * 8 + 4].view(torch.int32).item())
        if code:
            where = f"utterance {code - 1}" if code > 0 else "their sum differs from rows"
            raise RuntimeError(f"{who}: the lengths do not fit rows, max_t or max_u1 ({where}); "
                               "the output was filled with NaN")


class _PackJoiner(torch.autograd.Function):
    @staticmethod
    def forward(ctx, enc, dec, T, U, rows):
        n, max_t, d = enc.shape
        max_u1 = dec.size(1)
        out = torch.empty(rows, d, dtype=enc.dtype, device=enc.device)
        ws = _workspace(n, enc.device)
        with _on_device(enc.device.index):
            rc = _lib.load().ot_b200_pack_joiner_input(
                enc.data_ptr(), dec.data_ptr(), T.data_ptr(), U.data_ptr(), n, rows, d, max_t,
                max_u1, _flags(enc), ws.data_ptr(), out.data_ptr(), _stream(enc))
        _finish(rc, ws, n, "pack_joiner_input")
        ctx.meta = (T, U, n, rows, d, max_t, max_u1, enc.dtype)
        return out

    @staticmethod
    def backward(ctx, g):
        T, U, n, rows, d, max_t, max_u1, dtype = ctx.meta
        g = g.contiguous()
        genc = torch.empty(n, max_t, d, dtype=dtype, device=g.device)
        gdec = torch.empty(n, max_u1, d, dtype=dtype, device=g.device)
        ws = _workspace(n, g.device)
        with _on_device(g.device.index):
            rc = _lib.load().ot_b200_pack_joiner_input_backward(
                g.data_ptr(), T.data_ptr(), U.data_ptr(), n, rows, d, max_t, max_u1, _flags(g),
                ws.data_ptr(), genc.data_ptr(), gdec.data_ptr(), _stream(g))
        _finish(rc, ws, n, "pack_joiner_input (backward)")
        return genc, gdec, None, None, None


def pack_joiner_input(encoder_out, decoder_out, logit_lengths, target_lengths, rows=None):
    """Packed joiner input: row ``(b,t,u)`` is ``encoder_out[b,t] + decoder_out[b,u]``.

    ``encoder_out`` (N, maxT, D), ``decoder_out`` (N, maxU+1, D) (the decoder sees
    the blank-prepended targets), lengths int32 (N,).  Returns ``(rows, D)`` in
    the order :func:`~optimized_transducer_b200.transducer_loss` expects."""
    _check(encoder_out, logit_lengths, target_lengths, 3, "pack_joiner_input")
    _check(decoder_out, logit_lengths, target_lengths, 3, "pack_joiner_input")
    if encoder_out.size(2) != decoder_out.size(2) or encoder_out.dtype != decoder_out.dtype:
        raise RuntimeError("pack_joiner_input: encoder_out and decoder_out must share D and dtype")
    if rows is None:
        rows = packed_rows(logit_lengths, target_lengths)
    return _PackJoiner.apply(encoder_out, decoder_out, logit_lengths, target_lengths, int(rows))


def _copy(fn_name, src, out, T, U, rows):
    n, max_t, max_u1, d = (out.shape if fn_name == "ot_b200_unpack_to_padded" else src.shape)
    ws = _workspace(n, src.device)
    with _on_device(src.device.index):
        rc = getattr(_lib.load(), fn_name)(src.data_ptr(), T.data_ptr(), U.data_ptr(), n, rows, d,
                                           max_t, max_u1, _flags(src), ws.data_ptr(),
                                           out.data_ptr(), _stream(src))
    _finish(rc, ws, n, fn_name[len("ot_b200_"):])
    return out


class _PackPadded(torch.autograd.Function):
    @staticmethod
    def forward(ctx, padded, T, U, rows):
        out = torch.empty(rows, padded.size(3), dtype=padded.dtype, device=padded.device)
        ctx.meta = (T, U, rows, tuple(padded.shape))
        return _copy("ot_b200_pack_padded", padded, out, T, U, rows)

    @staticmethod
    def backward(ctx, g):
        T, U, rows, shape = ctx.meta
        out = torch.empty(shape, dtype=g.dtype, device=g.device)
        return _copy("ot_b200_unpack_to_padded", g.contiguous(), out, T, U, rows), None, None, None


class _UnpackPadded(torch.autograd.Function):
    @staticmethod
    def forward(ctx, packed, T, U, max_t, max_u1):
        out = torch.empty(T.numel(), max_t, max_u1, packed.size(1), dtype=packed.dtype,
                          device=packed.device)
        ctx.meta = (T, U, packed.size(0))
        return _copy("ot_b200_unpack_to_padded", packed, out, T, U, packed.size(0))

    @staticmethod
    def backward(ctx, g):
        T, U, rows = ctx.meta
        out = torch.empty(rows, g.size(3), dtype=g.dtype, device=g.device)
        return _copy("ot_b200_pack_padded", g.contiguous(), out, T, U, rows), None, None, None, None


def pack_padded(padded, logit_lengths, target_lengths, rows=None):
    """(N, maxT, maxU+1, D) -> packed (rows, D); entries outside the lattices are dropped."""
    _check(padded, logit_lengths, target_lengths, 4, "pack_padded")
    if rows is None:
        rows = packed_rows(logit_lengths, target_lengths)
    return _PackPadded.apply(padded, logit_lengths, target_lengths, int(rows))


def unpack_to_padded(packed, logit_lengths, target_lengths, max_t, max_u1):
    """packed (rows, D) -> (N, max_t, max_u1, D) with zeros outside the lattices."""
    if packed.dim() != 2 or not packed.is_contiguous() or not packed.is_cuda:
        raise RuntimeError("unpack_to_padded: expected a contiguous 2-D CUDA tensor")
    return _UnpackPadded.apply(packed, logit_lengths, target_lengths, int(max_t), int(max_u1))


def rnnt_loss(logits, targets, logit_lengths, target_lengths, blank=-1, reduction="mean",
              from_log_softmax=False, one_sym_per_frame=False):
    """Transducer loss on PADDED logits (N, maxT, maxU+1, V), the calling convention of
    ``torchaudio.functional.rnnt_loss`` (the oracle the reference tests against,
    python/tests/test_compute_transducer_loss.py:82-89).  ``blank=-1`` means the
    last class, as in torchaudio.  The gradient arrives in the padded layout,
    zero outside the lattices."""
    v = logits.size(-1)
    if blank < 0:
        blank += v
    packed = pack_padded(logits, logit_lengths, target_lengths)
    return transducer_loss(packed, targets, logit_lengths, target_lengths, blank, from_log_softmax,
                           one_sym_per_frame, reduction)
