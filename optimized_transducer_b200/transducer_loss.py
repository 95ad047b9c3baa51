"""Python surface of the transducer loss, a mirror of the reference's
``optimized_transducer/python/optimized_transducer/transducer_loss.py``.

Same names, argument order, defaults and error behaviour as the reference:

* :func:`transducer_loss` (reference ``transducer_loss.py:312-442``)
* :class:`TransducerLoss` (``:173-309``; the reference's module does not call
  ``super().__init__()`` and cannot be instantiated on current PyTorch, this
  one can)
* :class:`TransducerLossFunction` (``:7-170``)
* :func:`compute_transducer_loss`, the counterpart of the reference's private
  native entry ``_optimized_transducer.compute_transducer_loss``
  (``python/csrc/optimized_transducer.cc:15-19``).

All arithmetic runs in the sm_100a kernels of ``libot_b200.so``; PyTorch only
provides device memory and the current stream.  There is no CPU path: tensors
must live on a CUDA device.

Gradient scheduling.  The reference computes the gradient inside ``forward``
(overwriting ``logits`` there), divides it by N for ``reduction="mean"`` in a
second pass and multiplies it by the upstream gradient in a third.  Here
``forward`` stops after the alpha/beta recursions and ``backward`` runs one
fused pass that applies both factors while it overwrites ``logits``; the
observable results (loss, ``.grad`` of the leaves, ``logits`` overwritten by
its gradient after ``backward``) are the same.  ``OT_EAGER_GRAD=1`` restores
the reference's schedule, for callers that read ``logits`` between ``forward``
and ``backward``.
"""
import ctypes
import os

import torch

from . import _lib

__all__ = ["transducer_loss", "TransducerLoss", "TransducerLossFunction",
           "compute_transducer_loss", "stage_outputs", "transducer_loss_per_utterance",
           "PerUtteranceLossFunction"]


# Diagnostic: set to a list (and OT_TRACE=1) to collect, per backward call, a
# copy of the call's stage timeline (see _Call.stage("trace")).
trace_log = None


def _checks_enabled():
    return os.environ.get("OT_CHECKS", "1") != "0"


def _eager_grad():
    return os.environ.get("OT_EAGER_GRAD", "0") == "1"


def _fast_math():
    # Hardware ex2/lg2 in the alpha/beta recursions (float32 only).  On by
    # default: every parity test passes with it at the same tolerances, and the
    # recursions are a latency chain in which the library exp/log1p cost ~20 %.
    return os.environ.get("OT_FAST_MATH", "1") != "0"


def _validate(logits, targets, logit_lengths, target_lengths, blank):
    """The metadata checks of ot::ComputeTransducerLoss
    (optimized_transducer/csrc/transducer-loss.cc:33-46, 58-60, 77-79); the
    data-dependent ones (:49-56, :62-66) run on the device."""
    who = "ComputeTransducerLoss"
    if logits.dtype not in (torch.float32, torch.float64, torch.bfloat16, torch.float16):
        raise RuntimeError(f"{who}: expected logits to have scalar type Float "
                           f"(Double, BFloat16 and Half are accepted as extensions), got {logits.dtype}")
    for name, t in (("targets", targets), ("logit_lengths", logit_lengths),
                    ("target_lengths", target_lengths)):
        if t.dtype != torch.int32:
            raise RuntimeError(f"{who}: expected {name} to have scalar type Int, got {t.dtype}")
    for name, t in (("logits", logits), ("targets", targets),
                    ("logit_lengths", logit_lengths), ("target_lengths", target_lengths)):
        if not t.is_contiguous():
            raise RuntimeError(f"{who}: expected {name} to be contiguous")
    for name, t, d in (("logits", logits, 2), ("targets", targets, 2),
                       ("logit_lengths", logit_lengths, 1), ("target_lengths", target_lengths, 1)):
        if t.dim() != d:
            raise RuntimeError(f"{who}: expected {name} to be {d}-dimensional, got {t.dim()}")
    if logit_lengths.shape != target_lengths.shape:
        raise RuntimeError(f"{who}: expected logit_lengths and target_lengths to have the same size")
    if targets.size(0) != logit_lengths.size(0):
        raise RuntimeError(f"{who}: targets.size(0) must equal the batch size")
    if not logits.is_cuda:
        raise RuntimeError(
            "optimized_transducer_b200 runs on CUDA devices only (sm_100a kernels, no CPU path); "
            f"logits is on {logits.device}")
    for name, t in (("targets", targets), ("logit_lengths", logit_lengths),
                    ("target_lengths", target_lengths)):
        if t.device != logits.device:
            raise RuntimeError(f"{who}: expected {name} to be on {logits.device}, got {t.device}")
    if not (0 <= blank < logits.size(1)):
        raise RuntimeError(f"blank vs logits.size(1) is {blank} vs {logits.size(1)}. "
                           "Expect 0 <= blank < logits.size(1)")
    if logits.size(0) == 0 or logit_lengths.size(0) == 0:
        raise RuntimeError(f"{who}: empty batch")


def real_dtype(logits):
    """dtype of everything but the logits and their gradient: scores, loss,
    upstream factors, workspace arrays.  16-bit logits are computed in float32."""
    return logits.dtype if logits.dtype == torch.float64 else torch.float32


def _flags(logits, from_log_softmax, one_sym_per_frame, checks):
    f = 0
    if from_log_softmax:
        f |= _lib.FROM_LOG_SOFTMAX
    if one_sym_per_frame:
        f |= _lib.ONE_SYM_PER_FRAME
    if logits.dtype == torch.float64:
        f |= _lib.FP64
    elif logits.dtype == torch.bfloat16:
        f |= _lib.BF16
    elif logits.dtype == torch.float16:
        f |= _lib.FP16
    if checks:
        f |= _lib.CHECK_INPUTS
    if _fast_math():
        f |= _lib.FAST_MATH
    if os.environ.get("OT_TRACE", "0") == "1":
        f |= _lib.TRACE
    return f


class _Call:
    """Pointers and sizes of one loss evaluation, plus its workspace."""

    def __init__(self, logits, targets, logit_lengths, target_lengths, blank,
                 from_log_softmax, one_sym_per_frame, checks=None, share_sms=False):
        _validate(logits, targets, logit_lengths, target_lengths, blank)
        if checks is None:
            checks = _checks_enabled()
        self.lib = _lib.load()
        self.logits = logits
        self.n = int(logit_lengths.size(0))
        self.rows = int(logits.size(0))
        self.v = int(logits.size(1))
        self.max_u = int(targets.size(1))
        self.blank = int(blank)
        self.from_log_softmax = bool(from_log_softmax)
        self.modified = bool(one_sym_per_frame)
        self.flags = _flags(logits, from_log_softmax, one_sym_per_frame, checks)
        if share_sms:  # a collective runs beside this call (sharding.py)
            self.flags |= _lib.SHARE_SMS
        self.layout = _lib.workspace_layout(self.n, self.rows, self.max_u, self.flags)
        self.targets, self.t, self.u = targets, logit_lengths, target_lengths
        self.real = real_dtype(logits)
        with torch.cuda.device(logits.device):
            self.workspace = torch.empty(int(self.layout.total_bytes), dtype=torch.uint8,
                                         device=logits.device)
            self.scores = torch.empty(self.n, dtype=self.real, device=logits.device)

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.logits.device).cuda_stream)

    def forward(self, loss_out=None, loss_scale=1.0):
        """Enqueues the forward half.  ``loss_out``: optional 0-dim tensor that
        receives ``loss_scale * -(sum of scores)``."""
        with torch.cuda.device(self.logits.device):
            rc = self.lib.ot_b200_forward(
                self.logits.data_ptr(), self.targets.data_ptr() if self.max_u else None,
                self.t.data_ptr(), self.u.data_ptr(), self.n, self.rows, self.v, self.max_u,
                self.blank, self.flags, self.workspace.data_ptr(), int(self.layout.total_bytes),
                self.scores.data_ptr(), loss_out.data_ptr() if loss_out is not None else None,
                float(loss_scale), self._stream())
        _lib.check(rc)
        return self.scores

    def backward(self, grad_out, scale_tensor=None, scale_host=1.0, per_utterance=False):
        """Enqueues the gradient pass.  ``scale_tensor``: a device scalar, or with
        ``per_utterance`` an (N,) tensor of per-utterance factors."""
        flags = self.flags & ~_lib.CHECK_INPUTS
        if per_utterance:
            assert scale_tensor is not None and scale_tensor.numel() == self.n
            flags |= _lib.SCALE_PER_UTTERANCE
        with torch.cuda.device(self.logits.device):
            rc = self.lib.ot_b200_backward(
                self.logits.data_ptr(), grad_out.data_ptr(), self.n, self.rows, self.v,
                self.max_u, self.blank, flags,
                self.workspace.data_ptr(), int(self.layout.total_bytes),
                scale_tensor.data_ptr() if scale_tensor is not None else None,
                float(scale_host), self._stream())
        _lib.check(rc)
        return grad_out

    def stage(self, name):
        """A tensor view of one intermediate array inside the workspace, in the
        library's own order (per-cell arrays are NOT in packed-row order, see
        :meth:`cell_index`)."""
        dt = self.real
        es = 8 if dt == torch.float64 else 4
        cells = int(self.layout.max_cells)
        if name in ("split", "cell_split"):
            off, count, dtype, esz = getattr(self.layout, name + "_off"), self.n + 1, torch.int64, 8
        elif name == "trace":
            # with OT_TRACE=1: per stage (prepare, logprob, lattice, coef, gradient) the
            # %globaltimer (ns) at which its first block started and its last block ended
            off, count, dtype, esz = self.layout.status_off + 64, 10, torch.int64, 8
        elif name == "status":
            off, count, dtype, esz = self.layout.status_off, 16, torch.int32, 4
        else:
            off = getattr(self.layout, name + "_off")
            count = {"den": self.rows, "lp": 2 * cells, "alpha": cells,
                     "beta": cells, "scores_beta": self.n}[name]
            dtype, esz = dt, es
        return self.workspace[off:off + count * esz].view(dtype)

    def cell_index(self):
        """(rows,) int64 tensor: the cell of every packed row, i.e. the gather
        index that brings a per-cell array into packed-row order
        (``cell(b,t,u)`` as documented in ``include/ot_b200.h``)."""
        dev = self.logits.device
        T = self.t.to(torch.int64)
        U1 = self.u.to(torch.int64) + 1
        split = self.stage("split")[:-1]
        cell_split = self.stage("cell_split")[:-1]
        b = torch.repeat_interleave(torch.arange(self.n, device=dev), T * U1)
        idx = torch.arange(self.rows, device=dev) - split[b]
        t = idx // U1[b]
        u = idx - t * U1[b]
        pos = t * U1[b] + u if self.modified else (t + u) * U1[b] + u
        return cell_split[b] + pos


def compute_transducer_loss(logits, targets, logit_lengths, target_lengths, blank,
                            from_log_softmax, one_sym_per_frame):
    """Counterpart of ``_optimized_transducer.compute_transducer_loss``.

    Returns ``(scores, grad)``: ``scores[b] = log P(y_b | x_b)`` (the negated
    loss, as the reference's native function returns it) and the gradient of
    ``-scores.sum()``, or ``None`` if ``logits`` does not require grad.  With
    ``from_log_softmax=False`` the gradient is written over ``logits`` and the
    returned tensor shares its memory (reference ``cuda.cu:449``); otherwise it
    is a new tensor (``cuda.cu:444``).
    """
    call = _Call(logits, targets, logit_lengths, target_lengths, blank,
                 from_log_softmax, one_sym_per_frame)
    scores = call.forward()
    grad = None
    if logits.requires_grad:
        data = logits.detach()
        grad = data if not from_log_softmax else torch.empty_like(data)
        call.backward(grad)
    return scores, grad


def stage_outputs(logits, targets, logit_lengths, target_lengths, blank,
                  from_log_softmax=False, one_sym_per_frame=False):
    """Runs the forward half and returns its intermediate arrays (copies):
    ``scores``, ``scores_beta``, ``den`` (None for log-softmax input), ``lp``
    (rows, 2), ``alpha``, ``beta`` (rows) and ``split`` (N+1).  For tests and
    debugging; cells outside the band of the modified recursion are undefined."""
    call = _Call(logits, targets, logit_lengths, target_lengths, blank,
                 from_log_softmax, one_sym_per_frame)
    scores = call.forward()
    cell = call.cell_index()
    out = {"scores": scores.clone(), "scores_beta": call.stage("scores_beta").clone(),
           "den": None if from_log_softmax else call.stage("den").clone(),
           "lp": call.stage("lp").view(-1, 2)[cell], "alpha": call.stage("alpha")[cell],
           "beta": call.stage("beta")[cell], "split": call.stage("split").clone()}
    return out


class TransducerLossFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, logit_lengths, target_lengths, blank,
                from_log_softmax, one_sym_per_frame, reduction="mean"):
        assert reduction in ("mean", "sum")
        n = logit_lengths.size(0)
        if _eager_grad():
            # The reference's schedule (transducer_loss.py:135-154).
            scores, grad = compute_transducer_loss(
                logits, targets, logit_lengths, target_lengths, blank,
                from_log_softmax, one_sym_per_frame)
            loss = -1 * scores
            if reduction == "mean":
                loss = loss.mean()
                if grad is not None:
                    grad /= n
            else:
                loss = loss.sum()
            ctx.grad = grad
            ctx.call = None
            return loss

        call = _Call(logits.detach(), targets, logit_lengths, target_lengths, blank,
                     from_log_softmax, one_sym_per_frame)
        scale = (1.0 / n) if reduction == "mean" else 1.0
        loss = torch.empty((), dtype=call.real, device=logits.device)
        call.forward(loss_out=loss, loss_scale=scale)  # the reduction runs on the device too
        ctx.grad = None
        ctx.call = call if ctx.needs_input_grad[0] else None
        ctx.scale_host = scale
        return loss

    @staticmethod
    def backward(ctx, loss_grad):
        assert loss_grad.numel() == 1, loss_grad.numel()
        if ctx.call is None:
            if ctx.grad is None:
                raise RuntimeError("the gradient of this transducer loss was already consumed, "
                                   "or logits did not require grad")
            grad = ctx.grad.mul_(loss_grad)  # reference transducer_loss.py:162
            return (grad,) + (None,) * 7
        call, ctx.call = ctx.call, None  # the workspace is released after this pass
        data = call.logits
        grad = torch.empty_like(data) if call.from_log_softmax else data
        scale = loss_grad.detach().to(device=data.device, dtype=call.real).contiguous()
        call.backward(grad, scale_tensor=scale, scale_host=ctx.scale_host)
        if trace_log is not None:  # diagnostic, see OT_TRACE
            trace_log.append(call.stage("trace").clone())
        return (grad,) + (None,) * 7


class PerUtteranceLossFunction(torch.autograd.Function):
    """``reduction="none"``: the (N,) vector of per-utterance losses.  The
    reference has no such mode (transducer_loss.py:126-128 rejects it); its
    native function already returns per-utterance scores, and the gradient pass
    here takes one upstream factor per utterance."""

    @staticmethod
    def forward(ctx, logits, targets, logit_lengths, target_lengths, blank,
                from_log_softmax, one_sym_per_frame):
        call = _Call(logits.detach(), targets, logit_lengths, target_lengths, blank,
                     from_log_softmax, one_sym_per_frame)
        scores = call.forward()
        ctx.call = call if ctx.needs_input_grad[0] else None
        return scores.neg()

    @staticmethod
    def backward(ctx, loss_grad):
        if ctx.call is None:
            raise RuntimeError("the gradient of this transducer loss was already consumed, "
                               "or logits did not require grad")
        call, ctx.call = ctx.call, None
        assert loss_grad.numel() == call.n, (loss_grad.numel(), call.n)
        data = call.logits
        grad = torch.empty_like(data) if call.from_log_softmax else data
        scale = loss_grad.detach().to(device=data.device, dtype=call.real).contiguous()
        call.backward(grad, scale_tensor=scale, per_utterance=True)
        return (grad,) + (None,) * 6


def transducer_loss_per_utterance(logits: torch.Tensor, targets: torch.Tensor,
                                  logit_lengths: torch.Tensor, target_lengths: torch.Tensor,
                                  blank: int, from_log_softmax: bool,
                                  one_sym_per_frame: bool = False) -> torch.Tensor:
    """The unreduced transducer loss: an (N,) tensor, ``-log P(y_b | x_b)`` per
    utterance.  Arguments as for :func:`transducer_loss`.  ``backward`` accepts
    any (N,) upstream gradient and, like the reduced loss, overwrites ``logits``
    with its gradient unless ``from_log_softmax`` is True."""
    return PerUtteranceLossFunction.apply(
        logits, targets, logit_lengths, target_lengths, blank, from_log_softmax,
        one_sym_per_frame)


class TransducerLoss(torch.nn.Module):
    """Module form of :func:`transducer_loss` (reference ``transducer_loss.py:173-309``)."""

    def __init__(self, blank: int, reduction: str = "mean"):
        super().__init__()
        assert reduction in ("mean", "sum")
        self.blank = blank
        self.reduction = reduction

    def forward(self, logits, targets, logit_lengths, target_lengths,
                from_log_softmax, one_sym_per_frame=False):
        return TransducerLossFunction.apply(
            logits, targets, logit_lengths, target_lengths, self.blank,
            from_log_softmax, one_sym_per_frame, self.reduction)


def transducer_loss(logits: torch.Tensor, targets: torch.Tensor,
                    logit_lengths: torch.Tensor, target_lengths: torch.Tensor,
                    blank: int, from_log_softmax: bool,
                    one_sym_per_frame: bool = False,
                    reduction: str = "mean") -> torch.Tensor:
    """Transducer (RNN-T) loss over packed logits.

    Args:
      logits: (sum_b T_b*(U_b+1), V) float32 (float64, bfloat16 and float16 are
        accepted too; 16-bit logits are computed in float32, the loss is float32
        and the gradient is rounded back to the logits' type), contiguous,
        on a CUDA device: utterance b's (T_b, U_b+1, V) joiner output flattened
        to rows and the utterances concatenated (reference README.md:131-204).
        If it requires grad and ``from_log_softmax`` is False, ``backward``
        overwrites it with its gradient.
      targets: (N, max_b U_b) int32, not prepended with a blank.
      logit_lengths: (N,) int32, T_b.   target_lengths: (N,) int32, U_b.
      blank: id of the blank symbol.
      from_log_softmax: True if ``logits`` already holds log-softmax outputs.
      one_sym_per_frame: True for the modified transducer that emits at most
        one symbol per frame (needs U_b <= T_b - 1).
      reduction: "mean" (over utterances) or "sum"; "none" is not supported, as
        in the reference (transducer_loss.py:126-128).
    Returns: a 0-dim tensor with the reduced loss.
    """
    return TransducerLossFunction.apply(
        logits, targets, logit_lengths, target_lengths, blank, from_log_softmax,
        one_sym_per_frame, reduction)
