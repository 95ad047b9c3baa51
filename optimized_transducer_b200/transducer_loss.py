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

Input checks.  The data-dependent checks of the reference (lengths against the
number of rows, target range, ...) and its comparison of the two total scores
run on the device.  ``OT_CHECKS`` selects how a failure reaches the caller:

* ``1`` (default), "deferred": the call that failed returns a NaN loss and
  writes no gradient; the failure is raised as ``RuntimeError`` by the next
  call into this module on the same device that finds the report (usually the
  ``backward`` of the same loss, at the latest the next ``transducer_loss``),
  or by :func:`check_inputs`.  The host never waits for the GPU, so a training
  loop can run ahead of the device.
* ``2``, "strict": the call itself waits for its forward kernels and raises, as
  the reference does.  :func:`compute_transducer_loss` and
  :func:`stage_outputs` always work this way unless checks are off.
* ``0``: nothing is reported (the kernels still refuse to touch memory on
  inconsistent inputs, and the loss is NaN).

Gradient scheduling.  The reference computes the gradient inside ``forward``
(overwriting ``logits`` there), divides it by N for ``reduction="mean"`` in a
second pass and multiplies it by the upstream gradient in a third.  Two
schedules exist here, selected by ``OT_EAGER_GRAD``:

* ``1`` (default), the reference's: ``forward`` is ONE library call that
  computes loss and gradient (the 1/N of "mean" folded in), which lets the
  library overlap the stages of a large batch (see ``ot_b200_loss_and_gradient``);
  ``backward`` multiplies by the upstream gradient with a kernel that returns at
  once when that gradient is 1, the usual case, so the reference's two extra
  passes are gone.  An upstream gradient other than 1 (loss scaling) costs one
  extra pass.
* ``0``, deferred: ``forward`` stops after the alpha/beta recursions and
  ``backward`` runs one fused pass that applies both factors while it overwrites
  ``logits``: the cheapest schedule when the upstream gradient is not 1, and
  ``logits`` stays intact until ``backward``.

The observable results (loss, ``.grad`` of the leaves, ``logits`` holding its
gradient after ``backward``) are the same in both.
"""
import ctypes
import os

import torch

from . import _lib

__all__ = ["transducer_loss", "TransducerLoss", "TransducerLossFunction",
           "compute_transducer_loss", "stage_outputs", "transducer_loss_per_utterance",
           "PerUtteranceLossFunction", "check_inputs", "joiner_scores",
           "transducer_loss_and_grad", "group_cuts", "joiner_loss", "JoinerLossFunction"]


# Diagnostic: with OT_TRACE=1 and a list set here (collect_traces), every
# backward call appends a copy of its call's stage timeline (_Call.stage("trace")).
trace_log = None


def collect_traces(into):
    """``into``: a list that receives one stage timeline per backward call, or
    None to stop collecting.  (The package exports the FUNCTION transducer_loss
    under this module's name, so the module attribute is set through here.)"""
    global trace_log
    trace_log = into


def _record_trace(call):
    if trace_log is not None:
        trace_log.append(call.stage("trace").clone())


def _check_mode(default="deferred"):
    """"off", "deferred" or "strict", from ``OT_CHECKS`` (0 / 1 / 2)."""
    v = os.environ.get("OT_CHECKS", "1")
    if v == "0":
        return "off"
    if v == "2":
        return "strict"
    return default


def _eager_grad():
    return os.environ.get("OT_EAGER_GRAD", "1") != "0"


def _linear_domain():
    # OT_LATTICE=linear: float32 recursions in a scaled linear domain (every value
    # carried as m * 2^e) instead of the reference's log domain: alpha/beta land
    # within one float32 rounding of the float64 recursion and the gradient about
    # six to ten times closer to the float64 gradient than the reference's own
    # float32 output, for a recursion that takes 1.6 times as long.  Default: the
    # log domain, which repeats the reference's roundings almost step by step.
    return os.environ.get("OT_LATTICE", "log") == "linear"


def _fast_math(from_log_softmax=False):
    # Hardware ex2/lg2 in the log-adds of the recursions (float32, log domain).
    # OT_FAST_MATH=1 / 0 force it on / off.  Unset: on for raw logits (the
    # recursions are a latency chain in which the library exp/log1p cost ~20 %, and
    # against the reference's own build the approximations add less than a third to
    # a gradient difference that the order of the logsumexp sums dominates), off for
    # log-softmax input (no logsumexp there: with the exact log-add the gradient
    # matches the reference's to 2.5e-5 on the large-vocabulary benchmark batch,
    # with the approximations to 4.9e-4).
    v = os.environ.get("OT_FAST_MATH")
    if v is None or v == "":
        return not from_log_softmax
    return v != "0"


_LOGIT_DTYPES = (torch.float32, torch.float64, torch.bfloat16, torch.float16)


def _validate(logits, targets, logit_lengths, target_lengths, blank):
    """The metadata checks of ot::ComputeTransducerLoss
    (optimized_transducer/csrc/transducer-loss.cc:33-46, 58-60, 77-79); the
    data-dependent ones (:49-56, :62-66) run on the device."""
    dev = logits.device
    if (logits.dtype in _LOGIT_DTYPES and targets.dtype == torch.int32
            and logit_lengths.dtype == torch.int32 and target_lengths.dtype == torch.int32
            and logits.dim() == 2 and targets.dim() == 2 and logit_lengths.dim() == 1
            and target_lengths.dim() == 1 and logits.is_cuda and targets.device == dev
            and logit_lengths.device == dev and target_lengths.device == dev
            and logits.is_contiguous() and targets.is_contiguous()
            and logit_lengths.is_contiguous() and target_lengths.is_contiguous()
            and logit_lengths.size(0) == target_lengths.size(0) == targets.size(0) > 0
            and logits.size(0) > 0 and 0 <= blank < logits.size(1)):
        return  # the common case: one pass over the metadata
    _explain_invalid(logits, targets, logit_lengths, target_lengths, blank)


def _explain_invalid(logits, targets, logit_lengths, target_lengths, blank):
    """Raises the error for the first check of :func:`_validate` that fails."""
    who = "ComputeTransducerLoss"
    if logits.dtype not in _LOGIT_DTYPES:
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
    raise RuntimeError(f"{who}: empty batch")


def real_dtype(logits):
    """dtype of everything but the logits and their gradient: scores, loss,
    upstream factors, workspace arrays.  16-bit logits are computed in float32."""
    return logits.dtype if logits.dtype == torch.float64 else torch.float32


_DTYPE_FLAG = {torch.float32: 0, torch.float64: _lib.FP64, torch.bfloat16: _lib.BF16,
               torch.float16: _lib.FP16}
_CHECK_FLAG = {"off": 0, "deferred": _lib.REPORT_ERRORS, "strict": _lib.CHECK_INPUTS,
               False: 0, True: _lib.CHECK_INPUTS}
_LAYOUT_BITS = _lib.FROM_LOG_SOFTMAX | _lib.ONE_SYM_PER_FRAME | _lib.FP64
_LAYOUTS = {}  # (N, rows, max_u, layout bits) -> workspace layout: shapes repeat from step to step


def _flags(logits, from_log_softmax, one_sym_per_frame, checks):
    f = _DTYPE_FLAG[logits.dtype] | _CHECK_FLAG[checks]
    if from_log_softmax:
        f |= _lib.FROM_LOG_SOFTMAX
    if one_sym_per_frame:
        f |= _lib.ONE_SYM_PER_FRAME
    if _fast_math(from_log_softmax):
        f |= _lib.FAST_MATH
    if _linear_domain():
        f |= _lib.LINEAR_DOMAIN
    if os.environ.get("OT_TRACE", "0") == "1":
        f |= _lib.TRACE
    return f


def _layout(n, rows, max_u, flags):
    key = (n, rows, max_u, flags & _LAYOUT_BITS)
    lay = _LAYOUTS.get(key)
    if lay is None:
        if len(_LAYOUTS) > 4096:
            _LAYOUTS.clear()
        lay = _LAYOUTS[key] = _lib.workspace_layout(n, rows, max_u, key[3])
    return lay


class _on_device:
    """``with _on_device(index):`` makes the device current for the library call
    if it is not already (the library launches on the current device)."""
    __slots__ = ("index", "prev")

    def __init__(self, index):
        self.index = index

    def __enter__(self):
        cur = torch.cuda.current_device()
        self.prev = cur if cur != self.index else -1
        if self.prev >= 0:
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def check_inputs(device=None, wait=True):
    """Raises ``RuntimeError`` if a loss evaluated on ``device`` (default: the
    current one) with deferred checks (``OT_CHECKS=1``) failed its device-side
    checks since the last report.  ``wait=True`` first waits for the kernels on
    the device's current stream, so every loss enqueued so far has reported."""
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    code = ctypes.c_int32(0)
    with _on_device(index):
        stream = ctypes.c_void_p(torch.cuda.current_stream(index).cuda_stream)
        _lib.check(lib.ot_b200_poll_errors(ctypes.byref(code), None, None, stream, 1 if wait else 0))
    if code.value:
        raise RuntimeError(_lib.last_error())


class _Call:
    """Pointers and sizes of one loss evaluation, plus its workspace."""

    def __init__(self, logits, targets, logit_lengths, target_lengths, blank,
                 from_log_softmax, one_sym_per_frame, checks=None, share_sms=False):
        _validate(logits, targets, logit_lengths, target_lengths, blank)
        if checks is None:
            checks = _check_mode()
        self.lib = _lib.load()
        self.logits = logits
        self.n = logit_lengths.size(0)
        self.rows, self.v = logits.shape
        self.max_u = targets.size(1)
        self.blank = int(blank)
        self.from_log_softmax = bool(from_log_softmax)
        self.modified = bool(one_sym_per_frame)
        self.flags = _flags(logits, from_log_softmax, one_sym_per_frame, checks)
        if share_sms:  # a collective runs beside this call (sharding.py)
            self.flags |= _lib.SHARE_SMS
        self.layout = _layout(self.n, self.rows, self.max_u, self.flags)
        self.bytes = int(self.layout.total_bytes)
        self.targets, self.t, self.u = targets, logit_lengths, target_lengths
        self.real = real_dtype(logits)
        self.device = logits.device
        self.index = logits.device.index
        self.workspace = torch.empty(self.bytes, dtype=torch.uint8, device=self.device)
        self.scores = torch.empty(self.n, dtype=self.real, device=self.device)

    def _stream(self):
        return torch.cuda.current_stream(self.index).cuda_stream

    def forward(self, loss_out=None, loss_scale=1.0):
        """Enqueues the forward half.  ``loss_out``: optional 0-dim tensor that
        receives ``loss_scale * -(sum of scores)``."""
        with _on_device(self.index):
            rc = self.lib.ot_b200_forward(
                self.logits.data_ptr(), self.targets.data_ptr() if self.max_u else None,
                self.t.data_ptr(), self.u.data_ptr(), self.n, self.rows, self.v, self.max_u,
                self.blank, self.flags, self.workspace.data_ptr(), self.bytes,
                self.scores.data_ptr(), loss_out.data_ptr() if loss_out is not None else None,
                loss_scale, self._stream())
        if rc:
            _lib.check(rc)
        return self.scores

    def backward(self, grad_out, scale_tensor=None, scale_host=1.0, per_utterance=False):
        """Enqueues the gradient pass.  ``scale_tensor``: a device scalar, or with
        ``per_utterance`` an (N,) tensor of per-utterance factors."""
        flags = self.flags & ~_lib.CHECK_INPUTS
        if per_utterance:
            assert scale_tensor is not None and scale_tensor.numel() == self.n
            flags |= _lib.SCALE_PER_UTTERANCE
        with _on_device(self.index):
            rc = self.lib.ot_b200_backward(
                self.logits.data_ptr(), grad_out.data_ptr(), self.n, self.rows, self.v,
                self.max_u, self.blank, flags, self.workspace.data_ptr(), self.bytes,
                scale_tensor.data_ptr() if scale_tensor is not None else None,
                scale_host, self._stream())
        if rc:
            _lib.check(rc)
        return grad_out

    def loss_and_gradient(self, grad_out=None, loss_out=None, loss_scale=1.0, grad_scale=1.0, cuts=None):
        """Enqueues the whole step as one library call: scores, the reduced loss
        (``loss_out``, optional) and, into ``grad_out`` (optional; may be the
        logits), ``grad_scale`` times the gradient of ``-scores.sum()``.  ``cuts``:
        a ctypes int64 array of packed-row positions that cut the batch into groups
        (``ot_b200_loss_and_gradient_groups``), or None: the library decides."""
        with _on_device(self.index):
            rc = self.lib.ot_b200_loss_and_gradient_groups(
                self.logits.data_ptr(), grad_out.data_ptr() if grad_out is not None else None,
                self.targets.data_ptr() if self.max_u else None, self.t.data_ptr(), self.u.data_ptr(),
                self.n, self.rows, self.v, self.max_u, self.blank, self.flags,
                self.workspace.data_ptr(), self.bytes, self.scores.data_ptr(),
                loss_out.data_ptr() if loss_out is not None else None, loss_scale, grad_scale,
                cuts, (len(cuts) - 1) if cuts is not None else 0, self._stream())
        if rc:
            _lib.check(rc)
        return self.scores

    def scale_gradient(self, grad, loss_grad):
        """``grad *= loss_grad`` on the device; a no-op kernel when the factor is 1."""
        g = self.upstream(loss_grad)
        with _on_device(self.index):
            rc = self.lib.ot_b200_scale_gradient(grad.data_ptr(), grad.numel(), g.data_ptr(),
                                                 _DTYPE_FLAG[grad.dtype] | (self.flags & _lib.REPORT_ERRORS),
                                                 self._stream())
        if rc:
            _lib.check(rc)
        return grad

    def upstream(self, loss_grad):
        """The upstream gradient as a device tensor of the arithmetic type."""
        g = loss_grad.detach()
        if g.dtype != self.real or g.device != self.device:
            g = g.to(device=self.device, dtype=self.real)
        return g if g.is_contiguous() else g.contiguous()

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
            # %globaltimer (ns) at which its first block started and its last block ended;
            # then the same five pairs for the second, third and fourth group of a grouped call
            off, count, dtype, esz = self.layout.status_off + 64, 40, torch.int64, 8
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
                 from_log_softmax, one_sym_per_frame, checks=_check_mode("strict"))
    grad = None
    if logits.requires_grad:
        data = logits.detach()
        grad = data if not from_log_softmax else torch.empty_like(data)
    scores = call.loss_and_gradient(grad)
    return scores, grad


_PLANS = {}  # shape key -> _Call whose workspace the next call of that shape on that stream reuses


def _planned_call(logits, targets, logit_lengths, target_lengths, blank, from_log_softmax,
                  one_sym_per_frame, share_sms=False):
    """A :class:`_Call` for a step that is complete after ONE library call
    (``loss_and_gradient``), with the workspace of the previous such call of the
    same shape on the same stream: calls on one stream run in order, the step's
    kernels are the workspace's only readers, and a call that splits into groups
    on the library's own streams joins them before it ends.  Training batches
    repeat their shapes (bucketed sampling); a new shape costs one allocation."""
    _validate(logits, targets, logit_lengths, target_lengths, blank)
    index = logits.device.index
    env = os.environ
    key = (logits.shape, logits.dtype, index, torch.cuda.current_stream(index).cuda_stream,
           targets.size(1), logit_lengths.size(0), blank, from_log_softmax, one_sym_per_frame,
           share_sms, env.get("OT_CHECKS"), env.get("OT_FAST_MATH"), env.get("OT_LATTICE"),
           env.get("OT_TRACE"))
    call = _PLANS.get(key)
    if call is None:
        if len(_PLANS) >= 64:
            _PLANS.clear()
        call = _PLANS[key] = _Call(logits, targets, logit_lengths, target_lengths, blank,
                                   from_log_softmax, one_sym_per_frame, share_sms=share_sms)
    else:
        call.logits, call.targets, call.t, call.u = logits, targets, logit_lengths, target_lengths
        call.scores = torch.empty(call.n, dtype=call.real, device=call.device)
    return call


MAX_GROUPS = 4


def group_cuts(logit_lengths, target_lengths, max_groups=MAX_GROUPS):
    """Packed-row positions that cut a batch into at most ``max_groups`` groups of
    consecutive utterances, as a ctypes int64 array for
    ``ot_b200_loss_and_gradient_groups``: one utterance per group for up to
    ``max_groups`` utterances, else groups of about equal numbers of rows.
    ``logit_lengths`` / ``target_lengths``: HOST tensors or sequences (T_b, U_b)."""
    T = logit_lengths.tolist() if hasattr(logit_lengths, "tolist") else list(logit_lengths)
    U = target_lengths.tolist() if hasattr(target_lengths, "tolist") else list(target_lengths)
    ends, total = [], 0
    for t, u in zip(T, U):
        total += int(t) * (int(u) + 1)
        ends.append(total)
    n = len(ends)
    g = min(max_groups, n)
    cuts = [0]
    if n <= max_groups:
        cuts += ends
    else:
        b = 0
        for k in range(1, g):
            # the first utterance end at or beyond the k-th quantile, leaving one
            # utterance at least for every later group
            while ends[b] < total * k / g and b < n - (g - k) - 1:
                b += 1
            cuts.append(ends[b])
            b += 1
        cuts.append(total)
    return (ctypes.c_int64 * len(cuts))(*cuts)


def _cached_cuts(call, lengths_on_host):
    """The cuts for ``lengths_on_host`` = (T, U) host tensors, computed once per
    pair of tensors (and again when one of them is modified in place)."""
    if lengths_on_host is None:
        return None
    t, u = lengths_on_host
    key = (id(t), id(u), getattr(t, "_version", 0), getattr(u, "_version", 0))
    if getattr(call, "cuts_key", None) != key:
        call.cuts_key, call.cuts = key, group_cuts(t, u)
        call.cuts_owner = (t, u)  # keeps the ids alive for as long as the key is
    return call.cuts


def transducer_loss_and_grad(logits, targets, logit_lengths, target_lengths, blank,
                             from_log_softmax, one_sym_per_frame=False, reduction="mean",
                             lengths_on_host=None):
    """Loss AND gradient in one library call, without an autograd graph: the
    shape of the reference's native function, which returns its scores together
    with the gradient (``_optimized_transducer.compute_transducer_loss``,
    python/csrc/optimized_transducer.cc:15-19 and csrc/cuda.cu:402-457 of the
    reference), with the reduction of its Python layer (transducer_loss.py:
    135-154) folded in.

    Returns ``(loss, grad)``: the reduced loss as a 0-dim tensor and the gradient
    of that loss with respect to ``logits``: ``logits`` itself, overwritten, for
    raw logits; a new tensor for log-softmax input.  A training loop hands it to
    the joiner with ``joiner_out.backward(grad)``.  Arguments, checks
    (``OT_CHECKS``) and numerics are those of :func:`transducer_loss`, whose
    ``loss.backward()`` leaves the same values; what is saved is the autograd
    engine's and this module's per-step host work (about 130 us, against 40 us
    here), which decides the step time of a batch of a few utterances per GPU.
    The workspace is reused from call to call (same shape, same stream).

    ``lengths_on_host``: optionally the pair (logit_lengths, target_lengths) as
    HOST tensors (a data loader has them).  The library pipelines a batch by
    groups of utterances (see ``ot_b200_loss_and_gradient_groups``); with the
    lengths known on the host the groups are cut at utterance boundaries, one
    utterance per group for up to four, which overlaps best when the shortest
    utterances come first.  Results do not depend on it."""
    assert reduction in ("mean", "sum")
    data = logits.detach() if logits.requires_grad else logits
    call = _planned_call(data, targets, logit_lengths, target_lengths, blank,
                         from_log_softmax, one_sym_per_frame)
    scale = (1.0 / call.n) if reduction == "mean" else 1.0
    grad = torch.empty_like(data) if from_log_softmax else data
    loss = torch.empty((), dtype=call.real, device=call.device)
    call.loss_and_gradient(grad, loss, loss_scale=scale, grad_scale=scale,
                           cuts=_cached_cuts(call, lengths_on_host))
    _record_trace(call)
    return loss, grad


def stage_outputs(logits, targets, logit_lengths, target_lengths, blank,
                  from_log_softmax=False, one_sym_per_frame=False):
    """Runs the forward half and returns its intermediate arrays (copies):
    ``scores``, ``scores_beta``, ``den`` (None for log-softmax input), ``lp``
    (rows, 2), ``alpha``, ``beta`` (rows) and ``split`` (N+1).  For tests and
    debugging; cells outside the band of the modified recursion are undefined."""
    call = _Call(logits, targets, logit_lengths, target_lengths, blank,
                 from_log_softmax, one_sym_per_frame, checks=_check_mode("strict"))
    scores = call.forward()
    cell = call.cell_index()
    out = {"scores": scores.clone(), "scores_beta": call.stage("scores_beta").clone(),
           "den": None if from_log_softmax else call.stage("den").clone(),
           "lp": call.stage("lp").view(-1, 2)[cell], "alpha": call.stage("alpha")[cell],
           "beta": call.stage("beta")[cell], "split": call.stage("split").clone()}
    return out


def joiner_scores(joiner_in, weight, bias, targets, logit_lengths, target_lengths, blank,
                  reduction=None, stages=False, _trace=None):
    """Scores (or the reduced loss) straight from the joiner's last projection,
    WITHOUT materialising the logits: ``logits = joiner_in @ weight.T + bias`` is
    computed tile by tile on the tensor cores and reduced to the row logsumexp and
    the two gathered log-probabilities inside the same kernel
    (``ot_b200_forward_linear``); the (rows, V) tensor the reference needs never
    exists.  Forward only (scoring, validation): no gradient is defined.

    ``joiner_in`` (rows, D) bfloat16, packed like the logits would be; ``weight``
    (V, D) bfloat16 (the layout of ``torch.nn.Linear.weight``); ``bias`` (V,)
    float32 or None; D a multiple of 8; standard transducer.  Returns the (N,)
    scores ``log P(y_b | x_b)`` (float32), or with ``reduction`` "mean" / "sum" the
    0-dim loss.  ``stages=True`` returns a dict with scores, den, lp, alpha, beta in
    packed-row order instead (for tests)."""
    who = "joiner_scores"
    if joiner_in.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise RuntimeError(f"{who}: joiner_in and weight must be bfloat16")
    if joiner_in.dim() != 2 or weight.dim() != 2 or joiner_in.size(1) != weight.size(1):
        raise RuntimeError(f"{who}: expected joiner_in (rows, D) and weight (V, D)")
    if not (joiner_in.is_cuda and joiner_in.is_contiguous() and weight.is_contiguous()
            and weight.device == joiner_in.device):
        raise RuntimeError(f"{who}: contiguous CUDA tensors on one device are required (sm_100a kernels, no CPU path)")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != weight.size(0)
                             or bias.device != joiner_in.device or not bias.is_contiguous()):
        raise RuntimeError(f"{who}: bias must be a contiguous float32 tensor of V entries")
    if joiner_in.size(1) % 8 != 0:
        raise RuntimeError(f"{who}: D must be a multiple of 8, got {joiner_in.size(1)}")
    assert reduction in (None, "mean", "sum")
    rows, d = joiner_in.shape
    v = weight.size(0)
    proxy = torch.empty((rows, v), dtype=torch.float32, device="meta")  # shapes for the shared checks only
    for name, t in (("targets", targets), ("logit_lengths", logit_lengths), ("target_lengths", target_lengths)):
        if t.dtype != torch.int32 or not t.is_contiguous() or t.device != joiner_in.device:
            raise RuntimeError(f"{who}: expected {name} to be a contiguous int32 tensor on {joiner_in.device}")
    if targets.dim() != 2 or logit_lengths.dim() != 1 or logit_lengths.shape != target_lengths.shape \
            or targets.size(0) != logit_lengths.size(0) or not (0 <= blank < v) or rows == 0:
        raise RuntimeError(f"{who}: inconsistent argument shapes, or blank outside [0, V)")
    del proxy
    lib = _lib.load()
    n, max_u = int(logit_lengths.size(0)), int(targets.size(1))
    flags = (_CHECK_FLAG[_check_mode("strict")] | (_lib.FAST_MATH if _fast_math(False) else 0)
             | (_lib.LINEAR_DOMAIN if _linear_domain() else 0))
    if os.environ.get("OT_TRACE", "0") == "1":
        flags |= _lib.TRACE
    lay = _layout(n, rows, max_u, 0)
    dev = joiner_in.device
    ws = torch.empty(int(lay.total_bytes), dtype=torch.uint8, device=dev)
    scores = torch.empty(n, dtype=torch.float32, device=dev)
    loss = torch.empty((), dtype=torch.float32, device=dev) if reduction else None
    scale = (1.0 / n) if reduction == "mean" else 1.0
    with _on_device(dev.index):
        rc = lib.ot_b200_forward_linear(
            joiner_in.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
            targets.data_ptr() if max_u else None, logit_lengths.data_ptr(), target_lengths.data_ptr(),
            n, rows, d, v, max_u, int(blank), flags, ws.data_ptr(), int(lay.total_bytes),
            scores.data_ptr(), loss.data_ptr() if loss is not None else None, scale,
            torch.cuda.current_stream(dev.index).cuda_stream)
    if rc:
        _lib.check(rc)
    if _trace is not None:  # diagnostic (OT_TRACE=1): the stage timeline of this call
        _trace.append(ws[int(lay.status_off) + 64:int(lay.status_off) + 64 + 160].view(torch.int64).clone())
    if not stages:
        return loss if reduction else scores
    # the stage arrays, through a _Call-shaped view of the same workspace
    view = _Call.__new__(_Call)
    view.layout, view.workspace, view.real, view.n, view.rows = lay, ws, torch.float32, n, rows
    view.t, view.u, view.modified, view.logits = logit_lengths, target_lengths, False, joiner_in
    cell = view.cell_index()
    return {"scores": scores, "den": view.stage("den").clone(), "lp": view.stage("lp").view(-1, 2)[cell],
            "alpha": view.stage("alpha")[cell], "beta": view.stage("beta")[cell]}


def _padded_columns(v):
    """The number of columns the backward pass of :func:`joiner_loss` gives its
    bfloat16 gradient tile: ``v`` when rows of ``v`` entries already are a multiple
    of 16 bytes; else the next multiple of 64 when that adds at most 1/32, else
    the next multiple of 8."""
    if v % 8 == 0:
        return v
    v64 = -(-v // 64) * 64
    return v64 if (v64 - v) * 32 <= v else -(-v // 8) * 8


# The column sums of the gradient tile (the bias gradient) as a tensor-core
# contraction with eight rows of ones, float32 out: measured 0.11 ms against
# 0.21 ms for ``sum(0)`` on 686 128 x 512; for wide rows ``sum(0)`` is used.
_COLUMN_SUMS_BY_MATMUL_MAX_V = 1024
_ONES = {}


def _ones_rows(rows, device):
    key = (rows, device)
    t = _ONES.get(key)
    if t is None:
        _ONES.clear()  # one batch shape at a time: 16 bytes per row
        t = _ONES[key] = torch.ones((8, rows), dtype=torch.bfloat16, device=device)
    return t


class JoinerLossFunction(torch.autograd.Function):
    """Transducer loss straight from the joiner's last projection, forward AND
    backward, without the (rows, V) logits: see :func:`joiner_loss`."""

    @staticmethod
    def forward(ctx, joiner_in, weight, bias, targets, logit_lengths, target_lengths, blank, reduction):
        assert reduction in ("mean", "sum")
        x, w = joiner_in.detach(), weight.detach()
        b = bias.detach() if bias is not None else None
        rows, d = x.shape
        v = w.size(0)
        n, max_u = int(logit_lengths.size(0)), int(targets.size(1))
        lib = _lib.load()
        flags = (_CHECK_FLAG[_check_mode()] | (_lib.FAST_MATH if _fast_math(False) else 0)
                 | (_lib.LINEAR_DOMAIN if _linear_domain() else 0))
        if os.environ.get("OT_TRACE", "0") == "1":
            flags |= _lib.TRACE
        lay = _layout(n, rows, max_u, 0)
        dev = x.device
        ws = torch.empty(int(lay.total_bytes), dtype=torch.uint8, device=dev)
        scores = torch.empty(n, dtype=torch.float32, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        scale = (1.0 / n) if reduction == "mean" else 1.0
        with _on_device(dev.index):
            rc = lib.ot_b200_forward_linear(
                x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                targets.data_ptr() if max_u else None, logit_lengths.data_ptr(), target_lengths.data_ptr(),
                n, rows, d, v, max_u, int(blank), flags, ws.data_ptr(), int(lay.total_bytes),
                scores.data_ptr(), loss.data_ptr(), scale, torch.cuda.current_stream(dev.index).cuda_stream)
        if rc:
            _lib.check(rc)
        ctx.save_for_backward(x, w, b if b is not None else torch.empty(0, device=dev))
        ctx.meta = (n, rows, d, v, max_u, int(blank), flags & ~_lib.CHECK_INPUTS, ws, int(lay.total_bytes), scale,
                    b is not None, int(lay.status_off))
        return loss

    @staticmethod
    def backward(ctx, loss_grad):
        x, w, b = ctx.saved_tensors
        n, rows, d, v, max_u, blank, flags, ws, ws_bytes, scale, has_bias, status_off = ctx.meta
        lib = _lib.load()
        dev = x.device
        # The gradient tile the contractions read has rows of 2 * V bytes.  When that is
        # not a multiple of 16 (V = 500: 1000 bytes) the matmuls that read it fall off
        # the library's tensor-core kernels (measured, rows = 686 128, D = 512:
        # G @ W 1.40 ms and G.T @ X 1.15 ms with V = 500 against 0.33 ms each with the
        # rows padded to 512 columns).  So the projection is widened for this pass:
        # zero weight rows and a bias of -1e30 make the kernel write exact zeros into
        # the padding columns, which then drop out of all three contractions.
        vp = _padded_columns(v)
        wk, bk = w, (b if has_bias else None)
        if vp != v:
            wk = torch.zeros((vp, d), dtype=w.dtype, device=dev)
            wk[:v] = w
            bk = torch.full((vp,), -1e30, dtype=torch.float32, device=dev)
            if has_bias:
                bk[:v] = b
            else:
                bk[:v] = 0
        g = torch.empty((rows, vp), dtype=torch.bfloat16, device=dev)
        up = loss_grad.detach().to(device=dev, dtype=torch.float32).contiguous()
        with _on_device(dev.index):
            rc = lib.ot_b200_backward_linear(
                x.data_ptr(), wk.data_ptr(), bk.data_ptr() if bk is not None else None, n, rows, d, vp, max_u,
                blank, flags, ws.data_ptr(), ws_bytes, g.data_ptr(), up.data_ptr(), scale,
                torch.cuda.current_stream(dev.index).cuda_stream)
        if rc:
            _lib.check(rc)
        if trace_log is not None:  # diagnostic (OT_TRACE=1): the stage timeline of this loss
            trace_log.append(ws[status_off + 64:status_off + 64 + 320].view(torch.int64).clone())
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = g @ wk                     # (rows, V') x (V', D)
        if ctx.needs_input_grad[1]:
            # float32 out of the library's reduction over the rows, rounded once (a
            # bfloat16 output of this contraction measured 8e-3 of its largest entry
            # off the float64 result, the float32 one 1e-4, at the same speed)
            gw = torch.mm(g.t(), x, out_dtype=torch.float32)[:v].to(w.dtype)
        if has_bias and ctx.needs_input_grad[2]:
            if vp <= _COLUMN_SUMS_BY_MATMUL_MAX_V:
                gb = torch.mm(_ones_rows(rows, dev), g, out_dtype=torch.float32)[0, :v].contiguous()
            else:
                gb = g.sum(0, dtype=torch.float32)[:v].contiguous()
        return gx, gw, gb, None, None, None, None, None


def joiner_loss(joiner_in, weight, bias, targets, logit_lengths, target_lengths, blank,
                reduction="mean"):
    """The transducer loss of ``logits = joiner_in @ weight.T + bias`` with
    gradients for ``joiner_in``, ``weight`` and ``bias``, WITHOUT the (rows, V)
    logits in either direction.  Forward: :func:`joiner_scores` (projection,
    logsumexp and gather in one tensor-core kernel).  Backward: the library
    recomputes the logits tile by tile on the tensor cores and writes the gradient
    with respect to the logits in bfloat16 (``ot_b200_backward_linear``); the three
    contractions with it (``G @ weight``, ``G.T @ joiner_in``, column sums) are
    PyTorch matmuls; for a V whose rows of bfloat16 are not a multiple of 16 bytes
    the tile is given padding columns of exact zeros (see ``_padded_columns``),
    because those matmuls are three to four times slower on unaligned rows.  What is saved against the reference's path: the float
    logits (4 V bytes per row, written by the projection, read by the loss,
    overwritten by its gradient) never exist; the only (rows, V) tensor is the
    bfloat16 gradient, alive during ``backward`` only.

    ``joiner_in`` (rows, D) and ``weight`` (V, D) bfloat16, ``bias`` (V,) float32 or
    None; D a multiple of 8, V a multiple of 4; standard transducer; ``reduction``
    "mean" or "sum".  The gradient with respect to the logits is rounded to
    bfloat16 (2^-9 relative), like the activations around it."""
    who = "joiner_loss"
    if joiner_in.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise RuntimeError(f"{who}: joiner_in and weight must be bfloat16")
    if joiner_in.dim() != 2 or weight.dim() != 2 or joiner_in.size(1) != weight.size(1):
        raise RuntimeError(f"{who}: expected joiner_in (rows, D) and weight (V, D)")
    if not (joiner_in.is_cuda and joiner_in.is_contiguous() and weight.is_contiguous()
            and weight.device == joiner_in.device):
        raise RuntimeError(f"{who}: contiguous CUDA tensors on one device are required (sm_100a kernels, no CPU path)")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != weight.size(0)
                             or bias.device != joiner_in.device or not bias.is_contiguous()):
        raise RuntimeError(f"{who}: bias must be a contiguous float32 tensor of V entries")
    if joiner_in.size(1) % 8 != 0 or weight.size(0) % 4 != 0:
        raise RuntimeError(f"{who}: D must be a multiple of 8 and V a multiple of 4, got D={joiner_in.size(1)}, "
                           f"V={weight.size(0)}")
    for name, t in (("targets", targets), ("logit_lengths", logit_lengths), ("target_lengths", target_lengths)):
        if t.dtype != torch.int32 or not t.is_contiguous() or t.device != joiner_in.device:
            raise RuntimeError(f"{who}: expected {name} to be a contiguous int32 tensor on {joiner_in.device}")
    if targets.dim() != 2 or logit_lengths.dim() != 1 or logit_lengths.shape != target_lengths.shape \
            or targets.size(0) != logit_lengths.size(0) or not (0 <= blank < weight.size(0)) \
            or joiner_in.size(0) == 0:
        raise RuntimeError(f"{who}: inconsistent argument shapes, or blank outside [0, V)")
    return JoinerLossFunction.apply(joiner_in, weight, bias, targets, logit_lengths, target_lengths, blank,
                                    reduction)


class TransducerLossFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, logit_lengths, target_lengths, blank,
                from_log_softmax, one_sym_per_frame, reduction="mean"):
        assert reduction in ("mean", "sum")
        n = logit_lengths.size(0)
        if _eager_grad():
            # The reference's schedule (transducer_loss.py:135-154): the gradient is
            # computed here, over the logits, with the 1/N of "mean" already applied.
            data = logits.detach()
            call = _Call(data, targets, logit_lengths, target_lengths, blank,
                         from_log_softmax, one_sym_per_frame)
            scale = (1.0 / n) if reduction == "mean" else 1.0
            grad = None
            if ctx.needs_input_grad[0]:
                grad = torch.empty_like(data) if from_log_softmax else data
            loss = torch.empty((), dtype=call.real, device=logits.device)
            call.loss_and_gradient(grad, loss, loss_scale=scale, grad_scale=scale)
            ctx.grad = grad
            ctx.call = None
            ctx.eager = call if grad is not None else None
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
            grad, ctx.grad = ctx.grad, None
            call, ctx.eager = ctx.eager, None  # the workspace is released after this
            call.scale_gradient(grad, loss_grad)  # reference transducer_loss.py:162
            _record_trace(call)
            return (grad,) + (None,) * 7
        call, ctx.call = ctx.call, None  # the workspace is released after this pass
        data = call.logits
        grad = torch.empty_like(data) if call.from_log_softmax else data
        call.backward(grad, scale_tensor=call.upstream(loss_grad), scale_host=ctx.scale_host)
        _record_trace(call)  # diagnostic, see OT_TRACE
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
        call.backward(grad, scale_tensor=call.upstream(loss_grad), per_utterance=True)
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
