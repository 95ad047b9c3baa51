"""Utterance-level sharding of a batch across GPUs (one process per GPU).

The reference has no multi-device code (its only device awareness is the
``torch::DeviceGuard`` at optimized_transducer/csrc/cuda.cu:408).  Utterances
are independent up to the final reduction (``loss.sum()`` / ``loss.mean()``,
transducer_loss.py:147-152), so a batch shards by utterance with a single
exchange step: an all-reduce of the scalar loss.  Gradients never leave the
rank that owns the rows.

* :func:`partition_contiguous` / :func:`partition_lpt` split utterances by the
  streaming cost ``T_b * (U_b + 1) * V``.
* :func:`shard_batch` gives one rank its lengths, targets (re-padded to the
  shard's own max U, which the loss requires) and its row range.
* :func:`sharded_transducer_loss` evaluates the loss of the local shard with
  the sm_100a kernels and all-reduces the scalar; with ``overlap=True`` the
  all-reduce runs on a side stream and the main stream only waits for it after
  the gradient pass has been enqueued.
"""
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .transducer_loss import _Call, real_dtype

__all__ = ["utterance_costs", "partition_contiguous", "partition_lpt", "imbalance",
           "Shard", "shard_batch", "all_reduce_sum", "sharded_transducer_loss", "wait_loss"]


def utterance_costs(T, U, V: int) -> List[int]:
    """Streaming cost of each utterance: lattice cells times vocabulary size."""
    return [int(t) * (int(u) + 1) * int(V) for t, u in zip(T.tolist(), U.tolist())]


def partition_contiguous(costs: Sequence[int], world: int) -> List[Tuple[int, int]]:
    """Splits ``range(len(costs))`` into ``world`` consecutive ranges ``[b0, b1)``
    minimising the largest range cost (linear-partition dynamic programme).
    Ranges are non-empty while utterances last; surplus ranks get ``(n, n)``."""
    n = len(costs)
    parts = min(world, n)
    prefix = [0]
    for c in costs:
        prefix.append(prefix[-1] + c)
    inf = float("inf")
    # best[k][i]: minimal max-cost of splitting the first i utterances into k ranges
    best = [[inf] * (n + 1) for _ in range(parts + 1)]
    cut = [[0] * (n + 1) for _ in range(parts + 1)]
    best[0][0] = 0
    for k in range(1, parts + 1):
        for i in range(k, n + 1):
            for j in range(k - 1, i):
                cand = max(best[k - 1][j], prefix[i] - prefix[j])
                if cand < best[k][i]:
                    best[k][i], cut[k][i] = cand, j
    bounds, i = [], n
    for k in range(parts, 0, -1):
        j = cut[k][i]
        bounds.append((j, i))
        i = j
    bounds.reverse()
    bounds += [(n, n)] * (world - parts)
    return bounds


def partition_lpt(costs: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time bin packing: utterances in decreasing cost order,
    each to the least loaded rank.  Returns the (sorted) index list per rank."""
    loads = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for b in sorted(range(len(costs)), key=lambda i: (-costs[i], i)):
        r = min(range(world), key=lambda k: (loads[k], k))
        out[r].append(b)
        loads[r] += costs[b]
    return [sorted(ix) for ix in out]


def imbalance(costs: Sequence[int], parts: Sequence[Sequence[int]]) -> float:
    """max shard cost / mean shard cost (1.0 = perfectly balanced)."""
    loads = [sum(costs[b] for b in p) for p in parts]
    mean = sum(loads) / max(len(loads), 1)
    return max(loads) / mean if mean > 0 else 1.0


@dataclass
class Shard:
    rank: int
    indices: List[int]            # utterances of the global batch owned by this rank
    contiguous: bool              # True: indices is a range and rows is one slice
    T: torch.Tensor               # (n_local,) int32
    U: torch.Tensor               # (n_local,) int32
    targets: torch.Tensor         # (n_local, max local U) int32
    row_ranges: List[Tuple[int, int]]  # packed-row range of each owned utterance
    cost: int


def shard_batch(T: torch.Tensor, U: torch.Tensor, targets: torch.Tensor, V: int,
                world: int, rank: int, strategy: str = "auto",
                max_imbalance: float = 1.10) -> Shard:
    """The part of a global batch that ``rank`` owns.

    ``strategy``: "contiguous" keeps the utterance order, so the shard's rows
    are one slice of the packed logits (a view, and the in-place gradient lands
    in the caller's buffer); "lpt" balances better but permutes; "auto" uses
    contiguous unless its imbalance exceeds ``max_imbalance``."""
    costs = utterance_costs(T, U, V)
    bounds = partition_contiguous(costs, world)
    parts = [list(range(a, b)) for a, b in bounds]
    contiguous = True
    if strategy == "lpt" or (strategy == "auto" and imbalance(costs, parts) > max_imbalance):
        lpt = partition_lpt(costs, world)
        if strategy == "lpt" or imbalance(costs, lpt) < imbalance(costs, parts):
            parts, contiguous = lpt, False
    mine = parts[rank]
    cells = (T.to(torch.int64) * (U.to(torch.int64) + 1))
    starts = torch.cumsum(cells, 0) - cells
    idx = torch.tensor(mine, dtype=torch.long)
    Tl = T[idx].contiguous()
    Ul = U[idx].contiguous()
    max_u = int(Ul.max()) if len(mine) else 0
    tl = targets[idx, :max_u].contiguous()
    ranges = [(int(starts[b]), int(starts[b] + cells[b])) for b in mine]
    return Shard(rank, mine, contiguous, Tl, Ul, tl, ranges, sum(costs[b] for b in mine))


def slice_rows(packed: torch.Tensor, shard: Shard) -> torch.Tensor:
    """Rows of ``packed`` (global batch) that belong to ``shard``: a view for a
    contiguous shard, a gathered copy otherwise."""
    if not shard.row_ranges:
        return packed[:0]
    if shard.contiguous:
        return packed[shard.row_ranges[0][0]:shard.row_ranges[-1][1]]
    return torch.cat([packed[a:b] for a, b in shard.row_ranges])


def all_reduce_sum(x: torch.Tensor, group=None, overlap: bool = False):
    """Sum of ``x`` over the ranks of ``group``.  Returns ``(y, event)``.

    With ``overlap`` (CUDA only) the collective is issued on a side stream that
    first waits for the current stream; ``event`` marks its completion and ``y``
    must not be read before the reader's stream has waited for it.  Otherwise
    ``event`` is None and ``y`` is ready in stream order."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return x.clone(), None
    if not (overlap and x.is_cuda):
        y = x.clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y, None
    main = torch.cuda.current_stream(x.device)
    side = _side_stream(x.device)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        y = x.clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        event = side.record_event()
    x.record_stream(side)
    y.record_stream(main)
    return y, event


_SIDE = {}


def _side_stream(device):
    key = (device.type, device.index)
    if key not in _SIDE:
        # high priority: the collective's single CTA must not queue behind the
        # full-occupancy gradient kernel (also create the NCCL process group with
        # ProcessGroupNCCL.Options().is_high_priority_stream = True)
        _SIDE[key] = torch.cuda.Stream(device=device, priority=-1)
    return _SIDE[key]


def wait_loss(loss: torch.Tensor) -> torch.Tensor:
    """Makes the current stream wait for the all-reduce behind a loss returned by
    ``sharded_transducer_loss(..., overlap=True)``.  Call it before the value is
    read (``loss.item()``, logging, a device-side consumer on another stream)."""
    if loss.is_cuda:
        # every overlapped all-reduce of this device runs on the same side stream
        torch.cuda.current_stream(loss.device).wait_stream(_side_stream(loss.device))
    return loss


class _ShardedLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, logit_lengths, target_lengths, blank, from_log_softmax,
                one_sym_per_frame, reduction, global_batch, group, overlap):
        assert reduction in ("mean", "sum")
        if logit_lengths.numel() > 0:
            call = _Call(logits.detach(), targets, logit_lengths, target_lengths, blank,
                         from_log_softmax, one_sym_per_frame, share_sms=bool(overlap))
            local = torch.empty((), dtype=real_dtype(logits), device=logits.device)
            call.forward(loss_out=local, loss_scale=1.0)
        else:  # a rank without utterances still joins the collective
            call = None
            local = torch.zeros((), dtype=real_dtype(logits), device=logits.device)
        total, event = all_reduce_sum(local, group, overlap)
        scale = 1.0
        if reduction == "mean":
            scale = 1.0 / float(global_batch)
            if event is not None:
                with torch.cuda.stream(_side_stream(logits.device)):
                    total = total * scale
                    event = _side_stream(logits.device).record_event()
                total.record_stream(torch.cuda.current_stream(logits.device))
            else:
                total = total * scale
        ctx.call = call if ctx.needs_input_grad[0] else None
        ctx.scale_host = scale
        ctx.event = event
        ctx.empty_like = logits.detach() if call is None else None
        return total

    @staticmethod
    def backward(ctx, loss_grad):
        assert loss_grad.numel() == 1, loss_grad.numel()
        call, ctx.call = ctx.call, None
        grad = None
        if call is not None:
            data = call.logits
            grad = torch.empty_like(data) if call.from_log_softmax else data
            g = loss_grad.detach().to(device=data.device, dtype=call.real).contiguous()
            call.backward(grad, scale_tensor=g, scale_host=ctx.scale_host)
        elif ctx.empty_like is not None:
            grad = torch.zeros_like(ctx.empty_like)
        # Nothing here depends on the reduced VALUE, so the main stream does not
        # wait for the collective: the gradient kernel fills every SM until it
        # ends, the collective's kernel gets its slot only then, and a wait here
        # would put its whole latency behind the gradient pass.  It now runs
        # under whatever the main stream does next; wait_loss() orders a reader.
        return (grad,) + (None,) * 10


def sharded_transducer_loss(logits, targets, logit_lengths, target_lengths, blank,
                            from_log_softmax, one_sym_per_frame=False, reduction="mean",
                            global_batch: Optional[int] = None, group=None, overlap=False):
    """Transducer loss of a batch that is sharded by utterance over the ranks of
    ``group``.  Every rank passes ITS utterances (packed logits, targets padded
    to the local max U, lengths); every rank gets the loss of the whole batch.
    ``global_batch`` is the number of utterances over all ranks ("mean" divides
    by it; default: local count x world size).  Backward scales only the local
    rows: no gradient crosses ranks.

    ``overlap=True`` issues the scalar all-reduce on a side stream, off the
    critical path of the gradient pass; the VALUE of the returned tensor is then
    defined only after :func:`wait_loss` (or a device synchronisation)."""
    if global_batch is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        global_batch = int(logit_lengths.numel()) * world
    loss = _ShardedLoss.apply(logits, targets, logit_lengths, target_lengths, blank,
                              from_log_softmax, one_sym_per_frame, reduction, global_batch,
                              group, overlap)
    return loss
