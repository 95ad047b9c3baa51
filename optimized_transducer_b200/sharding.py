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


class PeerExchange:
    """Sum of one scalar per rank over peer-mapped device memory, the light
    alternative to an NCCL all-reduce of the 0-dim loss (see
    ``csrc/exchange.cu``): a one-warp kernel stores this rank's value into every
    rank's table, a second one-warp kernel sums the table once all values of the
    step are there.  Neither needs the room a collective's kernel needs, so both
    run beside the one-wave gradient kernel.

    ``PeerExchange(group)`` allocates the table with
    ``torch.distributed._symmetric_memory`` (one rendezvous, then no library
    call on the data path).  ``PeerExchange(tables=[...], rank=r)`` takes tables
    the caller made addressable itself (tests emulate several ranks on one
    device with it).  Ranks must not drift apart by ``ring`` steps or more.
    """

    RING = 256

    def __init__(self, group=None, device=None, tables=None, rank=None, max_wait_s=2.0):
        from . import _lib
        import ctypes
        self._lib, self._ct = _lib, ctypes
        self.lib = _lib.load()
        self.step = 0
        self.max_wait_ns = int(max_wait_s * 1e9)
        if tables is not None:
            self.world, self.rank = len(tables), int(rank)
            self.table = tables[self.rank]
            self._keep = list(tables)
            ptrs = [t.data_ptr() for t in tables]
            device = self.table.device
        else:
            import torch.distributed._symmetric_memory as symm_mem
            group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
            self.table = symm_mem.empty(self.table_doubles(self.world), dtype=torch.float64, device=device)
            self.table.zero_()
            self._keep = symm_mem.rendezvous(self.table, group)
            ptrs = [int(p) for p in self._keep.buffer_ptrs]
            torch.cuda.synchronize(device)
            dist.barrier(group)  # every table is zero before anyone publishes
        self.device = device
        self.ptrs = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)

    @classmethod
    def table_doubles(cls, world):
        """Size of one rank's table in float64 elements (16 bytes per entry)."""
        return 2 * cls.RING * world

    def _stream(self, stream):
        stream = torch.cuda.current_stream(self.device) if stream is None else stream
        return self._ct.c_void_p(stream.cuda_stream)

    def publish(self, local, step=None, stream=None):
        """Stores ``local`` (0-dim float32/float64) into every rank's table; never waits."""
        assert local.dtype in (torch.float32, torch.float64)
        flags = self._lib.FP64 if local.dtype == torch.float64 else 0
        with torch.cuda.device(self.device):
            self._lib.check(self.lib.ot_b200_exchange_publish(
                local.data_ptr(), flags, self.ptrs.data_ptr(), self.world, self.rank, self.RING,
                self.step if step is None else int(step), self._stream(stream)))

    def gather(self, out, scale=1.0, step=None, stream=None):
        """``out = scale * sum over ranks`` of what they published for the step
        (waits, bounded, for the values that are not there yet)."""
        assert out.dtype in (torch.float32, torch.float64)
        flags = self._lib.FP64 if out.dtype == torch.float64 else 0
        with torch.cuda.device(self.device):
            self._lib.check(self.lib.ot_b200_exchange_gather(
                self.table.data_ptr(), self.world, self.RING,
                self.step if step is None else int(step), out.data_ptr(), flags,
                float(scale), self.error.data_ptr(), self.max_wait_ns, self._stream(stream)))
        return out

    def all_reduce_sum(self, local, out, scale=1.0, stream=None):
        """Enqueues publish + gather of the next step on ``stream`` (default:
        the current one): ``out = scale * sum over ranks of local``."""
        assert local.dtype == out.dtype
        self.publish(local, stream=stream)
        self.gather(out, scale, stream=stream)
        self.step += 1
        return out

    def check(self):
        """Synchronises and raises if a gather gave up (a rank did not publish in time)."""
        code = int(self.error.item())
        if code:
            what = (f"rank {code - 101}'s entry was overwritten (ranks drifted apart by {self.RING} steps)"
                    if code > 100 else f"rank {code - 1} did not publish within {self.max_wait_ns / 1e9:.1f} s")
            raise RuntimeError("PeerExchange: " + what)


_PEER = {}


def peer_exchange(group=None, device=None):
    """The (cached) :class:`PeerExchange` of a process group; collective on first use."""
    key = (id(group), str(device))
    if key not in _PEER:
        _PEER[key] = PeerExchange(group, device)
    return _PEER[key]


class _ShardedLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, logit_lengths, target_lengths, blank, from_log_softmax,
                one_sym_per_frame, reduction, global_batch, group, overlap, exchange):
        assert reduction in ("mean", "sum")
        if logit_lengths.numel() > 0:
            call = _Call(logits.detach(), targets, logit_lengths, target_lengths, blank,
                         from_log_softmax, one_sym_per_frame,
                         share_sms=bool(overlap) and exchange is None)
            local = torch.empty((), dtype=real_dtype(logits), device=logits.device)
            call.forward(loss_out=local, loss_scale=1.0)
        else:  # a rank without utterances still joins the collective
            call = None
            local = torch.zeros((), dtype=real_dtype(logits), device=logits.device)
        scale = 1.0 / float(global_batch) if reduction == "mean" else 1.0
        if exchange is not None:
            # peer-memory exchange: two one-warp kernels on the side stream
            main = torch.cuda.current_stream(logits.device)
            side = _side_stream(logits.device)
            side.wait_stream(main)
            total = torch.empty_like(local)
            exchange.all_reduce_sum(local, total, scale, stream=side)
            local.record_stream(side)
            total.record_stream(side)
            ctx.call = call if ctx.needs_input_grad[0] else None
            ctx.scale_host = scale
            ctx.empty_like = logits.detach() if call is None else None
            return total
        total, event = all_reduce_sum(local, group, overlap)
        if reduction == "mean":
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
        return (grad,) + (None,) * 11


def sharded_transducer_loss(logits, targets, logit_lengths, target_lengths, blank,
                            from_log_softmax, one_sym_per_frame=False, reduction="mean",
                            global_batch: Optional[int] = None, group=None, overlap=False,
                            exchange: Optional[PeerExchange] = None):
    """Transducer loss of a batch that is sharded by utterance over the ranks of
    ``group``.  Every rank passes ITS utterances (packed logits, targets padded
    to the local max U, lengths); every rank gets the loss of the whole batch.
    ``global_batch`` is the number of utterances over all ranks ("mean" divides
    by it; default: local count x world size).  Backward scales only the local
    rows: no gradient crosses ranks.

    ``overlap=True`` issues the scalar all-reduce on a side stream, off the
    critical path of the gradient pass; the VALUE of the returned tensor is then
    defined only after :func:`wait_loss` (or a device synchronisation).

    ``exchange`` (a :class:`PeerExchange`, e.g. ``peer_exchange(group)``; GPUs of
    one node) replaces the NCCL all-reduce by two one-warp kernels over peer
    memory on the side stream; the value is likewise defined after
    :func:`wait_loss`."""
    if global_batch is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        global_batch = int(logit_lengths.numel()) * world
    loss = _ShardedLoss.apply(logits, targets, logit_lengths, target_lengths, blank,
                              from_log_softmax, one_sym_per_frame, reduction, global_batch,
                              group, overlap, exchange)
    return loss
