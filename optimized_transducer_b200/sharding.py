"""Utterance-level sharding of a batch across GPUs (one process per GPU).

The reference has no multi-device code (its only device awareness is the
``torch::DeviceGuard`` at optimized_transducer/csrc/cuda.cu:408).  Utterances
are independent up to the final reduction (``loss.sum()`` / ``loss.mean()``,
transducer_loss.py:147-152), so a batch shards by utterance with a single
exchange step: an all-reduce of the scalar loss.  Gradients never leave the
rank that owns the rows.

* :func:`partition_contiguous` / :func:`partition_lpt` split utterances by the
  streaming cost ``T_b * (U_b + 1) * V``; :func:`partition_lpt` can also weigh
  in the length ``T_b + U_b`` of the longest recursion of a shard, which is
  what a rank with only a few utterances waits for.
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

from .transducer_loss import (_Call, _cached_cuts, _eager_grad, _on_device, _planned_call,
                              _record_trace, real_dtype)

__all__ = ["utterance_costs", "chain_lengths", "shard_time", "partition_contiguous", "partition_lpt", "imbalance",
           "Shard", "shard_batch", "all_reduce_sum", "sharded_transducer_loss", "sharded_loss_and_grad",
           "wait_loss"]


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


# Step-time model of one rank: (12 bytes per cell) / (HBM bandwidth) for the
# three streaming passes over its cells, plus the dependent chain of the longest
# alpha/beta recursion it holds (one log-add per step of T+U).  Only the RATIO of
# the two constants matters for a partition; they are the measured B200 figures
# (6.5 TB/s copy bandwidth, 93 ns per recursion step).
SECONDS_PER_CELL = 12.0 / 6.5e12
SECONDS_PER_CHAIN_STEP = 93e-9


def chain_lengths(T, U) -> List[int]:
    """Steps of each utterance's alpha/beta recursion (standard transducer): T + U."""
    return [int(t) + int(u) for t, u in zip(T.tolist(), U.tolist())]


def shard_time(cost: float, chain: float) -> float:
    """Modelled step time of a shard with ``cost`` cells and a longest recursion of ``chain`` steps."""
    return cost * SECONDS_PER_CELL + chain * SECONDS_PER_CHAIN_STEP


def partition_lpt(costs: Sequence[int], world: int,
                  chains: Optional[Sequence[int]] = None) -> List[List[int]]:
    """Longest-processing-time bin packing: utterances in decreasing cost order,
    each to the rank whose load stays smallest.  Returns the (sorted) index list
    per rank.

    Without ``chains`` the load of a rank is the sum of its costs.  With
    ``chains`` (``T_b + U_b`` per utterance) it is the modelled step time
    :func:`shard_time` of (sum of costs, longest chain): with a handful of
    utterances per rank the recursion of the longest one is a fixed latency no
    other work hides, so long utterances are dealt first (ties in cost broken by
    chain length) and a rank that already holds a long chain takes more cells
    than one that does not."""
    n = len(costs)
    loads = [0] * world
    tails = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    if chains is None:
        order = sorted(range(n), key=lambda i: (-costs[i], i))
    else:
        order = sorted(range(n), key=lambda i: (-shard_time(costs[i], chains[i]), -chains[i], i))
    for b in order:
        if chains is None:
            r = min(range(world), key=lambda k: (loads[k], k))
        else:
            r = min(range(world),
                    key=lambda k: (shard_time(loads[k] + costs[b], max(tails[k], chains[b])), k))
            tails[r] = max(tails[r], chains[b])
        out[r].append(b)
        loads[r] += costs[b]
    if chains is not None:
        out = _refine(out, costs, chains)
    return [sorted(ix) for ix in out]


def _refine(parts, costs, chains, rounds=200):
    """Local search on a chain-aware partition: move one utterance off the slowest
    rank, or swap it against one of another rank, while that lowers the slowest
    rank's modelled time.  The greedy deal is within a few percent of the
    optimum; with a handful of utterances per rank these few percent are a
    whole utterance."""
    parts = [list(p) for p in parts]

    def time_of(p):
        return shard_time(sum(costs[b] for b in p), max((chains[b] for b in p), default=0))

    for _ in range(rounds):
        times = [time_of(p) for p in parts]
        worst = max(range(len(parts)), key=lambda k: times[k])
        best = (times[worst], None)
        for b in parts[worst]:
            rest = [x for x in parts[worst] if x != b]
            for k, other in enumerate(parts):
                if k == worst:
                    continue
                cand = max(time_of(rest), time_of(other + [b]))       # move b to rank k
                if cand < best[0] - 1e-12:
                    best = (cand, (b, k, None))
                for c in other:                                          # swap b against c
                    cand = max(time_of(rest + [c]), time_of([x for x in other if x != c] + [b]))
                    if cand < best[0] - 1e-12:
                        best = (cand, (b, k, c))
        if best[1] is None:
            break
        b, k, c = best[1]
        parts[worst].remove(b)
        parts[k].append(b)
        if c is not None:
            parts[k].remove(c)
            parts[worst].append(c)
    return parts


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
    in the caller's buffer); "lpt" balances the cells better but permutes;
    "lpt_chain" also accounts for the longest recursion per rank (see
    :func:`partition_lpt`), the choice when a rank gets only a few utterances;
    "auto" uses contiguous unless its imbalance exceeds ``max_imbalance``."""
    costs = utterance_costs(T, U, V)
    bounds = partition_contiguous(costs, world)
    parts = [list(range(a, b)) for a, b in bounds]
    contiguous = True
    if strategy == "lpt_chain":
        chains = chain_lengths(T, U)
        parts, contiguous = partition_lpt(costs, world, chains), False
        # Shortest recursion first within a rank: the grouped schedule of the library
        # (ot_b200_loss_and_gradient_groups) starts a group's recursion as soon as its
        # rows are staged and its gradient pass as soon as the recursion ends, so the
        # first group's gradient pass is runnable while stage 1 of the later groups is
        # still streaming and the memory system never waits for a recursion.  Measured
        # on shards of the benchmark batch (step time, longest first -> shortest first):
        # 8 utterances 0.224 -> 0.212 ms, 16 utterances 0.368 -> 0.360 ms.
        parts = [sorted(p_, key=lambda b: (chains[b], b)) for p_ in parts]
    elif strategy == "lpt" or (strategy == "auto" and imbalance(costs, parts) > max_imbalance):
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
        # every overlapped NCCL all-reduce of this device runs on the same side stream ...
        torch.cuda.current_stream(loss.device).wait_stream(_side_stream(loss.device))
        # ... and every peer-memory exchange on the library's own
        from . import _lib
        with torch.cuda.device(loss.device):
            _lib.check(_lib.load().ot_b200_exchange_wait(torch.cuda.current_stream(loss.device).cuda_stream))
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
        # Persistent slots for the values the one-call all-reduce reads and writes on
        # the library's own stream (step k uses slot k % RING): nothing the caching
        # allocator could hand to someone else while the exchange is still pending.
        self._slot_mem = torch.zeros(2 * self.RING, dtype=torch.float64, device=device)
        self._slots = {}

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

    def slots(self, dtype):
        """Per step slot k % RING: (0-dim tensor the local value is written to,
        0-dim tensor the sum arrives in), views of persistent memory."""
        views = self._slots.get(dtype)
        if views is None:
            mem = self._slot_mem.view(dtype).view(2 * self.RING, -1)  # row i: the 8 bytes of slot i
            views = self._slots[dtype] = [(mem[2 * i, 0], mem[2 * i + 1, 0]) for i in range(self.RING)]
        return views[self.step % self.RING]

    def all_reduce_next(self, local, out, scale=1.0):
        """One library call: publish + gather of the next step on the library's own
        high-priority stream, which first waits for what the current stream holds
        (i.e. for ``local``).  ``local`` / ``out`` should be a pair from
        :meth:`slots`; ``out`` is defined after :func:`wait_loss`."""
        flags = self._lib.FP64 if local.dtype == torch.float64 else 0
        rc = self.lib.ot_b200_exchange_allreduce(
            local.data_ptr(), out.data_ptr(), flags, self.ptrs.data_ptr(), self.table.data_ptr(),
            self.world, self.rank, self.RING, self.step, scale, self.error.data_ptr(), self.max_wait_ns,
            torch.cuda.current_stream(self.device).cuda_stream)
        if rc:
            self._lib.check(rc)
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
        scale = 1.0 / float(global_batch) if reduction == "mean" else 1.0
        ctx.grad = None
        if logit_lengths.numel() > 0:
            call = _Call(logits.detach(), targets, logit_lengths, target_lengths, blank,
                         from_log_softmax, one_sym_per_frame,
                         share_sms=bool(overlap) and exchange is None)
            if exchange is not None:
                local, total = exchange.slots(real_dtype(logits))
            else:
                local = torch.empty((), dtype=real_dtype(logits), device=logits.device)
            if _eager_grad():
                # one library call: local loss and gradient (the 1/N of "mean" uses
                # the GLOBAL batch size, known up front); see transducer_loss.py
                if ctx.needs_input_grad[0]:
                    ctx.grad = torch.empty_like(call.logits) if call.from_log_softmax else call.logits
                call.loss_and_gradient(ctx.grad, local, loss_scale=1.0, grad_scale=scale)
            else:
                call.forward(loss_out=local, loss_scale=1.0)
        else:  # a rank without utterances still joins the collective
            call = None
            if exchange is not None:
                local, total = exchange.slots(real_dtype(logits))
                local.zero_()
            else:
                local = torch.zeros((), dtype=real_dtype(logits), device=logits.device)
        if exchange is not None:
            # peer-memory exchange: two one-warp kernels on the library's own stream, one call
            with _on_device(logits.device.index):
                exchange.all_reduce_next(local, total, scale)
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
        if ctx.grad is not None:  # computed in forward: only the upstream factor is left
            grad, ctx.grad = ctx.grad, None
            call.scale_gradient(grad, loss_grad)
            _record_trace(call)
        elif call is not None:
            data = call.logits
            grad = torch.empty_like(data) if call.from_log_softmax else data
            call.backward(grad, scale_tensor=call.upstream(loss_grad), scale_host=ctx.scale_host)
            _record_trace(call)  # diagnostic, see OT_TRACE
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
    memory on a stream of the library's own; the value is likewise defined after
    :func:`wait_loss`.  The returned tensor then lives in one of the exchange's
    ``PeerExchange.RING`` persistent slots: it is overwritten that many steps
    later (clone it to keep it longer)."""
    if global_batch is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        global_batch = int(logit_lengths.numel()) * world
    loss = _ShardedLoss.apply(logits, targets, logit_lengths, target_lengths, blank,
                              from_log_softmax, one_sym_per_frame, reduction, global_batch,
                              group, overlap, exchange)
    return loss


def sharded_loss_and_grad(logits, targets, logit_lengths, target_lengths, blank,
                          from_log_softmax, one_sym_per_frame=False, reduction="mean",
                          global_batch: Optional[int] = None, group=None,
                          exchange: Optional[PeerExchange] = None, lengths_on_host=None):
    """:func:`sharded_transducer_loss` without an autograd graph: one library call
    for this rank's loss and gradient (see ``transducer_loss_and_grad``) and one
    for the exchange of the scalar.  Returns ``(loss, grad)``: the loss of the
    WHOLE batch on every rank (defined after :func:`wait_loss` when ``exchange``
    is given) and the gradient of that loss with respect to this rank's rows
    (``logits`` itself for raw logits).  No gradient crosses ranks; the only
    coupling is the sum the reference's Python layer takes over the batch
    (transducer_loss.py:147-152 of the reference).  ``lengths_on_host``: as for
    ``transducer_loss_and_grad`` (``Shard.T`` / ``Shard.U`` are host tensors)."""
    assert reduction in ("mean", "sum")
    if global_batch is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        global_batch = int(logit_lengths.numel()) * world
    scale = 1.0 / float(global_batch) if reduction == "mean" else 1.0
    data = logits.detach() if logits.requires_grad else logits
    dtype = real_dtype(data)
    if exchange is not None:
        local, total = exchange.slots(dtype)
    else:
        local = torch.empty((), dtype=dtype, device=data.device)
    if logit_lengths.numel() > 0:
        call = _planned_call(data, targets, logit_lengths, target_lengths, blank,
                             from_log_softmax, one_sym_per_frame)
        grad = torch.empty_like(data) if from_log_softmax else data
        call.loss_and_gradient(grad, local, loss_scale=1.0, grad_scale=scale,
                               cuts=_cached_cuts(call, lengths_on_host))
        _record_trace(call)
    else:  # a rank without utterances still joins the exchange
        local.zero_()
        grad = torch.zeros_like(data)
    if exchange is not None:
        with _on_device(data.device.index):
            exchange.all_reduce_next(local, total, scale)
        return total, grad
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local, group=group)
    return (local * scale if reduction == "mean" else local), grad
