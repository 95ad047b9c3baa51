"""Batch sharding across ranks: partitioning, per-rank views of a batch, and the
scalar all-reduce, the latter with two ``gloo`` ranks on the CPU.  The local
loss of each rank comes from the CPU oracle here (the CUDA kernels need a GPU);
what is tested is everything around them."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from optimized_transducer_b200 import sharding, synthetic
from oracle import oracle as O


def test_contiguous_partition_is_optimal_on_small_inputs():
    import itertools
    rng = np.random.default_rng(0)
    for _ in range(30):
        n, world = int(rng.integers(1, 9)), int(rng.integers(1, 5))
        costs = [int(c) for c in rng.integers(1, 100, n)]
        bounds = sharding.partition_contiguous(costs, world)
        assert len(bounds) == world and bounds[0][0] == 0
        assert all(bounds[i][1] == bounds[i + 1][0] for i in range(world - 1))
        assert max(b for _, b in bounds) == n
        got = max(sum(costs[a:b]) for a, b in bounds)
        best = min(max(sum(costs[a:b]) for a, b in zip((0,) + cuts, cuts + (n,)))
                   for k in range(min(world, n))
                   for cuts in itertools.combinations(range(1, n), k)) if n > 1 else costs[0]
        assert got == best
        if n >= world:
            assert all(b > a for a, b in bounds)


def test_lpt_covers_every_utterance_once_and_balances():
    w = synthetic.CONFIGS["cfg5"]
    T, U, _ = synthetic.make_lengths(w)
    costs = sharding.utterance_costs(T, U, w.v)
    parts = sharding.partition_lpt(costs, 8)
    assert sorted(b for p in parts for b in p) == list(range(w.n))
    assert sharding.imbalance(costs, parts) < 1.05
    cont = [list(range(a, b)) for a, b in sharding.partition_contiguous(costs, 8)]
    assert sharding.imbalance(costs, cont) < 1.25


def test_chain_aware_partition_lowers_the_modelled_step_time():
    """With a handful of utterances per rank the step time is (cells streamed) +
    (the longest recursion of the rank): the chain-aware deal must cover every
    utterance once and be no slower, in that model, than the deal by cells alone."""
    for name, world in (("cfg2", 8), ("cfg2", 4), ("cfg3", 8), ("cfg5", 8)):
        w = synthetic.CONFIGS[name]
        T, U, _ = synthetic.make_lengths(w)
        costs = sharding.utterance_costs(T, U, w.v)
        chains = sharding.chain_lengths(T, U)

        def slowest(parts):
            return max(sharding.shard_time(sum(costs[b] for b in p), max(chains[b] for b in p)) for p in parts)

        plain = sharding.partition_lpt(costs, world)
        aware = sharding.partition_lpt(costs, world, chains)
        assert sorted(b for p in aware for b in p) == list(range(w.n))
        assert all(p == sorted(p) and p for p in aware)
        assert slowest(aware) <= slowest(plain) + 1e-12
    # few, unequal utterances: the rank that holds the long chain takes fewer cells
    costs, chains = [100_000_000] * 6, [1200, 200, 200, 200, 200, 200]
    parts = sharding.partition_lpt(costs, 2, chains)
    with_long = next(p for p in parts if 0 in p)
    assert len(with_long) <= 3


@pytest.mark.parametrize("strategy", ["contiguous", "lpt", "lpt_chain", "auto"])
def test_shards_tile_the_batch(strategy):
    w = synthetic.CONFIGS["cfg2"]
    T, U, tg = synthetic.make_lengths(w)
    rows = synthetic.num_rows(T, U)
    packed = torch.arange(rows, dtype=torch.float32).unsqueeze(1).repeat(1, 2)
    seen = torch.zeros(rows, dtype=torch.int32)
    owners = []
    for rank in range(4):
        s = sharding.shard_batch(T, U, tg, w.v, 4, rank, strategy)
        owners += s.indices
        assert s.targets.shape == (len(s.indices), int(s.U.max()))  # re-padded to the local max U
        assert torch.equal(s.T, T[s.indices]) and torch.equal(s.U, U[s.indices])
        for local, b in enumerate(s.indices):
            assert torch.equal(s.targets[local, :int(U[b])], tg[b, :int(U[b])])
        local_rows = sharding.slice_rows(packed, s)
        assert local_rows.shape[0] == synthetic.num_rows(s.T, s.U)
        seen[local_rows[:, 0].long()] += 1
        if s.contiguous:
            assert local_rows.data_ptr() == packed[s.row_ranges[0][0]:].data_ptr()  # a view
    assert sorted(owners) == list(range(w.n)) and bool((seen == 1).all())


def test_chain_aware_shards_put_the_shortest_recursion_first():
    """lpt_chain orders a rank's utterances by the length of their recursion
    (T + U), shortest first: the order in which the library's grouped schedule
    overlaps best."""
    w = synthetic.CONFIGS["cfg2"]
    T, U, tg = synthetic.make_lengths(w)
    for world in (2, 4, 8):
        for rank in range(world):
            s = sharding.shard_batch(T, U, tg, w.v, world, rank, "lpt_chain")
            chains = (s.T + s.U).tolist()
            assert chains == sorted(chains)


def test_group_cuts_follow_utterance_boundaries():
    """The row positions handed to ot_b200_loss_and_gradient_groups: strictly
    rising from 0 to the number of rows, every cut at the end of an utterance, at
    most four groups, one utterance per group for up to four utterances."""
    from optimized_transducer_b200.transducer_loss import MAX_GROUPS, group_cuts
    rng = np.random.default_rng(5)
    for n in (1, 2, 3, 4, 5, 9, 32):
        T = torch.from_numpy(rng.integers(1, 60, n).astype(np.int32))
        U = torch.from_numpy(rng.integers(0, 12, n).astype(np.int32))
        ends = np.cumsum(T.numpy().astype(np.int64) * (U.numpy() + 1)).tolist()
        cuts = list(group_cuts(T, U))
        assert cuts[0] == 0 and cuts[-1] == ends[-1]
        assert all(a < b for a, b in zip(cuts, cuts[1:]))
        assert set(cuts[1:]) <= set(ends)
        assert len(cuts) - 1 == min(n, MAX_GROUPS)
    # lists work as well as tensors; a first utterance that holds most rows still leaves
    # every later group an utterance
    cuts = list(group_cuts([100, 1, 1, 1, 1, 1], [0] * 6))
    assert cuts == [0, 100, 101, 102, 105]


def test_more_ranks_than_utterances():
    T = torch.tensor([5, 7], dtype=torch.int32)
    U = torch.tensor([2, 3], dtype=torch.int32)
    tg = torch.ones(2, 3, dtype=torch.int32)
    shards = [sharding.shard_batch(T, U, tg, 10, 4, r) for r in range(4)]
    assert [len(s.indices) for s in shards] == [1, 1, 0, 0]
    assert shards[3].targets.shape == (0, 0) and shards[3].cost == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = synthetic.CONFIGS["cfg1"]
        T, U, tg = synthetic.make_lengths(w)
        x = synthetic.make_logits(w, T, U).double()
        shard = sharding.shard_batch(T, U, tg, w.v, world, rank)
        local_x = sharding.slice_rows(x, shard)
        out = O.oracle_loss(local_x.numpy(), shard.targets.numpy(), shard.T.numpy(), shard.U.numpy(), 0)
        local = torch.tensor(-out["scores"].sum(), dtype=torch.float64)
        total, event = sharding.all_reduce_sum(local, overlap=True)  # CPU: no overlap, no event
        assert event is None
        q.put((rank, float(total), shard.indices))
    finally:
        dist.destroy_process_group()


def test_two_rank_loss_equals_single_rank_loss():
    """world_size 2 over gloo: the all-reduced sum of the shard losses is the
    loss of the whole batch."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w = synthetic.CONFIGS["cfg1"]
    T, U, tg = synthetic.make_lengths(w)
    x = synthetic.make_logits(w, T, U).double()
    whole = -O.oracle_loss(x.numpy(), tg.numpy(), T.numpy(), U.numpy(), 0)["scores"].sum()
    for rank, total, _ in got:
        assert abs(total - whole) <= 1e-9 * abs(whole)
    assert sorted(b for _, _, ix in got for b in ix) == list(range(w.n))


def test_single_process_all_reduce_is_identity():
    x = torch.tensor(3.5)
    y, ev = sharding.all_reduce_sum(x)
    assert ev is None and float(y) == 3.5 and y.data_ptr() != x.data_ptr()
