"""The sharded loss with the peer-memory exchange on real peers: two processes,
one GPU each (needs two GPUs of one node; skipped otherwise)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from optimized_transducer_b200 import sharding, synthetic
        w = synthetic.CONFIGS["cfg1"]
        T, U, tg = synthetic.make_lengths(w)
        x = synthetic.make_logits(w, T, U)
        shard = sharding.shard_batch(T, U, tg, w.v, world, rank)
        local_x = sharding.slice_rows(x, shard).to(dev)
        args = (shard.targets.to(dev), shard.T.to(dev), shard.U.to(dev))
        ex = sharding.peer_exchange()
        out = {}
        for name, kw in (("nccl", {}), ("peer", {"exchange": ex})):
            for step in range(3):  # several steps: the sequence numbers advance
                leaf = local_x.clone().requires_grad_(True)
                loss = sharding.sharded_transducer_loss(leaf * 1.0, *args, blank=0, from_log_softmax=False,
                                                        reduction="mean", global_batch=w.n, overlap=True, **kw)
                loss.backward()
                sharding.wait_loss(loss)
            out[name] = (float(loss.item()), leaf.grad.cpu().numpy())
        ex.check()
        q.put((rank, out["nccl"][0], out["peer"][0], float(np.abs(out["nccl"][1] - out["peer"][1]).max())))
    finally:
        dist.destroy_process_group()


def test_peer_exchange_equals_nccl_all_reduce_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, nccl, peer, graddiff in got:
        assert peer == pytest.approx(nccl, rel=1e-6)
        assert graddiff == 0.0
    assert got[0][2] == got[1][2]  # the same bits on both ranks


def _sweep_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import optimized_transducer_b200 as ot
        from optimized_transducer_b200 import sharding
        ex = sharding.peer_exchange()
        rng = np.random.default_rng(5)  # the same batches on both ranks
        worst_loss, grad_mismatches, cases = 0.0, 0, 0
        for case in range(24):
            n = int(rng.integers(1, 11))  # n = 1: one rank has no utterance and still joins the exchange
            tmax, umax = int(rng.choice([3, 30, 150])), int(rng.choice([0, 4, 40]))
            v = int(rng.choice([37, 260, 500, 513]))
            from_ls, modified = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
            red = str(rng.choice(["mean", "sum"]))
            kind = str(rng.choice(["nccl", "peer"]))
            strategy = str(rng.choice(["auto", "contiguous", "lpt"]))
            T = rng.integers(1, tmax + 1, n).astype(np.int32)
            U = rng.integers(0, umax + 1, n).astype(np.int32)
            if modified:
                U = np.minimum(U, T - 1).astype(np.int32)
            rows = int((T.astype(np.int64) * (U + 1)).sum())
            x = torch.from_numpy((rng.standard_normal((rows, v)) * 2).astype(np.float32))
            if from_ls:
                x = x.log_softmax(-1)
            tg = torch.from_numpy(rng.integers(1, v, (n, max(int(U.max()), 0))).astype(np.int32))
            Tt, Ut = torch.from_numpy(T), torch.from_numpy(U)
            whole_loss, whole_grad = ot.transducer_loss_and_grad(x.to(dev), tg.to(dev), Tt.to(dev), Ut.to(dev), 0,
                                                                 from_ls, modified, red)
            shard = sharding.shard_batch(Tt, Ut, tg, v, world, rank, strategy=strategy)
            local = sharding.slice_rows(x, shard).to(dev)
            loss, grad = sharding.sharded_loss_and_grad(
                local, shard.targets.to(dev), shard.T.to(dev), shard.U.to(dev), 0, from_ls, modified, red,
                global_batch=n, exchange=ex if kind == "peer" else None, lengths_on_host=(shard.T, shard.U))
            if kind == "peer":
                sharding.wait_loss(loss)
            torch.cuda.synchronize()
            worst_loss = max(worst_loss, abs(loss.item() - whole_loss.item()) / max(1.0, abs(whole_loss.item())))
            want = torch.cat([whole_grad[a:b] for a, b in shard.row_ranges]) if shard.row_ranges else whole_grad[:0]
            grad_mismatches += int(want.shape != grad.shape or (want.numel() > 0 and not torch.equal(want, grad)))
            cases += 1
        ex.check()
        ot.check_inputs(dev)
        q.put((rank, cases, worst_loss, grad_mismatches))
    finally:
        dist.destroy_process_group()


def test_sharded_entry_point_on_random_batches_equals_the_whole_batch():
    """24 seeded random batches (1-10 utterances, so a rank may own none; both
    input kinds and recursions; both reductions; NCCL and the peer-memory exchange;
    every partition strategy) on two GPUs: the exchanged loss is the whole batch's to
    2e-6, and a rank's gradient carries the bits of its rows of the whole batch's
    gradient computed on one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sweep_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, cases, worst_loss, grad_mismatches in got:
        assert cases == 24 and worst_loss <= 2e-6 and grad_mismatches == 0, (rank, cases, worst_loss, grad_mismatches)
