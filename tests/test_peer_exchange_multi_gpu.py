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
