"""Seeded synthetic batches with the shapes of the five benchmark configurations.

No dataset is involved: "LibriSpeech-shaped" means only the ranges of T (frames
after 4x subsampling), U (BPE tokens) and V (vocabulary).  Lengths and targets
come from a CPU generator, so they are identical on every machine; the logits
are drawn on the requested device.
"""
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    n: int
    t_range: tuple
    u_range: tuple
    v: int
    scale: float = 1.0
    from_log_softmax: bool = False
    one_sym_per_frame: bool = False
    reduction: str = "mean"
    seed: int = 1000


CONFIGS = {
    "cfg1": Workload("cfg1", 4, (50, 100), (10, 20), 500, reduction="mean", seed=1001),
    "cfg2": Workload("cfg2", 32, (200, 500), (20, 100), 500, scale=2.0, reduction="sum", seed=1002),
    "cfg3": Workload("cfg3", 32, (200, 500), (20, 100), 500, one_sym_per_frame=True,
                     reduction="mean", seed=1003),
    "cfg4": Workload("cfg4", 16, (100, 300), (10, 60), 5000, from_log_softmax=True,
                     reduction="mean", seed=1004),
    "cfg5": Workload("cfg5", 64, (500, 1000), (100, 200), 1024, reduction="sum", seed=1005),
}


def make_lengths(w: Workload, n=None, seed=None):
    """Returns CPU int32 tensors ``(T, U, targets)``; ``targets`` is (N, max U)
    with entries in [1, V) (blank is 0)."""
    n = w.n if n is None else n
    g = torch.Generator().manual_seed(w.seed if seed is None else seed)
    T = torch.randint(w.t_range[0], w.t_range[1] + 1, (n,), generator=g, dtype=torch.int32)
    U = torch.randint(w.u_range[0], w.u_range[1] + 1, (n,), generator=g, dtype=torch.int32)
    if w.one_sym_per_frame:
        U = torch.minimum(U, T - 1)
    targets = torch.randint(1, w.v, (n, int(U.max())), generator=g, dtype=torch.int32)
    return T, U, targets


def num_rows(T, U):
    return int((T.to(torch.int64) * (U.to(torch.int64) + 1)).sum())


def make_logits(w: Workload, T, U, device="cpu", dtype=torch.float32, seed=None):
    """Packed (sum T*(U+1), V) input: N(0,1)*scale logits, or their log-softmax
    for a ``from_log_softmax`` workload."""
    rows = num_rows(T, U)
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed((w.seed if seed is None else seed) + 7919)
    x = torch.randn(rows, w.v, generator=g, device=dev, dtype=dtype)
    if w.scale != 1.0:
        x *= w.scale
    if w.from_log_softmax:
        x = torch.log_softmax(x, dim=-1)
    return x


def make_utterance_logits(w: Workload, T, U, indices, device="cpu", dtype=torch.float32):
    """Packed logits of the utterances ``indices`` of the workload's batch, in
    that order.  Every utterance has a generator of its own, seeded by the
    workload and the utterance's index in the WHOLE batch (``T`` and ``U`` are
    the whole batch's lengths): whichever rank holds an utterance, and however
    the batch is dealt, it consists of the same numbers."""
    dev = torch.device(device)
    parts = []
    for b in indices:
        g = torch.Generator(device=dev).manual_seed(w.seed * 1000003 + 7919 + int(b))
        x = torch.randn(int(T[b]) * (int(U[b]) + 1), w.v, generator=g, device=dev, dtype=dtype)
        if w.scale != 1.0:
            x *= w.scale
        if w.from_log_softmax:
            x = torch.log_softmax(x, dim=-1)
        parts.append(x)
    return torch.cat(parts) if len(parts) != 1 else parts[0]
