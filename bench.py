"""Benchmark of the transducer-loss hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2] [--scaling strong|weak]

A step is one forward+backward of ``transducer_loss`` over one synthetic batch.
Metric: lattice cells per second, cells = sum_b T_b * (U_b + 1) * V (the lattice
has U_b + 1 columns).  Rank 0 prints ONE JSON line.

``--impl ours`` (default): the sm_100a path.  Timed region = K steps, inputs
already resident in HBM (``value``); every step consumes its own pristine logits
buffer (the backward overwrites logits in place), so the inputs of consecutive
steps never share cache lines and are far larger than L2.  ``e2e`` repeats the
measurement with the logits in pinned host memory, the host-to-device copy and
the device-to-host read of the loss inside the timed region.  ``roofline``
describes the gradient kernel, the dominant one; ``cpu_baseline`` times the
reference's CPU implementation on this box's host cores.

With ``--gpus N`` (one process per GPU, launched by torch.distributed.run) the
SAME batch is dealt to the ranks by utterance ("strong" scaling, the default):
every utterance's logits depend only on the workload and the utterance's index,
so the batch, and its loss, are the same at every N.  ``--scaling weak`` gives
every rank a batch of the workload's size instead.  The ranks' losses are summed
over peer memory (or by NCCL); after the timed region the line's ``loss_check``
compares that sum with the float64 sum of the ranks' local losses.

``--impl reference``: the reference's own CPU implementation through its own
Python layer (``oracle/_ref``: its extension built from its sources plus its
``transducer_loss.py``; else the C port in ``oracle/``), on the same workload,
with all host threads.  Under torch.distributed.run only rank 0 works.

``--record-traffic FILE``: not a measurement; reads the csv log of an ncu run of
this script (metrics dram__bytes_read.sum, dram__bytes_write.sum) and stores the
gradient kernel's DRAM bytes per lattice cell, with a hash of the kernel's
source, in ``profiles/gradient_kernel_traffic.txt``, from which ``roofline.traffic``
is taken as long as the source has not changed since.
"""
import argparse
import csv
import hashlib
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fwd+bwd loss lattice cells (sum T*(U+1)*V)/s"
UNIT = "cells/s"
HBM_FALLBACK_GBS = 6650.0
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "gradient_kernel_traffic.txt")
GRADIENT_SOURCES = [os.path.join(ROOT, "optimized_transducer_b200", "csrc", f)
                    for f in ("gradient.cu", "ot_common.cuh")]
CACHE_NOTE = "inputs larger than cache: every step reads its own pristine copy of the logits"


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


def gradient_source_hash():
    h = hashlib.sha256()
    for path in GRADIENT_SOURCES:
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def recorded_traffic_per_cell(dtype, mode_b):
    """DRAM bytes per lattice cell of one gradient-kernel launch, from the last
    recorded ncu capture, or None when there is none for this kernel variant or
    the kernel's source has changed since."""
    try:
        with open(TRAFFIC_FILE) as f:
            rec = json.load(f)
        if rec["source_sha256"] != gradient_source_hash():
            return None
        if rec["dtype"] != dtype or bool(rec["from_log_softmax"]) != bool(mode_b):
            return None
        return float(rec["dram_bytes_per_cell"])
    except Exception:
        return None


def record_traffic(args, w):
    """Parses an ncu csv log (long format: one line per launch and metric).  The
    cells a gradient launch covers follow from its grid: one block per 8 rows (a
    launch of a two-group call covers about half the batch)."""
    per_launch = {}
    with open(args.record_traffic, newline="") as f:
        rows = [r for r in csv.reader(f) if len(r) >= 15 and r[0].isdigit()]
    for r in rows:
        name, grid, metric, value = r[4], r[8], r[12], float(r[14].replace(",", ""))
        if "gradient_kernel" in name and "scale" not in name and \
                metric in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
            rec = per_launch.setdefault(r[0], {"blocks": int(grid.strip("()").split(",")[0])})
            rec[metric] = value
    full = [v for v in per_launch.values() if len(v) == 3]
    if not full:
        raise SystemExit("no gradient-kernel launch with both DRAM metrics in " + args.record_traffic)
    total_bytes = sum(v["dram__bytes_read.sum"] + v["dram__bytes_write.sum"] for v in full)
    total_cells = sum(v["blocks"] * 8 * w.v for v in full)
    rec = {
        "kernel": "gradient_logsoftmax_kernel" if w.from_log_softmax else "gradient_kernel",
        "workload": f"{w.name}" + (f", first {args.utts} utterances" if args.utts else ", whole batch"),
        "dtype": args.dtype, "from_log_softmax": w.from_log_softmax, "launches": len(full),
        "cells_per_launch": total_cells / len(full),
        "dram_bytes_per_launch": total_bytes / len(full),
        "dram_bytes_per_cell": total_bytes / total_cells,
        "source_sha256": gradient_source_hash(),
        "sources": [os.path.relpath(p, ROOT) for p in GRADIENT_SOURCES],
        "made_by": "python bench.py --record-traffic <csv log of: ncu --metrics gpu__time_duration.sum,"
                   "dram__bytes_read.sum,dram__bytes_write.sum --clock-control none --csv --log-file <csv> "
                   "python bench.py --workload %s%s --dtype %s --steps 3 --warmup 3 --no-cpu-baseline "
                   "--no-e2e --no-timeline>" % (w.name, f" --utts {args.utts}" if args.utts else "", args.dtype),
    }
    with open(TRAFFIC_FILE, "w") as f:
        json.dump(rec, f, indent=1)
        f.write("\n")
    print(json.dumps(rec))


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)
    while the timed region runs."""

    def __init__(self, index, uuid=None, period=0.001):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:  # CUDA ordinals need not equal NVML indices: prefer the UUID
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(f"GPU-{uuid}".encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def workload_description(w, n_utt, rows):
    return (f"{w.name}: N={n_utt} utterances, T in [{w.t_range[0]},{w.t_range[1]}], "
            f"U in [{w.u_range[0]},{w.u_range[1]}], V={w.v}, logits N(0,1)*{w.scale:g}, "
            f"{'one_sym_per_frame' if w.one_sym_per_frame else 'standard'}, "
            f"{'log-softmax input' if w.from_log_softmax else 'raw logits'}, "
            f"reduction={w.reduction}, rows={rows}")


def global_batch(args, w, world):
    """Lengths and targets of the whole batch (CPU tensors) and the utterances
    the benchmark uses of it."""
    from optimized_transducer_b200 import synthetic
    n_global = w.n * world if args.scaling == "weak" else w.n
    T, U, tg = synthetic.make_lengths(w, n=n_global)
    if args.utts:  # a smaller case of the same workload, for profiler captures
        n_global = min(args.utts, n_global)
        T, U = T[:n_global].contiguous(), U[:n_global].contiguous()
        tg = tg[:n_global, :int(U.max())].contiguous()
    return n_global, T, U, tg


# ---------------------------------------------------------------------------
# reference arm / CPU baseline
# ---------------------------------------------------------------------------
REFERENCE_SAMPLE_BYTES = 4 << 30  # the reference arm takes the whole batch up to this size


def cpu_reference_step_factory(w, T, U, tg, n_sample):
    """Returns (step, cells, kind, cores, description) for the reference's CPU
    implementation on the first ``n_sample`` utterances of the batch.
    ``step()`` runs one forward+backward and returns its duration in seconds."""
    import numpy as np
    import torch
    from optimized_transducer_b200 import synthetic
    from oracle import oracle as O

    n_all = int(T.numel())
    T, U = T[:n_sample].contiguous(), U[:n_sample].contiguous()
    tg = tg[:n_sample, :int(U.max())].contiguous()
    x = synthetic.make_utterance_logits(w, T, U, range(n_sample), device="cpu")
    cells = synthetic.num_rows(T, U) * w.v
    torch.set_num_threads(os.cpu_count() or 1)  # torch.distributed.run exports OMP_NUM_THREADS=1
    cores = torch.get_num_threads()
    ref_py = O.load_ref_python()
    if ref_py is not None:
        work = torch.empty_like(x)

        class Feed(torch.autograd.Function):
            """The joiner's place: hands the loss a non-leaf tensor, as the
            reference's tests do (they torch.cat their leaves), and takes its
            gradient."""

            @staticmethod
            def forward(ctx, buf, anchor):
                return buf.view(buf.shape)

            @staticmethod
            def backward(ctx, grad):
                return None, None

        anchor = torch.zeros((), requires_grad=True)

        def step():
            work.copy_(x)  # restore the input (not timed)
            t0 = time.perf_counter()
            # The reference's own Python layer over its own extension
            # (transducer_loss.py:312-442 of the reference), then backward.
            loss = ref_py.transducer_loss(
                logits=Feed.apply(work, anchor), targets=tg, logit_lengths=T, target_lengths=U,
                blank=0, reduction=w.reduction, from_log_softmax=w.from_log_softmax,
                one_sym_per_frame=w.one_sym_per_frame)
            loss.backward()
            loss.item()
            return time.perf_counter() - t0
        kind = "reference"
        note = ("the reference's transducer_loss + backward on its own CPU build; only its logsumexp is "
                "multi-threaded (ATen), the rest of the reference is one thread")
    else:
        cores = O.set_threads(os.cpu_count() or 1)
        xn, tn, Tn, Un = x.numpy(), tg.numpy(), T.numpy(), U.numpy()
        work = np.empty_like(xn)

        def step():
            np.copyto(work, xn)  # restore the input (not timed)
            t0 = time.perf_counter()
            O.oracle_loss(work, tn, Tn, Un, 0, w.from_log_softmax, w.one_sym_per_frame,
                          in_place=not w.from_log_softmax)
            return time.perf_counter() - t0
        kind = "port"
        note = "C port of the reference's algorithm with OpenMP over rows and utterances"
    what = "all" if n_sample == n_all else f"first {n_sample} of"
    desc = (f"{what} {n_all} utterances of {w.name} ({synthetic.num_rows(T, U)} rows x V={w.v}); {note}")
    return step, cells, kind, cores, desc


def reference_sample_size(args, w, T, U, requested):
    """Utterances the CPU runs take: all of them, unless the logits exceed
    REFERENCE_SAMPLE_BYTES (then the longest prefix that fits) or a count is asked for."""
    n = int(T.numel())
    if requested:
        return min(requested, n)
    per_utt = (T.to(int) * (U.to(int) + 1) * w.v * 4).tolist()
    total, k = 0, 0
    while k < n and (k == 0 or total + per_utt[k] <= REFERENCE_SAMPLE_BYTES):
        total += per_utt[k]
        k += 1
    return k


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from optimized_transducer_b200 import synthetic
    n_global, T, U, tg = global_batch(args, w, args.gpus)
    n_sample = reference_sample_size(args, w, T, U, args.ref_utts)
    step, cells, kind, cores, desc = cpu_reference_step_factory(w, T, U, tg, n_sample)
    for _ in range(args.warmup):
        step()
    dt = sum(step() for _ in range(args.steps))
    value = cells * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_description(w, n_global, synthetic.num_rows(T, U)),
                   "cache": CACHE_NOTE},
        "setup": {"device": "host CPU", "sample": desc, "threads": cores},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_cuda(args, w):
    """The reference's own CUDA kernels on this GPU (its cuda.cu / kernels.cu built
    unmodified for sm_100 by oracle/build_ref.py --cuda), through its own Python
    layer: the like-for-like GPU comparison.  Not the reference arm the driver
    runs (that is the CPU build); one GPU, device-resident inputs, CUDA events."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from optimized_transducer_b200 import synthetic
    from oracle import oracle as O
    ref_py = O.load_ref_python(cuda=True)
    if ref_py is None:
        print(json.dumps({"impl": "reference-cuda",
                          "unavailable": "oracle/_ref/_optimized_transducer_cuda is not built "
                                         "(python oracle/build_ref.py --cuda)"}), flush=True)
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n_global, T, U, tg = global_batch(args, w, 1)
    rows = synthetic.num_rows(T, U)
    if rows * w.v >= 2 ** 31:
        print(json.dumps({"impl": "reference-cuda",
                          "unavailable": "the reference's kernels index with 32-bit element offsets "
                                         "(kernels.cu:49); this batch has more than 2^31 elements"}), flush=True)
        return
    pristine = synthetic.make_utterance_logits(w, T, U, range(n_global), device=dev)
    dT, dU, dtg = T.to(dev), U.to(dev), tg.to(dev)
    total = args.steps + args.warmup
    pool = [pristine.clone() for _ in range(total)]

    class Feed(torch.autograd.Function):
        @staticmethod
        def forward(ctx, buf, anchor):
            return buf.view(buf.shape)

        @staticmethod
        def backward(ctx, grad):
            return None, None

    anchor = torch.zeros((), device=dev, requires_grad=True)

    def step(buf):
        loss = ref_py.transducer_loss(
            logits=Feed.apply(buf, anchor), targets=dtg, logit_lengths=dT, target_lengths=dU, blank=0,
            reduction=w.reduction, from_log_softmax=w.from_log_softmax,
            one_sym_per_frame=w.one_sym_per_frame)
        loss.backward()
        return loss

    it = iter(pool)
    for _ in range(args.warmup):
        step(next(it))
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step(next(it))
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / args.steps
    cells = rows * w.v
    peak, peak_kind = measured_hbm_peak()
    line = {
        "impl": "reference-cuda", "metric": METRIC, "value": cells / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_description(w, n_global, rows), "cache": CACHE_NOTE},
        "setup": {"device": "cuda:0", "what": "the reference's CUDA kernels (sm_35-era SIMT code compiled for "
                  "sm_100 with its own options, -use_fast_math included) behind its Python layer; "
                  "row ids from a stand-in for moderngpu's load_balance_search"},
        "stages": {"whole_step_frac_of_peak": (12 if not w.from_log_softmax else 4) * cells / (ms * 1e-3) / 1e9 / peak},
        "loss": float(loss.item()),
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
STAGES = ("prepare", "logprob", "lattice", "coef", "gradient")


def timeline_summary(traces):
    """From the kernels' own %globaltimer stamps, as medians over the traced steps
    (microseconds): when every stage began and ended, relative to the start of the
    step's first kernel.  A call that ran as two groups of utterances has a second
    set of stages ("b:"; a call cut into more groups "c:", "d:" as well); stages of
    that did not run show -1."""
    out = {}
    rows = [t.reshape(20, 2).tolist() for t in traces]
    unused = -1  # a "first start" slot nobody wrote still holds its initial all-ones
    for i in range(20):
        name = ("", "b:", "c:", "d:")[i // 5] + STAGES[i % 5]
        spans = [((r[i][0] - r[0][0]) / 1e3, (r[i][1] - r[0][0]) / 1e3) for r in rows
                 if r[i][0] != unused and r[i][1] > 0]
        out[name] = ([round(statistics.median(s[0] for s in spans), 1),
                      round(statistics.median(s[1] for s in spans), 1)] if spans else [-1.0, -1.0])
    out["step_span"] = round(statistics.median(
        (max(r[i][1] for i in range(20)) - r[0][0]) / 1e3 for r in rows), 1)
    return out


def run_ours(args, w):
    import torch
    import torch.distributed as dist

    import optimized_transducer_b200 as ot
    from optimized_transducer_b200 import synthetic
    from optimized_transducer_b200.transducer_loss import collect_traces

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --impl ours needs a CUDA device: the loss has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        # The scalar all-reduce shares the GPU with the (persistent, full-occupancy)
        # gradient kernel: give NCCL's stream priority so its one CTA is placed first.
        opts = dist.ProcessGroupNCCL.Options()
        opts.is_high_priority_stream = True
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
        from optimized_transducer_b200 import sharding
    exchange, collective = None, "none"
    if world > 1:
        collective = "NCCL all-reduce of the 0-dim loss on a side stream"
        if args.collective == "peer":
            try:  # plain peer stores/loads only: no multicast object is wanted
                os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
                exchange = sharding.peer_exchange()
                collective = "peer-memory exchange (two one-warp kernels, no NCCL on the data path)"
            except Exception as e:  # symmetric memory unavailable: keep NCCL, say so
                collective += f" (peer exchange unavailable: {type(e).__name__})"

    # ----- the batch (global), and this rank's shard of it
    n_global, gT, gU, gtg = global_batch(args, w, world)
    rows_global = synthetic.num_rows(gT, gU)
    if world > 1:
        shard = sharding.shard_batch(gT, gU, gtg, w.v, world, rank, strategy=args.partition)
        T, U, tg, mine = shard.T, shard.U, shard.targets, shard.indices
    elif args.shard_of:
        # one GPU runs the shard that rank R of a W-rank job would hold (no exchange):
        # what a single rank of the strong-scaling run does, without the other W-1 GPUs
        from optimized_transducer_b200 import sharding
        w_, r_ = (int(v) for v in args.shard_of.split(":"))
        shard = sharding.shard_batch(gT, gU, gtg, w.v, w_, r_, strategy=args.partition)
        T, U, tg, mine = shard.T, shard.U, shard.targets, shard.indices
    else:
        T, U, tg, mine = gT, gU, gtg, list(range(n_global))
    rows = synthetic.num_rows(T, U)
    cells_local = rows * w.v
    dT, dU, dtg = T.to(dev), U.to(dev), tg.to(dev)
    # the lengths as the data loader has them (host tensors): the library cuts its
    # groups of utterances at utterance boundaries with them (--no-host-lengths: it
    # cuts at the quantiles of the rows instead)
    host_lengths = None if args.no_host_lengths else (T, U)
    pristine = synthetic.make_utterance_logits(w, gT, gU, mine, device=dev)
    if args.dtype != "f32":  # the 16-bit extension: same values, rounded once
        pristine = pristine.to(torch.bfloat16 if args.dtype == "bf16" else torch.float16)
    bytes_logits = pristine.numel() * pristine.element_size()

    # One logits buffer per step (the backward overwrites them), so that the K timed
    # steps run back to back.  Where the device cannot hold that many (the
    # long-utterance workload on one GPU) a few buffers rotate: each is restored
    # from the pristine copy before it is used again, and the steps are timed one by
    # one so that the restoring copies stay outside the timed spans.
    total_steps = args.steps + args.warmup
    free, _ = torch.cuda.mem_get_info(dev)
    fit = int((free - (8 << 30)) // bytes_logits) - 1  # leaves room for one more clone and the workspaces
    if fit < 2:
        raise RuntimeError("the device cannot hold this rank's logits four times over")
    rotating = fit < total_steps
    if rotating:
        args.no_e2e = True  # the host-buffer run needs two more device buffers and a pinned copy
    pool = [pristine.clone() for _ in range(min(fit, total_steps))]

    class Feed(torch.autograd.Function):
        """Stands for the joiner that produces the logits in training: the loss
        sees a non-leaf tensor (as in the reference's tests, which torch.cat
        their leaves), and its gradient is handed to this node instead of being
        accumulated into a leaf by a copy that is not part of the loss path."""

        @staticmethod
        def forward(ctx, buf, anchor):
            return buf.view(buf.shape)

        @staticmethod
        def backward(ctx, grad):
            return None, None

    anchor = torch.zeros((), device=dev, requires_grad=True)

    def loss_of(x, tg_, t_, u_):
        if world > 1:
            return sharding.sharded_transducer_loss(
                x, tg_, t_, u_, blank=0, from_log_softmax=w.from_log_softmax,
                one_sym_per_frame=w.one_sym_per_frame, reduction=w.reduction,
                global_batch=n_global, overlap=True, exchange=exchange)
        return ot.transducer_loss(x, tg_, t_, u_, blank=0, from_log_softmax=w.from_log_softmax,
                                  one_sym_per_frame=w.one_sym_per_frame, reduction=w.reduction)

    def one_step(buf):
        x = Feed.apply(buf, anchor)
        return x, loss_of(x, dtg, dT, dU)

    def run_step(buf, tg_, t_, u_, api):
        """One pass of the hot path over one batch: loss AND gradient (over ``buf``
        for raw logits).  "call": the one-call entry, the shape of the reference's
        native function; "autograd": transducer_loss(...) + loss.backward()."""
        if api == "autograd":
            loss = loss_of(Feed.apply(buf, anchor), tg_, t_, u_)
            loss.backward()
            return loss
        if world > 1:
            return sharding.sharded_loss_and_grad(
                buf, tg_, t_, u_, 0, w.from_log_softmax, w.one_sym_per_frame, w.reduction,
                global_batch=n_global, exchange=exchange, lengths_on_host=host_lengths)[0]
        return ot.transducer_loss_and_grad(buf, tg_, t_, u_, 0, w.from_log_softmax,
                                           w.one_sym_per_frame, w.reduction,
                                           lengths_on_host=host_lengths)[0]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def buffers():
        used = 0
        while True:
            for buf in pool:
                if used >= len(pool):
                    buf.copy_(pristine)  # only when rotating
                used += 1
                yield buf

    # ----- warm-up
    it = buffers()
    for _ in range(args.warmup):
        run_step(next(it), dtg, dT, dU, args.api)
    barrier()

    # ----- timed region: K steps, device resident
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    uuid = getattr(torch.cuda.get_device_properties(dev), "uuid", None)
    with ClockSampler(local_rank, uuid) as clocks:
        barrier()
        host_t0 = time.perf_counter()
        t_begin.record()
        for k in range(args.steps):
            buf = next(it)
            if rotating:
                ev[k][0].record()
            loss = run_step(buf, dtg, dT, dU, args.api)
            if rotating:
                ev[k][1].record()
        if world > 1:
            sharding.wait_loss(loss)  # the last step's exchange ends inside the timed region
        t_end.record()
        host_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps  # host time to ENQUEUE a step
        barrier()
    elapsed_ms = (sum(e[0].elapsed_time(e[1]) for e in ev) if rotating
                  else t_begin.elapsed_time(t_end))
    ot.check_inputs(dev)  # a failed device-side check in any step raises here
    last_loss = float(loss.item())

    # ----- the same K steps through the autograd surface (transducer_loss +
    #       loss.backward()), for the record: forward / backward split and what the
    #       autograd graph costs per step.  Not the headline when --api call.
    for b_ in pool:
        b_.copy_(pristine)
    it = buffers()
    for _ in range(min(args.warmup, 3)):
        run_step(next(it), dtg, dT, dU, "autograd")
    barrier()
    n_auto = min(args.steps, len(pool) - min(args.warmup, 3)) if not rotating else args.steps
    ev3 = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_auto)]
    for k in range(n_auto):
        buf = next(it)
        ev3[k][0].record()
        x, loss = one_step(buf)
        ev3[k][1].record()
        loss.backward()
        ev3[k][2].record()
    if world > 1:
        sharding.wait_loss(loss)
    barrier()
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev3)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev3)
    autograd_ms = (sum(e[0].elapsed_time(e[2]) for e in ev3) if rotating
                   else ev3[0][0].elapsed_time(ev3[-1][2])) / n_auto
    ot.check_inputs(dev)

    # ----- for the record: the same step with TWO independent batches in flight (two
    #       CUDA streams taking turns, as the micro-batches of a gradient-accumulation
    #       loop can): the recursion of one batch then runs beside the streaming
    #       kernels of the other.  Not the headline: `value` is one batch at a time.
    inflight_ms = 0.0
    if not rotating and args.api == "call" and len(pool) >= 8:
        for b_ in pool:
            b_.copy_(pristine)
        it = buffers()
        main = torch.cuda.current_stream(dev)
        lanes = [torch.cuda.Stream(device=dev) for _ in range(2)]
        for s_ in lanes:
            s_.wait_stream(main)
        for k in range(4):  # two warm-up steps per stream (plans, workspaces)
            with torch.cuda.stream(lanes[k % 2]):
                loss = run_step(next(it), dtg, dT, dU, "call")
        for s_ in lanes:
            main.wait_stream(s_)
        barrier()
        n2 = min(args.steps, len(pool) - 4)
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for s_ in lanes:
            s_.wait_stream(main)
        for k in range(n2):
            with torch.cuda.stream(lanes[k % 2]):
                loss = run_step(next(it), dtg, dT, dU, "call")
        for s_ in lanes:
            main.wait_stream(s_)
        if world > 1:
            sharding.wait_loss(loss)
        f1.record()
        barrier()
        inflight_ms = f0.elapsed_time(f1) / n2
        ot.check_inputs(dev)
    kbufs = pool[:2] if rotating else None
    del pool, it, x, loss, buf

    # ----- the dominant kernel by itself: CUDA events around each launch of the
    #       gradient pass, on the stream it is launched on, directly behind the
    #       forward kernels of the same step (as it runs inside a step; in the
    #       default schedule the pass overlaps other stages and has no span of its own)
    from optimized_transducer_b200.transducer_loss import _Call
    if kbufs is None:
        kbufs = [pristine.clone() for _ in range(2)]
    kout = torch.empty_like(pristine) if w.from_log_softmax else None
    kev = []
    for k in range(args.steps + 3):
        kb = kbufs[k % 2]
        kb.copy_(pristine)
        call = _Call(kb, dtg, dT, dU, 0, w.from_log_softmax, w.one_sym_per_frame, checks="off")
        call.forward()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        call.backward(kb if kout is None else kout)
        k1.record()
        kev.append((k0, k1))
    torch.cuda.synchronize(dev)
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in kev[3:])
    del kbufs, kout, kev, call

    # ----- the exchanged loss against the sum of the ranks' own losses, and a
    #       stage timeline of a few extra steps (neither is timed)
    loss_check, timeline = None, None
    if world > 1:
        buf = pristine.clone()
        total = run_step(buf, dtg, dT, dU, args.api)
        sharding.wait_loss(total)
        local = ot.transducer_loss(Feed.apply(pristine.clone(), anchor), dtg, dT, dU, blank=0,
                                   from_log_softmax=w.from_log_softmax,
                                   one_sym_per_frame=w.one_sym_per_frame, reduction="sum")
        mine_sum = torch.tensor([float(local.item())], dtype=torch.float64, device=dev)
        gathered = [torch.empty_like(mine_sum) for _ in range(world)]
        dist.all_gather(gathered, mine_sum)
        want = sum(float(g.item()) for g in gathered)  # float64, rank order, on the host
        if w.reduction == "mean":
            want /= n_global
        got = float(total.item())
        rel = abs(got - want) / max(abs(want), 1e-30)
        loss_check = {"exchanged": got, "sum_of_locals": want, "rel": rel}
        del buf, total, local
    if not args.no_timeline:
        os.environ["OT_TRACE"] = "1"
        traces = []
        collect_traces(traces)
        for _ in range(5):
            loss = run_step(pristine.clone(), dtg, dT, dU, args.api)
        torch.cuda.synchronize(dev)
        os.environ["OT_TRACE"] = "0"
        collect_traces(None)
        timeline = timeline_summary([t.cpu().numpy() for t in traces])
        del loss

    # ----- end to end: logits start in pinned host memory
    host = torch.empty(pristine.shape, dtype=pristine.dtype, pin_memory=True)
    host.copy_(pristine)
    hT, hU, htg = T.pin_memory(), U.pin_memory(), tg.pin_memory()
    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 10))
    # Double-buffered input pipeline, as a training loop would run it: the copy of
    # step k+1's inputs (own stream) overlaps step k's kernels.  Every step's
    # inputs cross PCIe inside the timed region, every step's loss is read back.
    main_stream = torch.cuda.current_stream(dev)
    copy_stream = torch.cuda.Stream(device=dev)
    dev_bufs = [torch.empty_like(pristine) for _ in range(2)]
    staged = [None, None]
    ready = [torch.cuda.Event() for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(2)]

    def e2e_prefetch(k):
        slot = k % 2
        copy_stream.wait_event(done[slot])  # the step that last used this buffer has finished with it
        with torch.cuda.stream(copy_stream):
            dev_bufs[slot].copy_(host, non_blocking=True)
            staged[slot] = (hT.to(dev, non_blocking=True), hU.to(dev, non_blocking=True),
                            htg.to(dev, non_blocking=True))
            ready[slot].record(copy_stream)

    def e2e_step(k, last):
        slot = k % 2
        if not last:
            e2e_prefetch(k + 1)
        main_stream.wait_event(ready[slot])
        t_, u_, g_ = staged[slot]
        for t in (dev_bufs[slot], t_, u_, g_):
            t.record_stream(main_stream)
        loss = run_step(dev_bufs[slot], g_, t_, u_, args.api)
        done[slot].record(main_stream)
        if world > 1:
            sharding.wait_loss(loss)
        return float(loss.item())  # device-to-host read of the result

    e2e_ms = 0.0
    if e2e_steps:
        for s_ in range(2):
            done[s_].record(main_stream)
        e2e_prefetch(0)
        e2e_step(0, True)  # warm-up
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_prefetch(0)   # the first step's copy is inside the timed region too
        for k in range(e2e_steps):
            e2e_step(k, k + 1 == e2e_steps)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # ----- max over ranks, whole-job totals
    stats = torch.tensor([elapsed_ms, e2e_ms, fwd_ms, bwd_ms, host_ms, kernel_ms, autograd_ms, inflight_ms], dtype=torch.float64, device=dev)
    cells = torch.tensor([float(cells_local)], dtype=torch.float64, device=dev)
    per_rank = None
    if world > 1:
        # every rank's own figures, for the record (the line reports the max)
        cols = ["ms_per_step", "forward_ms", "backward_ms", "host_enqueue_ms", "rows", "utterances",
                "longest_T_plus_U"]
        vals = [elapsed_ms / args.steps, fwd_ms, bwd_ms, host_ms, float(rows), float(T.numel()),
                float(int((T + U).max()))]
        if timeline is not None:
            for k, v in timeline.items():
                if isinstance(v, list):
                    cols += [f"us_{k}_begin", f"us_{k}_end"]
                    vals += [float(v[0]), float(v[1])]
                else:
                    cols.append("us_" + k)
                    vals.append(float(v))
        mine_t = torch.tensor(vals, dtype=torch.float64, device=dev)
        gathered = [torch.empty_like(mine_t) for _ in range(world)]
        dist.all_gather(gathered, mine_t)
        per_rank = {"columns": cols, "values": [[round(v, 4) for v in g.tolist()] for g in gathered]}
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(cells, op=dist.ReduceOp.SUM)
    elapsed_ms, e2e_ms, fwd_ms, bwd_ms, host_ms, kernel_ms, autograd_ms, inflight_ms = stats.tolist()
    cells_total = cells.item()

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        es = pristine.element_size()
        mode_b = w.from_log_softmax
        # Gradient kernel, per launch: read + in-place write of the local logits
        # (mode A), or the dense gradient write (mode B).
        grad_bytes = (1 if mode_b else 2) * es * cells_local
        achieved = grad_bytes / (kernel_ms * 1e-3) / 1e9
        eager = os.environ.get("OT_EAGER_GRAD", "1") != "0"
        two_groups = (eager and not mode_b and T.numel() >= 2 and cells_local >= (192 << 20)
                      and os.environ.get("OT_B200_PIPELINE", "1") != "0")
        # own kernels per step and rank: prepare, logprob, lattice, coef, gradient (twice
        # the last four + one closing kernel when the batch runs as two groups), the
        # scaling kernel of the eager schedule's backward, publish + gather of the exchange
        one_call = args.api == "call"
        # below the two-group size the one-call schedule chains up to four groups (one
        # utterance each with the lengths on the host): per group logprob, lattice,
        # coef, gradient, plus prepare and the closing kernel
        pipeline_on = os.environ.get("OT_B200_PIPELINE", "1") != "0"
        chained = 0
        if (eager and not mode_b and not two_groups and pipeline_on and T.numel() >= 2
                and cells_local >= (64 << 20) and rows >= 64):
            chained = min(4, int(T.numel()))
        launches = ((10 if two_groups else (2 + 4 * chained if chained >= 2 else 5))
                    + (1 if eager and not one_call else 0) + (2 if exchange is not None else 0))
        fwd_bytes = (0 if mode_b else es * cells_local)
        value = cells_total * args.steps / (elapsed_ms * 1e-3)
        per_cell = recorded_traffic_per_cell(args.dtype, mode_b)
        step_ms = elapsed_ms / args.steps
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f32" if args.dtype == "f32" else f"{args.dtype} logits and gradient, f32 arithmetic",
            "data": "synthetic",
            "config": {
                "workload": workload_description(w, n_global, rows_global)
                            + ("" if args.dtype == "f32" else f", logits stored as {args.dtype}"),
                "cache": CACHE_NOTE,
            },
            "setup": {
                "timed_region": ("the K steps one by one (CUDA events around each; a few logits buffers "
                                 "rotate and are restored between the steps)") if rotating else
                                "the K steps back to back, one pair of CUDA events",
                "sharding": "none" if world == 1 else
                            f"{world} ranks, whole utterances of the one batch ({args.partition} partition)"
                            if args.scaling == "strong" else
                            f"{world} ranks, {w.n} utterances per rank ({args.partition} partition)",
                "collective": collective,
                "checks": {"0": "off", "2": "strict (the call waits)"}.get(
                    os.environ.get("OT_CHECKS", "1"), "deferred (reported by a later call)"),
                "api": ("transducer_loss_and_grad: loss and in-place gradient from one call, no autograd graph "
                        "(the shape of the reference's native compute_transducer_loss, which returns scores "
                        "and gradient together)") if one_call else
                       "transducer_loss(...) + loss.backward() through torch.autograd",
                "autograd_api_ms_per_step": autograd_ms,
                "two_batches_in_flight_ms_per_step": inflight_ms if inflight_ms > 0 else None,
                "gradient_schedule": "eager (loss and gradient in one library call, as the reference)" if one_call else
                                     ("deferred (one fused pass in backward)"
                                      if os.environ.get("OT_EAGER_GRAD", "1") == "0" else
                                      "eager (loss and gradient in one library call, as the reference; "
                                      "backward only scales, and skips that when the upstream gradient is 1)"),
                "stage_overlap": ("off (OT_B200_PIPELINE=0)" if os.environ.get("OT_B200_PIPELINE", "1") == "0"
                                  else "two groups of utterances on three streams when a rank holds >= 192 Mi lattice cells "
                                       "(768 MB of float logits); below that up to four chained groups, each on streams of "
                                       "its own behind its part of stage 1" + (f" (here: {chained})" if chained >= 2 else "")),
                "host_enqueue_ms_per_step": host_ms,
            },
            "clocks": clocks.summary(),
            "e2e": None if not e2e_steps else {"value": cells_total / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": bytes_logits + 4 * (T.numel() + U.numel() + tg.numel()),
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": launches * args.steps,
            "roofline": {
                "kernel": "gradient_logsoftmax_kernel" if mode_b else "gradient_kernel",
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth",
                "traffic": None if per_cell is None else per_cell * cells_local,
                "bytes_per_launch": grad_bytes, "ms_per_launch": kernel_ms,
                "timing": "CUDA events around each launch of the kernel alone, behind the forward kernels "
                          "of the same batch (in the timed steps it overlaps other stages)",
            },
            "stages": {
                "measured_through": "transducer_loss + loss.backward() (CUDA events between them)",
                "forward_ms": fwd_ms, "backward_ms": bwd_ms,
                "forward_gbs": (fwd_bytes / (fwd_ms * 1e-3) / 1e9) if fwd_bytes else None,
                "whole_step_gbs": (fwd_bytes + grad_bytes) / (step_ms * 1e-3) / 1e9,
                "whole_step_frac_of_peak": (fwd_bytes + grad_bytes) / (step_ms * 1e-3) / 1e9 / peak,
            },
            "loss": last_loss,
        }
        if timeline is not None:  # unused later sets are left out of the line
            line["timeline_us"] = {k: v for k, v in timeline.items()
                                   if not (k[1:2] == ":" and v == [-1.0, -1.0])}
        if per_rank is not None:
            line["per_rank"] = per_rank
        if loss_check is not None:
            line["loss_check"] = loss_check
        if world == 1 and not args.no_cpu_baseline:
            n_sample = reference_sample_size(args, w, gT, gU, args.cpu_utts)
            step, c_cells, kind, cores, desc = cpu_reference_step_factory(w, gT, gU, gtg, n_sample)
            step()
            t0 = time.perf_counter()
            reps, spent = 0, 0.0
            while reps < 2 or (time.perf_counter() - t0 < 10.0 and reps < 20):
                spent += step()
                reps += 1
            dt = spent / reps
            line["cpu_baseline"] = {"value": c_cells / dt, "unit": UNIT, "cores": cores, "kind": kind,
                                    "sample": desc + f"; {reps} repetitions"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if loss_check is not None and loss_check["rel"] > 1e-6:
        raise SystemExit(f"loss check failed on rank {rank}: {loss_check}")


def run_pack(args, w):
    """Measurement of the packing helpers (callers' side of the packed layout) on
    the workload's shapes with D = 512 features: forward = one pass that writes
    rows*D*4 bytes, backward = both sums from one read of them (two reads for small batches)."""
    import torch
    from optimized_transducer_b200 import packing, synthetic

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    d = 512
    T, U, _ = synthetic.make_lengths(w)
    if args.utts:  # a smaller case of the same workload, for profiler captures
        T, U = T[:args.utts].contiguous(), U[:args.utts].contiguous()
    n_utt = int(T.numel())
    rows = synthetic.num_rows(T, U)
    dT, dU = T.to(dev), U.to(dev)
    enc = torch.randn(n_utt, int(T.max()), d, device=dev, requires_grad=True)
    dec = torch.randn(n_utt, int(U.max()) + 1, d, device=dev, requires_grad=True)
    g = torch.randn(rows, d, device=dev)
    # No synchronisation between iterations: the host runs ahead of the device, so
    # the events bracket kernel time, not the host's launch latency.
    n_it = args.warmup + args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_it)]
    for it in range(n_it):
        ev[it][0].record()
        x = packing.pack_joiner_input(enc, dec, dT, dU, rows=rows)
        ev[it][1].record()
        x.backward(g)
        ev[it][2].record()
        del x
        enc.grad = dec.grad = None
    torch.cuda.synchronize()
    fwd = [ev[it][0].elapsed_time(ev[it][1]) for it in range(args.warmup, n_it)]
    bwd = [ev[it][1].elapsed_time(ev[it][2]) for it in range(args.warmup, n_it)]
    peak, peak_kind = measured_hbm_peak()
    f_ms, b_ms = statistics.median(fwd), statistics.median(bwd)
    bytes_out = rows * d * 4
    # the library's own choice (pack.cu): one read needs U + 1 <= 128 and two device-fills of CTAs
    two_reads = (os.environ.get("OT_B200_PACK_SUM") == "two" or int(U.max()) + 1 > 128
                 or n_utt * ((d // 4 + 7) // 8) < 2 * torch.cuda.get_device_properties(dev).multi_processor_count)
    line = {
        "metric": "packed joiner-input elements (rows*D)/s, forward", "value": rows * d / (f_ms * 1e-3),
        "unit": "elements/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": f_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"pack_joiner_input on {w.name} lengths, D={d}, rows={rows}"},
        "roofline": {"kernel": "pack_add_frames_kernel", "bound": "hbm", "achieved": bytes_out / (f_ms * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s", "frac": bytes_out / (f_ms * 1e-3) / 1e9 / peak,
                     "peak_source": f"{peak_kind} copy bandwidth", "traffic": None},
        "backward": {"ms": b_ms,
                     "kernels": "prepare + pack_sum_kernel x2, two reads of the gradient (OT_B200_PACK_SUM=two)"
                     if two_reads else "prepare + pack_sum_slab_kernel: both sums from one read of the gradient",
                     "achieved_gbs": (2 if two_reads else 1) * bytes_out / (b_ms * 1e-3) / 1e9,
                     "frac_of_peak_one_read": bytes_out / (b_ms * 1e-3) / 1e9 / peak},
        "gpu_launches": (5 if two_reads else 4) * args.steps,  # forward: prepare + add; backward: prepare + sums
    }
    print(json.dumps(line), flush=True)


def run_fused(args, w):
    """The forward half computed from the joiner's operands (no logits): D = 512
    bfloat16 features on the workload's lengths, weight (V, 512).  The bound of the
    fused kernel is the tensor pipe: 2*rows*D*V flops against the measured dense
    bfloat16 peak."""
    import torch
    import optimized_transducer_b200 as ot
    from optimized_transducer_b200 import synthetic

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    d = 512
    T, U, tg = synthetic.make_lengths(w)
    if args.utts:
        n = min(args.utts, w.n)
        T, U = T[:n].contiguous(), U[:n].contiguous()
        tg = tg[:n, :int(U.max())].contiguous()
    rows = synthetic.num_rows(T, U)
    g = torch.Generator(device=dev).manual_seed(w.seed)
    x = torch.randn(rows, d, device=dev, generator=g).to(torch.bfloat16)
    wt = (torch.randn(w.v, d, device=dev, generator=g) * (w.scale / d ** 0.5)).to(torch.bfloat16)
    bias = torch.zeros(w.v, device=dev)
    dT, dU, dtg = T.to(dev), U.to(dev), tg.to(dev)
    os.environ["OT_TRACE"] = "1"
    os.environ.setdefault("OT_CHECKS", "0")
    n_it = args.warmup + args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(n_it)]
    spans = []
    for it in range(n_it):
        ev[it][0].record()
        out = ot.joiner_scores(x, wt, bias, dtg, dT, dU, 0, stages=False, reduction="sum", _trace=spans)
        ev[it][1].record()
    torch.cuda.synchronize()
    ms = statistics.median(ev[it][0].elapsed_time(ev[it][1]) for it in range(args.warmup, n_it))
    k_us = statistics.median((int(t[3]) - int(t[2])) / 1e3 for t in (s.cpu() for s in spans[args.warmup:]))
    # forward + backward without logits (joiner_loss): the library recomputes the logits
    # tile in backward and writes the bfloat16 gradient with respect to the logits; the
    # three contractions with it are PyTorch matmuls
    from optimized_transducer_b200.transducer_loss import collect_traces
    xa, wa, ba = (t.clone().requires_grad_(True) for t in (x, wt, bias))
    ev3 = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_it)]
    bspans = []
    collect_traces(bspans)
    for it in range(n_it):
        xa.grad = wa.grad = ba.grad = None
        ev3[it][0].record()
        jl = ot.joiner_loss(xa, wa, ba, dtg, dT, dU, 0, reduction="sum")
        ev3[it][1].record()
        jl.backward()
        ev3[it][2].record()
    torch.cuda.synchronize()
    collect_traces(None)
    jf_ms = statistics.median(ev3[it][0].elapsed_time(ev3[it][1]) for it in range(args.warmup, n_it))
    jb_ms = statistics.median(ev3[it][1].elapsed_time(ev3[it][2]) for it in range(args.warmup, n_it))
    g_us = statistics.median((int(t[9]) - int(t[8])) / 1e3 for t in (s_.cpu() for s_ in bspans[args.warmup:]))
    # the same loss with the logits materialised in bfloat16 (projection by the library
    # GEMM, the 16-bit transducer loss of this package, autograd through both): what
    # joiner_loss is an alternative to
    from optimized_transducer_b200.transducer_loss import _padded_columns

    def materialised(wt_, bias_):
        xm, wm, bm = (t.clone().requires_grad_(True) for t in (x, wt_, bias_))
        evm = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_it)]
        for it in range(n_it):
            xm.grad = wm.grad = bm.grad = None
            evm[it][0].record()
            ml = ot.transducer_loss(torch.nn.functional.linear(xm, wm, bm.to(torch.bfloat16)), dtg, dT, dU, 0,
                                    False, reduction="sum")
            evm[it][1].record()
            ml.backward()
            evm[it][2].record()
        torch.cuda.synchronize()
        return {"forward_ms": statistics.median(evm[it][0].elapsed_time(evm[it][1]) for it in range(args.warmup, n_it)),
                "backward_ms": statistics.median(evm[it][1].elapsed_time(evm[it][2]) for it in range(args.warmup, n_it)),
                "loss": float(ml.item())}

    mat = materialised(wt, bias)
    mat["what"] = ("the same loss and gradients through torch.nn.functional.linear -> (rows, V) bfloat16 logits "
                   "-> transducer_loss -> autograd (library GEMMs on both sides)")
    vp = _padded_columns(w.v)
    mat_padded = None
    if vp != w.v:
        # a model whose vocabulary is padded so that rows of logits are a multiple of 16
        # bytes (zero weight rows, a bias of -1e30: the same loss): the library GEMMs of
        # the materialised path stay on their tensor-core kernels
        wp = torch.zeros((vp, d), dtype=wt.dtype, device=dev)
        wp[:w.v] = wt
        bp = torch.full((vp,), -1e30, dtype=torch.float32, device=dev)
        bp[:w.v] = bias
        mat_padded = materialised(wp, bp)
        mat_padded["what"] = f"the same with the vocabulary padded from {w.v} to {vp} entries by the caller"
    from optimized_transducer_b200.transducer_loss import _padded_columns
    flops = 2.0 * rows * d * w.v
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, kind = float(json.load(f)["bf16_tflops"]), "measured (burst)"
    except Exception:
        peak, kind = 1590.0, "fallback"
    line = {
        "metric": "lattice rows/s of the logits-free forward half (projection + logsumexp + recursions)",
        "value": rows / (ms * 1e-3), "unit": "rows/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 operands, f32 accumulators", "data": "synthetic",
        "config": {"workload": f"joiner_scores on {w.name} lengths: rows={rows}, D={d}, V={w.v}"},
        "roofline": {"kernel": "linear_logprob_kernel", "bound": "tensor", "achieved": flops / (k_us * 1e-6) / 1e12,
                     "peak": peak, "unit": "TFLOP/s", "frac": flops / (k_us * 1e-6) / 1e12 / peak,
                     "peak_source": f"{kind} dense bf16 GEMM", "traffic": None,
                     "us_per_launch": k_us, "timing": "the kernel's own %globaltimer span (first block start to last block end)"},
        "bytes_never_written": rows * w.v * 4,
        "joiner_loss": {
            "what": "forward + backward from the joiner's operands, no float logits: forward as above; backward = "
                    "linear_gradient_kernel (logits tile recomputed on the tensor cores, bfloat16 gradient "
                    "with respect to the logits written) + three PyTorch contractions with that tile",
            "forward_ms": jf_ms, "backward_ms": jb_ms,
            "linear_gradient_kernel_us": g_us,
            "linear_gradient_kernel_tflops": flops / (g_us * 1e-6) / 1e12,
            "linear_gradient_kernel_frac_of_peak": flops / (g_us * 1e-6) / 1e12 / peak,
            "gradient_bytes_written": rows * _padded_columns(w.v) * 2,
            "materialised_bf16_logits": mat,
            "materialised_bf16_logits_padded_vocabulary": mat_padded,
        },
        "gpu_launches": 4 * args.steps,
        "loss": float(out.item()),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference", "reference-cuda"], default="ours",
                    help="ours: the sm_100a path; reference: the reference's CPU implementation (the arm "
                         "the driver compares with); reference-cuda: the reference's own CUDA kernels on "
                         "this GPU (an extra, like-for-like comparison)")
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong",
                    help="strong (default): the workload's one batch is dealt to the ranks; "
                         "weak: every rank gets a batch of the workload's size")
    ap.add_argument("--dtype", choices=["f32", "bf16", "f16"], default="f32",
                    help="storage type of the logits (the reference's is f32; 16-bit is an extension)")
    ap.add_argument("--collective", choices=["peer", "nccl"], default="peer",
                    help="how the ranks' losses are summed: over peer memory (default) or by NCCL")
    ap.add_argument("--api", choices=["call", "autograd"], default="call",
                    help="the timed step: 'call' = transducer_loss_and_grad (one call, loss + in-place gradient, "
                         "no autograd graph); 'autograd' = transducer_loss(...) + loss.backward().  The other "
                         "one is measured too and reported under setup / stages")
    ap.add_argument("--shard-of", default="", metavar="W:R",
                    help="diagnostic, one GPU: run the shard rank R of a W-rank job would hold")
    ap.add_argument("--no-host-lengths", action="store_true",
                    help="do not hand the host copies of the lengths to the one-call entry")
    ap.add_argument("--partition", choices=["auto", "contiguous", "lpt", "lpt_chain"], default="lpt_chain",
                    help="how utterances are dealt to the ranks (each rank creates its own shard, so a "
                         "permuting partition costs nothing here); lpt_chain balances cells and the "
                         "longest recursion per rank")
    ap.add_argument("--ref-utts", type=int, default=0,
                    help="utterances per step of the reference arm (0: the whole batch, up to 4 GB of logits)")
    ap.add_argument("--cpu-utts", type=int, default=0,
                    help="utterances of the CPU-baseline sample of our arm (0: as --ref-utts 0)")
    ap.add_argument("--op", choices=["loss", "pack", "fused"], default="loss",
                    help="loss: the transducer loss (default, the benchmark); pack: the packing helpers; "
                         "fused: the logits-free forward half (projection fused with the logsumexp)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer measurement")
    ap.add_argument("--no-timeline", action="store_true", help="skip the traced extra steps")
    ap.add_argument("--utts", type=int, default=0,
                    help="use only the first UTTS utterances (small case for profiler captures)")
    ap.add_argument("--record-traffic", default="",
                    help="csv log of an ncu run of this script: store the gradient kernel's DRAM traffic")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    from optimized_transducer_b200 import synthetic
    w = synthetic.CONFIGS[args.workload]
    if args.record_traffic:
        record_traffic(args, w)
    elif args.op == "pack":
        run_pack(args, w)
    elif args.op == "fused":
        run_fused(args, w)
    elif args.impl == "reference":
        run_reference_arm(args, w)
    elif args.impl == "reference-cuda":
        run_reference_cuda(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
