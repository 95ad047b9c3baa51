"""Benchmark of the transducer-loss hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2] [--scaling weak|strong]

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
reference's CPU implementation on this box's host cores on a bounded sample.

``--impl reference``: the reference's CPU implementation alone (its own build
from ``oracle/_ref`` when present, else the C port in ``oracle/``), each step a
bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one full-size cfg2 launch of the
# gradient kernel, from the one-pass ncu capture summarised in profiles/gradient_kernel_cfg2.md.
CFG2_GRADIENT_TRAFFIC_BYTES = 2706.0e6
CFG2_ROWS = 686128

METRIC = "fwd+bwd loss lattice cells (sum T*(U+1)*V)/s"
UNIT = "cells/s"
HBM_FALLBACK_GBS = 6650.0


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


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


# ---------------------------------------------------------------------------
# reference arm / CPU baseline
# ---------------------------------------------------------------------------
def cpu_reference_step_factory(w, n_sample):
    """Returns (step, cells, kind, cores, description) for the reference's CPU
    implementation on the first ``n_sample`` utterances of the workload.
    ``step()`` runs one forward+backward and returns its duration in seconds."""
    import numpy as np
    import torch
    from optimized_transducer_b200 import synthetic
    from oracle import oracle as O

    T, U, tg = synthetic.make_lengths(w)
    T, U = T[:n_sample].contiguous(), U[:n_sample].contiguous()
    tg = tg[:n_sample, :int(U.max())].contiguous()
    x = synthetic.make_logits(w, T, U, device="cpu")
    cells = synthetic.num_rows(T, U) * w.v
    cores = torch.get_num_threads()
    ref = O.load_ref()
    if ref is not None:
        ext = ref[0]
        work = torch.empty_like(x)

        def step():
            # What the reference's Python layer does around its native call
            # (transducer_loss.py:135-170): loss = -scores, reduce, divide the
            # gradient for "mean", multiply it by the upstream gradient.
            work.copy_(x)  # restore the input (not timed)
            lx = work.requires_grad_(True)
            t0 = time.perf_counter()
            scores, grad = ext.compute_transducer_loss(
                logits=lx, targets=tg, logit_lengths=T, target_lengths=U, blank=0,
                from_log_softmax=w.from_log_softmax, one_sym_per_frame=w.one_sym_per_frame)
            with torch.no_grad():  # both run inside an autograd.Function there
                loss = -1 * scores
                if w.reduction == "mean":
                    loss = loss.mean()
                    grad /= T.size(0)
                else:
                    loss = loss.sum()
                grad.mul_(torch.ones(()))
            dt = time.perf_counter() - t0
            work.requires_grad_(False)
            return dt
        kind = "reference"
        note = "only its logsumexp is multi-threaded (ATen); the rest of the reference is one thread"
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
    desc = (f"first {n_sample} of {w.n} utterances of {w.name} "
            f"({synthetic.num_rows(T, U)} rows x V={w.v}); {note}")
    return step, cells, kind, cores, desc


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from optimized_transducer_b200 import synthetic
    step, cells, kind, cores, desc = cpu_reference_step_factory(w, min(args.ref_utts, w.n))
    for _ in range(args.warmup):
        step()
    dt = sum(step() for _ in range(args.steps))
    value = cells * args.steps / dt
    T, U, _ = synthetic.make_lengths(w)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_description(w, w.n, synthetic.num_rows(T, U)),
                   "device": "host CPU", "sample": desc},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def run_ours(args, w):
    import torch
    import torch.distributed as dist

    import optimized_transducer_b200 as ot
    from optimized_transducer_b200 import synthetic

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
    n_global = w.n * world if args.scaling == "weak" else w.n
    T, U, tg = synthetic.make_lengths(w, n=n_global)
    if args.utts:  # a smaller case of the same workload, for profiler captures
        n_global = min(args.utts, n_global)
        T, U = T[:n_global].contiguous(), U[:n_global].contiguous()
        tg = tg[:n_global, :int(U.max())].contiguous()
    if world > 1:
        shard = sharding.shard_batch(T, U, tg, w.v, world, rank, strategy=args.partition)
        T, U, tg = shard.T, shard.U, shard.targets
    rows = synthetic.num_rows(T, U)
    cells_local = rows * w.v
    dT, dU, dtg = T.to(dev), U.to(dev), tg.to(dev)
    pristine = synthetic.make_logits(w, T, U, device=dev, seed=w.seed + 31 * rank)
    if args.dtype != "f32":  # the 16-bit extension: same values, rounded once
        pristine = pristine.to(torch.bfloat16 if args.dtype == "bf16" else torch.float16)
    bytes_logits = pristine.numel() * pristine.element_size()

    total_steps = args.steps + args.warmup
    free, _ = torch.cuda.mem_get_info(dev)
    if (total_steps + 2) * bytes_logits > 0.85 * free:
        raise RuntimeError("steps + warmup need one logits buffer each; lower --steps")
    pool = [pristine.clone() for _ in range(total_steps)]

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

    def one_step(buf):
        x = Feed.apply(buf, anchor)
        if world > 1:
            loss = sharding.sharded_transducer_loss(
                x, dtg, dT, dU, blank=0, from_log_softmax=w.from_log_softmax,
                one_sym_per_frame=w.one_sym_per_frame, reduction=w.reduction,
                global_batch=n_global, overlap=True, exchange=exchange)
        else:
            loss = ot.transducer_loss(x, dtg, dT, dU, blank=0, from_log_softmax=w.from_log_softmax,
                                      one_sym_per_frame=w.one_sym_per_frame, reduction=w.reduction)
        return x, loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ----- warm-up
    it = iter(pool)
    for _ in range(args.warmup):
        x, loss = one_step(next(it))
        loss.backward()
    barrier()

    # ----- timed region: K steps, device resident
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    uuid = getattr(torch.cuda.get_device_properties(dev), "uuid", None)
    with ClockSampler(local_rank, uuid) as clocks:
        barrier()
        t_begin.record()
        for k in range(args.steps):
            ev[k][0].record()
            x, loss = one_step(next(it))
            ev[k][1].record()
            loss.backward()
            ev[k][2].record()
        if world > 1:
            sharding.wait_loss(loss)  # the last step's all-reduce ends inside the timed region
        t_end.record()
        barrier()
    elapsed_ms = t_begin.elapsed_time(t_end)
    last_loss = float(loss.item())
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    del pool, it, x, loss

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
        x = Feed.apply(dev_bufs[slot], anchor)
        if world > 1:
            loss = sharding.sharded_transducer_loss(
                x, g_, t_, u_, blank=0, from_log_softmax=w.from_log_softmax,
                one_sym_per_frame=w.one_sym_per_frame, reduction=w.reduction,
                global_batch=n_global, overlap=True, exchange=exchange)
        else:
            loss = ot.transducer_loss(x, g_, t_, u_, blank=0, from_log_softmax=w.from_log_softmax,
                                      one_sym_per_frame=w.one_sym_per_frame, reduction=w.reduction)
        loss.backward()
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
    stats = torch.tensor([elapsed_ms, e2e_ms, fwd_ms, bwd_ms], dtype=torch.float64, device=dev)
    cells = torch.tensor([float(cells_local)], dtype=torch.float64, device=dev)
    per_rank = None
    if world > 1:
        # every rank's own figures, for the record (the line reports the max)
        mine = torch.tensor([elapsed_ms / args.steps, fwd_ms, bwd_ms, float(rows)], dtype=torch.float64, device=dev)
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        per_rank = [[round(v, 4) for v in g.tolist()] for g in gathered]
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(cells, op=dist.ReduceOp.SUM)
    elapsed_ms, e2e_ms, fwd_ms, bwd_ms = stats.tolist()
    cells_total = cells.item()

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        es = pristine.element_size()
        mode_b = w.from_log_softmax
        # Gradient kernel, per launch: read + in-place write of the local logits
        # (mode A), or the dense gradient write (mode B).
        grad_bytes = (1 if mode_b else 2) * es * cells_local
        achieved = grad_bytes / (bwd_ms * 1e-3) / 1e9
        fwd_bytes = (0 if mode_b else es * cells_local)
        value = cells_total * args.steps / (elapsed_ms * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f32" if args.dtype == "f32" else f"{args.dtype} logits and gradient, f32 arithmetic",
            "data": "synthetic",
            "config": {
                "workload": workload_description(w, n_global, rows if world == 1 else "sharded")
                            + ("" if args.dtype == "f32" else f", logits stored as {args.dtype}"),
                "sharding": "none" if world == 1 else
                            f"{world} ranks, whole utterances, balanced by T*(U+1)*V ({args.partition} partition)",
                "collective": collective,
                "cache": "inputs larger than L2: every step reads its own pristine logits buffer",
                "checks": os.environ.get("OT_CHECKS", "1"),
                "gradient_schedule": "eager" if os.environ.get("OT_EAGER_GRAD", "0") == "1" else "deferred (fused into backward)",
            },
            "clocks": clocks.summary(),
            "e2e": None if not e2e_steps else {"value": cells_total / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": bytes_logits + 4 * (T.numel() + U.numel() + tg.numel()),
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms, "steps": e2e_steps},
            # own kernels per step and rank: prepare, logprob, lattice, coef, gradient
            # (+ publish and gather of the peer-memory exchange)
            "gpu_launches": (5 + (2 if exchange is not None else 0)) * args.steps,
            "roofline": {
                "kernel": "gradient_logsoftmax_kernel" if mode_b else "gradient_kernel",
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth",
                "traffic": (CFG2_GRADIENT_TRAFFIC_BYTES
                            if (w.name == "cfg2" and world == 1 and rows == CFG2_ROWS
                                and args.dtype == "f32") else None),
                "bytes_per_launch": grad_bytes, "ms_per_launch": bwd_ms,
            },
            "stages": {
                "forward_ms": fwd_ms, "backward_ms": bwd_ms,
                "forward_gbs": (fwd_bytes / (fwd_ms * 1e-3) / 1e9) if fwd_bytes else None,
                "whole_step_gbs": (fwd_bytes + grad_bytes) / ((elapsed_ms / args.steps) * 1e-3) / 1e9,
                "whole_step_frac_of_peak": (fwd_bytes + grad_bytes) / ((elapsed_ms / args.steps) * 1e-3) / 1e9 / peak,
            },
            "loss": last_loss,
        }
        if per_rank is not None:
            line["per_rank"] = {"columns": ["ms_per_step", "forward_ms", "backward_ms", "rows"], "values": per_rank}
        if world == 1 and not args.no_cpu_baseline:
            step, c_cells, kind, cores, desc = cpu_reference_step_factory(w, min(args.cpu_utts, w.n))
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


def run_pack(args, w):
    """Measurement of the packing helpers (callers' side of the packed layout) on
    the workload's shapes with D = 512 features: forward = one pass that writes
    rows*D*4 bytes, backward = two summation passes that read them."""
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
    line = {
        "metric": "packed joiner-input elements (rows*D)/s, forward", "value": rows * d / (f_ms * 1e-3),
        "unit": "elements/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": f_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"pack_joiner_input on {w.name} lengths, D={d}, rows={rows}"},
        "roofline": {"kernel": "pack_add_frames_kernel", "bound": "hbm", "achieved": bytes_out / (f_ms * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s", "frac": bytes_out / (f_ms * 1e-3) / 1e9 / peak,
                     "peak_source": f"{peak_kind} copy bandwidth", "traffic": None},
        "backward": {"ms": b_ms, "kernels": "pack_sum_kernel x2 (+ autograd's gradient copy)",
                     "achieved_gbs": 2 * bytes_out / (b_ms * 1e-3) / 1e9},
        "gpu_launches": 5 * args.steps,  # forward: prepare + add; backward: prepare + two sums
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--dtype", choices=["f32", "bf16", "f16"], default="f32",
                    help="storage type of the logits (the reference's is f32; 16-bit is an extension)")
    ap.add_argument("--collective", choices=["peer", "nccl"], default="peer",
                    help="how the ranks' losses are summed: over peer memory (default) or by NCCL")
    ap.add_argument("--partition", choices=["auto", "contiguous", "lpt"], default="lpt",
                    help="how utterances are dealt to the ranks (each rank creates its own shard, "
                         "so the permuting, better balanced \"lpt\" costs nothing here)")
    ap.add_argument("--ref-utts", type=int, default=4,
                    help="utterances per step of the reference arm (bounded sample)")
    ap.add_argument("--cpu-utts", type=int, default=8,
                    help="utterances of the CPU-baseline sample of our arm")
    ap.add_argument("--op", choices=["loss", "pack"], default="loss",
                    help="loss: the transducer loss (default, the benchmark); pack: the packing helpers")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer measurement")
    ap.add_argument("--utts", type=int, default=0,
                    help="use only the first UTTS utterances (small case for profiler captures)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    from optimized_transducer_b200 import synthetic
    w = synthetic.CONFIGS[args.workload]
    if args.op == "pack":
        run_pack(args, w)
    elif args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
