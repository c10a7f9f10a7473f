#!/usr/bin/env python
"""Benchmark of the LoGo attention hot path: ``sq_full_attn`` forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--ratio R] [--impl reference]

Workload (the configuration the metric is quoted on): bf16 Q/K/V, 4 sequences x 8192 tokens
packed to ``[1, 32768, 16, 128]``, causal, Q/K ~ N(0,1) * 128**-0.25 (so that q.k has the
variance of N(0,1)/sqrt(128)-scaled inputs), V, dO ~ N(0,1), a Bernoulli(R) row mask.
One step = select/compact + forward + backward over one such batch. Synthetic, seeded.

Metric: TFLOP/s on the EFFECTIVE FLOPs of the selected rows,
``F_fwd = 4 * 128 * HQ * sum_{selected rows}(pos + 1)``, ``F_step = 3.5 * F_fwd``.
Masked / padded tile work and the recomputation of S in the backward are not counted.

The K timed steps are replays of one CUDA graph (the step's three C-ABI calls captured once) and
carry one CUDA event per step and nothing else; the per-kernel durations behind
``roofline`` and ``kernel_ms`` come from a second pass of the same K steps with an event pair
around every kernel (those pairs cost several per cent of the step, see ``kernel_ms_pass``).

With N > 1 (one process per GPU under torchrun) every rank runs its own batch (weak
scaling, no collective on the data path); the value is the sum of FLOPs over ranks divided
by the slowest rank's device time.

After the headline the default run also measures, with a few steps each, the other workloads of
the same path and reports them INSIDE the same JSON line (keys ``fuse``, ``decode``, ``layer_train``,
``prefill``): the norm / blend kernels and decode attention as HBM GB/s, and the two model-level
configurations with the partitioning the reference's configurations prescribe (sequences dealt to
the ranks for the layer training step, batch for the 1.5B prefill, KV heads for decode), each with
its one NCCL all-gather. ``--no-legs`` leaves them out; ``--workload X`` runs one of them alone.

``--impl reference`` times the CPU restatement of the reference's algorithm (the oracle) on
the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np
import torch

T_SEQ, N_SEQ, HQ, H, D = 8192, 4, 16, 16, 128
N_TOK = T_SEQ * N_SEQ
SCALE = D ** -0.5
METRIC = "sq_full_attn_fwd_bwd_effective_tflops"


def profiled_traffic(kernel: str, ratio: float):
    """DRAM bytes of one launch of `kernel` at `ratio`, as recorded by the ncu summaries under profiles/
    in lines of the form ``traffic_bytes kernel=<name> ratio=<r>: <bytes>``; None when there is none."""
    import re

    for f in sorted((ROOT / "profiles").glob("*.md")):
        for m in re.finditer(r"traffic_bytes kernel=(\S+) ratio=(\S+): ([0-9.eE+]+)", f.read_text()):
            if m.group(1) == kernel and abs(float(m.group(2)) - ratio) < 1e-9:
                return float(m.group(3))
    return None


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(bf16=d.get("bf16_tflops", 1590.0), bf16_sustained=d.get("bf16_tflops_sustained", 1400.0),
                    hbm=d.get("hbm_gbs", 6650.0), source="measured")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


# ----------------------------------------------------------------------------------------------
# CPU leg: the oracle on a bounded sample (used for cpu_baseline and for --impl reference)
# ----------------------------------------------------------------------------------------------
def cpu_sample_step(ratio: float, seed: int, t: int = 2048, heads: int = 4):
    """One forward + backward of the oracle on one sequence of `t` tokens and `heads` heads.
    Returns (seconds, effective FLOPs)."""
    from oracle import logo_oracle as orc

    rs = np.random.RandomState(seed)
    mk = lambda s: torch.from_numpy((rs.standard_normal((t, heads, D)) * s).astype(np.float32))
    q, k, v, do = mk(D ** -0.25).requires_grad_(True), mk(D ** -0.25).requires_grad_(True), \
        mk(1.0).requires_grad_(True), mk(1.0)
    sel = torch.from_numpy(rs.uniform(size=t) < ratio) if ratio < 1.0 else torch.ones(t, dtype=torch.bool)
    t0 = time.perf_counter()
    o, _ = orc.attention_dense_ref(q, k, v, [0, t], SCALE, None, sel)
    o.backward(do)
    dt = time.perf_counter() - t0
    pos = torch.nonzero(sel).flatten().double()
    flops = 3.5 * 4.0 * D * heads * float((pos + 1).sum())
    return dt, flops


def run_cpu(steps: int, warmup: int, ratio: float):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    for i in range(warmup):
        cpu_sample_step(ratio, 1000 + i)
    total_t, total_f = 0.0, 0.0
    for i in range(steps):
        dt, fl = cpu_sample_step(ratio, i)
        total_t += dt
        total_f += fl
    return total_f / total_t / 1e12, total_t / max(steps, 1) * 1e3, cores


# ----------------------------------------------------------------------------------------------
# clocks sampling during the timed region
# ----------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.recording = False   # the thread starts before the warm-up (its first NVML calls are slow); samples count from begin()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        while not self._stop_evt.is_set():
            try:
                mhz = self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM)
                get = getattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    self.nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.handle)
                if self.recording:
                    self.samples.append(mhz)
                    for bit, name in self.REASONS.items():
                        if mask & bit and name != "gpu_idle":
                            self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(0.002)

    def begin(self):
        self.recording = True

    def finish(self):
        self.recording = False
        self._stop_evt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def make_batch(device, ratio, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda h, s: (torch.randn(N_TOK, h, D, device=device, generator=g) * s).to(torch.bfloat16)
    q, k, v, do = mk(HQ, D ** -0.25), mk(H, D ** -0.25), mk(H, 1.0), mk(HQ, 1.0)
    sel = (torch.rand(N_TOK, device=device, generator=g) < ratio) if ratio < 1.0 else \
        torch.ones(N_TOK, dtype=torch.bool, device=device)
    cu = torch.arange(0, N_TOK + 1, T_SEQ, dtype=torch.int32, device=device)
    return q, k, v, do, sel, cu


def effective_flops_fwd(sel):
    pos = (torch.nonzero(sel).flatten() % T_SEQ).double()
    return 4.0 * D * HQ * float((pos + 1).sum().item())


def device_step(batch):
    """The hot path with inputs resident in HBM: select -> forward -> backward (raw C-ABI launches)."""
    from logo_b200 import ops, ops_bwd

    q, k, v, do, sel, cu = batch
    m = ops.select_rows(sel, None, cu)
    o, lse = ops.sq_attn_fwd_raw(q, k, v, m, SCALE)
    dq, dk, dv = ops_bwd.sq_attn_bwd_raw(q, k, v, o, lse, do, m, SCALE)
    return m, o, dq, dk, dv


def run_gpu(args):
    from logo_b200 import _lib, ops

    ctx = Ctx()
    dist, world, rank, local_rank, device, peaks = ctx.dist, ctx.world, ctx.rank, ctx.local_rank, ctx.device, ctx.peaks
    lib = _lib.load()

    batch = make_batch(device, args.ratio, seed=1234 + rank)
    f_fwd = effective_flops_fwd(batch[4])
    f_step = 3.5 * f_fwd

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: inputs resident in HBM ----
    # Every event the timed region uses exists before it starts (the step marks are recorded once,
    # the library's per-kernel events are reserved): creating CUDA events inside a timed loop can
    # stall the stream for milliseconds when the driver grows its event pool.
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    for ev in [e0, e1] + marks:
        ev.record()
    _lib.check(lib.logo_profile_reserve(8 * (args.steps + 2)), "logo_profile_reserve")
    lib.logo_profile_enable(0)
    # One step = three C-ABI calls = nine launches, the shortest 10 us long. They are captured once and
    # replayed as one CUDA graph per step: launched one by one from Python, the first step after the
    # barrier waits on the host for every launch (0.3 ms alone, several ms with 8 ranks and their NCCL
    # threads on the same cores), which a 20-step measurement shows as 1-8 % of the total.
    launch = "one CUDA graph per step (select + forward + backward captured once)"
    try:
        for _ in range(2):
            m, *_ = device_step(batch)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            m, *_ = device_step(batch)
        run_step = graph.replay
    except Exception as exc:   # noqa: BLE001 - any capture problem means: measure the plain launches
        print(f"step not captured ({type(exc).__name__}: {exc}); timing plain launches", file=sys.stderr)
        launch = "plain launches"
        m, *_ = device_step(batch)

        def run_step():
            device_step(batch)
    for _ in range(args.warmup):
        run_step()
    torch.cuda.synchronize()
    ops.check_device_status(m.status, "warm-up")
    barrier()
    sampler.begin()
    e0.record()
    for i in range(args.steps):
        run_step()
        marks[i].record()
    e1.record()
    barrier()
    per_step = [a.elapsed_time(b) for a, b in zip([e0] + marks[:-1], marks)]
    clocks = sampler.finish()
    ms_total = e0.elapsed_time(e1)
    ops.check_device_status(m.status, "timed region")

    # ---- per-kernel durations: the same K steps once more, with a CUDA event pair around every kernel.
    # The pairs cost several per cent of the step (a dozen extra stream operations between kernels that
    # are 20 us to 1.4 ms long), so they stay out of the pass that gives `value`.
    import ctypes
    lib.logo_profile_enable(1)
    for _ in range(2):
        device_step(batch)
    torch.cuda.synchronize()
    lib.logo_profile_read(None, None, 7)      # drop those two steps (their events go back to the pool)
    ek0, ek1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ek0.record()
    for i in range(args.steps):
        device_step(batch)
    ek1.record()
    torch.cuda.synchronize()
    lib.logo_profile_enable(0)
    ms_step_with_events = ek0.elapsed_time(ek1) / args.steps
    kinds = ["select", "attn_fwd", "bwd_preprocess", "bwd_dkv", "bwd_dq", "bwd_fused", "bwd_finish"]
    tot = (ctypes.c_double * len(kinds))()
    cnt = (ctypes.c_int * len(kinds))()
    lib.logo_profile_read(ctypes.cast(tot, ctypes.c_void_p), ctypes.cast(cnt, ctypes.c_void_p), len(kinds))
    kernel_ms = {name: (tot[i] / cnt[i] if cnt[i] else None) for i, name in enumerate(kinds)}
    # select = 2 kernels per call; the two-kernel backward launches one zero_unselected_rows_kernel (counted
    # with the preprocess kernel; the forward and the single-pass backward write those zeros themselves);
    # the count is that of K steps
    launches = 2 * cnt[0] + cnt[1] + cnt[2] + (cnt[2] if cnt[5] == 0 else 0) + cnt[3] + cnt[4] + cnt[5] + cnt[6]

    # ---- e2e: public API, host buffers, copies inside the timed region ----
    # Every step copies ITS inputs from pinned host memory and reads ITS results back to pinned host
    # memory. The three phases run on three streams with two sets of device buffers, so the upload of
    # step i+1 and the download of step i-1 overlap the compute of step i (PCIe is full duplex): the
    # steady-state step costs the longest phase instead of their sum.
    host = [t.cpu().pin_memory() for t in batch[:5]]
    cu_host = batch[5].cpu()
    main_s = torch.cuda.current_stream(device)
    h2d_s, d2h_s = torch.cuda.Stream(device), torch.cuda.Stream(device)
    dev_in = [[torch.empty_like(t, device=device) for t in host] for _ in range(2)]
    outs_host = None
    ev_in = [torch.cuda.Event() for _ in range(2)]       # inputs of buffer set b are on the device
    ev_used = [torch.cuda.Event() for _ in range(2)]     # compute no longer reads buffer set b
    ev_out = [torch.cuda.Event() for _ in range(2)]      # results of buffer set b are on the host
    keep = [None, None]                                   # device results stay referenced until downloaded
    step_no = 0

    def e2e_step():
        nonlocal outs_host, step_no
        b = step_no & 1
        with torch.cuda.stream(h2d_s):
            if step_no >= 2:
                h2d_s.wait_event(ev_used[b])
            for dst, src in zip(dev_in[b], host):
                dst.copy_(src, non_blocking=True)
            ev_in[b].record(h2d_s)
        main_s.wait_event(ev_in[b])
        q, k, v, do, sel = dev_in[b]
        q, k, v = (t.detach()[None].requires_grad_(True) for t in (q, k, v))
        o = ops.sq_full_attn(q, k, v, sel[None], scale=SCALE, cu_seqlens=cu_host)
        o.backward(do[None])
        res = (o.detach(), q.grad, k.grad, v.grad)
        ev_used[b].record(main_s)
        if outs_host is None:
            outs_host = [[torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in res] for _ in range(2)]
        with torch.cuda.stream(d2h_s):
            d2h_s.wait_event(ev_used[b])
            if step_no >= 2:
                d2h_s.wait_event(ev_out[b])
            for dst, src in zip(outs_host[b], res):
                dst.copy_(src, non_blocking=True)
                src.record_stream(d2h_s)
            ev_out[b].record(d2h_s)
        keep[b] = res
        step_no += 1

    def e2e_drain():
        main_s.wait_stream(h2d_s)
        main_s.wait_stream(d2h_s)

    if args.skip_e2e:
        ms_e2e, h2d, d2h = float("nan"), 0, 0
    else:
        for _ in range(max(args.warmup, 2)):
            e2e_step()
        e2e_drain()
        barrier()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record()
        for _ in range(args.steps):
            e2e_step()
        e2e_drain()      # the last download is inside the timed region
        e3.record()
        barrier()
        ms_e2e = e2.elapsed_time(e3)
        h2d = sum(t.numel() * t.element_size() for t in host)
        d2h = sum(t.numel() * t.element_size() for t in outs_host[0])

    # ---- reduce over ranks: slowest rank's time, summed FLOPs ----
    stats = torch.tensor([ms_total, ms_e2e, f_step], dtype=torch.float64, device=device)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms_total, ms_e2e, f_sum = mx[0].item(), mx[1].item(), sm[2].item()
    else:
        f_sum = f_step
    # ---- the further workloads of the path (every rank takes part; rank 0 reports) ----
    del host, dev_in, outs_host, keep
    torch.cuda.empty_cache()
    legs = {} if args.no_legs else run_legs(ctx, args)
    if rank != 0:
        ctx.barrier()     # rank 0 still runs its single-rank extras; every rank leaves the group together
        ctx.close()
        return

    value = f_sum * args.steps / (ms_total * 1e-3) / 1e12
    e2e_value = f_sum * args.steps / (ms_e2e * 1e-3) / 1e12

    # Dominant kernel: the single-pass backward (five tile products over the visible (query, key) pairs
    # = 2.5 * F_fwd per launch); with the two-kernel backward selected it is the dK/dV kernel (four
    # products = 2 * F_fwd).
    if kernel_ms["bwd_fused"]:
        dom, dom_name, dom_flops = "bwd_fused", "attn_bwd_fused_kernel", 2.5 * f_fwd
    else:
        dom, dom_name, dom_flops = "bwd_dkv", "attn_bwd_dkv_kernel", 2.0 * f_fwd
    achieved = dom_flops / (kernel_ms[dom] * 1e-3) / 1e12 if kernel_ms[dom] else None
    roofline = {"bound": "tensor", "kernel": dom_name, "achieved": achieved, "peak": peaks["bf16"],
                "unit": "TFLOP/s", "frac": (achieved / peaks["bf16"]) if achieved else None,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this very
                # workload, from the ncu capture summarised under profiles/ (null if none for this ratio)
                "traffic": profiled_traffic(dom_name, args.ratio),
                "peak_source": f"{peaks['source']} cuBLAS bf16 burst"}
    kernel_tflops = {
        "attn_fwd": f_fwd / (kernel_ms["attn_fwd"] * 1e-3) / 1e12 if kernel_ms["attn_fwd"] else None,
        "bwd_fused": 2.5 * f_fwd / (kernel_ms["bwd_fused"] * 1e-3) / 1e12 if kernel_ms["bwd_fused"] else None,
        "bwd_dkv": 2.0 * f_fwd / (kernel_ms["bwd_dkv"] * 1e-3) / 1e12 if kernel_ms["bwd_dkv"] else None,
        "bwd_dq": 1.5 * f_fwd / (kernel_ms["bwd_dq"] * 1e-3) / 1e12 if kernel_ms["bwd_dq"] else None,
    }

    # the other ratios of the configuration's sweep (same step, 20 timed steps each; not the headline)
    sweep = {f"{args.ratio:g}": round(value / world, 1)}
    if not args.skip_e2e:
        for r in (0.125, 0.25, 0.5, 1.0):
            if abs(r - args.ratio) < 1e-9:
                continue
            b2 = make_batch(device, r, seed=99)
            f2 = 3.5 * effective_flops_fwd(b2[4])
            for _ in range(2):
                device_step(b2)
            torch.cuda.synchronize()
            run2 = lambda: device_step(b2)   # noqa: E731
            if launch.startswith("one CUDA graph"):   # as for the headline: at r = 0.125 a step is 0.8 ms of GPU work
                try:
                    g2 = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g2):
                        device_step(b2)
                    run2 = g2.replay
                except Exception:   # noqa: BLE001
                    pass
            for _ in range(10):
                run2()
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(20):
                run2()
            s1.record()
            torch.cuda.synchronize()
            sweep[f"{r:g}"] = round(f2 * 20 / (s0.elapsed_time(s1) * 1e-3) / 1e12, 1)
            del b2

    if args.skip_cpu:
        cpu_value, cpu_ms, cores = None, float("nan"), 0
    else:
        cpu_value, cpu_ms, cores = run_cpu(steps=3, warmup=1, ratio=args.ratio)
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "step_ms_rank0": {"median": float(np.median(per_step)), "min": float(np.min(per_step)),
                          "max": float(np.max(per_step)), "argmax": int(np.argmax(per_step))},
        "config": {"workload": "sq_full_attn fwd+bwd, 4x8192 tokens packed [1,32768,16,128], causal, "
                               f"Bernoulli({args.ratio}) row mask", "ratio": args.ratio,
                   "l2": "inputs (671 MB per step) exceed the 126 MB L2; no flush needed",
                   "effective_flops_per_step": f_step, "launch": launch},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
        "kernel_ms": kernel_ms, "kernel_tflops": kernel_tflops,
        "kernel_ms_pass": {"what": "the same K steps repeated with a CUDA event pair around every kernel",
                           "ms_per_step_with_events": ms_step_with_events},
        "frac_of_peak_fwd_bwd": value / world / peaks["bf16"],
        # the step slows by ~10 % over its first ~25 repetitions as the power controller settles
        # (2.38 -> 2.65 ms): short runs compare with the burst peak, long ones with the sustained one
        "frac_of_sustained_peak_fwd_bwd": value / world / peaks["bf16_sustained"],
        "ratio_sweep_tflops_rank0": sweep,
        "cpu_baseline": {"value": cpu_value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": "oracle fwd+bwd on 1 sequence x 2048 tokens x 4 heads, fp32, 3 steps "
                                   f"({cpu_ms:.0f} ms each)"},
    }
    line.update(legs)
    print(json.dumps(line), flush=True)
    ctx.barrier()
    ctx.close()


# ----------------------------------------------------------------------------------------------
# further workloads of the same path: legs of the default run, or one alone with --workload
# ----------------------------------------------------------------------------------------------
class Ctx:
    """Process-group state shared by the legs of one run."""

    def __init__(self):
        import torch.distributed as dist

        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for the product path")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1 and not dist.is_initialized():
            dist.init_process_group("nccl", device_id=self.device)
        self.peaks = measured_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def close(self):
        if self.world > 1 and self.dist.is_initialized():
            self.dist.destroy_process_group()


def _timed(fn, steps, warmup, ctx):
    """Device time of `steps` calls in ms (max over ranks), after `warmup` calls."""
    for _ in range(warmup):
        fn()
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    ctx.barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=ctx.device)
    if ctx.world > 1:
        ctx.dist.all_reduce(ms, op=ctx.dist.ReduceOp.MAX)
    return ms.item()


def decode_batch_for(world: int) -> int:
    """Sequences of the decode configuration (64 x 32768 cached tokens x 24 layers = 384 GiB of global
    cache) that fit the ranks: 96 GiB per GPU, i.e. 16 / 32 / 64 / 64 sequences at 1 / 2 / 4 / 8 GPUs."""
    return {1: 16, 2: 32}.get(world, 64)


def leg_decode(ctx, steps, warmup, batch=None):
    """One layer-step of decode attention: B sequences x 32768 cached tokens, Bernoulli(0.5) active
    sequences, KV heads sharded over the ranks; step = decode attention + norm / blend of this rank's
    heads, then the all-gather of the head slices every rank needs before the replicated o_proj.
    Reports achieved HBM GB/s on the algorithmic bytes, with the gather outside and inside the graph."""
    from logo_b200 import Cache, ops
    from logo_b200.layers import decode_attention

    dist, world, device, peaks = ctx.dist, ctx.world, ctx.device, ctx.peaks
    B, ctx_len, heads, window = batch or decode_batch_for(world), 32768, 16 // world, 128
    g = torch.Generator(device=device).manual_seed(7)
    mk = lambda *sh: torch.randn(*sh, device=device, generator=g).to(torch.bfloat16)
    cache = Cache(max_length=ctx_len + 8)
    chunk = 4096
    for _ in range(ctx_len // chunk):   # fill the cache in chunks to bound the staging memory
        cache.append(0, mk(B, chunk, heads, D), mk(B, chunk, heads, D), mk(B, chunk, heads, D), mk(B, chunk, heads, D),
                     window)
    st = cache.layer_buffers(0)
    ql, qg = mk(B, heads, D), mk(B, heads, D)
    gate = torch.rand(B, device=device, generator=torch.Generator(device=device).manual_seed(11)).to(torch.bfloat16)
    thres = torch.tensor([0.5], device=device)
    n_active = int((gate.float() >= 0.5).sum().item())
    bytes_step = (n_active * 2 * ctx_len + B * 2 * min(ctx_len, window + 1)) * heads * D * 2 + 4 * B * heads * D * 2
    wl, wg = (mk(D) * 0.1 + 1), (mk(D) * 0.1 + 1)
    slices = torch.empty(world, B, heads * D, dtype=torch.bfloat16, device=device) if world > 1 else None
    fused_out = torch.empty(B, heads * D, dtype=torch.bfloat16, device=device)

    def step():     # this rank's heads: attention over the cache, then norm / blend
        local, glob = decode_attention(ql, qg, st, gate, thres, SCALE)
        fused_out.copy_(ops.fuse_norm_blend(local, glob, gate, thres, wl, wg, 1e-5, True))

    def gather():   # every rank gets the attention output of all heads
        if world > 1:
            dist.all_gather_into_tensor(slices, fused_out)

    def capture(body):
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(3):
                body()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            body()
        return graph

    # The layer-step is a handful of small launches: replayed as one CUDA graph (what a decode loop does).
    out = {"B": B, "ctx": ctx_len, "kv_heads_per_rank": heads, "active": n_active, "partition": "kv heads",
           "collective": "all_gather of the [B, heads*128] output slices" if world > 1 else None,
           "bytes_per_step": bytes_step * world}
    try:
        graph = capture(step)
        run, out["cuda_graph"] = (lambda: (graph.replay(), gather())), True
    except Exception as exc:   # noqa: BLE001 - any capture problem means: measure the plain launches
        print(f"decode step not captured ({type(exc).__name__}: {exc}); timing plain launches", file=sys.stderr)
        torch.cuda.synchronize()
        run, out["cuda_graph"] = (lambda: (step(), gather())), False
    ms = _timed(run, steps, warmup, ctx)
    out["ms_per_step"] = ms / steps
    out["gbs"] = bytes_step * world * steps / (ms * 1e-3) / 1e9
    out["gbs_per_gpu"] = out["gbs"] / world
    out["frac_of_hbm"] = out["gbs_per_gpu"] / peaks["hbm"]
    out["tokens_per_s_layer_step"] = B * steps / (ms * 1e-3)
    if world > 1 and out["cuda_graph"]:
        # the same step with the collective captured in the graph: no launch gap between the kernels and NCCL
        try:
            graph2 = capture(lambda: (step(), gather()))
            ms2 = _timed(graph2.replay, steps, warmup, ctx)
            out["gather_in_graph"] = {"ms_per_step": ms2 / steps, "gbs": bytes_step * world * steps / (ms2 * 1e-3) / 1e9}
        except Exception as exc:   # noqa: BLE001
            out["gather_in_graph"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
            torch.cuda.synchronize()
    out["roofline"] = {"bound": "hbm", "kernel": "decode_attn_kernel", "achieved": out["gbs_per_gpu"],
                       "peak": peaks["hbm"], "unit": "GB/s", "frac": out["frac_of_hbm"],
                       "traffic": profiled_traffic("decode_attn_kernel", 0.5),
                       "peak_source": f"{peaks['source']} copy bandwidth"}
    del cache, st
    return out


def leg_fuse(ctx, steps, warmup, ratio=0.5):
    """Fused RMSNorm + gate blend, forward and backward, 32768 tokens x 16 heads (every rank the same)."""
    from logo_b200 import _lib

    device, peaks = ctx.device, ctx.peaks
    lib = _lib.load()
    n, h = N_TOK, HQ
    g = torch.Generator(device=device).manual_seed(3)
    mk = lambda *sh: torch.randn(*sh, device=device, generator=g).to(torch.bfloat16)
    local, glob, d_out = mk(n, h, D), mk(n, h, D), mk(n, h * D)
    gate = torch.rand(n, device=device, generator=g).to(torch.bfloat16)
    thres = torch.tensor([1.0 - ratio], device=device)
    wl, wg = mk(D) * 0.1 + 1, mk(D) * 0.1 + 1
    out, d_local, d_glob, d_gate = torch.empty_like(d_out), torch.empty_like(local), torch.empty_like(glob), \
        torch.empty_like(gate)
    d_wl, d_wg = torch.empty_like(wl), torch.empty_like(wg)
    ws = torch.empty(lib.logo_fuse_bwd_workspace_bytes(n), dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device).cuda_stream
    sq = int((gate.float() >= thres.item()).sum().item())

    def fwd():
        _lib.check(lib.logo_fuse_fwd(local.data_ptr(), glob.data_ptr(), gate.data_ptr(), 0, thres.data_ptr(), 1,
                                     wl.data_ptr(), wg.data_ptr(), 0, out.data_ptr(), n, h, D, 1e-5, 1, stream), "fuse")

    def bwd():
        _lib.check(lib.logo_fuse_bwd(d_out.data_ptr(), local.data_ptr(), glob.data_ptr(), gate.data_ptr(), 0,
                                     thres.data_ptr(), 1, wl.data_ptr(), wg.data_ptr(), 0, d_local.data_ptr(),
                                     d_glob.data_ptr(), d_gate.data_ptr(), d_wl.data_ptr(), d_wg.data_ptr(), n, h, D,
                                     1e-5, 1, ws.data_ptr(), ws.numel(), stream), "fuse bwd")

    row = h * D * 2
    bytes_fwd = (2 * n + sq) * row + 2 * n
    bytes_bwd = (4 * n + 2 * sq) * row + 4 * n        # reads d_out, local, glob(sel); writes d_local, d_glob
    ms_f = _timed(fwd, steps, warmup, ctx)
    ms_b = _timed(bwd, steps, warmup, ctx)
    gf = bytes_fwd * steps / (ms_f * 1e-3) / 1e9
    gb = bytes_bwd * steps / (ms_b * 1e-3) / 1e9
    return {"tokens": n, "selected": sq, "bytes_fwd": bytes_fwd, "bytes_bwd": bytes_bwd,
            "fwd_gbs": gf, "fwd_ms": ms_f / steps, "fwd_frac_of_hbm": gf / peaks["hbm"],
            "bwd_gbs": gb, "bwd_ms": ms_b / steps, "bwd_frac_of_hbm": gb / peaks["hbm"],
            "roofline": {"bound": "hbm", "kernel": "fuse_fwd_kernel", "achieved": gf, "peak": peaks["hbm"],
                         "unit": "GB/s", "frac": gf / peaks["hbm"], "traffic": profiled_traffic("fuse_fwd_kernel", ratio),
                         "peak_source": f"{peaks['source']} copy bandwidth"}}


def lpt_partition(lens, world, ratio, window=128):
    """Whole sequences -> ranks, longest-processing-time first on the estimated attention cost
    ratio * L^2 / 2 + (window + 1) * L (global causal rows + local window rows). Returns the list of
    sequence indices of every rank; deterministic, so every rank computes the same plan."""
    cost = [ratio * l * l / 2 + (window + 1) * l for l in lens]
    order = sorted(range(len(lens)), key=lambda i: (-cost[i], i))
    load, plan = [0.0] * world, [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        plan[r].append(i)
        load[r] += cost[i]
    return plan


def _varlen_lengths(total, count, lo, hi, seed):
    rs = np.random.RandomState(seed)
    raw = rs.uniform(lo, hi, count)
    lens = np.maximum((raw / raw.sum() * total).astype(np.int64), 1)
    lens[-1] += total - lens.sum()
    return lens.tolist()


def leg_layer(ctx, steps, warmup):
    """Training step (forward + backward) of one LoGo attention layer: 8 packed sequences with
    lengths ~U[512, 8192] summing to 32768 tokens, hidden 2048, 16 x 128, global ratio 0.25.
    With N ranks whole sequences are dealt to the ranks (longest cost first), weights replicated; the
    one collective of the step gathers every rank's layer outputs (un-padded: the plan gives every
    rank's row count) and runs asynchronously under the backward."""
    from logo_b200 import LoGoAttention
    from logo_b200.config import LoGoConfig

    dist, world, rank, device = ctx.dist, ctx.world, ctx.rank, ctx.device
    lens = sorted(_varlen_lengths(N_TOK, 8, 512, 8192, 5), reverse=True)
    plan = lpt_partition(lens, world, 0.25)
    mine = [lens[i] for i in plan[rank]]
    rows = [sum(lens[i] for i in p_) for p_ in plan]
    cfg = LoGoConfig(hidden_size=2048, num_attention_heads=16, num_key_value_heads=16, window_size=128,
                     global_qk_param="linear_proj", num_hidden_layers=1, rms_norm_eps=1e-5,
                     max_position_embeddings=8192)
    torch.manual_seed(0)
    layer = LoGoAttention(cfg, 0).to(device=device, dtype=torch.bfloat16).train()
    n = sum(mine)
    g = torch.Generator(device=device).manual_seed(1 + rank)
    hidden = torch.randn(1, n, 2048, device=device, generator=g).to(torch.bfloat16).requires_grad_(True)
    d_out = torch.randn(1, n, 2048, device=device, generator=g).to(torch.bfloat16)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(mine)]), dtype=torch.int32, device=device)
    pos = torch.cat([torch.arange(l, device=device) for l in mine])[None]
    with torch.no_grad():   # threshold at the 75th percentile of the gates: 25 % of the tokens go global
        gate = torch.sigmoid(layer.gate_proj(hidden)).float().flatten()
        layer.gate_thres.fill_(torch.quantile(gate, 0.75).item())
    gathered = [torch.empty(r, 2048, dtype=torch.bfloat16, device=device) for r in rows] if world > 1 else None

    def step(overlap=True):
        hidden.grad = None
        out, _, _ = layer(hidden, position_ids=pos, cu_seqlens=cu)
        work = None
        if world > 1:   # every rank ends up with all layer outputs
            work = dist.all_gather(gathered, out.detach()[0].contiguous(), async_op=True)
            if not overlap:
                work.wait()
        out.backward(d_out)
        if work is not None and overlap:
            work.wait()

    ms = _timed(step, steps, warmup, ctx)
    ms_sync = None
    if world > 1:
        # the first timed block also pays NCCL's one-off set-up for this gather: time the overlapped form
        # again after the other one and keep the better of its two measurements
        ms_sync = _timed(lambda: step(False), steps, warmup, ctx)
        ms = min(ms, _timed(step, steps, warmup, ctx))
    # The step is about 60 launches; with a sequence or two per rank its GPU time falls under the time the
    # host needs to issue them (8 processes share the cores). The whole step (forward, gather, backward) is
    # also timed as one CUDA graph: every rank captures the same sequence, nothing in it synchronises the host.
    ms_graph = None
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(2):
                step()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        ms_graph = _timed(graph.replay, steps, warmup, ctx)
    except Exception as exc:   # noqa: BLE001 - any capture problem means: keep the plain measurement
        print(f"layer step not captured ({type(exc).__name__}: {exc})", file=sys.stderr)
        torch.cuda.synchronize()
    res = {"tokens": N_TOK, "sequence_lengths": lens, "tokens_per_rank": rows, "partition": "whole sequences, "
           "longest estimated cost first", "collective": "all_gather of the layer outputs (un-padded), overlapped "
           "with the backward" if world > 1 else None,
           "ms_per_step": ms / steps, "tokens_per_s": N_TOK * steps / (ms * 1e-3),
           "note": "a sequence is never split: with 8 ranks each holds one, and the longest (6286 of 32768 tokens) "
                   "sets the step time"}
    if ms_sync is not None:
        res["ms_per_step_gather_not_overlapped"] = ms_sync / steps
    if ms_graph is not None:
        res["ms_per_step_plain_launches"] = res["ms_per_step"]
        res["ms_per_step"] = min(res["ms_per_step"], ms_graph / steps)
        res["ms_per_step_cuda_graph"] = ms_graph / steps
        res["tokens_per_s"] = N_TOK / (res["ms_per_step"] * 1e-3)
    del layer
    return res


def leg_prefill(ctx, steps, warmup):
    """Prefill of a 24-layer, hidden-2048 LoGo decoder stack (the 1.5B configuration with vocabulary
    32000): the attention layers, the RMSNorm and the gated activation of the MLP are this package's
    kernels, the rest (embedding, MLP projections, residuals, lm_head on the last token) is plain torch.
    B = 8 x 8192 tokens, batch-sharded over the ranks, gate threshold 0.5. Random bf16 weights."""
    import torch.nn as nn
    import torch.nn.functional as F

    from logo_b200 import LoGoAttention, ops
    from logo_b200.config import LoGoConfig
    from logo_b200.layers import RMSNorm

    dist, world, rank, device = ctx.dist, ctx.world, ctx.rank, ctx.device
    cfg = LoGoConfig(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=24,
                     num_attention_heads=16, num_key_value_heads=16, window_size=128, global_qk_param="linear_proj",
                     gate_thres_init=0.5, rms_norm_eps=1e-5, max_position_embeddings=8192)

    class Block(nn.Module):
        def __init__(self, i):
            super().__init__()
            self.ln1, self.ln2 = RMSNorm(2048, 1e-5), RMSNorm(2048, 1e-5)
            self.attn = LoGoAttention(cfg, i)
            self.gate_up = nn.Linear(2048, 2 * 5632, bias=False)
            self.down = nn.Linear(5632, 2048, bias=False)

        def forward(self, x, pos_emb, pos):
            x = x + self.attn(self.ln1(x), position_ids=pos, position_embeddings=pos_emb)[0]
            gu = self.gate_up(self.ln2(x))
            a, b = gu.chunk(2, dim=-1)
            return x + self.down(ops.silu_mul(a, b))

    torch.manual_seed(0)
    with torch.device(device):     # parameters are created on the GPU: 1.3 B values are slow to draw on the host
        emb = nn.Embedding(32000, 2048)
        blocks = nn.ModuleList([Block(i) for i in range(24)])
        norm_f = RMSNorm(2048, 1e-5)
    for m in list(blocks.modules()) + [emb]:
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
    emb, blocks, norm_f = emb.to(torch.bfloat16), blocks.to(torch.bfloat16).eval(), norm_f.to(torch.bfloat16)
    b_local, t = 8 // world, 8192
    ids = torch.randint(0, 32000, (b_local, t), device=device, generator=torch.Generator(device=device).manual_seed(rank))
    pos = torch.arange(t, device=device)[None].expand(b_local, -1)
    logits_all = torch.empty(8, 32000, dtype=torch.bfloat16, device=device) if world > 1 else None

    @torch.no_grad()
    def step():
        x = emb(ids)
        pos_emb = blocks[0].attn.rotary_emb(x, pos)
        for blk in blocks:
            x = blk(x, pos_emb, pos)
        logits = F.linear(norm_f(x[:, -1]), emb.weight)
        if world > 1:   # last-token logits of the whole batch on every rank
            dist.all_gather_into_tensor(logits_all, logits.contiguous())
            return logits_all
        return logits

    ms = _timed(step, steps, warmup, ctx)
    # about a thousand launches per step: with one sequence per rank (8 GPUs) the host, shared by the eight
    # processes, can fall behind the GPU, so the step is also timed as one CUDA graph
    ms_graph = None
    try:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        ms_graph = _timed(graph.replay, steps, warmup, ctx)
    except Exception as exc:   # noqa: BLE001 - any capture problem means: keep the plain measurement
        print(f"prefill step not captured ({type(exc).__name__}: {exc})", file=sys.stderr)
        torch.cuda.synchronize()
    best = ms if ms_graph is None else min(ms, ms_graph)
    res = {"tokens": 8 * t, "batch_per_rank": b_local, "partition": "batch",
           "collective": "all_gather of the last-token logits [8, 32000]" if world > 1 else None,
           "ms_per_step": best / steps, "tokens_per_s": 8 * t * steps / (best * 1e-3),
           "ms_per_step_plain_launches": ms / steps,
           "ms_per_step_cuda_graph": None if ms_graph is None else ms_graph / steps,
           "model": "24 layers, hidden 2048, MLP 5632, 16 x 128 heads, vocab 32000, window 128, gate threshold 0.5"}
    del blocks, emb
    torch.cuda.empty_cache()
    return res


def run_legs(ctx, args):
    """The further workloads, a few steps each; a leg that fails reports its error and the run goes on."""
    legs = {}
    for name, fn, st, wu in (("fuse", leg_fuse, 20, 3), ("decode", leg_decode, 20, 3), ("layer_train", leg_layer, 6, 3),
                             ("prefill", leg_prefill, 3, 1)):
        t0 = time.perf_counter()
        try:
            legs[name] = fn(ctx, st, wu)
            legs[name]["steps"], legs[name]["n_gpus"] = st, ctx.world
        except Exception as exc:   # noqa: BLE001
            legs[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        legs[name]["wall_s"] = round(time.perf_counter() - t0, 1)
        torch.cuda.empty_cache()
    return legs


def run_one_leg(args):
    """--workload X: one leg alone, as its own JSON line."""
    ctx = Ctx()
    fn, metric, unit, key, scaling = {
        "decode": (leg_decode, "decode_attn_hbm_gbs", "GB/s", "gbs", "strong"),
        "fuse": (leg_fuse, "fuse_fwd_hbm_gbs", "GB/s", "fwd_gbs", "weak"),
        "layer": (leg_layer, "logo_layer_train_tokens_per_s", "tokens/s", "tokens_per_s", "strong"),
        "prefill": (leg_prefill, "logo_1b5_prefill_tokens_per_s", "tokens/s", "tokens_per_s", "strong"),
    }[args.workload]
    kwargs = {"batch": args.decode_batch} if (args.workload == "decode" and args.decode_batch) else {}
    res = fn(ctx, args.steps, args.warmup, **kwargs)
    if ctx.rank == 0:
        print(json.dumps({"metric": metric, "value": res[key], "unit": unit, "n_gpus": ctx.world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": res.get("ms_per_step", res.get("fwd_ms")),
                          "higher_is_better": True, "scaling": scaling, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": fn.__doc__.split("\n\n")[0].replace("\n    ", " ")}, "detail": res}),
              flush=True)
    ctx.barrier()
    ctx.close()


def run_decode_model(args):
    """Decode step of the 24-layer, hidden-2048 stack (the 1.5B configuration): B sequences with a
    32768-token cached context generate one token each. Attention layers (projections, rotary kernel,
    in-place cache append, split-KV decode attention, norm/blend) are this package's; norms use the
    row-wise RMSNorm kernel; the MLP is plain torch. The step is replayed as one CUDA graph.
    B = 16 holds 103 GB of cache on one GPU (the 64-sequence configuration needs four GPUs)."""
    import torch.nn as nn

    from logo_b200 import Cache, LoGoAttention, ops
    from logo_b200.config import LoGoConfig
    from logo_b200.layers import RMSNorm

    ctx = Ctx()
    world, device, peaks = ctx.world, ctx.device, ctx.peaks
    if world > 1:
        raise SystemExit("decode_model measures the 1-GPU point; the sharded layer-step is --workload decode")
    B, ctx_len, n_layers = args.decode_batch or 16, 32768, 24
    cfg = LoGoConfig(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=n_layers,
                     num_attention_heads=16, num_key_value_heads=16, window_size=128, global_qk_param="linear_proj",
                     gate_thres_init=0.5, rms_norm_eps=1e-5, max_position_embeddings=ctx_len + 64)

    class Block(nn.Module):
        def __init__(self, i):
            super().__init__()
            self.ln1, self.ln2 = RMSNorm(2048, 1e-5), RMSNorm(2048, 1e-5)
            self.attn = LoGoAttention(cfg, i)
            self.gate_up = nn.Linear(2048, 2 * 5632, bias=False)
            self.down = nn.Linear(5632, 2048, bias=False)

        def forward(self, x, cache, pos):
            x = x + self.attn(self.ln1(x), position_ids=pos, past_key_value=cache, use_cache=True)[0]
            a, b = self.gate_up(self.ln2(x)).chunk(2, dim=-1)
            return x + self.down(ops.silu_mul(a, b))

    torch.manual_seed(0)
    with torch.device(device):
        blocks = nn.ModuleList([Block(i) for i in range(n_layers)])
    for m in blocks.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
    blocks = blocks.to(torch.bfloat16).eval()
    g = torch.Generator(device=device).manual_seed(7)
    mk = lambda *sh: torch.randn(*sh, device=device, generator=g).to(torch.bfloat16)
    cache = Cache(max_length=ctx_len + 32)
    chunk = 4096
    for layer in range(n_layers):      # synthetic context: fill every layer's cache in chunks
        for _ in range(ctx_len // chunk):
            cache.append(layer, mk(B, chunk, 16, D), mk(B, chunk, 16, D), mk(B, chunk, 16, D), mk(B, chunk, 16, D), 128)
    x = mk(B, 1, 2048)
    out = torch.empty_like(x)

    @torch.no_grad()
    def step():
        # every eager call appends one token; the captured graph re-writes the slot it was captured at
        pos = torch.full((B, 1), cache.layers[0].length, dtype=torch.long, device=device)
        h = x
        for blk in blocks:
            h = blk(h, cache, pos)
        out.copy_(h)

    run, graphed = step, False
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run, graphed = graph.replay, True
    except Exception as exc:   # noqa: BLE001 - any capture problem means: measure the plain launches
        print(f"decode step not captured ({type(exc).__name__}: {exc}); timing plain launches", file=sys.stderr)
        torch.cuda.synchronize()
    ms = _timed(run, args.steps, args.warmup, ctx)
    with torch.no_grad():
        gate = torch.sigmoid(blocks[0].attn.gate_proj(blocks[0].ln1(x))).float().flatten()
    n_active = int((gate >= 0.5).sum().item())
    t_step = ms / args.steps * 1e-3
    n_param = sum(p.numel() for p in blocks.parameters())
    cache_bytes = n_layers * (0.5 * B * 2 * ctx_len + B * 2 * 129) * 16 * D * 2     # half the sequences active per layer
    print(json.dumps({
        "metric": "logo_1b5_decode_tokens_per_s", "value": B / t_step, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"24-layer LoGo decoder stack, one decode step, B={B}, cached context {ctx_len}, "
                               "gate threshold 0.5 (about half the sequences take the global branch per layer); "
                               "no embedding / lm_head", "cuda_graph": graphed, "active_in_layer_0": n_active},
        "roofline": {"bound": "hbm", "achieved": (cache_bytes + 2 * n_param) / t_step / 1e9, "peak": peaks["hbm"],
                     "unit": "GB/s", "frac": (cache_bytes + 2 * n_param) / t_step / 1e9 / peaks["hbm"], "traffic": None,
                     "note": "expected bytes: K/V of the active sequences + local rings + every weight once",
                     "peak_source": f"{peaks['source']} copy bandwidth"}}))


def run_ref_gpu(args):
    """The reference's OWN GPU kernels on this GPU (the kernels to beat): its Triton ``sq_full_attn``
    (logo/ops/selected_full_attn.py, unmodified, JIT-compiled here) forward + backward on the headline
    configuration for the four ratios, and the flash-attn call of its local branch (window 128).
    Needs the reference package under baseline/_ref (pip install --target); a part that does not run
    on this box is reported as unavailable with the error text."""
    ref = ROOT / "baseline" / "_ref"
    out = {"metric": "reference_gpu_kernels", "n_gpus": 1, "data": "synthetic", "dtype": "bf16",
           "config": {"workload": "reference Triton sq_full_attn fwd+bwd, 4x8192 tokens packed [1,32768,16,128]; "
                                  "flash-attn varlen window-128 fwd+bwd on the same tokens"}}
    if not (ref / "logo").is_dir():
        out["unavailable"] = "no reference package under baseline/_ref"
        print(json.dumps(out))
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --workload ref_gpu needs a CUDA device")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    sys.path.insert(0, str(ref))

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    try:
        from logo.ops import sq_full_attn as ref_sq_full_attn

        # a small case first: does the JIT produce kernels for this GPU at all?
        n0 = 1024
        q0, k0, v0 = (torch.randn(1, n0, 2, D, device=device, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
        o0 = ref_sq_full_attn(q0, k0, v0, torch.rand(1, n0, device=device) < 0.5,
                              cu_seqlens=torch.tensor([0, n0], dtype=torch.int32, device=device))
        o0.sum().backward()
        torch.cuda.synchronize()
        res = {}
        for r in (0.125, 0.25, 0.5, 1.0):
            q, k, v, do, sel, cu = make_batch(device, r, seed=1234)
            q, k, v = (t[None].requires_grad_(True) for t in (q, k, v))
            f_step = 3.5 * effective_flops_fwd(sel)

            def step():
                q.grad = k.grad = v.grad = None
                o = ref_sq_full_attn(q, k, v, sel[None], scale=SCALE, cu_seqlens=cu)
                o.backward(do[None])

            ms = timed(step, args.steps, max(args.warmup, 2))
            res[f"{r:g}"] = {"ms_per_step": ms, "tflops": f_step / (ms * 1e-3) / 1e12}
            del q, k, v, do
        out["triton_sq_full_attn"] = res
    except Exception as exc:   # noqa: BLE001
        out["triton_sq_full_attn"] = {"unavailable": f"unavailable on this box: {type(exc).__name__}: {exc}"[:400]}
        torch.cuda.synchronize()
    try:
        from flash_attn import flash_attn_varlen_func

        q, k, v, do, _, cu = make_batch(device, 1.0, seed=1234)
        q, k, v = (t.requires_grad_(True) for t in (q, k, v))

        def step_l():
            q.grad = k.grad = v.grad = None
            o = flash_attn_varlen_func(q, k, v, cu, cu, T_SEQ, T_SEQ, softmax_scale=SCALE, causal=True,
                                       window_size=(128, 128))
            o.backward(do)

        ms = timed(step_l, args.steps, max(args.warmup, 2))
        out["flash_attn_window128"] = {"ms_per_step": ms}
        # this package's local branch on the same tensors, for the ratio
        from logo_b200 import ops
        ql, kl, vl = (t.detach().clone().requires_grad_(True) for t in (q, k, v))

        def step_m():
            ql.grad = kl.grad = vl.grad = None
            o = ops.swa_attn(ql, kl, vl, cu, 128, SCALE)
            o.backward(do)

        out["logo_b200_window128"] = {"ms_per_step": timed(step_m, args.steps, max(args.warmup, 2))}
    except Exception as exc:   # noqa: BLE001
        out["flash_attn_window128"] = {"unavailable": f"unavailable on this box: {type(exc).__name__}: {exc}"[:400]}
    print(json.dumps(out))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    value, ms, cores = run_cpu(args.steps, args.warmup, args.ratio)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "sq_full_attn fwd+bwd on a bounded SLICE of the 4x8192x16x128 configuration: each "
                               f"step = 1 sequence x 2048 tokens x 4 heads, causal, Bernoulli({args.ratio}) row mask "
                               "(the dense-masked CPU restatement cannot run the full size in bench time)",
                   "ratio": args.ratio},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": "each step = oracle fwd+bwd on 1 sequence x 2048 tokens x 4 heads, fp32"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--ratio", type=float, default=0.5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="sq_attn", choices=["sq_attn", "decode", "decode_model", "fuse", "layer", "prefill", "ref_gpu"],
                    help="sq_attn is the headline metric; the others measure further rows of the same path")
    ap.add_argument("--decode-batch", type=int, default=0, help="sequences of the decode workloads (0: by rank count)")
    ap.add_argument("--bwd-mode", default=None, choices=["single_pass", "two_kernel"],
                    help="backward implementation of the global branch (default: the library's)")
    ap.add_argument("--no-legs", action="store_true", help="headline only: leave out the fuse / decode / layer / prefill legs")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: leave out the host-buffer leg")
    ap.add_argument("--skip-cpu", action="store_true", help="profiling runs: leave out the CPU baseline leg")
    args = ap.parse_args()
    if args.bwd_mode and args.impl == "ours":
        import logo_b200
        logo_b200.set_backward_mode("global", args.bwd_mode)
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "sq_attn":
        run_gpu(args)
    elif args.workload == "decode_model":
        run_decode_model(args)
    elif args.workload == "ref_gpu":
        run_ref_gpu(args)
    else:
        run_one_leg(args)


if __name__ == "__main__":
    main()
