#!/usr/bin/env python
"""Benchmark of the FPx x FP16 linear layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A *step* is one pass over every (layer shape, batch size) pair of the workload; the default workload is the
LLaMA-2-70B linear-layer set in FP6 at batch sizes 1/4/16/64/128 (the set the OC-sharded runs divide).  Rank 0 prints
ONE JSON line:

  value      whole-job TFLOP/s (2*OC*IC*BS summed over the step / device time), inputs resident in HBM,
             the step replayed as a CUDA graph, weights rotated over replicas so that every launch reads
             its weights from HBM and not from L2; K steps are timed several times over (at least 0.25 s in
             all) and the median repeat is reported
  weight_gbs packed-weight bytes streamed per second (same timing)
  e2e        same metric through the host-buffer C entry point (pinned host activations in, host output back,
             copies and synchronisation inside the timed region)
  roofline   algorithmic bytes per launch / average launch time, against the measured HBM copy bandwidth
  cpu_baseline  the reference's CPU path (dequantise, then fp32 matmul) timed on this box's cores on a bounded sample
  workloads  (single GPU, default workload) the same figures for the other workloads: LLaMA-2-7B FP6, LLaMA-2-13B FP5
             with a split-K sweep, and the LLaMA-2-70B prefill shapes next to the fp16 library GEMM

With --gpus N > 1 (launched by torch.distributed.run) every layer is sharded by output channels, each rank runs
the kernel on its shard and the ranks exchange the [BS, OC] result; total work is fixed (strong scaling).
`--impl reference` times the reference's CPU implementation only (rank 0).
"""
import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (e_bits, m_bits, [(layer, OC, IC)], [batch sizes])
    "llama2-7b-fp6": (3, 2, [("qkv", 12288, 4096), ("o", 4096, 4096), ("gate_up", 22016, 4096), ("down", 4096, 11008)],
                      [1, 8, 32, 128]),
    "llama2-13b-fp5": (2, 2, [("qkv", 15360, 5120), ("o", 5120, 5120), ("gate_up", 27648, 5120), ("down", 5120, 13824)],
                       [1, 16, 64]),
    "llama2-70b-fp6": (3, 2, [("qkv", 10240, 8192), ("o", 8192, 8192), ("gate_up", 57344, 8192), ("down", 8192, 28672)],
                       [1, 4, 16, 64, 128]),
    "llama2-70b-prefill-fp6": (3, 2, [("gate_up", 57344, 8192), ("down", 8192, 28672)], [512, 1024, 2048]),
    "single-4096-fp6": (3, 2, [("square", 4096, 4096)], [8]),
}
DEFAULT_WORKLOAD = "llama2-70b-fp6"
EXTRA_WORKLOADS = ("llama2-7b-fp6", "llama2-13b-fp5", "llama2-70b-prefill-fp6")
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1590.0
MIN_TIMED_SECONDS = 0.25
# DRAM bytes (read + write) per GEMM launch as a multiple of the launch's algorithmic bytes, from a profiler capture of
# one layer of the workload (too large to capture whole); recorded when the capture was made, NOT measured in this run.
RECORDED_TRAFFIC_RATIO = {
    "llama2-70b-fp6": (1.01, "profiler captures of single launches of this workload (gate_up at 1, 16 and 64 tokens: DRAM read + write "
                             "= 1.010, 1.010 and 0.996 x the launch's algorithmic bytes; summaries under profiles/), scaled to the "
                             "average launch of a step; recorded, not measured in this run"),
}


def alg_bytes(oc, ic, bs, bw, world=1):
    """Algorithmic bytes of one launch on one GPU: its shard of the weights and scales, all activations, all output."""
    return oc * ic * bw / 8 / world + 2 * oc / world + 2 * bs * ic + 2 * bs * oc


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", FALLBACK_TFLOPS)), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_TFLOPS, "fallback"


# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _poll(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while True:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            if self._stop.wait(0.002):
                return

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------- CPU reference arm
def cpu_reference_step(e, m, layer, batches, rows=None, seed=0, cache={}):
    """One bounded sample of the reference's CPU path on the first `rows` output channels of `layer`: for every
    batch size, weight_dequant (single thread, as the reference wrote it) followed by an fp32 matmul on all cores.
    Returns (flops, seconds, dequant_seconds, kind)."""
    import torch
    import oracle
    from fp6_llm_b200.formats import random_codes_layer
    use_ref = oracle.have_ref()
    dequant = oracle.ref_dequant if use_ref else oracle.dequant
    _, oc, ic = layer
    rows = oc if rows is None else rows
    key = (e, m, rows, ic, seed)
    if key not in cache:
        w, s = random_codes_layer(rows, ic, e, m, seed=seed, scale_lo=1e-3, scale_hi=1e-2)
        cache[key] = (w.numpy(), s.numpy())
    wn, sn = cache[key]
    flops, total, t_deq = 0.0, 0.0, 0.0
    for bs in batches:
        x = torch.randn(bs, ic, generator=torch.Generator().manual_seed(bs)).half()
        t0 = time.perf_counter()
        w16 = dequant(wn, sn, e, m)
        t1 = time.perf_counter()
        y = x.float() @ torch.from_numpy(w16).float().T
        t2 = time.perf_counter()
        assert y.shape == (bs, rows)
        t_deq += t1 - t0
        total += t2 - t0
        flops += 2.0 * rows * ic * bs
    return flops, total, t_deq, ("reference" if use_ref else "port")


def cpu_sample_plan(e, m, layers, batches, budget_s):
    """Rows (a multiple of 64, the same fraction of every layer) one CPU pass over all layers and batch sizes may cover so
    that it takes about budget_s seconds."""
    _, probe_s, _, _ = cpu_reference_step(e, m, layers[0], batches, rows=64)
    est = probe_s / (64 * layers[0][2]) * sum(l[1] * l[2] for l in layers)
    frac = min(1.0, budget_s / max(est, 1e-9))
    return [max(64, int(l[1] * frac) // 64 * 64) for l in layers]


def cpu_pass(e, m, layers, batches, rows):
    fl = secs = deq = 0.0
    kind = "port"
    for layer, r in zip(layers, rows):
        f_l, s_l, d_l, kind = cpu_reference_step(e, m, layer, batches, r)
        fl, secs, deq = fl + f_l, secs + s_l, deq + d_l
    return fl, secs, deq, kind


def select_cases(args, workload=None):
    """The workload's (e, m, layers, batches); --case LAYER:BATCH narrows it to one launch shape (small profiler runs)."""
    e, m, layers, batches = WORKLOADS[workload or args.workload]
    if args.case and workload is None:
        name, bs = args.case.split(":")
        layers = [l for l in layers if l[0] == name]
        if not layers:
            raise SystemExit(f"--case: workload {args.workload} has no layer {name!r}")
        batches = [int(bs)]
    return e, m, layers, batches


def run_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(len(os.sched_getaffinity(0)))   # torchrun pins OMP_NUM_THREADS to 1; the baseline gets every core
    e, m, layers, batches = select_cases(args)
    # every step covers every layer at every batch size, cut to the same fraction of the output channels, sized so that the
    # whole run (warm-up included) takes about two minutes
    rows = cpu_sample_plan(e, m, layers, batches, budget_s=120.0 / max(args.steps + args.warmup, 1))
    for _ in range(args.warmup):
        cpu_pass(e, m, layers, batches, rows)
    flops = secs = deq = 0.0
    kind = "port"
    for _ in range(args.steps):
        f, t, d, kind = cpu_pass(e, m, layers, batches, rows)
        flops, secs, deq = flops + f, secs + t, deq + d
    value = flops / secs / 1e12
    parts = ", ".join(f"{l[0]} {r}/{l[1]}" for l, r in zip(layers, rows))
    sample = (f"per step: the first output channels of every layer ({parts}) at batch sizes {batches}; dequantisation "
              f"single-threaded as in the reference ({deq / secs:.0%} of the time), matmul on all cores")
    line = {
        "impl": "reference", "metric": "w6a16_linear_tflops" if e == 3 else "w5a16_linear_tflops", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs / max(args.steps, 1) * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload + (f" [{args.case} only]" if args.case else ""), "format": f"e{e}m{m}",
                   "layers": [list(l) for l in layers], "batch_sizes": batches,
                   "path": "weight_dequant_cpu + fp32 matmul on host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------- our arm
class Bench:
    """One workload resident on this rank's GPU: prepacked (sharded) weights in rotating replicas, activations, graphs."""

    TARGET = 512 * 1024 * 1024   # a weight buffer is re-read only after this many bytes of other weights went by

    def __init__(self, ctx, e, m, layers, batches, split_k=0, exchange=None):
        import torch
        import fp6_llm_b200 as f
        from fp6_llm_b200.formats import bit_width, synth_layer
        from fp6_llm_b200.sharding import ShardedFPxLinear, plan_rows
        self.ctx, self.e, self.m, self.layers, self.batches = ctx, e, m, layers, batches
        self.f, self.torch = f, torch
        self.bw = bit_width(e, m)
        dev, world, rank = ctx["dev"], ctx["world"], ctx["rank"]
        self.models = []
        shard_bytes = 0      # of the LARGEST shard of every layer: replica counts must be the same on every rank, because
        for li, (name, oc, ic) in enumerate(layers):   # every rank has to make the same sequence of layer calls
            plan = plan_rows(oc, world)
            r0, r1 = plan[rank]
            w, s = synth_layer(oc, ic, e, m, seed=100 + li, device=dev)
            w, s = w[r0:r1].contiguous(), s[r0:r1].contiguous()
            packed = f.weight_prepacking_eXmY_cpu(e, m, w)
            del w
            widest = max(b - a for a, b in plan) * ic * self.bw // 8
            shard_bytes += widest
            self.models.append({"name": name, "oc": oc, "ic": ic, "plan": plan, "packed": packed, "scale": s, "widest": widest})
        # Cold-L2 protocol: in the step graph batch index bi of step s uses replica (s*len(batches)+bi) % replicas of every
        # layer; the per-case pass rotates over enough replicas of that one layer.
        self.shard_bytes = shard_bytes
        self.replicas = min(48, max(1, -(-self.TARGET // max(shard_bytes, 1))))
        for mdl in self.models:
            n_rep = min(64, max(self.replicas, -(-self.TARGET // mdl["widest"])))
            mdl["replicas"] = [ShardedFPxLinear(mdl["packed"] if r == 0 else mdl["packed"].clone(), mdl["scale"], mdl["plan"], rank, e, m,
                                                exchange=exchange, native=ctx.get("native", True))
                               for r in range(n_rep)]
        torch.cuda.synchronize(dev)
        self.acts = {(mdl["name"], bs): torch.randn(bs, mdl["ic"], device=dev, dtype=torch.float16)
                     for mdl in self.models for bs in batches}
        self.cases = [(mdl, bs) for bs in batches for mdl in self.models]
        self.split = {(mdl["name"], bs): max(split_k, 0) for mdl, bs in self.cases}
        self.graphs = []

    # -- the step
    def run_step(self, step_index):
        outs = []
        nb = len(self.batches)
        for bi, bs in enumerate(self.batches):
            rep = (step_index * nb + bi) % self.replicas
            for mdl in self.models:
                outs.append(mdl["replicas"][rep].forward(self.acts[(mdl["name"], bs)], self.split[(mdl["name"], bs)]))
        return outs

    def capture(self, warmup):
        torch, ctx = self.torch, self.ctx
        n_graphs = self.replicas // math.gcd(self.replicas, len(self.batches))
        with torch.cuda.stream(ctx["stream"]):
            for i in range(max(warmup, 3)):
                self.run_step(i)
        torch.cuda.synchronize(ctx["dev"])
        assert self.f.device_status() == 0, "a GEMM CTA timed out during warm-up"
        with torch.cuda.stream(ctx["stream"]):
            for r in range(n_graphs):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=ctx["stream"]):
                    keep = self.run_step(r)
                self.graphs.append((g, keep))
            for i in range(max(warmup, 3)):
                self.graphs[i % n_graphs][0].replay()
        torch.cuda.synchronize(ctx["dev"])

    def time_steps(self, steps, sample_clocks=False):
        """Times `steps` graph replays, repeated until at least MIN_TIMED_SECONDS have been measured; returns
        (median ms per step with the max over ranks taken per repeat, repeats, clock record or None)."""
        torch, ctx = self.torch, self.ctx
        stream, dev, n_graphs = ctx["stream"], ctx["dev"], len(self.graphs)

        def block(events, repeats, first_step):
            with torch.cuda.stream(stream):
                events[0].record(stream)
                for r in range(repeats):
                    for i in range(steps):
                        self.graphs[(first_step + r * steps + i) % n_graphs][0].replay()
                    events[r + 1].record(stream)
            torch.cuda.synchronize(dev)
            return [events[r].elapsed_time(events[r + 1]) for r in range(repeats)]

        probe = block([torch.cuda.Event(enable_timing=True) for _ in range(2)], 1, 0)[0]
        repeats = max(3, min(400, int(math.ceil(MIN_TIMED_SECONDS * 1e3 / max(probe, 1e-3)))))
        if ctx["world"] > 1:   # the same count on every rank
            t = torch.tensor([repeats], device=dev)
            ctx["dist"].all_reduce(t, op=ctx["dist"].ReduceOp.MAX)
            repeats = int(t.item())
        events = [torch.cuda.Event(enable_timing=True) for _ in range(repeats + 1)]
        ctx["barrier"]()
        torch.cuda.synchronize(dev)
        sampler = ClockSampler(ctx["local_rank"]) if sample_clocks else None
        if sampler:
            sampler.start()
        ms = block(events, repeats, 0)
        clocks = sampler.stop() if sampler else None
        ctx["barrier"]()
        if ctx["world"] > 1:
            t = torch.tensor(ms, device=dev)
            ctx["dist"].all_reduce(t, op=ctx["dist"].ReduceOp.MAX)
            ms = [float(v) for v in t.tolist()]
        return statistics.median(ms) / steps, repeats, clocks

    # -- figures of the step
    def flops_step(self):
        return sum(2.0 * mdl["oc"] * mdl["ic"] * bs for mdl, bs in self.cases)

    def weight_bytes_step(self):
        return sum(mdl["oc"] * mdl["ic"] * self.bw / 8 for mdl, bs in self.cases)

    def alg_bytes_step(self):
        return sum(alg_bytes(mdl["oc"], mdl["ic"], bs, self.bw, self.ctx["world"]) for mdl, bs in self.cases)

    def launches_step(self, with_barrier):
        L = self.f.lib()
        n = 0
        for mdl, bs in self.cases:
            r0, r1 = mdl["plan"][self.ctx["rank"]]
            if mdl["replicas"][0].use_native(bs, self.split[(mdl["name"], bs)]):
                n += L.fp6b200_native_kernel_launches(r1 - r0, bs, mdl["ic"]) + (1 if with_barrier else 0)
            else:
                n += L.fp6b200_kernel_launches(r1 - r0, bs, mdl["ic"], self.split[(mdl["name"], bs)]) + (1 if with_barrier else 0)
        return n

    # -- every case alone
    def time_graph(self, fn, n_calls, min_ms=15.0):
        """Device microseconds per call of a graph that makes n_calls calls of fn(i)."""
        torch, ctx = self.torch, self.ctx
        stream, dev = ctx["stream"], ctx["dev"]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g, stream=stream):
                keep = [fn(i) for i in range(n_calls)]
            g.replay()
            torch.cuda.synchronize(dev)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            g.replay()
            b.record(stream)
            torch.cuda.synchronize(dev)
            reps = max(3, min(200, int(math.ceil(min_ms / max(a.elapsed_time(b), 1e-3)))))
            a.record(stream)
            for _ in range(reps):
                g.replay()
            b.record(stream)
        torch.cuda.synchronize(dev)
        us = a.elapsed_time(b) * 1e3 / (reps * n_calls)
        del g, keep
        if ctx["world"] > 1:
            t = torch.tensor([us], device=dev)
            ctx["dist"].all_reduce(t, op=ctx["dist"].ReduceOp.MAX)
            us = float(t.item())
        return us

    def per_case(self, compare_cublas=False, split_sweep=None, compare_reference=False):
        torch, f, ctx = self.torch, self.f, self.ctx
        hbm_peak, tc_peak, _ = ctx["peaks"]
        world = ctx["world"]
        out = []
        for mdl, bs in self.cases:
            key = (mdl["name"], bs)
            n_rep = len(mdl["replicas"])
            x = self.acts[key]
            us = self.time_graph(lambda r: mdl["replicas"][r].forward(x, self.split[key]), n_rep)
            ab = alg_bytes(mdl["oc"], mdl["ic"], bs, self.bw, world)
            fl = 2.0 * mdl["oc"] * mdl["ic"] * bs
            t_roof = max(ab / (hbm_peak * 1e9), fl / world / (tc_peak * 1e12))
            entry = {"layer": mdl["name"], "oc": mdl["oc"], "ic": mdl["ic"], "bs": bs, "split_k": self.split[key],
                     "us": round(us, 3), "tflops": round(fl / us / 1e6, 3),
                     "weight_gbs": round(mdl["oc"] * mdl["ic"] * self.bw / 8 / us / 1e3, 1),
                     "roofline_frac": round(t_roof / (us * 1e-6), 4),
                     "bound": "hbm" if ab / (hbm_peak * 1e9) >= fl / world / (tc_peak * 1e12) else "tensor",
                     "kernel": "fp6 tensor-core inputs" if mdl["replicas"][0].use_native(bs, self.split[key]) else "fp16 patterns"}
            if split_sweep and world == 1:
                # the reference's explicit split-K scheme on this kernel: the given splits, and the library's K-aware choice
                chosen = f.heuristic_split_k_b200(mdl["oc"], bs, mdl["ic"], ctx["sms"])
                sweep = {}
                for k in sorted(set(list(split_sweep) + [chosen])):
                    sweep[str(k)] = round(self.time_graph(lambda r: mdl["replicas"][r].forward_local(x, k), n_rep), 3)
                entry["split_k_sweep_us"] = sweep
                entry["choose_split_k"] = chosen
                entry["reference_heuristic_split_k"] = f.HeuristicFuntion_SplitK(mdl["oc"], bs, ctx["sms"])
            if compare_reference and world == 1 and (self.e, self.m) in ((3, 2), (2, 2)):
                # the reference's own kernel (sm_80 code: mma.sync, ldmatrix, cp.async) recompiled for sm_100a, on the same
                # packed weights, with the split-K its heuristic picks; cold L2 like everything else
                import oracle
                R = oracle.ref_gpu()
                sk = f.HeuristicFuntion_SplitK(mdl["oc"], bs, ctx["sms"])
                ws_ref = torch.empty(max(sk, 1) * mdl["oc"] * bs, dtype=torch.float32, device=ctx["dev"])
                out_ref = torch.empty(bs, mdl["oc"], dtype=torch.float16, device=ctx["dev"])

                def ref_call(r):
                    rc = R.ref_gpu_linear(self.e, self.m, torch.cuda.current_stream().cuda_stream, mdl["replicas"][r].packed.data_ptr(),
                                          mdl["scale"].data_ptr(), x.data_ptr(), out_ref.data_ptr(), mdl["oc"], bs, mdl["ic"],
                                          ws_ref.data_ptr(), sk)
                    assert rc == 0, f"reference kernel returned {rc}"
                with torch.cuda.stream(ctx["stream"]):
                    ref_call(0)
                torch.cuda.synchronize(ctx["dev"])
                mine = mdl["replicas"][0].forward(x, self.split[key]).float()
                rel = float((out_ref.float() - mine).norm() / mine.norm())
                us_ref = self.time_graph(ref_call, n_rep)
                entry["reference_kernel_us"] = round(us_ref, 3)
                entry["reference_kernel_split_k"] = sk
                entry["speedup_vs_reference_kernel"] = round(us_ref / us, 3)
                entry["reference_kernel_rel_diff"] = round(rel, 6)
                del ws_ref, out_ref
            if compare_cublas and world == 1:
                # the same layer as a library fp16 GEMM on weights dequantised on the GPU (2.67x / 3.2x the bytes), cold L2
                w16 = f.dequant_packed_cuda(self.e, self.m, mdl["packed"], mdl["scale"])
                n16 = max(2, -(-self.TARGET // (w16.numel() * 2)))
                reps16 = [w16] + [w16.clone() for _ in range(n16 - 1)]
                with torch.cuda.stream(ctx["stream"]):
                    torch.nn.functional.linear(x, reps16[0])
                torch.cuda.synchronize(ctx["dev"])
                us16 = self.time_graph(lambda r: torch.nn.functional.linear(x, reps16[r]), n16)
                entry["cublas_fp16_us"] = round(us16, 3)
                entry["speedup_vs_cublas_fp16"] = round(us16 / us, 3)
                del reps16, w16
            out.append(entry)
        return out

    def free(self):
        self.graphs = []
        for mdl in self.models:
            mdl.clear()
        self.models, self.cases, self.acts = [], [], {}
        self.torch.cuda.empty_cache()


def summarise(bench, ms_per_step, ctx):
    sec = ms_per_step / 1e3
    hbm_peak = ctx["peaks"][0]
    return {"value": bench.flops_step() / sec / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_per_step,
            "weight_gbs": bench.weight_bytes_step() / sec / 1e9,
            "roofline_frac_hbm": bench.alg_bytes_step() / sec / 1e9 / hbm_peak}


def run_ours(args):
    import torch
    import torch.distributed as dist
    import fp6_llm_b200 as f
    from fp6_llm_b200.sharding import PeerExchange

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # the exchange uses plain peer stores only
        dist.init_process_group("nccl", device_id=dev)
    f.lib()   # raises if the CUDA library is missing: there is no fallback
    # N > 1: the kernel stores its rows into every rank's output buffer (peer-mapped symmetric memory) and ends with an
    # arrival barrier; the NCCL all-gather variant is timed next to it.
    exchange = PeerExchange() if (world > 1 and args.exchange == "fused") else None
    ctx = {"dev": dev, "world": world, "rank": rank, "local_rank": local_rank, "dist": dist, "peaks": peaks(),
           "stream": torch.cuda.Stream(dev), "sms": torch.cuda.get_device_properties(dev).multi_processor_count,
           "barrier": (lambda: dist.barrier()) if world > 1 else (lambda: None), "native": not args.no_native}
    hbm_peak, tc_peak, peak_kind = ctx["peaks"]

    e, m, layers, batches = select_cases(args)
    bench = Bench(ctx, e, m, layers, batches, args.split_k, exchange)
    # The weights are prepacked above and only read from here on: let the GEMMs request them while the previous kernel
    # of the stream is still finishing (see fp6b200_set_option in include/fp6_llm_b200.h).
    f.set_static_weights(not args.no_static_weights)
    f.set_programmatic_launch(not args.no_programmatic_launch)
    bench.capture(args.warmup)
    ms_step, repeats, clocks = bench.time_steps(args.steps, sample_clocks=True)
    status = f.device_status()
    sec_step = ms_step / 1e3
    flops_step, abytes_step, n_cases = bench.flops_step(), bench.alg_bytes_step(), len(bench.cases)
    launches_step = bench.launches_step(exchange is not None)

    # ---- N > 1: the exchanged result of one step against the plain single-GPU entry point on this rank's shard, and
    # against the other ranks' copies; then the same step with one NCCL all-gather per layer instead of the fused exchange
    multi = None
    if world > 1:
        worst, agree = 0.0, True
        with torch.cuda.stream(ctx["stream"]):
            for mdl, bs in bench.cases:
                layer = mdl["replicas"][0]
                x = bench.acts[(mdl["name"], bs)]
                full = layer.forward(x, bench.split[(mdl["name"], bs)]).clone()
                local = layer.forward_local(x, bench.split[(mdl["name"], bs)])
                r0, r1 = mdl["plan"][rank]
                worst = max(worst, float((full[:, r0:r1].float() - local.float()).abs().max().item()))
                digest = full.view(torch.int16).to(torch.int64).sum().reshape(1)
                lo, hi = digest.clone(), digest.clone()
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                agree = agree and bool((lo == hi).item())
        torch.cuda.synchronize(dev)
        t = torch.tensor([worst, float(f.device_status())], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        multi = {"cases_checked": len(bench.cases), "max_abs_diff_vs_own_shard": float(t[0].item()),
                 "all_ranks_hold_the_same_result": agree, "device_status_max_over_ranks": int(t[1].item())}
        status = max(status, int(t[1].item()))
        if exchange is not None and not args.no_nccl_comparison:
            for mdl in bench.models:
                for layer in mdl["replicas"]:
                    layer.exchange = None
            bench.graphs = []
            bench.capture(3)
            ms_nccl, _, _ = bench.time_steps(args.steps)
            multi["nccl_all_gather"] = {"value": flops_step / (ms_nccl / 1e3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_nccl,
                                        "note": "same step with ONE NCCL all-gather of [BS, OC] per layer instead of the fused exchange"}
            for mdl in bench.models:
                for layer in mdl["replicas"]:
                    layer.exchange = exchange
            bench.graphs = []

    # ---- per-case device times (separate pass, each case alone in a graph over its replicas)
    import oracle as _oracle
    ref_kernel = world == 1 and not args.no_reference_kernel and _oracle.have_ref_gpu()
    per_case = (bench.per_case(compare_cublas=args.compare_cublas, compare_reference=ref_kernel)
                if (world == 1 or args.per_case_multi) else [])

    # ---- end to end through the batched host-buffer entry point (single GPU only: it is a per-GPU call)
    e2e = None
    if world == 1:
        host_in = {k: v.cpu().pin_memory() for k, v in bench.acts.items()}
        host_out = {(mdl["name"], bs): torch.empty(bs, mdl["oc"], dtype=torch.float16).pin_memory() for mdl, bs in bench.cases}
        nb, nm = len(batches), len(bench.models)

        def e2e_step(i):
            calls = []
            for j, (mdl, bs) in enumerate(bench.cases):
                key = (mdl["name"], bs)
                layer = mdl["replicas"][(i * nb + j // nm) % bench.replicas]
                calls.append((e, m, host_in[key], layer.packed, layer.scale, host_out[key], bench.split[key], layer.native))
            f.linear_forward_host_batch(calls)
        for i in range(3):
            e2e_step(i)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        e2e_step(0)
        n_e2e = max(3, min(400, int(math.ceil(MIN_TIMED_SECONDS / max(time.perf_counter() - t0, 1e-6)))))
        t0 = time.perf_counter()
        for i in range(n_e2e):
            e2e_step(i)
        torch.cuda.synchronize(dev)
        e2e_sec = (time.perf_counter() - t0) / n_e2e
        key0 = (bench.models[0]["name"], batches[-1])
        ref0 = f.linear_forward_eXmY_cuda(e, m, bench.acts[key0], bench.models[0]["replicas"][0].packed, bench.models[0]["scale"], 0)
        e2e = {"value": flops_step / e2e_sec / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(sum(2 * bs * mdl["ic"] for mdl, bs in bench.cases)),
               "d2h_bytes_per_step": int(sum(2 * bs * mdl["oc"] for mdl, bs in bench.cases)),
               "ms_per_step": e2e_sec * 1e3, "steps": n_e2e,
               "matches_device_path": bool(torch.equal(ref0.cpu(), host_out[key0])),
               "note": "one fp6b200_linear_host_io_batch call per step: pinned host activations -> device, kernels, device -> "
                       "pinned host output, pipelined over three streams, one synchronise per step; wall clock"}
        del host_in, host_out

    # ---- CPU baseline (rank 0, single GPU run only): bounded sample of the same workload
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        # every layer of the workload at every batch size, cut to the same fraction of its output channels so that
        # the whole sample takes about 20 s
        rows = cpu_sample_plan(e, m, layers, batches, budget_s=20.0)
        fl, secs, deq, kind = cpu_pass(e, m, layers, batches, rows)
        parts = ", ".join(f"{l[0]} {r}/{l[1]}" for l, r in zip(layers, rows))
        cpu = {"value": fl / secs / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
               "sample": f"one pass over the first output channels of every layer ({parts}) at batch sizes "
                         f"{batches}: {secs:.2f} s, of which single-threaded dequantisation {deq:.2f} s"}

    # ---- the other workloads (single GPU, default run): value, roofline fraction and per-case table of each
    others = None
    if world == 1 and not args.case and not args.no_extra_workloads and args.workload == DEFAULT_WORKLOAD:
        replicas_main, shard_main = bench.replicas, bench.shard_bytes
        bench.free()
        others = {}
        for name in EXTRA_WORKLOADS:
            e2, m2, layers2, batches2 = WORKLOADS[name]
            b2 = Bench(ctx, e2, m2, layers2, batches2, 0, None)
            b2.capture(3)
            ms2, rep2, _ = b2.time_steps(max(2, min(args.steps, 20)))
            entry = summarise(b2, ms2, ctx)
            entry["format"] = f"e{e2}m{m2}"
            entry["batch_sizes"] = batches2
            entry["repeats"] = rep2
            entry["cases"] = b2.per_case(compare_cublas=name.endswith("prefill-fp6"),
                                         split_sweep=(1, 2, 4, 8) if name == "llama2-13b-fp5" else None,
                                         compare_reference=ref_kernel)
            if name.endswith("prefill-fp6"):
                entry["tensor_peak_tflops"] = tc_peak
                entry["frac_of_tensor_peak"] = entry["value"] / tc_peak
            others[name] = entry
            b2.free()
            del b2
    else:
        replicas_main, shard_main = bench.replicas, bench.shard_bytes

    if rank == 0:
        ratio = RECORDED_TRAFFIC_RATIO.get(args.workload) if (world == 1 and not args.case) else None
        per_launch = abytes_step / n_cases
        line = {
            "metric": "w6a16_linear_tflops" if e == 3 else "w5a16_linear_tflops",
            "value": flops_step / sec_step / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload + (f" [{args.case} only]" if args.case else ""), "format": f"e{e}m{m}",
                       "layers": [list(l) for l in layers], "batch_sizes": batches,
                       "split_k": "0 (library: tile waves + stream-K remainder)" if args.split_k <= 0 else args.split_k,
                       "parallelism": "single GPU" if world == 1 else (
                           f"OC-sharded x{world}, rows stored into every rank's [BS, OC] by the kernel over NVLink + arrival barrier" if exchange is not None
                           else f"OC-sharded x{world} + NCCL all-gather of [BS, OC]"),
                       "l2": f"inputs larger than L2: {replicas_main} replica(s) of the layer set ({shard_main * replicas_main / 2**20:.0f} MiB) rotated so a buffer is re-read only after >= 512 MiB of other weights",
                       "launch": "whole step replayed as a CUDA graph; kernels launched programmatically (prologue overlaps the previous kernel's tail)",
                       "timing": f"median of {repeats} repeats of {args.steps} steps (CUDA events, max over ranks per repeat)",
                       "kernels": (f"batch <= {f.NATIVE_AUTO_MAX}: codes straight into the tensor cores as e3m2 / e2m3 operands (weights also held in the 128x128 tile layout at 6 bits per weight, activations as four exact e5m2 planes); larger batches: codes unpacked to fp16 patterns in tensor memory"
                                   if ctx.get("native", True) and f.native_supported(e, m, 256, 64, 1) else "codes unpacked to fp16 patterns in tensor memory"),
                       "static_weights": bool(f.static_weights()),
                       "programmatic_gemm_launch": bool(f.lib().fp6b200_get_option(2) == 1)},
            "weight_gbs": bench_weight_gbs(layers, batches, e, m, sec_step),
            "roofline": {"bound": "hbm", "achieved": abytes_step / sec_step / 1e9, "peak": hbm_peak, "unit": "GB/s",
                         "frac": abytes_step / sec_step / 1e9 / hbm_peak,
                         "traffic": per_launch * ratio[0] if ratio else None,
                         "traffic_source": ratio[1] if ratio else "not captured for this configuration",
                         "algorithmic_bytes_per_launch": per_launch, "peak_source": peak_kind,
                         "note": "per-GPU algorithmic bytes (own weight shard + all activations + all output) of the launches of a step / device time of the step; per-case fractions use min(HBM, tensor) roofline"},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_step * args.steps * repeats, "clocks": clocks,
            "device_status": status, "cases": per_case,
        }
        timed_ref = [c for c in per_case if "reference_kernel_us" in c]
        if timed_ref and len(timed_ref) == len(per_case):
            ref_us, own_us = sum(c["reference_kernel_us"] for c in timed_ref), sum(c["us"] for c in timed_ref)
            line["reference_kernel"] = {
                "us_per_step": round(ref_us, 1), "ours_us_per_step": round(own_us, 1), "speedup": round(ref_us / own_us, 3),
                "what": "the reference's own GPU kernel (fp6_llm/csrc/fp6_linear.cu: sm_80 code - mma.sync, ldmatrix, cp.async - recompiled "
                        "for sm_100a into oracle/_ref) on the same prepacked weights and activations, split-K from its heuristic for "
                        f"{ctx['sms']} SMs, every case alone in a graph with cold L2; sums over the cases of a step",
                "max_rel_diff_to_ours": max(c["reference_kernel_rel_diff"] for c in timed_ref)}
        if multi is not None:
            line["multi_gpu_check"] = multi
        if others is not None:
            line["workloads"] = others
        print(json.dumps(line), flush=True)
    if world > 1:
        # Orderly teardown: graphs (they hold captured work) and exchange buffers go first, every rank waits for the
        # others, then the process group; a watchdog ends the process if the communicator's own teardown does not return.
        bench.free()
        if exchange is not None:
            exchange.close()
        torch.cuda.synchronize(dev)
        dist.barrier()
        sys.stdout.flush()
        watchdog = threading.Timer(30.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        dist.destroy_process_group()


def bench_weight_gbs(layers, batches, e, m, sec_step):
    bw = 1 + e + m
    return sum(oc * ic * bw / 8 for _, oc, ic in layers) * len(batches) / sec_step / 1e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD)
    ap.add_argument("--split-k", type=int, default=0, help="0 = let the library decompose the work")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-workloads", action="store_true", help="single GPU: skip the `workloads` summary of the other workloads")
    ap.add_argument("--exchange", choices=["fused", "nccl"], default="fused", help="N > 1: how the ranks' rows reach each other")
    ap.add_argument("--no-nccl-comparison", action="store_true", help="N > 1: do not also time the NCCL all-gather variant")
    ap.add_argument("--per-case-multi", action="store_true",
                    help="N > 1: also time every (layer, batch) pair alone (off by default: the step time is the result)")
    ap.add_argument("--compare-cublas", action="store_true",
                    help="also time torch's fp16 GEMM on GPU-dequantised weights for every case (single GPU)")
    ap.add_argument("--no-programmatic-launch", action="store_true",
                    help="plain stream order between a GEMM and the kernel before it")
    ap.add_argument("--no-reference-kernel", action="store_true",
                    help="single GPU: do not also time the reference's own GPU kernel (recompiled for sm_100a, oracle/_ref) per case")
    ap.add_argument("--no-native", action="store_true",
                    help="run every batch size on the fp16-pattern kernel (by default batches <= 32 use the tensor cores' own FP6 inputs)")
    ap.add_argument("--no-static-weights", action="store_true",
                    help="do not let a GEMM read its (prepacked, read-only) weights before the previous kernel has completed")
    ap.add_argument("--case", default=None, help="LAYER:BATCH - run only this launch shape of the workload (for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
