#!/usr/bin/env python
"""Benchmark of the FPx x FP16 linear layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A *step* is one pass over every (layer shape, batch size) pair of the workload; the default workload is the
LLaMA-2-7B linear-layer set in FP6 at batch sizes 1/8/32/128.  Rank 0 prints ONE JSON line:

  value      whole-job TFLOP/s (2*OC*IC*BS summed over the step / device time), inputs resident in HBM,
             the step replayed as a CUDA graph, weights rotated over replicas so that every launch reads
             its weights from HBM and not from L2
  weight_gbs packed-weight bytes streamed per second (same timing)
  e2e        same metric through the host-buffer C entry point (pinned host activations in, host output back,
             copies and synchronisation inside the timed region)
  roofline   algorithmic bytes of all launches / device time, against the measured HBM copy bandwidth
  cpu_baseline  the reference's CPU path (dequantise, then fp32 matmul) timed on this box's cores on a bounded sample

With --gpus N > 1 (launched by torch.distributed.run) every layer is sharded by output channels, each rank runs
the kernel on its shard and the ranks all-gather the [BS, OC] result over NCCL; total work is fixed (strong scaling).
`--impl reference` times the reference's CPU implementation only (rank 0).
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
DEFAULT_WORKLOAD = "llama2-7b-fp6"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum per GEMM launch, averaged over the launches of one step, from the ncu
# launch list of this command (profiles/launch_list_llama2-7b-fp6_bench_step.md).  A recorded figure, not measured live.
NCU_TRAFFIC_BYTES = {"llama2-7b-fp6": 38.53e6}


def alg_bytes(oc, ic, bs, bw):
    return oc * ic * bw / 8 + 2 * oc + 2 * bs * ic + 2 * bs * oc


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
        cache.clear()
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


def cpu_sample_rows(e, m, layer, batches, n_steps, budget_s):
    """Rows of `layer` (multiple of 64) one CPU step may cover so that n_steps steps take about budget_s seconds."""
    _, oc, ic = layer
    _, secs, _, _ = cpu_reference_step(e, m, layer, batches, rows=64)
    per_row = secs / 64
    rows = int(budget_s / max(n_steps, 1) / per_row) // 64 * 64
    return max(64, min(oc, rows))


def select_cases(args):
    """The workload's (e, m, layers, batches); --case LAYER:BATCH narrows it to one launch shape (small profiler runs)."""
    e, m, layers, batches = WORKLOADS[args.workload]
    if args.case:
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
    e, m, layers, batches = WORKLOADS[args.workload]
    layer = min(layers, key=lambda l: l[1] * l[2])          # the smallest layer of the set
    rows = cpu_sample_rows(e, m, layer, batches, args.steps + args.warmup, budget_s=120.0)
    for _ in range(args.warmup):
        cpu_reference_step(e, m, layer, batches, rows)
    flops = secs = deq = 0.0
    kind = "port"
    for _ in range(args.steps):
        f, t, d, kind = cpu_reference_step(e, m, layer, batches, rows)
        flops, secs, deq = flops + f, secs + t, deq + d
    value = flops / secs / 1e12
    sample = (f"per step: first {rows} output channels of layer {layer[0]} {layer[1]}x{layer[2]} at batch sizes {batches}; "
              f"dequantisation single-threaded as in the reference ({deq / secs:.0%} of the time), matmul on all cores")
    line = {
        "impl": "reference", "metric": "w6a16_linear_tflops" if e == 3 else "w5a16_linear_tflops", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs / max(args.steps, 1) * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload + (f" [{args.case} only]" if args.case else ""), "format": f"e{e}m{m}", "layers": [list(l) for l in layers], "batch_sizes": batches,
                   "path": "weight_dequant_cpu + fp32 matmul on host cores"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    import fp6_llm_b200 as f
    from fp6_llm_b200.formats import bit_width, synth_layer
    from fp6_llm_b200.sharding import PeerExchange, ShardedFPxLinear, plan_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    f.lib()   # raises if the CUDA library is missing: there is no fallback
    # N > 1: the kernel stores its rows into every rank's output buffer (peer-mapped symmetric memory) and ends with an
    # arrival barrier; --exchange nccl selects one NCCL all-gather per layer instead.
    exchange = PeerExchange() if (world > 1 and args.exchange == "fused") else None
    sms = torch.cuda.get_device_properties(dev).multi_processor_count

    e, m, layers, batches = select_cases(args)
    bw = bit_width(e, m)
    # ---- weights: seeded N(0, 0.02) -> per-row scale -> round-to-nearest codes -> GPU prepack; replicas for cold L2
    shard_bytes = 0      # of the LARGEST shard of every layer: replica counts must be the same on every rank, because
    models = []          # every rank has to make the same sequence of layer calls          # per layer: dict(name, oc, ic, plan, replicas=[ShardedFPxLinear...])
    for li, (name, oc, ic) in enumerate(layers):
        plan = plan_rows(oc, world)
        r0, r1 = plan[rank]
        w, s = synth_layer(oc, ic, e, m, seed=100 + li, device=dev)
        w, s = w[r0:r1].contiguous(), s[r0:r1].contiguous()
        packed = f.weight_prepacking_eXmY_cpu(e, m, w)
        del w
        widest = max(b - a for a, b in plan) * ic * bw // 8
        shard_bytes += widest
        models.append({"name": name, "oc": oc, "ic": ic, "plan": plan, "packed": packed, "scale": s, "widest": widest})
    # Cold-L2 protocol: a (layer, replica) buffer is re-read only after >= 512 MiB of other weights went by.
    # In the step graph batch index bi of step s uses replica (s*len(batches)+bi) % replicas of every layer;
    # the per-case pass below rotates over enough replicas of that one layer.
    target = 512 * 1024 * 1024
    replicas = min(48, max(1, -(-target // max(shard_bytes, 1))))
    for mdl in models:
        n_rep = min(64, max(replicas, -(-target // mdl["widest"])))
        mdl["replicas"] = [ShardedFPxLinear(mdl["packed"] if r == 0 else mdl["packed"].clone(), mdl["scale"], mdl["plan"], rank, e, m,
                                            exchange=exchange)
                           for r in range(n_rep)]
    # The weights are prepacked above and only read from here on: let the GEMMs request them while the previous kernel
    # of the stream is still finishing (see fp6b200_set_option in include/fp6_llm_b200.h).
    torch.cuda.synchronize(dev)
    f.set_static_weights(not args.no_static_weights)
    f.set_programmatic_launch(not args.no_programmatic_launch)
    acts = {(mdl["name"], bs): torch.randn(bs, mdl["ic"], device=dev, dtype=torch.float16) for mdl in models for bs in batches}
    cases = [(mdl, bs) for bs in batches for mdl in models]
    # split_k = 0: the library decomposes the work itself (tile waves + stream-K remainder + fix-up kernel)
    split = {(mdl["name"], bs): max(args.split_k, 0) for mdl, bs in cases}
    nb = len(batches)

    def run_step(step_index):
        outs = []
        for bi, bs in enumerate(batches):
            rep = (step_index * nb + bi) % replicas
            for mdl in models:
                outs.append(mdl["replicas"][rep].forward(acts[(mdl["name"], bs)], split[(mdl["name"], bs)]))
        return outs

    # eager warm-up (configures kernels, sizes the workspace), then capture the distinct step graphs
    import math
    n_graphs = replicas // math.gcd(replicas, nb)
    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            run_step(i)
    torch.cuda.synchronize(dev)
    assert f.device_status() == 0, "a GEMM CTA timed out during warm-up"
    graphs = []
    with torch.cuda.stream(stream):
        for r in range(n_graphs):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                keep = run_step(r)
            graphs.append((g, keep))
    torch.cuda.synchronize(dev)

    def barrier():
        if world > 1:
            dist.barrier()

    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            graphs[i % n_graphs][0].replay()
    torch.cuda.synchronize(dev)
    barrier()
    sampler = ClockSampler(local_rank)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    sampler.start()
    with torch.cuda.stream(stream):
        start.record(stream)
        for i in range(args.steps):
            graphs[i % n_graphs][0].replay()
        end.record(stream)
    torch.cuda.synchronize(dev)
    clocks = sampler.stop()
    barrier()
    ms_total = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    status = f.device_status()

    flops_step = sum(2.0 * mdl["oc"] * mdl["ic"] * bs for mdl, bs in cases)
    wbytes_step = sum(mdl["oc"] * mdl["ic"] * bw / 8 for mdl, bs in cases)
    abytes_step = sum(alg_bytes(mdl["oc"], mdl["ic"], bs, bw) for mdl, bs in cases)
    sec_step = ms_total / 1e3 / args.steps
    launches_step = sum(1 + (1 if split[(mdl["name"], bs)] != 1 else 0) + (1 if exchange is not None else 0)
                        for mdl, bs in cases)   # GEMM + reduce/fix-up (+ arrival barrier)
    hbm_peak, tc_peak, peak_kind = peaks()

    # ---- per-case device times (separate pass, each case alone in a graph of `replicas` launches)
    per_case = []
    if world == 1 or args.per_case_multi:
        for mdl, bs in cases:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                n_rep = len(mdl["replicas"])
                with torch.cuda.graph(g, stream=stream):
                    keep = [mdl["replicas"][r].forward(acts[(mdl["name"], bs)], split[(mdl["name"], bs)]) for r in range(n_rep)]
                g.replay()
                torch.cuda.synchronize(dev)
                reps = max(3, min(50, args.steps))
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(reps):
                    g.replay()
                b.record(stream)
            torch.cuda.synchronize(dev)
            us = a.elapsed_time(b) * 1e3 / (reps * n_rep)
            if world > 1:
                t = torch.tensor([us], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                us = float(t.item())
            ab = alg_bytes(mdl["oc"], mdl["ic"], bs, bw)
            fl = 2.0 * mdl["oc"] * mdl["ic"] * bs
            t_roof = max(ab / world / (hbm_peak * 1e9), fl / world / (tc_peak * 1e12))
            entry = {"layer": mdl["name"], "oc": mdl["oc"], "ic": mdl["ic"], "bs": bs, "split_k": split[(mdl["name"], bs)],
                     "us": round(us, 3), "tflops": round(fl / us / 1e6, 3),
                     "weight_gbs": round(mdl["oc"] * mdl["ic"] * bw / 8 / us / 1e3, 1),
                     "roofline_frac": round(t_roof / (us * 1e-6), 4)}
            del g, keep
            if args.compare_cublas and world == 1:
                # the same layer as a library fp16 GEMM on weights dequantised on the GPU (2.67x / 3.2x the bytes), cold L2
                w16 = f.dequant_packed_cuda(e, m, mdl["packed"], mdl["scale"])
                n16 = max(2, -(-target // (w16.numel() * 2)))
                reps16 = [w16] + [w16.clone() for _ in range(n16 - 1)]
                x = acts[(mdl["name"], bs)]
                g = torch.cuda.CUDAGraph()
                with torch.cuda.stream(stream):
                    torch.nn.functional.linear(x, reps16[0])
                    torch.cuda.synchronize(dev)
                    with torch.cuda.graph(g, stream=stream):
                        keep = [torch.nn.functional.linear(x, w) for w in reps16]
                    g.replay()
                    torch.cuda.synchronize(dev)
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    for _ in range(reps):
                        g.replay()
                    b.record(stream)
                torch.cuda.synchronize(dev)
                us16 = a.elapsed_time(b) * 1e3 / (reps * n16)
                entry["cublas_fp16_us"] = round(us16, 3)
                entry["speedup_vs_cublas_fp16"] = round(us16 / us, 3)
                del g, keep, reps16, w16
            per_case.append(entry)

    # ---- end to end through the host-buffer entry point (single GPU only: it is a per-GPU call)
    e2e = None
    if world == 1:
        host_in = {k: v.cpu().pin_memory() for k, v in acts.items()}
        host_out = {(mdl["name"], bs): torch.empty(bs, mdl["oc"], dtype=torch.float16).pin_memory() for mdl, bs in cases}
        def e2e_step(i):
            for j, (mdl, bs) in enumerate(cases):
                key = (mdl["name"], bs)
                layer = mdl["replicas"][(i * nb + j // len(models)) % replicas]
                f.linear_forward_host(e, m, host_in[key], layer.packed, layer.scale, host_out[key], split[key])
        for i in range(3):
            e2e_step(i)
        n_e2e = max(3, min(args.steps, 50))
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for i in range(n_e2e):
            e2e_step(i)
        torch.cuda.synchronize(dev)
        e2e_sec = (time.perf_counter() - t0) / n_e2e
        e2e = {"value": flops_step / e2e_sec / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(sum(2 * bs * mdl["ic"] for mdl, bs in cases)),
               "d2h_bytes_per_step": int(sum(2 * bs * mdl["oc"] for mdl, bs in cases)),
               "ms_per_step": e2e_sec * 1e3, "steps": n_e2e,
               "note": "pinned host activations -> device, kernels, device -> pinned host output, synchronise, per call; wall clock"}

    # ---- CPU baseline (rank 0, single GPU run only): bounded sample of the same workload
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        # every layer of the workload at every batch size, cut to the same fraction of its output channels so that
        # the whole sample takes about 20 s
        _, probe_s, _, _ = cpu_reference_step(e, m, layers[0], batches, rows=64)
        est = probe_s / (64 * layers[0][2]) * sum(l[1] * l[2] for l in layers)
        frac = min(1.0, 20.0 / max(est, 1e-9))
        fl = secs = deq = 0.0
        parts = []
        for layer in layers:
            rows = max(64, int(layer[1] * frac) // 64 * 64)
            f_l, s_l, d_l, kind = cpu_reference_step(e, m, layer, batches, rows)
            fl, secs, deq = fl + f_l, secs + s_l, deq + d_l
            parts.append(f"{layer[0]} {rows}/{layer[1]}")
        cpu = {"value": fl / secs / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
               "sample": f"one pass over the first output channels of every layer ({', '.join(parts)}) at batch sizes "
                         f"{batches}: {secs:.2f} s, of which single-threaded dequantisation {deq:.2f} s"}

    if rank == 0:
        traffic = NCU_TRAFFIC_BYTES.get(args.workload) if (world == 1 and not args.case) else None
        line = {
            "metric": "w6a16_linear_tflops" if e == 3 else "w5a16_linear_tflops",
            "value": flops_step / sec_step / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sec_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload + (f" [{args.case} only]" if args.case else ""), "format": f"e{e}m{m}", "layers": [list(l) for l in layers], "batch_sizes": batches,
                       "split_k": "0 (library: tile waves + stream-K remainder)" if args.split_k <= 0 else args.split_k,
                       "parallelism": "single GPU" if world == 1 else (
                           f"OC-sharded x{world}, rows stored into every rank's [BS, OC] by the kernel over NVLink + arrival barrier" if exchange is not None
                           else f"OC-sharded x{world} + NCCL all-gather of [BS, OC]"),
                       "l2": f"inputs larger than L2: {replicas} replicas of the layer set ({shard_bytes * replicas / 2**20:.0f} MiB) rotated so a buffer is re-read only after >= 512 MiB of other weights",
                       "launch": "whole step replayed as a CUDA graph; kernels launched programmatically (prologue overlaps the previous kernel's tail)",
                       "static_weights": bool(f.static_weights()),
                       "programmatic_gemm_launch": bool(f.lib().fp6b200_get_option(2) == 1)},
            "weight_gbs": wbytes_step / sec_step / 1e9,
            "roofline": {"bound": "hbm", "achieved": abytes_step / world / sec_step / 1e9, "peak": hbm_peak, "unit": "GB/s",
                         "frac": abytes_step / world / sec_step / 1e9 / hbm_peak, "traffic": traffic,
                         "algorithmic_bytes_per_launch": abytes_step / world / len(cases), "peak_source": peak_kind,
                         "note": "per-GPU algorithmic bytes of all launches of a step / device time of the step; per-case fractions use min(HBM, tensor) roofline"},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_step * args.steps, "clocks": clocks,
            "device_status": status, "cases": per_case,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Orderly teardown: the graphs hold captured collectives, so they go first; a watchdog ends the process
        # if the communicator's own teardown does not return.
        import threading
        del graphs
        torch.cuda.synchronize(dev)
        dist.barrier()
        sys.stdout.flush()
        watchdog = threading.Timer(20.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        dist.destroy_process_group()
        os._exit(0)   # skip interpreter teardown: nothing is left to flush and no destructor may wait on a peer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD)
    ap.add_argument("--split-k", type=int, default=0, help="0 = let the library decompose the work")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", choices=["fused", "nccl"], default="fused", help="N > 1: how the ranks' rows reach each other")
    ap.add_argument("--per-case-multi", action="store_true",
                    help="N > 1: also time every (layer, batch) pair alone (off by default: the step time is the result)")
    ap.add_argument("--compare-cublas", action="store_true",
                    help="also time torch's fp16 GEMM on GPU-dequantised weights for every case (single GPU)")
    ap.add_argument("--no-programmatic-launch", action="store_true",
                    help="plain stream order between a GEMM and the kernel before it")
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
