#!/usr/bin/env python
"""LoRA-delta throughput benchmark (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 2..5]

A step is one pass of the hot path over one batch: for every transformer layer, the q/k/v LoRA deltas
(shrink + expand) and the o LoRA delta of all tokens of the batch.  The default workload is the S1-shaped decode
batch (configuration 2: hidden 4096, 32 layers, 1000 rank-8 adapters paged randomly into a [262144, 4096] fp16
pool, 256 tokens with Zipf(1.0) adapter ids), drawn from seeded generators.

* ``value``: tokens/s with every input resident in HBM, the step replayed from a CUDA graph, CUDA-event timed.
* ``e2e``: the same metric through the public Python API (LoraBatchOps) with activations starting in pinned host
  memory and the deltas read back to the host inside the timed region.
* ``roofline``: the dominant kernel's algorithmic bytes per launch over its CUDA-event time, against the measured
  HBM copy bandwidth.
* ``cpu_baseline`` / ``--impl reference``: the reference's torch per-token formula on the host cores.

Multi-GPU: configurations 2 and 3 (7B-shaped, one GPU holds everything) run as independent replicas, one batch per
GPU ("weak"); configurations 4 and 5 run under S-LoRA tensor parallelism ("strong").
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--phys-layers", type=int, default=8,
                    help="distinct layers held in HBM and cycled over the model's layer count")
    ap.add_argument("--mode", default="auto", choices=["auto", "dp", "tp"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-plan", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--pool-rows", type=int, default=None)
    ap.add_argument("--adapters", type=int, default=None,
                    help="resident adapters, when fewer than the configuration's (small cases for the profiler)")
    ap.add_argument("--layers", type=int, default=None,
                    help="override the model's layer count (small cases for profiling; not a benchmark number)")
    ap.add_argument("--tp-exchange", default="fused", choices=["fused", "p2p", "nccl"],
                    help="tensor-parallel runs: exchange the intermediates over peer memory from inside the shrink and "
                         "expand kernels (fused), by one kernel over peer memory (p2p), or with NCCL all-gather")
    ap.add_argument("--prefill", action="store_true",
                    help="secondary line: the segment (prefill) API on long sequences, served by the tensor-core kernels")
    ap.add_argument("--prefill-seqs", type=int, default=8)
    ap.add_argument("--prefill-len", type=int, default=512)
    ap.add_argument("--adapter-swap", action="store_true",
                    help="secondary line: pool row allocation, adapter load and offload, the library's kernels beside "
                         "the same steps on torch ops (slora_b200/pool_bench.py)")
    return ap.parse_args()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

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

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return False

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ------------------------------------------------------------------------------------------------------------------
# the reference arm: the reference's CPU formulation of the path on the host cores
# ------------------------------------------------------------------------------------------------------------------
def cpu_workload(cfg, pool_rows):
    from slora_b200.workloads import build_workload
    return build_workload(cfg, device="cpu", phys_layers=1, pool_rows=pool_rows)


def run_cpu_baseline(cfg, pool_rows, seconds):
    from oracle import cpu_baseline as cb
    wl = cpu_workload(cfg, pool_rows)
    sec_per_layer, reps = cb.time_layer(wl, min_seconds=seconds)
    sec_grouped, reps_grouped = cb.time_layer(wl, min_seconds=min(seconds, 3.0), fn=cb.grouped_layer)
    L = wl.spec.layers
    return {"value": wl.T / (sec_per_layer * L), "unit": "tokens/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "grouped_by_adapter": {"value": wl.T / (sec_grouped * L), "unit": "tokens/s",
                                   "sample": f"same layer, tokens of one adapter multiplied together, {reps_grouped} "
                                             f"repetitions, {sec_grouped:.3f} s per layer"},
            "sample": f"1 of {L} layers (q,k,v,o over the whole {wl.T}-token batch) x {reps} repetitions, "
                      f"{sec_per_layer:.3f} s per layer, extrapolated x{L}; torch per-token formula, fp32, "
                      f"{torch.get_num_threads()} threads of {os.cpu_count()} cpus"}, wl


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_baseline as cb
    from slora_b200.workloads import SPECS
    pool_rows = args.pool_rows or min(SPECS[args.config].pool_rows, 65536 if args.config != 4 else 327680)
    wl = cpu_workload(args.config, pool_rows)
    L = wl.spec.layers
    call = (wl.x_qkv[0], wl.x_o[0], wl.pools_a[0], wl.pools_b[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids,
            wl.a_scaling, wl.proj_dims())
    for _ in range(max(1, min(args.warmup, 3))):
        cb.per_token_layer(*call)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        cb.per_token_layer(*call)
        times.append(time.perf_counter() - t0)
    sec_per_layer = sum(times) / len(times)
    value = wl.T / (sec_per_layer * L)
    sample = (f"each step = 1 of {L} layers (q,k,v,o over the whole {wl.T}-token batch), extrapolated x{L}; "
              f"torch per-token formula, fp32, {torch.get_num_threads()} threads")
    line = {"impl": "reference", "metric": "lora_delta_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sec_per_layer * L * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl.spec.name, "tokens": wl.T, "layers": L, "hidden": wl.spec.hidden,
                       "adapters": wl.spec.n_adapters, "pool_rows": pool_rows},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------------------
class Runner:
    """Holds one GPU's resident workload and issues steps through the public API."""

    def __init__(self, args, cfg, device, seed_shift=0):
        import slora_b200 as sl
        from slora_b200.workloads import build_workload
        self.sl = sl
        self.args = args
        wl = build_workload(cfg, device=device, phys_layers=args.phys_layers, pool_rows=args.pool_rows,
                            n_adapters=args.adapters)
        if seed_shift:
            # replicas serve different batches: redraw the per-token adapter ids
            from slora_b200.workloads import build_batch
            g = torch.Generator().manual_seed(3000 + cfg + 7919 * seed_shift)
            ids, seg = build_batch(wl.spec, g)
            wl.ids, wl.segments = ids.to(device), seg
        self.wl = wl
        self.L = args.layers or wl.spec.layers
        self.P = args.phys_layers
        H, K = wl.spec.hidden, wl.spec.h_kv
        dt = wl.dtype
        self.q = [torch.zeros((wl.T, H), dtype=dt, device=device) for _ in range(self.P)]
        self.k = [torch.zeros((wl.T, K), dtype=dt, device=device) for _ in range(self.P)]
        self.v = [torch.zeros((wl.T, K), dtype=dt, device=device) for _ in range(self.P)]
        self.o = [torch.zeros((wl.T, H), dtype=dt, device=device) for _ in range(self.P)]
        self.ops = sl.LoraBatchOps(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling, wl.pools_a, wl.pools_b, wl.max_rank,
                                   use_pdl=not args.no_pdl)
        self.ops.prepare(wl.ids, use_plan=not args.no_plan)
        self.launches_per_step = 4 * self.L  # replaced by the library's own count of the first eager step
        self.graph = None

    def zero_outputs(self):
        for bufs in (self.q, self.k, self.v, self.o):
            for b in bufs:
                b.zero_()

    def step_eager(self):
        ops, wl = self.ops, self.wl
        for l in range(self.L):
            p = l % self.P
            ops.lora_get_qkv(p, wl.x_qkv[p], self.q[p], self.k[p], self.v[p])
            ops.lora_get_o(p, wl.x_o[p], self.o[p])

    def capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.step_eager()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            self.step_eager()
        self.graph = g

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_eager()


def _graph_time(fn, launches, iters=5):
    """Microseconds per launch of `fn`'s launches, replayed from a CUDA graph (no host time between kernels)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters / launches


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in
# profiles/lora_pipe_kernels_cfg2_decode.md (same batch and per-launch work as the benchmark's; y stays in L2 there)
NCU_TRAFFIC = {(2, "lora_pipe_kernel<expand>(qkv)"): 32.76e6 + 0.016e6,
               (2, "lora_pipe_kernel<shrink>(qkv)"): 28.54e6 + 0.002e6}


def kernel_roofline(run, peak_gbs, peak_kind):
    """Average duration of the q/k/v expand launch (the largest kernel of the step) and of the q/k/v shrink launch:
    a CUDA graph holding one launch per layer of that kernel alone, CUDA-event timed."""
    from slora_b200 import batch_infer, _lib
    wl, ops = run.wl, run.ops
    dims = wl.proj_dims()
    distinct = torch.unique(wl.ids).tolist()
    es = 2
    b_bytes = sum(wl.ranks[a] * dims[p][1] * es for a in distinct for p in range(3))
    y_bytes = wl.T * sum(2 * dims[p][1] * es for p in range(3))
    a_bytes = sum(wl.ranks[a] * dims[p][0] * es for a in distinct for p in range(3))
    x_bytes = wl.T * dims[0][0] * es
    flags = ops.flags  # programmatic launch and tensor-core routing as the step itself uses them

    def shrinks():
        for l in range(run.L):
            p = l % run.P
            batch_infer.shrink_multi(ops.plan, wl.ids, [0, 1, 2], ops.delta, wl.x_qkv[p], wl.pools_a[p], wl.a_start,
                                     wl.a_len, wl.a_loc, flags)

    def expands():
        for l in range(run.L):
            p = l % run.P
            batch_infer.expand_multi(ops.plan, wl.ids, [0, 1, 2], [run.q[p], run.k[p], run.v[p]], ops.delta,
                                     wl.pools_b[p], wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling,
                                     ops.delta[0].stride(0), wl.max_rank, flags=flags)

    t_shrink = _graph_time(shrinks, run.L) * 1e-6
    t_expand = _graph_time(expands, run.L) * 1e-6
    out = {}
    for name, t, nbytes in (("lora_pipe_kernel<expand>(qkv)", t_expand, b_bytes + y_bytes),
                            ("lora_pipe_kernel<shrink>(qkv)", t_shrink, a_bytes + x_bytes)):
        out[name] = {"bound": "hbm", "achieved": nbytes / t / 1e9, "peak": peak_gbs, "unit": "GB/s",
                     "frac": nbytes / t / 1e9 / peak_gbs, "traffic": NCU_TRAFFIC.get((wl.spec.cfg, name)),
                     "kernel": name,
                     "us_per_launch": t * 1e6, "algorithmic_bytes_per_launch": nbytes, "peak_kind": peak_kind,
                     "how": "CUDA graph of one launch per layer of this kernel alone, CUDA events around the replay"}
    return out


def e2e_measure(run, steps, warmup):
    """Steps through LoraBatchOps with activations in pinned host memory and results copied back to the host."""
    sl, wl = run.sl, run.wl
    L, T, H, K = run.L, wl.T, wl.spec.hidden, wl.spec.h_kv
    dt = wl.dtype
    dev = wl.ids.device
    g = torch.Generator().manual_seed(77)
    x_host = torch.randn((L, 2, T, H), generator=g, dtype=torch.float32).to(dt).pin_memory()
    ids_host = wl.ids.cpu().pin_memory()
    x_dev = torch.empty((L, 2, T, H), dtype=dt, device=dev)
    ids_dev = torch.empty_like(wl.ids)
    y_dev = torch.zeros((L, T, 2 * H + 2 * K), dtype=dt, device=dev)
    y_host = torch.empty((L, T, 2 * H + 2 * K), dtype=dt).pin_memory()
    ops = sl.LoraBatchOps(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling, wl.pools_a, wl.pools_b, wl.max_rank,
                          use_pdl=not run.args.no_pdl)
    h2d = x_host.numel() * x_host.element_size() + ids_host.numel() * 8
    d2h = y_host.numel() * y_host.element_size()
    # Three streams: activations of layer l+1.. upload and deltas of layer l-1.. download while layer l computes
    # (PCIe is full duplex), the way a serving loop would feed a layer-by-layer model.
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(L)]
    ev_done = [torch.cuda.Event() for _ in range(L)]
    times = []
    for it in range(warmup + steps):
        y_dev.zero_()
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            for l in range(L):
                x_dev[l].copy_(x_host[l], non_blocking=True)
                ev_in[l].record(s_in)
        ids_dev.copy_(ids_host, non_blocking=True)
        ops.prepare(ids_dev, use_plan=not run.args.no_plan)
        for l in range(L):
            p = l % run.P
            yl = y_dev[l]
            cur.wait_event(ev_in[l])
            ops.lora_get_qkv(p, x_dev[l, 0], yl[:, :H], yl[:, H:H + K], yl[:, H + K:H + 2 * K])
            ops.lora_get_o(p, x_dev[l, 1], yl[:, H + 2 * K:])
            ev_done[l].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[l])
                y_host[l].copy_(yl, non_blocking=True)
        cur.wait_stream(s_out)
        t1.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(t0.elapsed_time(t1) * 1e-3)
    return sum(times), h2d, d2h


def prefill_bench(args, device, peak_gbs):
    """Secondary workload: the reference's prefill entry points (lora_get_qkvo_fwd_shrink / _expand) over long
    same-adapter sequences, S2-shaped (hidden 4096, ranks 8..64).  Sequences of 32 tokens or more run on the tensor
    cores.  A step is q, k, v, o shrink + expand of every layer; prints its own JSON line."""
    import slora_b200 as sl
    from slora_b200.workloads import build_workload
    peak, peak_kind = peak_gbs
    P = args.phys_layers
    wl = build_workload(3, device=device, phys_layers=P, pool_rows=args.pool_rows or 65536, decode_tokens=0,
                        prefill=("seqs", args.prefill_seqs, args.prefill_len, args.prefill_len))
    L, H, R = args.layers or wl.spec.layers, wl.spec.hidden, wl.max_rank
    seg = wl.segments
    b_start = torch.tensor([s for s, _, _ in seg], dtype=torch.int32, device=device)
    b_len = torch.tensor([n for _, n, _ in seg], dtype=torch.int32, device=device)
    req = torch.tensor([a for _, _, a in seg], dtype=torch.int64, device=device)
    max_len = max(n for _, n, _ in seg)
    delta = torch.zeros((wl.T, R), dtype=wl.dtype, device=device)
    ys = [[torch.zeros((wl.T, H), dtype=wl.dtype, device=device) for _ in range(4)] for _ in range(P)]

    def step():
        for l in range(L):
            p = l % P
            for proj in range(4):
                x = wl.x_o[p] if proj == 3 else wl.x_qkv[p]
                sl.lora_get_qkvo_fwd_shrink(x, wl.pools_a[p], delta, wl.a_loc, wl.a_start, wl.a_len, b_start, b_len,
                                            req, H, proj, R, max_len)
                sl.lora_get_qkvo_fwd_expand(delta, wl.pools_b[p], ys[p][proj], wl.a_scaling, wl.a_loc, wl.a_start,
                                            wl.a_len, b_start, b_len, req, H, proj, R, max_len)

    before = sl.launch_counts()
    step()
    torch.cuda.synchronize()
    after = sl.launch_counts()
    per_step = {k: after[k] - before[k] for k in after}
    graph = None
    if not args.no_graph:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            step()
    run = graph.replay if graph is not None else step
    for _ in range(max(args.warmup, 3)):
        run()
    torch.cuda.synchronize()
    with ClockSampler(physical_gpu_index(device.index or 0)) as clocks:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            run()
        t1.record()
        torch.cuda.synchronize()
    elapsed = t0.elapsed_time(t1) * 1e-3
    es = 2
    distinct = sorted(set(a for _, _, a in seg))
    w_bytes = sum(wl.ranks[a] * 2 * H * es for a in distinct) * 4
    act_bytes = wl.T * H * es * (2 + 8)  # x read for q/k/v and for o; y read and written for four projections
    step_bytes = (w_bytes + act_bytes) * L
    flops = sum(2 * n * wl.ranks[a] * 2 * H for _, n, a in seg) * 4 * L
    gbs = step_bytes / (elapsed / args.steps) / 1e9
    line = {"metric": "lora_prefill_tokens_per_s", "value": wl.T * args.steps / elapsed, "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 in, f32 accumulate (tcgen05)", "data": "synthetic",
            "config": {"workload": "cfg3-S2-prefill-segments", "sequences": len(seg), "tokens": wl.T, "layers": L,
                       "hidden": H, "ranks": sorted(set(wl.ranks[a] for a in distinct)), "phys_layers": P,
                       "graph": graph is not None},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                         "traffic": None, "peak_kind": peak_kind, "tflops": flops / (elapsed / args.steps) / 1e12,
                         "kernel": "whole step (lora_shrink_mma_kernel + lora_expand_mma_kernel per projection)"},
            "gpu_launches": sum(per_step.values()) * args.steps, "launches_per_step": per_step,
            "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    mode = args.mode
    if mode == "auto":
        mode = "tp" if (args.config in (4, 5) and world > 1) else "dp"
    if mode == "tp" and world > 1:
        from slora_b200 import tp_bench
        tp_bench.run(args, dist, rank, world, device)
        return

    peak_gbs, peak_kind = load_peaks()
    if args.prefill:
        prefill_bench(args, device, peak_gbs=load_peaks())
        return
    if args.adapter_swap:
        from slora_b200 import pool_bench
        if rank == 0:
            print(json.dumps(pool_bench.run()), flush=True)
        return
    run = Runner(args, args.config, device, seed_shift=rank)
    wl = run.wl
    before = sum(run.sl.launch_counts().values())
    run.step_eager()
    torch.cuda.synchronize()
    run.launches_per_step = sum(run.sl.launch_counts().values()) - before
    run.ops.plan and run.ops.plan.check()
    if not args.no_graph:
        run.capture()
    for _ in range(max(args.warmup, 3)):
        run.step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            run.step()
        t1.record()
        torch.cuda.synchronize()
    elapsed = t0.elapsed_time(t1) * 1e-3
    if dist is not None:
        dist.barrier()
        t = torch.tensor([elapsed], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = float(t.item())
    tokens = wl.T * args.steps * world
    value = tokens / elapsed
    ms_per_step = elapsed / args.steps * 1e3
    bytes_layer = wl.algorithmic_bytes_per_layer()
    step_gbs = bytes_layer * run.L / (elapsed / args.steps) / 1e9

    roof = kernel_roofline(run, peak_gbs, peak_kind)
    e2e = None
    if not args.no_e2e:
        e_time, h2d, d2h = e2e_measure(run, max(3, min(args.steps, 10)), 3)
        e_steps = max(3, min(args.steps, 10))
        if dist is not None:
            t = torch.tensor([e_time], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_time = float(t.item())
        e2e = {"value": wl.T * e_steps * world / e_time, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": e_steps, "ms_per_step": e_time / e_steps * 1e3}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu, _ = run_cpu_baseline(args.config, min(wl.spec.pool_rows, 65536 if args.config != 4 else 327680),
                                  args.cpu_seconds)
    if rank == 0:
        main_roof = roof["lora_pipe_kernel<expand>(qkv)"]
        line = {
            "metric": "lora_delta_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": {"workload": wl.spec.name, "tokens_per_gpu": wl.T, "layers": run.L, "hidden": wl.spec.hidden,
                       "kv_width": wl.spec.h_kv, "adapters": wl.spec.n_adapters, "max_rank": wl.max_rank,
                       "distinct_adapters_in_batch": len(torch.unique(wl.ids)), "pool_rows": wl.spec.pool_rows,
                       "phys_layers": run.P, "parallelism": f"replicas x{world}" if world > 1 else "1 gpu",
                       "l2": "inputs larger than L2: %d MiB of adapter rows and activations touched per step, no "
                             "reuse between layers" % (bytes_layer * min(run.P, run.L) // 2 ** 20),
                       "graph": not args.no_graph, "pdl": not args.no_pdl, "plan": not args.no_plan},
            "roofline": main_roof,
            "roofline_shrink": roof["lora_pipe_kernel<shrink>(qkv)"],
            "step_hbm": {"algorithmic_bytes_per_step": bytes_layer * run.L, "achieved": step_gbs, "peak": peak_gbs,
                         "frac": step_gbs / peak_gbs, "unit": "GB/s", "peak_kind": peak_kind,
                         "gathered_bytes_per_step": wl.gathered_bytes_per_layer() * run.L,
                         "frac_of_nominal_8TBs": step_gbs / 8000.0},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": run.launches_per_step * args.steps,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
