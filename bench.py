#!/usr/bin/env python
"""LoRA-delta throughput benchmark (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 2..5]

A step is one pass of the hot path over one batch: for every transformer layer, the q/k/v LoRA deltas
(shrink + expand) and the o LoRA delta of all tokens of the batch.

The default workload is the S4-shaped batch (configuration 4: hidden 5120, 40 layers, 2000 adapters of rank 16/32/64
paged randomly into a [327680, 5120] fp16 pool, 512 tokens, Zipf(0.8) adapter ids) under S-LoRA tensor parallelism
over the N GPUs of the run ("strong" scaling: the same batch at every N; N = 1 is that batch on one GPU).  On one
GPU the line also carries, under ``decode_cfg2``, the S1-shaped decode batch (configuration 2: hidden 4096, 32
layers, 1000 rank-8 adapters in a [262144, 4096] pool, 256 tokens, Zipf(1.0)), the configuration the 70 %-of-roofline
target is stated on.  ``--config 2`` / ``3`` run those batches alone (replicas on N GPUs, "weak").

* ``value``: tokens/s with every input resident in HBM, the step replayed from a CUDA graph, CUDA-event timed.
* ``e2e``: the same metric through the public Python API with activations starting in pinned host memory and the
  deltas read back to the host inside the timed region.
* ``roofline``: the dominant kernel's algorithmic bytes per launch over its CUDA-event time, against the measured
  HBM copy bandwidth.
* ``parity``: one layer of the batch against the CPU oracle, before anything is timed.
* ``cpu_baseline`` / ``--impl reference``: the reference's torch per-token formula on the host cores.
* ``gpu_reference``: the reference's own BGMV CUDA kernels (compiled from the reference tree by ``oracle/Makefile``
  where that tree is present) on the same inputs, outside the timed region.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def load_workloads():
    """The workload builders, loaded by path: the CPU arm must not import the package (which loads the CUDA library)."""
    name = "slora_b200_workloads_by_path"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "slora_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=4)
    ap.add_argument("--phys-layers", type=int, default=None,
                    help="distinct layers held in HBM and cycled over the model's layer count (default: 8 for the "
                         "7B-shaped configurations, 4 for the larger ones)")
    ap.add_argument("--mode", default="auto", choices=["auto", "dp", "tp"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-plan", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-decode-extra", action="store_true",
                    help="leave out the configuration-2 figures that the default single-GPU line carries")
    ap.add_argument("--no-gpu-reference", action="store_true")
    ap.add_argument("--replays", type=int, default=100, help="graph replays behind the median figure")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--pool-rows", type=int, default=None)
    ap.add_argument("--adapters", type=int, default=None,
                    help="resident adapters, when fewer than the configuration's (small cases for the profiler)")
    ap.add_argument("--layers", type=int, default=None,
                    help="override the model's layer count (small cases for profiling; not a benchmark number)")
    ap.add_argument("--tp-exchange", default="fused", choices=["fused", "p2p", "nccl"],
                    help="tensor-parallel runs: exchange the intermediates over peer memory from inside the shrink and "
                         "expand kernels (fused), by one kernel over peer memory (p2p), or with NCCL all-gather")
    ap.add_argument("--tp-o", default="both", choices=["both", "replicated", "sharded"],
                    help="tensor-parallel runs: input of the o projection replicated, head-sharded (the rule of the "
                         "reference's figure for a row-parallel projection), or both measured (headline: replicated)")
    ap.add_argument("--prefill", action="store_true",
                    help="secondary line: long same-adapter sequences, served by the tensor-core kernels")
    ap.add_argument("--prefill-seqs", type=int, default=8)
    ap.add_argument("--prefill-len", type=int, default=512)
    ap.add_argument("--rope", action="store_true",
                    help="secondary line: rotary embedding and KV-pool scatter in the q/k/v expand's epilogue against "
                         "the same two steps as a pass of their own (configuration 2)")
    ap.add_argument("--warm-outputs", action="store_true",
                    help="secondary line: the step with the outputs written just before every call (as the base "
                         "projection's epilogue leaves them, in L2) against the step on cold outputs: what writing "
                         "y = xW + delta from one kernel could save at most")
    ap.add_argument("--scheduler", action="store_true",
                    help="secondary line: what the adapter-clustering request queue is worth on the LoRA path "
                         "(bench_sched.py)")
    ap.add_argument("--adapter-swap", action="store_true",
                    help="secondary line: pool row allocation, adapter load and offload, the library's kernels beside "
                         "the same steps on torch ops (bench_pool.py)")
    return ap.parse_args(argv)


def phys_layers_for(args, cfg):
    if args.phys_layers:
        return args.phys_layers
    return 8 if cfg in (2, 3) else 4


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
def cpu_workload(cfg, pool_rows=None, n_adapters=None):
    """The same workload (same tables, same batch, same pool size) on CPU tensors; only the rows the batch reads are
    filled."""
    return load_workloads().build_workload(cfg, device="cpu", phys_layers=1, pool_rows=pool_rows,
                                           n_adapters=n_adapters, fill="batch")


def pick_threads(call, cb):
    """The per-token loop at 1, n/2 and n torch threads, one repetition each: its speed swings by an order of
    magnitude with the thread count (tiny matrix products), so the arm runs at the fastest of the three."""
    n = os.cpu_count() or 1
    sweep = {}
    for t in sorted({1, max(1, n // 2), n}):
        torch.set_num_threads(t)
        cb.per_token_layer(*call)                     # warm-up at this setting
        t0 = time.perf_counter()
        cb.per_token_layer(*call)
        sweep[t] = time.perf_counter() - t0
    best = min(sweep, key=sweep.get)
    torch.set_num_threads(best)
    return best, {str(k): round(v, 4) for k, v in sweep.items()}


def cpu_call(wl):
    return (wl.x_qkv[0], wl.x_o[0], wl.pools_a[0], wl.pools_b[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids,
            wl.a_scaling, wl.proj_dims())


def run_cpu_baseline(cfg, seconds, pool_rows=None, n_adapters=None):
    from oracle import cpu_baseline as cb
    wl = cpu_workload(cfg, pool_rows, n_adapters)
    threads, sweep = pick_threads(cpu_call(wl), cb)
    sec_per_layer, reps = cb.time_layer(wl, min_seconds=seconds)
    sec_grouped, reps_grouped = cb.time_layer(wl, min_seconds=min(seconds, 3.0), fn=cb.grouped_layer)
    L = wl.spec.layers
    return {"value": wl.T / (sec_per_layer * L), "unit": "tokens/s", "cores": threads, "kind": "port",
            "thread_sweep_s_per_layer": sweep, "cpus": os.cpu_count(),
            "grouped_by_adapter": {"value": wl.T / (sec_grouped * L), "unit": "tokens/s",
                                   "sample": f"same layer, tokens of one adapter multiplied together, {reps_grouped} "
                                             f"repetitions, {sec_grouped:.3f} s per layer"},
            "sample": f"1 of {L} layers (q,k,v,o over the whole {wl.T}-token batch) x {reps} repetitions, "
                      f"{sec_per_layer:.3f} s per layer, extrapolated x{L}; torch per-token formula, fp32, "
                      f"{threads} threads (fastest of {sweep}) of {os.cpu_count()} cpus"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_baseline as cb
    wmod = load_workloads()
    wl = cpu_workload(args.config, args.pool_rows, args.adapters)
    L = args.layers or wl.spec.layers
    call = cpu_call(wl)
    threads, sweep = pick_threads(call, cb)
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
              f"torch per-token formula, fp32, {threads} threads (fastest of {sweep} s per layer) of "
              f"{os.cpu_count()} cpus")
    line = {"impl": "reference", "metric": "lora_delta_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sec_per_layer * L * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.config in (4, 5) else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": wmod.workload_config(wl, L, args.gpus if args.config in (4, 5) else 1),
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "thread_sweep_s_per_layer": sweep, "cpus": os.cpu_count(), "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------------
# our arm, one GPU (and independent replicas)
# ------------------------------------------------------------------------------------------------------------------
class Runner:
    """Holds one GPU's resident workload and issues steps through the public API."""

    def __init__(self, args, cfg, device, seed_shift=0):
        import slora_b200 as sl
        from slora_b200.workloads import build_workload
        self.sl = sl
        self.args = args
        self.P = phys_layers_for(args, cfg)
        wl = build_workload(cfg, device=device, phys_layers=self.P, pool_rows=args.pool_rows,
                            n_adapters=args.adapters)
        if seed_shift:
            # replicas serve different batches: redraw the per-token adapter ids
            from slora_b200.workloads import build_batch
            g = torch.Generator().manual_seed(3000 + cfg + 7919 * seed_shift)
            ids, seg = build_batch(wl.spec, g)
            wl.ids, wl.segments = ids.to(device), seg
        self.wl = wl
        self.L = args.layers or wl.spec.layers
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
        self.graph = capture_graph(self.step_eager)

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_eager()


def capture_graph(fn):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        fn()
    return g


def _graph_time(fn, launches, iters=5):
    """Microseconds per launch of `fn`'s launches, replayed from a CUDA graph (no host time between kernels)."""
    g = capture_graph(fn)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters / launches


def replay_median(step, replays, warmups=20):
    """Median (and spread) of single replays of the step, each timed by its own pair of CUDA events."""
    for _ in range(warmups):
        step()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(replays)]
    for e0, e1 in evs:
        e0.record()
        step()
        e1.record()
    torch.cuda.synchronize()
    ms = sorted(e0.elapsed_time(e1) for e0, e1 in evs)
    return {"ms_per_step_median": ms[len(ms) // 2], "ms_per_step_min": ms[0], "ms_per_step_p90": ms[int(0.9 * len(ms))],
            "replays": replays, "warmups": warmups}


# dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the same launch, from the ncu captures
# of small cases summarised under profiles/ (the same kernels on a batch of the same shape with fewer resident
# adapters; traffic grows with the adapter rows and token rows a launch streams, as the algorithmic bytes do, so the
# ratio carries over to the full launch).  Configurations without a capture print null.
NCU_TRAFFIC_RATIO = {
    (2, "expand"): ((32.76e6 + 0.016e6) / 38.93e6, "profiles/lora_pipe_kernels_cfg2_decode.md"),
    (2, "shrink"): ((28.54e6 + 0.002e6) / 28.44e6, "profiles/lora_pipe_kernels_cfg2_decode.md"),
    (4, "expand"): ((254.1e6 + 16.6e6) / 269.4e6, "profiles/lora_pipe_kernels_cfg4_mixed_ranks.md"),
    (4, "shrink"): ((243.4e6 + 4.4e6) / 243.1e6, "profiles/lora_pipe_kernels_cfg4_mixed_ranks.md"),
}


def kernel_roofline(run, peak_gbs, peak_kind):
    """Average duration of the q/k/v expand launch (the largest kernel of the step) and of the q/k/v shrink launch:
    a CUDA graph holding one launch per layer of that kernel alone, CUDA-event timed."""
    from slora_b200 import batch_infer
    wl, ops = run.wl, run.ops
    dims = wl.proj_dims()
    distinct = torch.unique(wl.ids).tolist()
    es = 2
    b_bytes = sum(wl.ranks[a] * dims[p][1] * es for a in distinct for p in range(3))
    y_bytes = wl.T * sum(2 * dims[p][1] * es for p in range(3))
    a_bytes = sum(wl.ranks[a] * dims[p][0] * es for a in distinct for p in range(3))
    x_bytes = wl.T * dims[0][0] * es
    flags = ops.flags  # programmatic launch, exact item count and tensor-core routing as the step itself uses them

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
    rows = [("lora_expand_pipe_kernel(qkv)", "expand", t_expand, b_bytes + y_bytes),
            ("lora_shrink_pipe_kernel(qkv)", "shrink", t_shrink, a_bytes + x_bytes)]
    for name, kind, t, nbytes in rows:
        ratio = NCU_TRAFFIC_RATIO.get((wl.spec.cfg, kind))
        out[kind] = {"bound": "hbm", "achieved": nbytes / t / 1e9, "peak": peak_gbs, "unit": "GB/s",
                     "frac": nbytes / t / 1e9 / peak_gbs,
                     "traffic": None if ratio is None else ratio[0] * nbytes,
                     "traffic_how": "no ncu capture of this kernel on this configuration" if ratio is None else
                     f"ncu dram bytes / algorithmic bytes of the small case in {ratio[1]}, times this launch's "
                     f"algorithmic bytes",
                     "kernel": name, "us_per_launch": t * 1e6, "algorithmic_bytes_per_launch": nbytes,
                     "peak_kind": peak_kind,
                     "how": "CUDA graph of one launch per layer of this kernel alone, CUDA events around the replay"}
    return out


def parity_check(run):
    """One layer of the batch through the public API from zeroed outputs, against the CPU oracle (adapter-grouped
    form of the per-token formula): the two normalised errors, worst projection."""
    import numpy as np
    from oracle import lora_oracle as orc
    wl, ops = run.wl, run.ops
    run.zero_outputs()
    ops.lora_get_qkv(0, wl.x_qkv[0], run.q[0], run.k[0], run.v[0])
    ops.lora_get_o(0, wl.x_o[0], run.o[0])
    torch.cuda.synchronize()
    worst = [0.0, 0.0]
    for p, got in enumerate((run.q[0], run.k[0], run.v[0], run.o[0])):
        x = wl.x_o[0] if p == 3 else wl.x_qkv[0]
        ref = orc.lora_delta_grouped(np.zeros(tuple(got.shape), dtype=np.float32), x, wl.pools_a[0], wl.pools_b[0],
                                     wl.a_start, wl.a_len, wl.a_loc, wl.ids, p, wl.a_scaling)
        mx, mn = orc.error_metrics(got, ref)
        worst = [max(worst[0], mx), max(worst[1], mn)]
    run.zero_outputs()
    return {"max_rel": worst[0], "mean_rel": worst[1], "tolerance": {"max_rel": 1e-2, "mean_rel": 1e-3},
            "ok": worst[0] <= 1e-2 and worst[1] <= 1e-3,
            "how": "layer 0, q/k/v/o deltas from zeroed outputs vs the fp32 CPU oracle, worst projection; "
                   "max|y-ref|/max|ref| and mean|y-ref|/mean|ref|"}


def gpu_reference(run, steps=5):
    """The reference's own BGMV kernels (bgmv_impl.cuh built for sm_100a into oracle/_ref/libref_bgmv.so) on this
    workload: its eight launches per layer on the legacy default stream, per-token adapter ids.  Outside every timed
    region of this library; a comparison point on the same GPU, not the oracle."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libref_bgmv.so")
    wl = run.wl
    H, R, T, L, P = wl.spec.hidden, wl.max_rank, wl.T, run.L, run.P
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libref_bgmv.so was not built (no reference tree at build time)"}
    if wl.spec.h_kv != H:
        return {"unavailable": "the reference kernels need k/v as wide as a pool row"}
    lib = ctypes.CDLL(path)
    lib.ref_dispatch_bgmv.restype = ctypes.c_int
    lib.ref_dispatch_bgmv.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                                             ctypes.c_int, ctypes.c_void_p]
    delta = [torch.zeros((T, R), dtype=wl.dtype, device=wl.ids.device) for _ in range(3)]
    ys = [run.q, run.k, run.v, run.o]

    def ref_step():
        for l in range(L):
            p = l % P
            for proj in range(4):
                x = wl.x_o[p] if proj == 3 else wl.x_qkv[p]
                d = delta[0] if proj == 3 else delta[proj]
                for out, inp, pool, hi, ho in ((d, x, wl.pools_a[p], H, R), (ys[proj][p], d, wl.pools_b[p], R, H)):
                    rc = lib.ref_dispatch_bgmv(out.data_ptr(), inp.data_ptr(), pool.data_ptr(), wl.a_start.data_ptr(),
                                               wl.a_len.data_ptr(), wl.a_loc.data_ptr(), wl.ids.data_ptr(), proj, T,
                                               hi, ho, wl.a_scaling.data_ptr())
                    if rc != 0:
                        return rc
        return 0

    torch.cuda.synchronize()
    if ref_step() != 0:
        torch.cuda.synchronize()
        return {"unavailable": f"the reference has no kernel instance for ({H}, {R})"}
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ref_step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    run.zero_outputs()
    return {"value": T / ms * 1e3, "unit": "tokens/s", "ms_per_step": ms, "launches_per_step": 8 * L, "steps": steps,
            "how": "the reference's bgmv kernels compiled for sm_100a from its own sources, eager, legacy default "
                   "stream, same inputs; timed after this library's figures were taken"}


def host_topology(local_rank):
    """NUMA node of this rank's GPU and the node count, read from sysfs (nothing is changed)."""
    out = {"numa_nodes": None, "gpu_numa_node": None}
    try:
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        out["numa_nodes"] = len(nodes)
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev = torch.cuda.get_device_properties(local_rank).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        if os.path.exists(path):
            out["gpu_numa_node"] = int(open(path).read().strip())
    except Exception:
        pass
    return out


def bind_to_gpu_node(topo):
    """With more than one NUMA node, run this process (and first-touch its pinned buffers) on the GPU's own node."""
    try:
        node = topo.get("gpu_numa_node")
        if topo.get("numa_nodes", 1) and topo["numa_nodes"] > 1 and node is not None and node >= 0:
            cpus = set()
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
            if cpus:
                os.sched_setaffinity(0, cpus)
                return True
    except Exception:
        pass
    return False


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


def measure_single(args, cfg, device, rank, world, dist, peak, extras=True):
    """Everything the line says about one configuration on one GPU (or one replica per GPU)."""
    from slora_b200.workloads import workload_config
    peak_gbs, peak_kind = peak
    local_rank = device.index or 0
    run = Runner(args, cfg, device, seed_shift=rank)
    wl = run.wl
    out = {}
    if not args.no_parity:
        out["parity"] = parity_check(run)
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
    bytes_layer = wl.algorithmic_bytes_per_layer()
    step_gbs = bytes_layer * run.L / (elapsed / args.steps) / 1e9
    out.update({
        "value": tokens / elapsed, "ms_per_step": elapsed / args.steps * 1e3,
        "us_per_layer": elapsed / args.steps / run.L * 1e6,
        "config": dict(workload_config(wl, run.L, 1), **({"parallelism": f"replicas x{world}"} if world > 1 else {}),
                       l2="inputs larger than L2: %d MiB of adapter rows and activations touched per step over %d "
                          "physical layers, no reuse between layers" % (bytes_layer * min(run.P, run.L) // 2 ** 20,
                                                                        run.P)),
        "run": {"phys_layers": run.P, "graph": not args.no_graph, "pdl": not args.no_pdl, "plan": not args.no_plan,
                "flags": run.ops.flags, "launches_per_step": run.launches_per_step},
        "step_hbm": {"algorithmic_bytes_per_step": bytes_layer * run.L, "achieved": step_gbs, "peak": peak_gbs,
                     "frac": step_gbs / peak_gbs, "unit": "GB/s", "peak_kind": peak_kind,
                     "gathered_bytes_per_step": wl.gathered_bytes_per_layer() * run.L,
                     "frac_of_nominal_8TBs": step_gbs / 8000.0},
        "gpu_launches": run.launches_per_step * args.steps, "clocks": clocks.summary(),
    })
    if not args.no_graph and args.replays > 0:
        med = replay_median(run.step, args.replays)
        med["tokens_per_s_median"] = wl.T / med["ms_per_step_median"] * 1e3
        out["replay_median"] = med
    roof = kernel_roofline(run, peak_gbs, peak_kind)
    out["roofline"] = roof["expand"]
    out["roofline_kernels"] = roof
    if extras and not args.no_e2e:
        e_steps = max(3, min(args.steps, 10))
        e_time, h2d, d2h = e2e_measure(run, e_steps, 3)
        if dist is not None:
            t = torch.tensor([e_time], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_time = float(t.item())
        out["e2e"] = {"value": wl.T * e_steps * world / e_time, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": d2h, "steps": e_steps, "ms_per_step": e_time / e_steps * 1e3,
                      "h2d_gbs_per_gpu": h2d / (e_time / e_steps) / 1e9, "d2h_gbs_per_gpu": d2h / (e_time / e_steps) / 1e9,
                      "host": host_topology(local_rank)}
    if extras and rank == 0 and not args.no_gpu_reference:
        out["gpu_reference"] = gpu_reference(run)
    del run
    torch.cuda.empty_cache()
    return out


def prefill_bench(args, device, peak):
    """Secondary workload: long same-adapter sequences, S2-shaped (hidden 4096, ranks 8..64).  Sequences of 32 tokens
    or more run on the tensor cores.  Two ways in: the reference's prefill entry points (lora_get_qkvo_fwd_shrink /
    _expand, one call per projection and direction) and LoraBatchOps (one q/k/v call and one o call per layer, the
    activations read once for q, k and v).  A step is q, k, v, o shrink + expand of every layer; prints its own line."""
    import slora_b200 as sl
    from slora_b200.workloads import build_workload
    peak_gbs, peak_kind = peak
    P = phys_layers_for(args, 3)
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
    ops = sl.LoraBatchOps(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling, wl.pools_a, wl.pools_b, R,
                          use_pdl=not args.no_pdl)
    ops.prepare(wl.ids)

    def step_segments():
        for l in range(L):
            p = l % P
            for proj in range(4):
                x = wl.x_o[p] if proj == 3 else wl.x_qkv[p]
                sl.lora_get_qkvo_fwd_shrink(x, wl.pools_a[p], delta, wl.a_loc, wl.a_start, wl.a_len, b_start, b_len,
                                            req, H, proj, R, max_len)
                sl.lora_get_qkvo_fwd_expand(delta, wl.pools_b[p], ys[p][proj], wl.a_scaling, wl.a_loc, wl.a_start,
                                            wl.a_len, b_start, b_len, req, H, proj, R, max_len)

    def step_batch_ops():
        for l in range(L):
            p = l % P
            ops.lora_get_qkv(p, wl.x_qkv[p], ys[p][0], ys[p][1], ys[p][2])
            ops.lora_get_o(p, wl.x_o[p], ys[p][3])

    es = 2
    distinct = sorted(set(a for _, _, a in seg))
    w_bytes = sum(wl.ranks[a] * 2 * H * es for a in distinct) * 4
    act_bytes = wl.T * H * es * (2 + 8)  # x read for q/k/v and for o; y read and written for four projections
    step_bytes = (w_bytes + act_bytes) * L
    flops = sum(2 * n * wl.ranks[a] * 2 * H for _, n, a in seg) * 4 * L
    results = {}
    clocks = None
    for name, step in (("segment_api", step_segments), ("batch_ops", step_batch_ops)):
        before = sl.launch_counts()
        step()
        torch.cuda.synchronize()
        after = sl.launch_counts()
        per_step = {k: after[k] - before[k] for k in after}
        graph = None if args.no_graph else capture_graph(step)
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
        sec = t0.elapsed_time(t1) * 1e-3 / args.steps
        gbs = step_bytes / sec / 1e9
        results[name] = {"value": wl.T / sec, "unit": "tokens/s", "ms_per_step": sec * 1e3,
                         "hbm": {"achieved": gbs, "peak": peak_gbs, "frac": gbs / peak_gbs, "unit": "GB/s"},
                         "tflops": flops / sec / 1e12, "launches_per_step": per_step, "graph": graph is not None}
    best = max(results, key=lambda k: results[k]["value"])
    r = results[best]
    line = {"metric": "lora_prefill_tokens_per_s", "value": r["value"], "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 in, f32 accumulate (tcgen05)", "data": "synthetic",
            "config": {"workload": "cfg3-S2-prefill-segments", "sequences": len(seg), "tokens": wl.T, "layers": L,
                       "hidden": H, "ranks": sorted(set(wl.ranks[a] for a in distinct)), "phys_layers": P,
                       "entry": best},
            "roofline": {"bound": "hbm", "achieved": r["hbm"]["achieved"], "peak": peak_gbs, "unit": "GB/s",
                         "frac": r["hbm"]["frac"], "traffic": None, "peak_kind": peak_kind, "tflops": r["tflops"],
                         "kernel": "whole step (lora_shrink_mma_kernel + lora_expand_mma_kernel)"},
            "entries": results,
            "gpu_launches": sum(r["launches_per_step"].values()) * args.steps, "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


def rope_bench(args, device, peak):
    """What folding the rotary embedding of q, k and the KV-pool scatter of k, v into the q/k/v expand saves
    (S1-shaped decode batch): per layer, the plain q/k/v call; the call with both steps in the expand's epilogue; the
    call followed by the two steps as one pass of their own (the reference runs four more launches here: rotary q,
    rotary k, scatter k, scatter v)."""
    import subprocess
    import slora_b200 as sl
    from slora_b200.workloads import build_workload
    if os.environ.get("SLORA_ROPE_EPILOGUE") is None and not args.no_graph:
        # the separate-pass figure needs the library's switch, read once per process: a child process measures it
        env = dict(os.environ, SLORA_ROPE_EPILOGUE="0")
        child = subprocess.run([sys.executable, os.path.abspath(__file__), "--rope"], env=env, capture_output=True,
                               text=True)
        separate = json.loads(child.stdout.strip().splitlines()[-1]) if child.returncode == 0 else None
    else:
        separate = None
    peak_gbs, _ = peak
    P = phys_layers_for(args, 2)
    wl = build_workload(2, device=device, phys_layers=P, pool_rows=args.pool_rows)
    L, T, H = args.layers or wl.spec.layers, wl.T, wl.spec.hidden
    dt = wl.dtype
    ops = sl.LoraBatchOps(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling, wl.pools_a, wl.pools_b, wl.max_rank,
                          use_pdl=not args.no_pdl)
    ops.prepare(wl.ids)
    q = [torch.zeros((T, H), dtype=dt, device=device) for _ in range(P)]
    k = [torch.zeros((T, H), dtype=dt, device=device) for _ in range(P)]
    v = [torch.zeros((T, H), dtype=dt, device=device) for _ in range(P)]
    kpool = [torch.zeros((4096, H), dtype=dt, device=device) for _ in range(P)]
    vpool = [torch.zeros((4096, H), dtype=dt, device=device) for _ in range(P)]
    rows = torch.randperm(4096, device=device)[:T].to(torch.int64)
    ang = torch.rand((T, 64), device=device) * 6.28
    cos, sin = torch.cos(ang).to(dt), torch.sin(ang).to(dt)

    def plain():
        for l in range(L):
            p = l % P
            ops.lora_get_qkv(p, wl.x_qkv[p], q[p], k[p], v[p])

    def with_steps():
        for l in range(L):
            p = l % P
            ops.lora_get_qkv(p, wl.x_qkv[p], q[p], k[p], v[p], rope=(cos, sin), kv_dest=(rows, kpool[p], vpool[p]))

    t_plain = _graph_time(plain, L)
    t_steps = _graph_time(with_steps, L)
    es = 2
    extra_bytes = T * (2 * H * es * 2 + 2 * H * es * 2)      # rotary q, k read + write; k, v rows read + written
    line = {"metric": "rotary_and_kv_scatter_cost_per_layer", "unit": "us per layer (q/k/v call)",
            "workload": wl.spec.name, "layers": L, "tokens": T,
            "qkv_call_plain_us": t_plain,
            "qkv_call_with_both_steps_us": t_steps,
            "how_the_steps_ran": "a pass of their own after the expand" if os.environ.get("SLORA_ROPE_EPILOGUE") == "0"
            else "in the expand's epilogue",
            "bytes_of_a_separate_pass_per_layer": extra_bytes,
            "separate_pass_at_measured_hbm_peak_us": extra_bytes / peak_gbs / 1e3}
    if separate is not None:
        line["qkv_call_with_separate_pass_us"] = separate["qkv_call_with_both_steps_us"]
        line["value"] = separate["qkv_call_with_both_steps_us"] - t_steps
        line["value_is"] = "us per layer saved by the epilogue against the separate pass"
    return line


def warm_outputs_bench(args, device, peak):
    """Upper bound of what a fused base projection + delta kernel would save: in the reference's layer the base
    torch.mm writes y right before the LoRA calls read it, so y is in the 126 MB L2, not in HBM.  Per layer: the LoRA
    step on outputs nobody touched since the previous pass over the physical layers (the main benchmark's setting:
    y read from HBM); the same step with a fill of q, k, v (and o) issued before each call, minus the fills alone."""
    import slora_b200 as sl
    from slora_b200.workloads import build_workload
    cfg = args.config if args.config in (2, 4) else 2
    P = phys_layers_for(args, cfg)
    wl = build_workload(cfg, device=device, phys_layers=P, pool_rows=args.pool_rows)
    L, T, H, K = args.layers or wl.spec.layers, wl.T, wl.spec.hidden, wl.spec.h_kv
    dt = wl.dtype
    ops = sl.LoraBatchOps(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling, wl.pools_a, wl.pools_b, wl.max_rank,
                          use_pdl=not args.no_pdl)
    ops.prepare(wl.ids)
    q = [torch.zeros((T, H), dtype=dt, device=device) for _ in range(P)]
    k = [torch.zeros((T, K), dtype=dt, device=device) for _ in range(P)]
    v = [torch.zeros((T, K), dtype=dt, device=device) for _ in range(P)]
    o = [torch.zeros((T, H), dtype=dt, device=device) for _ in range(P)]

    # A kernel of another library between the calls (here a fill, in the reference's layer the base projection and
    # the attention) also ends the chain of programmatic dependent launches, so both settings get one: a fill of the
    # whole output ("warm": y is in L2 when the call reads it) or of one element of it ("cold").
    def step(lora, whole):
        for l in range(L):
            p = l % P
            for t in (q[p], k[p], v[p]):
                (t if whole else t[:1, :8]).fill_(0.5)
            if lora:
                ops.lora_get_qkv(p, wl.x_qkv[p], q[p], k[p], v[p])
            (o[p] if whole else o[p][:1, :8]).fill_(0.5)
            if lora:
                ops.lora_get_o(p, wl.x_o[p], o[p])

    cold = _graph_time(lambda: step(True, False), L) - _graph_time(lambda: step(False, False), L)
    both = _graph_time(lambda: step(True, True), L)
    fills = _graph_time(lambda: step(False, True), L)
    y_bytes = T * (2 * H + 2 * K) * 2
    return {"metric": "lora_step_with_outputs_in_l2", "unit": "us per layer", "workload": wl.spec.name, "layers": L,
            "tokens": T, "cold_outputs_us": cold, "fills_then_lora_us": both, "fills_alone_us": fills,
            "warm_outputs_us": both - fills, "value": cold - (both - fills),
            "value_is": "us per layer that reading y from L2 instead of HBM saves: the most a fused base projection "
                        "+ delta kernel could add on top of what the L2 already gives",
            "y_bytes_per_layer": y_bytes, "y_read_at_measured_hbm_peak_us": y_bytes / peak[0] / 1e3}


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
    bind_to_gpu_node(host_topology(local_rank))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    peak = load_peaks()
    mode = args.mode
    if mode == "auto":
        mode = "tp" if (args.config in (4, 5) and world > 1) else "dp"
    if mode == "tp" and world > 1:
        import bench_tp
        bench_tp.run(args, dist, rank, world, device, peak)
        return
    if args.prefill:
        prefill_bench(args, device, peak)
        return
    if args.rope:
        if rank == 0:
            print(json.dumps(rope_bench(args, device, peak)), flush=True)
        return
    if args.warm_outputs:
        if rank == 0:
            print(json.dumps(warm_outputs_bench(args, device, peak)), flush=True)
        return
    if args.scheduler:
        import bench_sched
        if rank == 0:
            print(json.dumps(bench_sched.run(device)), flush=True)
        return
    if args.adapter_swap:
        import bench_pool
        if rank == 0:
            print(json.dumps(bench_pool.run()), flush=True)
        return

    cfg = args.config
    m = measure_single(args, cfg, device, rank, world, dist, peak)
    decode = None
    if cfg == 4 and world == 1 and not args.no_decode_extra and not (args.adapters or args.pool_rows or args.layers):
        decode = measure_single(args, 2, device, rank, world, dist, peak, extras=False)
    cpu, bad = None, []
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = run_cpu_baseline(cfg, args.cpu_seconds, args.pool_rows, args.adapters)
    if rank == 0:
        line = {
            "metric": "lora_delta_tokens_per_s", "value": m["value"], "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": m["ms_per_step"],
            "higher_is_better": True, "scaling": "strong" if cfg in (4, 5) else "weak",
            # no published number exists for this metric (the reference records end-to-end requests/s only), so there
            # is nothing to divide by; the ratio to the CPU arm is the driver's to compute from the two lines
            "vs_baseline": None,
            "dtype": "f16 in, f32 accumulate", "data": "synthetic", "config": m["config"], "run": m["run"],
            "us_per_layer": m["us_per_layer"], "parity": m.get("parity"), "roofline": m["roofline"],
            "roofline_kernels": m["roofline_kernels"], "step_hbm": m["step_hbm"],
            "replay_median": m.get("replay_median"), "cpu_baseline": cpu, "e2e": m.get("e2e"),
            "gpu_reference": m.get("gpu_reference"), "gpu_launches": m["gpu_launches"], "clocks": m["clocks"],
        }
        if decode is not None:
            line["decode_cfg2"] = {k: decode.get(k) for k in ("value", "ms_per_step", "us_per_layer", "config", "run",
                                                              "parity", "roofline", "roofline_kernels", "step_hbm",
                                                              "replay_median", "clocks")}
            line["decode_cfg2"]["unit"] = "tokens/s"
            line["gpu_launches"] += decode["gpu_launches"]
        bad = [p for p in (line.get("parity"), (line.get("decode_cfg2") or {}).get("parity")) if p and not p["ok"]]
        if bad:
            line["invalid"] = "parity check against the CPU oracle failed; the figures of this line do not count"
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and bad:
        raise SystemExit(4)


if __name__ == "__main__":
    main()
