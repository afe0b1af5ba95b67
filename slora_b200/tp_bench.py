"""Tensor-parallel leg of the benchmark: one process per GPU, NCCL all-gather of the rank-r intermediates.

Each rank holds its shard of every adapter (A: r/N rank rows, B: h_out/N output rows) for a few physical layers and
runs the model's layer count over them; activations are replicated, outputs are the rank's [T, h_out/N] slices.
Time is CUDA-event time of K steps, maximum over ranks; tokens/s counts the batch once (strong scaling).
"""
from __future__ import annotations

import json
import os

import torch


def run(args, dist, rank, world, device):
    from . import tp
    from .workloads import build_workload

    cfg = args.config
    pool_rows = args.pool_rows
    wl = build_workload(cfg, device=device, phys_layers=args.phys_layers, pool_rows=pool_rows, rank_div=world)
    spec = wl.spec
    H, K, T, L, P = spec.hidden, spec.h_kv, wl.T, spec.layers, args.phys_layers
    tables = tp.TpTables(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling)
    ops = tp.TpLoraOps(tables, wl.pools_a, wl.pools_b, wl.max_rank, world, rank,
                       tp.CudaBackend(use_pdl=not args.no_pdl, fused=args.tp_exchange == "fused"),
                       peer_exchange=args.tp_exchange != "nccl").prepare(wl.ids)
    dt = wl.dtype
    q = [torch.zeros((T, H // world), dtype=dt, device=device) for _ in range(P)]
    k = [torch.zeros((T, K // world), dtype=dt, device=device) for _ in range(P)]
    v = [torch.zeros((T, K // world), dtype=dt, device=device) for _ in range(P)]
    o = [torch.zeros((T, H // world), dtype=dt, device=device) for _ in range(P)]

    def step():
        for l in range(L):
            p = l % P
            ops.lora_qkv(p, wl.x_qkv[p], q[p], k[p], v[p])
            ops.lora_o(p, wl.x_o[p], o[p])

    import slora_b200 as sl
    before = sum(sl.launch_counts().values())
    step()
    torch.cuda.synchronize()
    launches_per_step = sum(sl.launch_counts().values()) - before
    graph = None
    if ops.px is not None and not args.no_graph:
        # with the exchange over peer memory the step holds no library collective and replays from a CUDA graph
        # (the exchange kernels keep their sequence numbers on the device); with NCCL all-gathers it runs eagerly
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            step()
        torch.cuda.synchronize()
        dist.barrier()
    run = graph.replay if graph is not None else step
    for _ in range(max(args.warmup, 3)):
        run()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        run()
    t1.record()
    torch.cuda.synchronize()
    dist.barrier()
    el = torch.tensor([t0.elapsed_time(t1) * 1e-3], dtype=torch.float64, device=device)
    dist.all_reduce(el, op=dist.ReduceOp.MAX)
    elapsed = float(el.item())
    ops.plan.check()
    if rank == 0:
        es = 2
        distinct = torch.unique(wl.ids).tolist()
        dims = wl.proj_dims()
        w_bytes = sum(wl.ranks[a] * (hi + ho) * es for a in distinct for hi, ho in dims) // world
        act = T * 2 * H * es + T * sum(2 * ho * es for _, ho in dims) // world
        exch = L * (3 + 1) * T * wl.max_rank * es  # bytes every rank receives per step
        per_rank_bytes = (w_bytes + act) * L
        line = {
            "metric": "lora_delta_tokens_per_s", "value": T * args.steps / elapsed, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": {"workload": spec.name, "tokens": T, "layers": L, "hidden": H, "kv_width": K,
                       "adapters": spec.n_adapters, "max_rank": wl.max_rank, "phys_layers": P,
                       "parallelism": f"slora-tp{world}: A rank-sharded, B output-sharded, [T, 3R/N] and [T, R/N] "
                                      f"exchanged per layer by " + ("peer memory from inside the shrink / expand kernels (NVLink stores + flags)"
                                                                    if ops.px is not None and args.tp_exchange == "fused"
                                                                    else "one kernel over peer memory (NVLink stores + flags)"
                                                                    if ops.px is not None else "NCCL all-gather + regroup"),
                       "l2": "inputs larger than L2", "graph": graph is not None, "pdl": not args.no_pdl},
            "per_rank_hbm": {"algorithmic_bytes_per_step": per_rank_bytes,
                             "achieved": per_rank_bytes / (elapsed / args.steps) / 1e9, "unit": "GB/s"},
            "exchange_bytes_per_step_per_rank": exch,
            "gpu_launches": args.steps * launches_per_step, "collectives_per_step": 2 * L, "e2e": None,
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    del graph
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
