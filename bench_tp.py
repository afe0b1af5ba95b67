"""Tensor-parallel leg of the benchmark (``bench.py --gpus N`` on configurations 4 and 5): one process per GPU, S-LoRA
tensor parallelism for the adapter path.

Each rank holds its shard of every adapter (A: r/N rank rows, B: h_out/N output rows) for a few physical layers and
runs the model's layer count over them; q/k/v see replicated activations, their rank-r intermediates are exchanged
over NVLink from inside the kernels (peer-memory stores, signalled in band; ``--tp-exchange p2p|nccl`` select the one-kernel
exchange or NCCL all-gather + regroup).  The o projection runs by either rule: input replicated (the q/k/v rule), or
input head-sharded ``[T, H/N]`` with the partial intermediates summed over the ranks, which is what a tensor-parallel
base model hands over (the rule of the reference's figure for a row-parallel projection, ``figures/slora_tp.png``);
the headline is the replicated-input rule (every intermediate all-gathered), the other figure sits beside it.

Time is CUDA-event time of K graph replays, maximum over ranks; tokens/s counts the batch once (strong scaling).
The line also carries: per-rank roofline of the largest kernel, the cost of the exchange (step time minus the same
kernels with nothing exchanged and nothing waited for), parity of one layer (local shrink against the oracle, the
exchanged intermediate bit for bit against every rank's local one, expand against the oracle) and the end-to-end
figure with host buffers.
"""
from __future__ import annotations

import json
import os

import torch


def _capture(fn, dist):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    return g


def _timed(run, steps, warmup, dist, device):
    """Seconds for `steps` calls of run(), CUDA events, bracketed by barriers, maximum over ranks."""
    for _ in range(max(warmup, 3)):
        run()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        run()
    t1.record()
    torch.cuda.synchronize()
    dist.barrier()
    el = torch.tensor([t0.elapsed_time(t1) * 1e-3], dtype=torch.float64, device=device)
    mine = float(el.item())
    dist.all_reduce(el, op=dist.ReduceOp.MAX)
    return float(el.item()), mine


def tp_parity(ops, wl, world, rank, dist, q, k, v, o, o_rule):
    """One layer under tensor parallelism against the CPU oracle: (1) this rank's shrink of q/k/v (its r/N rows of
    every adapter) against the oracle on its own pool; (2) the exchanged intermediate this rank's expand reads, bit
    for bit against every rank's local result (gathered with NCCL, outside any timed region); (3) this rank's output
    slices against the oracle's expand of that intermediate over its own B shard."""
    import numpy as np
    from oracle import lora_oracle as orc
    from slora_b200 import tp as tpmod
    t = ops.t
    T, N, R, Rl = wl.T, world, ops.R, ops.Rl
    be = ops.backend
    worst = [0.0, 0.0]

    def note(got, ref):
        mx, mn = orc.error_metrics(got, ref)
        worst[0], worst[1] = max(worst[0], mx), max(worst[1], mn)

    for buf in (q, k, v, o):
        buf.zero_()
    # (1) local shrink through the plain entry point
    local = torch.zeros((3, T, Rl), dtype=wl.dtype, device=q.device)
    be.shrink(ops.plan, ops.ids, [0, 1, 2], [local[0], local[1], local[2]], wl.x_qkv[0], wl.pools_a[0], t)
    torch.cuda.synchronize()
    for p in range(3):
        ref = orc.lora_shrink_ref(wl.x_qkv[0], wl.pools_a[0], t.a_start, t.a_len, t.a_loc, ops.ids, p, out_width=Rl)
        note(local[p], ref)
    # (2) the real call: shrink + exchange + expand.  With the exchange fused into the kernels the two halves of the
    # call are issued apart, so that the delta buffer can be looked at in between (with in-band signalling the expand
    # empties it again): every rank's shrink has completed and been synchronised with before anybody reads.
    fused = ops.px is not None and getattr(be, "fused", False)
    if fused:
        be.shrink_push(ops.px, ops.plan, ops.ids, [0, 1, 2], wl.x_qkv[0], wl.pools_a[0], t, Rl, 0)
        torch.cuda.synchronize()
        dist.barrier()
        # (rotating thirds: the shrink left the exchange's number, which picks the part, for its expand)
        part = int(ops.px.inband_seq[1].item()) % 3 if ops.px.inband == 3 else 0
        full = ops.px.full[part][:, :T].clone()       # [3, T, R] as this rank's expand is about to read it
        be.expand_wait(ops.px, ops.plan, ops.ids, [0, 1, 2], [q, k, v], wl.pools_b[0], t, Rl, 0)
    else:
        ops.lora_qkv(0, wl.x_qkv[0], q, k, v)
    torch.cuda.synchronize()
    dist.barrier()
    exchange_exact = None
    if ops.px is not None:
        everyone = torch.zeros((N, 3, T, Rl), dtype=wl.dtype, device=q.device)
        dist.all_gather_into_tensor(everyone.view(-1), local.view(-1))
        if not fused:
            full = ops.px.full[0][:, :T].clone()      # [3, T, R] as this rank's expand read it
        ev, full_np = everyone.cpu().numpy(), full.cpu().numpy()
        rows_per_rank = (np.asarray(wl.ranks)[ops.ids.cpu().numpy()] // N).tolist()
        exchange_exact = True
        for tok, rs in enumerate(rows_per_rank):
            for g in range(N):
                if not np.array_equal(full_np[:, tok, g * rs:(g + 1) * rs], ev[g, :, tok, :rs]):
                    exchange_exact = False
        delta_full = full
    else:
        delta_full = None
    # (3) expand of that intermediate over this rank's B shard
    if delta_full is not None:
        for p, got in enumerate((q, k, v)):
            ref = orc.lora_expand_ref(np.zeros(tuple(got.shape), dtype=np.float32), delta_full[p], wl.pools_b[0],
                                      t.a_start, t.a_len, t.a_loc, ops.ids, p, t.a_scaling, rank_mult=N)
            note(got, ref)
    for buf in (q, k, v, o):
        buf.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    ok = worst[0] <= 1e-2 and worst[1] <= 1e-3 and exchange_exact is not False
    flag = torch.tensor([1 if ok else 0], device=q.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return {"max_rel": worst[0], "mean_rel": worst[1], "exchange_bit_exact": exchange_exact,
            "tolerance": {"max_rel": 1e-2, "mean_rel": 1e-3}, "ok": bool(flag.item()),
            "how": "rank 0's figures; layer 0: local q/k/v shrink vs the fp32 CPU oracle, the exchanged intermediate "
                   "vs every rank's local result, q/k/v expand vs the oracle; 'ok' holds on every rank"}


def run(args, dist, rank, world, device, peak):
    import bench
    from slora_b200 import tp
    from slora_b200.workloads import build_workload, workload_config
    import slora_b200 as sl

    peak_gbs, peak_kind = peak
    cfg = args.config
    P = bench.phys_layers_for(args, cfg)
    wl = build_workload(cfg, device=device, phys_layers=P, pool_rows=args.pool_rows, rank_div=world,
                        n_adapters=args.adapters)
    spec = wl.spec
    H, K, T, L = spec.hidden, spec.h_kv, wl.T, args.layers or spec.layers
    tables = tp.TpTables(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling)
    ops = tp.TpLoraOps(tables, wl.pools_a, wl.pools_b, wl.max_rank, world, rank,
                       tp.CudaBackend(use_pdl=not args.no_pdl, fused=args.tp_exchange == "fused"),
                       peer_exchange=args.tp_exchange != "nccl").prepare(wl.ids)
    dt = wl.dtype
    q = [torch.zeros((T, H // world), dtype=dt, device=device) for _ in range(P)]
    k = [torch.zeros((T, K // world), dtype=dt, device=device) for _ in range(P)]
    v = [torch.zeros((T, K // world), dtype=dt, device=device) for _ in range(P)]
    o = [torch.zeros((T, H // world), dtype=dt, device=device) for _ in range(P)]
    x_o_shard = [x[:, rank * (H // world):(rank + 1) * (H // world)].contiguous() for x in wl.x_o]

    parity = None
    if not args.no_parity:
        parity = tp_parity(ops, wl, world, rank, dist, q[0], k[0], v[0], o[0], args.tp_o)

    def step_rule(sharded_o):
        def step():
            for l in range(L):
                p = l % P
                ops.lora_qkv(p, wl.x_qkv[p], q[p], k[p], v[p])
                if sharded_o:
                    ops.lora_o_sharded(p, x_o_shard[p], o[p])
                else:
                    ops.lora_o(p, wl.x_o[p], o[p])
        return step

    def local_step_rule(sharded_o):
        """The same kernels on the same bytes with nothing exchanged and nothing waited for: shrinks into local
        buffers, expands from this rank's (stale) full-width delta buffer."""
        be, t = ops.backend, ops.t
        R, N = ops.R, ops.N
        src = ops.px.full if ops.px is not None else torch.zeros((2, 3, T, R), dtype=dt, device=device)
        sum_in = torch.zeros((T, R), dtype=dt, device=device)

        def step():
            for l in range(L):
                p = l % P
                be.shrink(ops.plan, ops.ids, [0, 1, 2], [ops.local[0], ops.local[1], ops.local[2]], wl.x_qkv[p],
                          wl.pools_a[p], t)
                be.expand(ops.plan, ops.ids, [0, 1, 2], [q[p], k[p], v[p]], [src[0][j][:T] for j in range(3)],
                          wl.pools_b[p], t, delta_stride=R, delta_width=R, delta_parts=1, delta_part_stride=0,
                          rank_mult=N)
                if sharded_o:
                    be.shrink(ops.plan, ops.ids, [3], [sum_in], x_o_shard[p], wl.pools_a[p], t, rank_mult=N)
                    be.expand(ops.plan, ops.ids, [3], [o[p]], [sum_in], wl.pools_b[p], t, delta_stride=R,
                              delta_width=R, delta_parts=1, delta_part_stride=0, rank_mult=N)
                else:
                    be.shrink(ops.plan, ops.ids, [3], [ops.local[0]], wl.x_o[p], wl.pools_a[p], t)
                    be.expand(ops.plan, ops.ids, [3], [o[p]], [src[1][0][:T]], wl.pools_b[p], t, delta_stride=R,
                              delta_width=R, delta_parts=1, delta_part_stride=0, rank_mult=N)
        return step

    rules = {"both": [True, False], "sharded": [True], "replicated": [False]}[args.tp_o]
    use_graph = ops.px is not None and not args.no_graph
    results = {}
    launches_per_step = None
    clocks = None
    for sharded_o in rules:
        step = step_rule(sharded_o)
        before = sum(sl.launch_counts().values())
        step()
        torch.cuda.synchronize()
        n_launch = sum(sl.launch_counts().values()) - before
        dist.barrier()
        graph = _capture(step, dist) if use_graph else None
        runner = graph.replay if graph is not None else step
        if launches_per_step is None:
            with bench.ClockSampler(bench.physical_gpu_index(device.index or 0)) as clocks:
                elapsed, mine = _timed(runner, args.steps, args.warmup, dist, device)
            launches_per_step = n_launch
        else:
            elapsed, mine = _timed(runner, args.steps, args.warmup, dist, device)
        ops.plan.check()
        res = {"ms_per_step": elapsed / args.steps * 1e3, "value": T * args.steps / elapsed,
               "us_per_layer": elapsed / args.steps / L * 1e6, "this_rank_ms_per_step": mine / args.steps * 1e3,
               "launches_per_step": n_launch, "graph": graph is not None}
        # the same kernels with nothing exchanged: what is left of the step is kernels and launch gaps
        lstep = local_step_rule(sharded_o)
        lgraph = _capture(lstep, dist) if not args.no_graph else None
        l_el, _ = _timed(lgraph.replay if lgraph is not None else lstep, args.steps, args.warmup, dist, device)
        res["kernels_only_ms_per_step"] = l_el / args.steps * 1e3
        res["kernels_only_us_per_layer"] = l_el / args.steps / L * 1e6
        res["exchange_us_per_layer"] = (elapsed - l_el) / args.steps / L * 1e6
        if graph is not None and args.replays > 0:
            med = bench.replay_median(graph.replay, args.replays)
            t_med = torch.tensor([med["ms_per_step_median"]], dtype=torch.float64, device=device)
            dist.all_reduce(t_med, op=dist.ReduceOp.MAX)
            med["ms_per_step_median"] = float(t_med.item())
            med["tokens_per_s_median"] = T / med["ms_per_step_median"] * 1e3
            res["replay_median"] = med
        results["sharded_o" if sharded_o else "replicated_o"] = res
        del graph, lgraph
        torch.cuda.synchronize()
        dist.barrier()
    # headline: the rule the task's statement of the scheme gives (rank-r intermediates all-gathered for all four
    # projections, i.e. replicated inputs); the head-sharded o rule of the reference's figure is reported beside it
    head_rule = "replicated_o" if False in rules else "sharded_o"
    head = results[head_rule]

    # per-rank roofline of the largest kernel (the q/k/v expand of this rank's output slice), timed alone
    from slora_b200 import batch_infer
    es = 2
    distinct = torch.unique(wl.ids).tolist()
    dims = wl.proj_dims()
    b_bytes = sum(wl.ranks[a] * dims[p][1] * es for a in distinct for p in range(3)) // world
    y_bytes = T * sum(2 * dims[p][1] * es for p in range(3)) // world
    R = ops.R
    src = ops.px.full if ops.px is not None else torch.zeros((2, 3, T, R), dtype=dt, device=device)

    def expands():
        for l in range(L):
            p = l % P
            ops.backend.expand(ops.plan, ops.ids, [0, 1, 2], [q[p], k[p], v[p]], [src[0][j][:T] for j in range(3)],
                               wl.pools_b[p], ops.t, delta_stride=R, delta_width=R, delta_parts=1, delta_part_stride=0,
                               rank_mult=world)
    eg = _capture(expands, dist)
    e_el, _ = _timed(eg.replay, 5, 3, dist, device)
    t_expand = e_el / 5 / L
    roofline = {"bound": "hbm", "achieved": (b_bytes + y_bytes) / t_expand / 1e9, "peak": peak_gbs, "unit": "GB/s",
                "frac": (b_bytes + y_bytes) / t_expand / 1e9 / peak_gbs, "traffic": None,
                "traffic_how": "no ncu capture under tensor parallelism (a multi-rank command is never profiled)",
                "kernel": "lora_expand_pipe_kernel(qkv), this rank's h_out/N slice", "us_per_launch": t_expand * 1e6,
                "algorithmic_bytes_per_launch": b_bytes + y_bytes, "peak_kind": peak_kind,
                "how": "CUDA graph of one launch per layer of this kernel alone on every rank, slowest rank"}
    del eg

    # end to end: activations from pinned host memory, slices back to the host, through TpLoraOps
    e2e = None
    if not args.no_e2e:
        e2e = e2e_tp(args, ops, wl, world, rank, dist, device, L, P, head_rule == "sharded_o", q, k, v, o)

    w_bytes = sum(wl.ranks[a] * (hi + ho) * es for a in distinct for hi, ho in dims) // world
    x_o_bytes = T * H * es // (world if head_rule == "sharded_o" else 1)
    act = T * H * es + x_o_bytes + T * sum(2 * ho * es for _, ho in dims) // world
    exch = L * (3 + 1) * T * wl.max_rank * es  # bytes every rank receives per step
    per_rank_bytes = (w_bytes + act) * L
    sec = head["ms_per_step"] * 1e-3
    if rank == 0:
        signalling = {3: "in-band signalling, early start, buffers of three rotating parts",
                      2: "in-band signalling, early start", 1: "in-band signalling",
                      0: "flags"}.get(int(getattr(ops.px, "inband", 0)), "flags") if ops.px is not None else ""
        how = ("peer memory from inside the shrink / expand kernels (NVLink stores; %s)" % signalling
               if ops.px is not None and args.tp_exchange == "fused" else
               "one kernel over peer memory (NVLink stores + flags)" if ops.px is not None else
               "NCCL all-gather + regroup")
        config = workload_config(wl, L, world)
        config["l2"] = "inputs larger than L2: every rank streams its shard of %d physical layers" % P
        line = {
            "metric": "lora_delta_tokens_per_s", "value": head["value"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": config,
            "run": {"phys_layers": P, "graph": head["graph"], "pdl": not args.no_pdl, "o_rule": head_rule,
                    "split": "A over rank rows (q,k,v) / input columns (o, head-sharded rule), B over output rows",
                    "exchange": "[T, 3R/N] (q,k,v) and [T, R/N] or partial [T, R] (o) per layer by " + how,
                    "launches_per_step": launches_per_step},
            "us_per_layer": head["us_per_layer"], "parity": parity, "roofline": roofline,
            "per_rank_hbm": {"algorithmic_bytes_per_step": per_rank_bytes, "achieved": per_rank_bytes / sec / 1e9,
                             "peak": peak_gbs, "frac": per_rank_bytes / sec / 1e9 / peak_gbs, "unit": "GB/s",
                             "peak_kind": peak_kind},
            "exchange": {"bytes_received_per_step_per_rank": exch, "exchanges_per_step": 2 * L,
                         "us_per_layer": head["exchange_us_per_layer"],
                         "kernels_only_us_per_layer": head["kernels_only_us_per_layer"],
                         "how": "step time minus the same kernels on the same bytes with nothing exchanged and no "
                                "flag waited for (both graph replays, maximum over ranks)"},
            "o_rules": results, "replay_median": head.get("replay_median"),
            "gpu_launches": args.steps * launches_per_step, "collectives_per_step": 2 * L, "e2e": e2e,
            "cpu_baseline": None, "clocks": clocks.summary() if clocks is not None else None,
        }
        if not line["parity"]["ok"]:
            line["invalid"] = "parity check against the CPU oracle failed; the figures of this line do not count"
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0 and not line["parity"]["ok"]:
        raise SystemExit(4)


def e2e_tp(args, ops, wl, world, rank, dist, device, L, P, sharded_o, q, k, v, o):
    """Steps through TpLoraOps with the activations starting in pinned host memory and the output slices copied back.

    The q/k/v activations are replicated over the ranks.  Pushing the same rows through every GPU's PCIe link would
    multiply the host traffic by N, so each rank uploads rows [rank*T/N, (rank+1)*T/N) and the ranks all-gather them
    over NVLink (NCCL); the o input is uploaded as this rank's column slice (head-sharded rule) or the same way
    (replicated rule).  The layers are cut into chunks: one upload, one graph replay (the chunk's all-gathers and LoRA
    calls, captured through the public API) and one download per chunk, on three streams, so that the host issues a
    few dozen operations per step instead of several hundred - at 8 ranks the step would otherwise be bound by the
    Python loop, not by PCIe or the GPUs."""
    T, H, K = wl.T, wl.spec.hidden, wl.spec.h_kv
    dt = wl.dtype
    N = world
    rows = (T + N - 1) // N
    Tp = rows * N
    g = torch.Generator().manual_seed(77 + rank)
    Ho = H // N if sharded_o else H
    orow = T if sharded_o else rows
    x_host = torch.randn((L, rows, H), generator=g, dtype=torch.float32).to(dt).pin_memory()
    xo_host = torch.randn((L, orow, Ho), generator=g, dtype=torch.float32).to(dt).pin_memory()
    x_part = torch.empty((L, rows, H), dtype=dt, device=device)
    x_full = torch.empty((L, Tp, H), dtype=dt, device=device)
    xo_part = torch.empty((L, orow, Ho), dtype=dt, device=device)
    xo_full = xo_part if sharded_o else torch.empty((L, Tp, H), dtype=dt, device=device)
    W = (2 * H + 2 * K) // N
    y_dev = torch.zeros((L, T, W), dtype=dt, device=device)
    y_host = torch.empty((L, T, W), dtype=dt).pin_memory()
    h2d = x_host.numel() * 2 + xo_host.numel() * 2
    d2h = y_host.numel() * 2
    hq, hk = H // N, K // N
    chunk = 8 if L % 8 == 0 else (5 if L % 5 == 0 else 1)
    chunks = [(c, min(L, c + chunk)) for c in range(0, L, chunk)]

    def run_layers(lo, hi):
        for l in range(lo, hi):
            p = l % P
            yl = y_dev[l]
            dist.all_gather_into_tensor(x_full[l].view(-1), x_part[l].view(-1))
            if not sharded_o:
                dist.all_gather_into_tensor(xo_full[l].view(-1), xo_part[l].view(-1))
            ops.lora_qkv(p, x_full[l][:T], yl[:, :hq], yl[:, hq:hq + hk], yl[:, hq + hk:hq + 2 * hk])
            if sharded_o:
                ops.lora_o_sharded(p, xo_full[l], yl[:, hq + 2 * hk:])
            else:
                ops.lora_o(p, xo_full[l][:T], yl[:, hq + 2 * hk:])

    graphs, how = None, "eager"
    if ops.px is not None and not args.no_graph:
        try:
            graphs = [_capture(lambda lo=lo, hi=hi: run_layers(lo, hi), dist) for lo, hi in chunks]
            how = "one CUDA graph per chunk of %d layers (NCCL all-gathers of the uploads and the LoRA calls)" % chunk
        except Exception as e:    # a stack that cannot capture the collectives: issue the same calls eagerly
            graphs, how = None, "eager (graph capture failed: %s)" % type(e).__name__
            torch.cuda.synchronize()
        dist.barrier()
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in chunks]
    ev_done = [torch.cuda.Event() for _ in chunks]
    steps, warmup = max(3, min(args.steps, 10)), 3
    times = []
    for it in range(warmup + steps):
        torch.cuda.synchronize()
        dist.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            for c, (lo, hi) in enumerate(chunks):
                x_part[lo:hi].copy_(x_host[lo:hi], non_blocking=True)
                xo_part[lo:hi].copy_(xo_host[lo:hi], non_blocking=True)
                ev_in[c].record(s_in)
        for c, (lo, hi) in enumerate(chunks):
            cur.wait_event(ev_in[c])
            if graphs is not None:
                graphs[c].replay()
            else:
                run_layers(lo, hi)
            ev_done[c].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[c])
                y_host[lo:hi].copy_(y_dev[lo:hi], non_blocking=True)
        cur.wait_stream(s_out)
        t1.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(t0.elapsed_time(t1) * 1e-3)
    el = torch.tensor([sum(times)], dtype=torch.float64, device=device)
    dist.all_reduce(el, op=dist.ReduceOp.MAX)
    e_time = float(el.item())
    del graphs
    import bench
    return {"value": T * steps / e_time, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "bytes_are": "per rank", "steps": steps, "ms_per_step": e_time / steps * 1e3,
            "h2d_gbs_per_gpu": h2d / (e_time / steps) / 1e9, "d2h_gbs_per_gpu": d2h / (e_time / steps) / 1e9,
            "host": bench.host_topology(device.index or 0), "issue": how,
            "how": "each rank uploads T/N rows of the replicated activations and the ranks all-gather them over "
                   "NVLink; outputs are this rank's column slices"}
