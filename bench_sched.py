"""What the scheduler hook is worth on the LoRA path (``bench.py --scheduler``): the same request stream admitted in
arrival order (``ReqQueue``) and with adapter clustering (``ClusterReqQueue``, the reference's
``slora/server/router/cluster_req_queue.py``), the running decode batches of both handed to the LoRA kernels.

A request stream over the S1-shaped adapter set (1000 rank-8 adapters, hidden 4096; adapter of a request drawn as the
reference's trace generator does, ``floor(power(alpha) * n)``, ``benchmarks/trace.py:42-43``) is fed to each queue
with a serving loop that keeps up to 256 requests running.  At fixed intervals the running batch (one decode token per
request) is snapshotted; for every snapshot the line reports the distinct adapters, the algorithmic bytes of one
layer, and the measured time of the q/k/v + o LoRA deltas of one layer (CUDA events over a graph of 8 physical
layers).  Prints one JSON line.
"""
from __future__ import annotations

import json

import numpy as np
import torch


def _serve(queue, n_adapters, alpha, total, per_step, seed, snapshot_every, running_cap):
    from slora_b200.req_queue import Req
    rng = np.random.default_rng(seed)
    ranks = {a: 8 for a in range(n_adapters)}
    running, snaps, nxt, step = None, [], 0, 0
    while nxt < total or running is not None:
        for _ in range(per_step):
            if nxt < total:
                a = int(np.floor(rng.power(alpha) * n_adapters))
                queue.append(Req(a, nxt, int(rng.integers(8, 512)), int(rng.integers(8, 512))))
                nxt += 1
        new = queue.generate_new_batch(running, ranks)
        if new is not None:
            if running is None:
                running = new
            else:
                running.merge(new)
        if running is not None:
            if step % snapshot_every == 0 and len(running.reqs) >= running_cap // 2:
                snaps.append([r.adapter_dir for r in running.reqs])
            for r in running.reqs:
                r.output_ids.append(0)
                if len(r.output_ids) >= r.max_output_len:
                    r.has_generate_finished = True
            running.filter_finished()
            if running.is_clear():
                running = None
        step += 1
        if step > 20000:
            break
    return snaps


def run(device, batch_num_adapters=32, n_requests=1500, per_step=2, alpha=0.3, phys_layers=8, max_snaps=12):
    import slora_b200 as sl
    from slora_b200.req_queue import ClusterReqQueue, ReqQueue
    from slora_b200.workloads import build_workload
    wl = build_workload(2, device=device, phys_layers=phys_layers, pool_rows=65536)
    H, dt = wl.spec.hidden, wl.dtype
    cap = 256
    qargs = dict(max_total_tokens=cap * 1100, batch_max_tokens=16384, running_max_req_size=cap)
    out = {"metric": "scheduler_hook_effect_on_lora_path", "unit": "us per layer", "requests": n_requests,
           "adapters": wl.spec.n_adapters, "power_alpha": alpha, "running_cap": cap,
           "batch_num_adapters": batch_num_adapters, "queues": {}}
    for name, q in (("arrival_order", ReqQueue(**qargs)),
                    ("adapter_clustering", ClusterReqQueue(batch_num_adapters=batch_num_adapters, **qargs))):
        snaps = _serve(q, wl.spec.n_adapters, alpha, n_requests, per_step, 5, 25, cap)
        snaps = snaps[:: max(1, len(snaps) // max_snaps)][:max_snaps]
        rows = []
        for ids_list in snaps:
            ids = torch.tensor(ids_list, dtype=torch.int64, device=device)
            T = ids.numel()
            ops = sl.LoraBatchOps(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling, wl.pools_a, wl.pools_b, wl.max_rank)
            ops.prepare(ids)
            x = torch.randn((T, H), device=device, dtype=torch.float32).to(dt)
            ys = [torch.zeros((T, H), dtype=dt, device=device) for _ in range(4)]

            def layers():
                for p in range(phys_layers):
                    ops.lora_get_qkv(p, x, ys[0], ys[1], ys[2])
                    ops.lora_get_o(p, x, ys[3])
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                layers()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                layers()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / 10 / phys_layers
            distinct = len(set(ids_list))
            layer_bytes = distinct * 4 * 8 * 2 * H * 2 + T * 2 * H * 2 + T * 4 * 2 * H * 2
            rows.append({"tokens": T, "distinct_adapters": distinct, "us_per_layer": round(us, 2),
                         "tokens_per_s_per_layer": round(T / us * 1e6), "algorithmic_bytes_per_layer": layer_bytes})
            ops.plan.check()
        n = max(1, len(rows))
        out["queues"][name] = {
            "snapshots": rows,
            "mean_tokens": sum(r["tokens"] for r in rows) / n,
            "mean_distinct_adapters": sum(r["distinct_adapters"] for r in rows) / n,
            "mean_us_per_layer": sum(r["us_per_layer"] for r in rows) / n,
            "mean_us_per_token_layer": sum(r["us_per_layer"] / r["tokens"] for r in rows) / n,
        }
    a, c = out["queues"]["arrival_order"], out["queues"]["adapter_clustering"]
    if a["snapshots"] and c["snapshots"]:
        out["value"] = a["mean_us_per_token_layer"] / c["mean_us_per_token_layer"]
        out["value_is"] = "LoRA-path time per token and layer, arrival order over adapter clustering"
    return out


if __name__ == "__main__":
    print(json.dumps(run(torch.device("cuda", 0))), flush=True)
