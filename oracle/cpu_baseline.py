"""The reference's CPU arm for the LoRA hot path: its torch per-token formula, run on host cores.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see oracle/lora_oracle.py).  The reference has no CPU kernel for this path;
what it has is the torch loop its kernel scripts compare against
(``test/kernel/test_kernel_correctness_multi_rank.py:97-106``): per token, slice the adapter's rows out of the pool,
reshape, and do a ``[1, r] @ [r, H]``-sized matmul.  This file times exactly that loop (with the ``a_loc`` gather of
``slora/csrc/bgmv/bgmv_impl.cuh:34-38,174-179`` and the ``alpha/r`` scale of ``:180,197``) in float32 on CPU tensors,
using every thread torch has (``torch.get_num_threads()``).
"""
from __future__ import annotations

import time

import torch


@torch.no_grad()
def per_token_layer(x_qkv, x_o, pool_a, pool_b, a_start, a_len, a_loc, ids, scales, proj_dims):
    """q, k, v, o LoRA deltas of one layer, one token at a time (float32 CPU tensors in, list of [T, h_out] out)."""
    T = ids.numel()
    outs = []
    for p, (h_in, h_out) in enumerate(proj_dims):
        x = x_o if p == 3 else x_qkv
        rows = []
        for i in range(T):
            a = int(ids[i])
            r = int(a_len[a]) // 4
            base = int(a_start[a]) + p * r
            loc = a_loc[base: base + r]
            wa = pool_a[loc].reshape(-1)[: r * h_in].float().reshape(r, h_in).T
            nb = -(-(h_out * r) // pool_b.shape[1])
            wb = pool_b[loc[:nb]].reshape(-1)[: h_out * r].float().reshape(h_out, r).T
            delta = x[i:i + 1].float() @ wa
            rows.append((delta @ wb) * float(scales[a]))
        outs.append(torch.cat(rows))
    return outs


@torch.no_grad()
def grouped_layer(x_qkv, x_o, pool_a, pool_b, a_start, a_len, a_loc, ids, scales, proj_dims):
    """The same deltas with the tokens of one adapter multiplied together (two small matmuls per distinct adapter and
    projection): a fairer CPU arrangement than the reference's per-token loop, reported beside it."""
    outs = []
    groups = {}
    for i, a in enumerate(ids.tolist()):
        groups.setdefault(a, []).append(i)
    for p, (h_in, h_out) in enumerate(proj_dims):
        x = (x_o if p == 3 else x_qkv).float()
        y = torch.zeros((ids.numel(), h_out), dtype=torch.float32)
        for a, tok in groups.items():
            r = int(a_len[a]) // 4
            base = int(a_start[a]) + p * r
            loc = a_loc[base: base + r]
            wa = pool_a[loc].reshape(-1)[: r * h_in].float().reshape(r, h_in)
            nb = -(-(h_out * r) // pool_b.shape[1])
            wb = pool_b[loc[:nb]].reshape(-1)[: h_out * r].float().reshape(h_out, r)
            sel = torch.tensor(tok)
            y[sel] = (x[sel] @ wa.T) @ wb.T * float(scales[a])
        outs.append(y)
    return outs


def time_layer(wl_cpu, min_seconds=10.0, min_reps=2, max_reps=50, fn=None):
    """Seconds per layer (all four projections over the whole batch), averaged over enough repetitions to fill
    ``min_seconds`` of CPU work; returns ``(seconds_per_layer, reps)``."""
    args = (wl_cpu.x_qkv[0], wl_cpu.x_o[0], wl_cpu.pools_a[0], wl_cpu.pools_b[0], wl_cpu.a_start, wl_cpu.a_len,
            wl_cpu.a_loc, wl_cpu.ids, wl_cpu.a_scaling, wl_cpu.proj_dims())
    fn = fn or per_token_layer
    fn(*args)  # warm-up (thread pool, allocator)
    reps, t0 = 0, time.perf_counter()
    while True:
        fn(*args)
        reps += 1
        el = time.perf_counter() - t0
        if (el >= min_seconds and reps >= min_reps) or reps >= max_reps:
            return el / reps, reps
