"""Seeded synthetic workloads shaped like the reference's benchmark settings.

The reference measures on synthetic request traces (``benchmarks/trace.py:33-61``) over dummy adapters
(``slora/models/peft/layer_weights/lora_layer_weight.py:36-95``) with the model settings S1..S6 of
``benchmarks/exp_suite.py:4-20``.  For the LoRA hot path a workload is: adapter ranks, the three index tables over a
pool with a random page permutation (as in ``slora/models/peft/triton_kernel/tests/bench_ops.py:118-124``), pool
contents for a few layers, one batch of per-token adapter ids (plus prefill segments) and activations.

Everything is drawn from ``torch.Generator`` objects seeded from the configuration number, so the CPU oracle and the
CUDA kernels see bit-identical inputs.  Value distributions: ``x ~ N(0,1)``, ``A ~ N(0, 1/h_in)`` (std ``h_in**-0.5``),
``B ~ N(0, 0.02**2)`` (std 0.02), ``scale = alpha / r`` with ``alpha = 16``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

ALPHA = 16.0


@dataclass
class WorkloadSpec:
    name: str
    hidden: int
    h_kv: int              # k/v output width (== hidden unless GQA)
    layers: int
    n_adapters: int
    rank_choices: Tuple[int, ...]
    pool_rows: int
    decode_tokens: int
    zipf_alpha: Optional[float]   # None: uniform adapter ids
    prefill: Optional[Tuple[str, int, int, int]] = None  # (kind, count_or_budget, min_len, max_len)
    cfg: int = 0


SPECS = {
    # config 1: CPU-runnable correctness case
    1: WorkloadSpec("cfg1-correctness", 4096, 4096, 1, 4, (8,), 256, 32, None, None, 1),
    # config 2: S1-shaped decode
    2: WorkloadSpec("cfg2-S1-decode", 4096, 4096, 32, 1000, (8,), 262144, 256, 1.0, None, 2),
    # config 3: S2-shaped mixed batch
    3: WorkloadSpec("cfg3-S2-mixed", 4096, 4096, 32, 500, (64, 32, 16, 8), 262144, 248, 1.0, ("seqs", 8, 8, 512), 3),
    # config 4: S4-shaped, Llama-13B
    4: WorkloadSpec("cfg4-S4-13B", 5120, 5120, 40, 2000, (64, 32, 16), 327680, 461, 0.8, ("budget", 51, 16, 256), 4),
    # config 5: S6-shaped, Llama-70B with GQA
    5: WorkloadSpec("cfg5-S6-70B-gqa", 8192, 1024, 80, 200, (64,), 65536, 1024, None, None, 5),
}


@dataclass
class Workload:
    spec: WorkloadSpec
    dtype: torch.dtype
    ranks: List[int]
    a_start: torch.Tensor
    a_len: torch.Tensor
    a_loc: torch.Tensor
    a_scaling: torch.Tensor
    ids: torch.Tensor                    # [T] int64 per-token adapter
    segments: List[Tuple[int, int, int]]  # (start, len, adapter) for prefill sequences; decode tokens are 1-token
    pools_a: List[torch.Tensor] = field(default_factory=list)   # per physical layer [rows, hidden]
    pools_b: List[torch.Tensor] = field(default_factory=list)
    x_qkv: List[torch.Tensor] = field(default_factory=list)     # per physical layer [T, hidden]
    x_o: List[torch.Tensor] = field(default_factory=list)

    @property
    def T(self):
        return self.ids.numel()

    @property
    def max_rank(self):
        return max(self.ranks)

    def to(self, device):
        out = Workload(self.spec, self.dtype, self.ranks, self.a_start.to(device), self.a_len.to(device),
                       self.a_loc.to(device), self.a_scaling.to(device), self.ids.to(device), self.segments)
        out.pools_a = [p.to(device) for p in self.pools_a]
        out.pools_b = [p.to(device) for p in self.pools_b]
        out.x_qkv = [p.to(device) for p in self.x_qkv]
        out.x_o = [p.to(device) for p in self.x_o]
        return out

    def proj_dims(self):
        """(h_in, h_out) of q, k, v, o."""
        H, K = self.spec.hidden, self.spec.h_kv
        return [(H, H), (H, K), (H, K), (H, H)]

    def algorithmic_bytes_per_layer(self):
        """Compulsory HBM traffic of one layer's q/k/v/o LoRA deltas: each distinct adapter's rows once, x once for
        q/k/v and once for o, y read and written; intermediates excluded."""
        esize = 2
        distinct = torch.unique(self.ids.cpu()).tolist()
        dims = self.proj_dims()
        w = sum(self.ranks[a] * (hi + ho) * esize for a in distinct for hi, ho in dims)
        x = self.T * 2 * self.spec.hidden * esize
        y = self.T * sum(2 * ho * esize for _, ho in dims)
        return w + x + y

    def gathered_bytes_per_layer(self):
        """Per-token gathered bytes (adapter rows counted once per token): the secondary figure."""
        esize = 2
        dims = self.proj_dims()
        ids = self.ids.cpu().tolist()
        w = sum(self.ranks[a] * (hi + ho) * esize for a in ids for hi, ho in dims)
        return w + self.T * 2 * self.spec.hidden * esize + self.T * sum(2 * ho * esize for _, ho in dims)


def workload_config(wl: "Workload", layers=None, world=1):
    """The ``config`` object of a benchmark line for this workload (identical for every arm that runs it)."""
    spec = wl.spec
    return {"workload": spec.name, "tokens": wl.T, "layers": layers or spec.layers, "hidden": spec.hidden,
            "kv_width": spec.h_kv, "adapters": spec.n_adapters, "ranks": sorted(set(spec.rank_choices)),
            "max_rank": wl.max_rank, "pool_rows": spec.pool_rows,
            "distinct_adapters_in_batch": len(set(wl.ids.tolist())),
            "parallelism": "1 gpu" if world == 1 else f"slora-tp{world}"}


def zipf_probs(n, alpha):
    p = torch.arange(1, n + 1, dtype=torch.float64) ** (-alpha)
    return p / p.sum()


def draw_ids(n_adapters, count, alpha, gen):
    if count == 0:
        return torch.empty(0, dtype=torch.int64)
    if alpha is None:
        return torch.randint(0, n_adapters, (count,), generator=gen, dtype=torch.int64)
    return torch.multinomial(zipf_probs(n_adapters, alpha), count, replacement=True, generator=gen)


def make_tables(ranks, pool_rows, seed, permute=True):
    """``a_start / a_len / a_loc`` for adapters of the given ranks over a pool of ``pool_rows`` rows.

    ``a_loc`` is the head of a seeded random permutation of the pool's rows (scattered pages) or the identity."""
    lens = torch.tensor([4 * r for r in ranks], dtype=torch.int64)
    total = int(lens.sum())
    if total > pool_rows:
        raise ValueError(f"pool of {pool_rows} rows cannot hold {total} adapter rows")
    start = torch.zeros_like(lens)
    start[1:] = torch.cumsum(lens, 0)[:-1]
    if permute:
        g = torch.Generator().manual_seed(seed)
        loc = torch.randperm(pool_rows, generator=g)[:total].to(torch.int64)
    else:
        loc = torch.arange(total, dtype=torch.int64)
    return start, lens, loc


def build_batch(spec: WorkloadSpec, gen):
    """Per-token adapter ids and prefill segments of one batch."""
    ids, segments, pos = [], [], 0
    if spec.prefill is not None:
        kind, count, lo, hi = spec.prefill
        lens = []
        if kind == "seqs":
            lens = torch.randint(lo, hi + 1, (count,), generator=gen).tolist()
        else:  # token budget cut into chunks
            left = count
            while left > 0:
                n = min(left, int(torch.randint(lo, hi + 1, (1,), generator=gen)))
                lens.append(n)
                left -= n
        seq_adapters = draw_ids(spec.n_adapters, len(lens), spec.zipf_alpha, gen).tolist()
        for n, a in zip(lens, seq_adapters):
            segments.append((pos, n, a))
            ids.extend([a] * n)
            pos += n
    dec = draw_ids(spec.n_adapters, spec.decode_tokens, spec.zipf_alpha, gen).tolist()
    for a in dec:
        segments.append((pos, 1, a))
        ids.append(a)
        pos += 1
    return torch.tensor(ids, dtype=torch.int64), segments


def fill_pool_rows(pool, loc, std, gen, chunk=8192):
    """Write N(0, std^2) values into the rows ``loc`` of ``pool`` (rows outside ``loc`` stay as they are)."""
    dev = pool.device
    loc = loc.to(dev)
    for i in range(0, loc.numel(), chunk):
        rows = loc[i:i + chunk]
        vals = torch.randn((rows.numel(), pool.shape[1]), generator=gen, device=dev, dtype=torch.float32) * std
        pool[rows] = vals.to(pool.dtype)


def build_workload(cfg: int, device="cpu", dtype=torch.float16, phys_layers=1, pool_rows=None, n_adapters=None,
                   decode_tokens=None, hidden=None, h_kv=None, permute=True, rank_choices=None, prefill="default",
                   with_activations=True, rank_div=1, fill="all") -> Workload:
    """Build configuration ``cfg`` (1..5), optionally shrunk (fewer adapters / rows / tokens) for tests.

    Tables and batch composition are always drawn on CPU; pool contents and activations are drawn on ``device``
    (seeded per device type, so CPU-built and CUDA-built workloads differ in values but not in structure).
    ``rank_div`` > 1 gives the tables and (random) pool contents of one rank of an N-way tensor-parallel group.
    ``fill="batch"`` writes only the rows of adapters that occur in the batch (the other rows of the full-size pool
    stay uninitialised: nothing on the path reads them); the host-side timing legs use it to build a full-size pool
    in seconds.
    """
    base = SPECS[cfg]
    spec = WorkloadSpec(base.name, hidden or base.hidden, h_kv or (hidden if hidden and base.h_kv == base.hidden
                                                                   else base.h_kv),
                        base.layers, n_adapters or base.n_adapters, tuple(rank_choices or base.rank_choices),
                        pool_rows or base.pool_rows,
                        base.decode_tokens if decode_tokens is None else decode_tokens, base.zipf_alpha,
                        base.prefill if prefill == "default" else prefill, cfg)
    g_w = torch.Generator().manual_seed(1000 + cfg)
    g_b = torch.Generator().manual_seed(3000 + cfg)
    choice = torch.randint(0, len(spec.rank_choices), (spec.n_adapters,), generator=g_w).tolist()
    ranks = [spec.rank_choices[c] for c in choice]
    # rank_div = N builds one tensor-parallel rank's tables: slots of r / N rows (Workload.ranks keeps the full r)
    a_start, a_len, a_loc = make_tables([r // rank_div for r in ranks], spec.pool_rows, 2000 + cfg, permute)
    a_scaling = torch.tensor([ALPHA / r for r in ranks], dtype=dtype)
    ids, segments = build_batch(spec, g_b)
    wl = Workload(spec, dtype, ranks, a_start, a_len, a_loc, a_scaling, ids, segments)
    dev = torch.device(device)
    g_dev = torch.Generator(device=dev).manual_seed(4000 + cfg)
    for _ in range(phys_layers):
        pa = torch.empty((spec.pool_rows, spec.hidden), dtype=dtype, device=dev)
        pb = torch.empty((spec.pool_rows, spec.hidden), dtype=dtype, device=dev)
        if dev.type == "cpu" and fill == "all":
            pa.zero_()
            pb.zero_()
        rows = a_loc
        if fill == "batch":
            used = sorted(set(ids.tolist()))
            rows = torch.cat([a_loc[int(a_start[a]): int(a_start[a]) + int(a_len[a])] for a in used]) if used else a_loc[:0]
        fill_pool_rows(pa, rows, spec.hidden ** -0.5, g_dev)
        fill_pool_rows(pb, rows, 0.02, g_dev)
        wl.pools_a.append(pa)
        wl.pools_b.append(pb)
        if with_activations:
            wl.x_qkv.append(torch.randn((wl.T, spec.hidden), generator=g_dev, device=dev,
                                        dtype=torch.float32).to(dtype))
            wl.x_o.append(torch.randn((wl.T, spec.hidden), generator=g_dev, device=dev,
                                      dtype=torch.float32).to(dtype))
    if dev.type != "cpu":
        wl.a_start, wl.a_len, wl.a_loc = a_start.to(dev), a_len.to(dev), a_loc.to(dev)
        wl.a_scaling, wl.ids = a_scaling.to(dev), ids.to(dev)
    return wl
