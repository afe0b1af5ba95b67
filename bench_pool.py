"""Adapter swap cost on one GPU: rows allocated from the free map, an adapter's rows written into every layer's pool
buffers, and adapters dropped again - the library's kernels beside the same steps done the reference's way with torch
ops on the same GPU (``slora/common/mem_allocator.py:30-39``, ``slora/server/router/model_infer/infer_adapter.py:41-90``
and ``:186-250``).  Times are per call: ``gpu_us`` from CUDA events, ``host_us`` the wall clock until the call returns
(a call that reads a size back from the device blocks the host for the whole of it).

    python bench_pool.py [--layers 32] [--pool-rows 65536] [--map-rows 262144] [--rank 64]

Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from slora_b200.infer_adapter import InferAdapter
from slora_b200.mem_allocator import MemoryAllocator


class _Layer:
    def __init__(self, w):
        self.w_combined = w


class _Adapter:
    def __init__(self, name, r, heads, hd, layers, gen):
        self.lora_dir, self.r, self.scaling = name, r, 16.0 / r
        self.layers = [_Layer(torch.randn((2, 4 * r, heads, hd), device="cuda", generator=gen).to(torch.float16))
                       for _ in range(layers)]


class _TorchOpsAllocator(MemoryAllocator):
    """``alloc`` / ``free`` as the reference computes them: full-map cumulative sum, mask, nonzero; indexed store."""

    def alloc(self, need_size):
        if need_size > self.can_use_mem_size:
            raise Exception("no enough pool space")
        running = torch.cumsum(self.mem_state, dim=0, dtype=torch.int32)
        select_index = torch.nonzero(torch.logical_and(running <= need_size, self.mem_state), as_tuple=False).view(-1)
        self.mem_state[select_index] = False
        self.can_use_mem_size -= int(select_index.numel())
        return select_index

    def free(self, free_index):
        self.can_use_mem_size += free_index.shape[0]
        self.mem_state[free_index] = True


class _TorchOpsAdapters(InferAdapter):
    """Row copies per layer with indexed stores, compaction with gathers: the steps of the reference on torch ops."""

    def _copy_rows_cuda(self, adapter, loc, prefetch):
        return False

    def _compact_cuda(self, keep):
        dev = self.a_loc.device
        keep_t = torch.tensor(keep, dtype=torch.long, device=dev)
        drop = sorted(set(range(len(self.adapter_dirs))) - set(keep))
        starts, lens = self.a_start.tolist(), self.a_len.tolist()
        rows = torch.cat([self.a_loc[starts[i]: starts[i] + lens[i]] for i in drop])
        self.mem_manager.mem_state[rows] = True
        self.mem_manager.can_use_mem_size += int(rows.numel())
        new_len = self.a_len[keep_t]
        new_start = torch.zeros_like(new_len)
        new_start[1:] = torch.cumsum(new_len, dim=0)[:-1]
        tot = int(new_len.sum().item())
        src = torch.repeat_interleave(self.a_start[keep_t] - new_start, new_len) + torch.arange(tot, device=dev)
        self.a_loc, self.a_scaling = self.a_loc[src], self.a_scaling[keep_t]
        self.a_start, self.a_len = new_start, new_len
        self.adapter_dirs = [self.adapter_dirs[i] for i in keep]
        self.idx_map = {d: i for i, d in enumerate(self.adapter_dirs)}
        self.host_lens = [self.host_lens[i] for i in keep]


def _timed(fn, reps, setup=None):
    gpu, host = [], []
    for _ in range(reps):
        if setup is not None:
            setup()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        fn()
        e1.record()
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        gpu.append(e0.elapsed_time(e1) * 1e3)
        host.append((t1 - t0) * 1e6)
    gpu.sort()
    host.sort()
    return {"gpu_us": round(gpu[len(gpu) // 2], 1), "host_us": round(host[len(host) // 2], 1)}


def run(layers=32, pool_rows=65536, map_rows=262144, rank=64, heads=32, hd=128, n_adapters=32, reps=9):
    gen = torch.Generator(device="cuda").manual_seed(7)
    out = {"metric": "adapter_swap", "unit": "us per call", "layers": layers, "pool_rows": pool_rows,
           "map_rows": map_rows, "rank": rank, "row_bytes": heads * hd * 2, "n_adapters": n_adapters}
    # (1) 4*rank rows out of a fragmented free map of map_rows rows (no pool buffers behind it)
    frag = torch.rand((map_rows,), device="cuda", generator=gen) < 0.3
    for name, cls in (("kernels", MemoryAllocator), ("torch_ops", _TorchOpsAllocator)):
        mm = cls(map_rows, 0, torch.float16, heads, hd, 0, device="cuda", allocate_buffers=False)

        def reset(mm=mm):
            mm.mem_state.copy_(frag)
            mm.can_use_mem_size = map_rows        # the bench never runs the map dry; the count is not under test
        reset()
        mm.alloc(4 * rank)                        # first call builds the workspace
        out.setdefault("alloc", {})[name] = _timed(lambda mm=mm: mm.alloc(4 * rank), reps, reset)
    # (2) one adapter into every layer, (3) half of the resident adapters dropped
    ads = [_Adapter(f"a{i}", rank, heads, hd, layers, gen) for i in range(n_adapters)]
    mm = MemoryAllocator(pool_rows, 0, torch.float16, heads, hd, layers, device="cuda")
    for name, cls, mm_cls in (("kernels", InferAdapter, MemoryAllocator),
                              ("torch_ops", _TorchOpsAdapters, _TorchOpsAllocator)):
        mm.__class__ = mm_cls                     # same pool, the other bookkeeping
        ia = cls.init(mm, None)
        ia.load_adapters(ads[:2])
        state = {"next": 2}

        def load_one(ia=ia, state=state):
            ia.load_adapters([ads[state["next"]]])
            state["next"] += 1
        res = _timed(load_one, min(reps, n_adapters - 2))
        res["bytes"] = 2 * 4 * rank * heads * hd * 2 * layers
        res["gbs_read_write"] = round(2 * res["bytes"] / res["gpu_us"] / 1e3, 1)
        out.setdefault("load_one_adapter", {})[name] = res
        ia.load_adapters(ads)                     # everything resident

        def refill(ia=ia):
            ia.load_adapters(ads)
        keep = [a.lora_dir for a in ads[::2]]
        out.setdefault("offload_half", {})[name] = _timed(lambda ia=ia: ia.offload_adapters(keep), reps, refill)
        ia.offload_adapters([])
        torch.cuda.synchronize()
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--pool-rows", type=int, default=65536)
    ap.add_argument("--map-rows", type=int, default=262144)
    ap.add_argument("--rank", type=int, default=64)
    ap.add_argument("--adapters", type=int, default=32)
    a = ap.parse_args(argv)
    print(json.dumps(run(a.layers, a.pool_rows, a.map_rows, a.rank, n_adapters=a.adapters)), flush=True)


if __name__ == "__main__":
    main()
