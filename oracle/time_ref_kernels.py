"""Times the REFERENCE's own BGMV CUDA kernels (compiled from the reference tree by oracle/Makefile into
oracle/_ref/libref_bgmv.so) on the S1-shaped decode batch, beside this library on the same inputs.

TEST / MEASUREMENT INFRASTRUCTURE ONLY: nothing in the package imports this file.  Needs a GPU and the reference
library.  Run from the repository root:  python oracle/time_ref_kernels.py [--config 2] [--phys-layers 4]

The reference's call pattern is kept (lora_unordered_batch_infer.py:254-318,428-448): per layer eight dispatch_bgmv
launches (shrink + expand for q, k, v, o) on the legacy default stream, per-token adapter ids.  A step is all layers
of the model; the time is CUDA-event time of whole steps.  One JSON line on stdout.
"""
import argparse
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--phys-layers", type=int, default=4)
    ap.add_argument("--pool-rows", type=int, default=65536)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    import slora_b200 as sl
    from slora_b200.workloads import build_workload
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_bgmv.so"))
    lib.ref_dispatch_bgmv.restype = ctypes.c_int
    lib.ref_dispatch_bgmv.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                                             ctypes.c_int, ctypes.c_void_p]
    w = build_workload(args.config, device="cuda", phys_layers=args.phys_layers, pool_rows=args.pool_rows)
    L, P, T, H, R = w.spec.layers, args.phys_layers, w.T, w.spec.hidden, w.max_rank
    assert w.spec.h_kv == H, "the reference kernels need k/v as wide as the pool rows"
    delta = [torch.zeros((T, R), dtype=w.dtype, device="cuda") for _ in range(3)]
    ys = [[torch.zeros((T, H), dtype=w.dtype, device="cuda") for _ in range(4)] for _ in range(P)]

    def ref_step():
        for l in range(L):
            p = l % P
            for proj in range(4):
                x = w.x_o[p] if proj == 3 else w.x_qkv[p]
                d = delta[0] if proj == 3 else delta[proj]
                for out, inp, pool, hi, ho in ((d, x, w.pools_a[p], H, R), (ys[p][proj], d, w.pools_b[p], R, H)):
                    rc = lib.ref_dispatch_bgmv(out.data_ptr(), inp.data_ptr(), pool.data_ptr(), w.a_start.data_ptr(),
                                               w.a_len.data_ptr(), w.a_loc.data_ptr(), w.ids.data_ptr(), proj, T, hi,
                                               ho, w.a_scaling.data_ptr())
                    if rc != 0:
                        raise RuntimeError(f"the reference has no kernel for ({hi}, {ho})")

    ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, R)
    ops.prepare(w.ids)

    def our_step():
        for l in range(L):
            p = l % P
            ops.lora_get_qkv(p, w.x_qkv[p], ys[p][0], ys[p][1], ys[p][2])
            ops.lora_get_o(p, w.x_o[p], ys[p][3])

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    ms_ref = timed(ref_step)
    ms_ours = timed(our_step)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        our_step()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        our_step()
    ms_graph = timed(g.replay)
    print(json.dumps({
        "workload": w.spec.name, "tokens": T, "layers": L, "phys_layers": P, "pool_rows": args.pool_rows,
        "reference_kernels": {"ms_per_step": ms_ref, "tokens_per_s": T / ms_ref * 1e3, "launches_per_step": 8 * L,
                              "how": "the reference's bgmv kernels, sm_100a build, eager, legacy default stream"},
        "this_library_eager": {"ms_per_step": ms_ours, "tokens_per_s": T / ms_ours * 1e3, "launches_per_step": 4 * L},
        "this_library_graph": {"ms_per_step": ms_graph, "tokens_per_s": T / ms_graph * 1e3},
        "speedup_eager": ms_ref / ms_ours, "speedup_graph": ms_ref / ms_graph}), flush=True)


if __name__ == "__main__":
    main()
