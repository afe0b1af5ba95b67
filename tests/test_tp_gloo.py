"""S-LoRA tensor parallelism on two CPU ranks (gloo): shard builder, intermediate exchange and the layout the
kernels are given, with the oracle standing in for the CUDA kernels.  Concatenating the ranks' output slices must
reproduce the single-rank oracle."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.helpers import ROOT, orc
from slora_b200 import tp
from slora_b200.workloads import make_tables

H, WORLD, T = 64, 2, 12
RANKS = [8, 16, 8]


class OracleBackend:
    """Same contract as tp.CudaBackend, computed with the CPU oracle (test infrastructure)."""

    def make_plan(self, ids, t, local_width=None):
        return None

    def shrink(self, plan, ids, qkvo, deltas, x, pool_a, t, rank_mult=1):
        for p, d in zip(qkvo, deltas):
            out = orc.lora_shrink_ref(x, pool_a, t.a_start, t.a_len, t.a_loc, ids, p, out_width=d.shape[1],
                                      rank_mult=rank_mult)
            d.copy_(torch.from_numpy(out))

    def expand(self, plan, ids, qkvo, ys, deltas, pool_b, t, delta_stride, delta_width, delta_parts, delta_part_stride,
               rank_mult):
        for p, y, d in zip(qkvo, ys, deltas):
            # rebuild delta[t, k] from the gathered parts exactly as the kernel indexes them
            flat = d.reshape(-1) if d.is_contiguous() else None
            base = d.storage_offset()
            store = torch.as_strided(d, (d.untyped_storage().nbytes() // d.element_size(),), (1,), 0)
            Tn = y.shape[0]
            full = torch.zeros((Tn, delta_width * delta_parts), dtype=torch.float32)
            for tok in range(Tn):
                a = int(ids[tok])
                rk = int(t.a_len[a]) // 4 * rank_mult
                rs = rk // delta_parts
                for k in range(rk):
                    part, j = divmod(k, rs)
                    full[tok, k] = store[base + part * delta_part_stride + tok * delta_stride + j]
            out = orc.lora_expand_ref(y, full, pool_b, t.a_start, t.a_len, t.a_loc, ids, p, t.a_scaling, rank_mult)
            y.copy_(torch.from_numpy(out))


class OracleRegroupBackend(OracleBackend):
    """The same with the regroup step of tp.CudaBackend (slora_tp_regroup), restated in torch."""

    def regroup(self, out, gathered, ids, t, n_parts, nproj, part_width, part_stride):
        store = torch.as_strided(gathered, (gathered.untyped_storage().nbytes() // gathered.element_size(),), (1,), 0)
        base = gathered.storage_offset()
        Tn = ids.numel()
        for p in range(nproj):
            for tok in range(Tn):
                rs = int(t.a_len[int(ids[tok])]) // 4
                for g in range(n_parts):
                    src = base + g * part_stride + (p * Tn + tok) * part_width
                    out[p, tok, g * rs:(g + 1) * rs] = store[src:src + rs]


def _logical_adapters(seed):
    g = torch.Generator().manual_seed(seed)
    ads = []
    for r in RANKS:
        A = [torch.randn((r, H), generator=g) / 8 for _ in range(4)]
        B = [torch.randn((H, r), generator=g) / 8 for _ in range(4)]
        ads.append((A, B))
    return ads


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, port, out_dir, regroup, o_sharded=False):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    ads = _logical_adapters(11)
    pool_rows = 128
    local_ranks = [r // WORLD for r in RANKS]
    a_start, a_len, a_loc = make_tables(local_ranks, pool_rows, 100 + rank, True)
    pool_a = torch.zeros((pool_rows, H))
    pool_b = torch.zeros((pool_rows, H))
    for i, (A, B) in enumerate(ads):
        ra, rb = tp.shard_adapter(A, B, rank, WORLD, H, o_input_sharded=o_sharded)
        loc = a_loc[a_start[i]: a_start[i] + a_len[i]]
        pool_a[loc] = ra
        pool_b[loc] = rb
    tables = tp.TpTables(a_start, a_len, a_loc, torch.tensor([16.0 / r for r in RANKS]))
    g = torch.Generator().manual_seed(5)
    x_qkv, x_o = torch.randn((T, H), generator=g), torch.randn((T, H), generator=g)
    ids = torch.randint(0, len(RANKS), (T,), generator=g)
    backend = OracleRegroupBackend() if regroup else OracleBackend()
    ops = tp.TpLoraOps(tables, [pool_a], [pool_b], max(RANKS), WORLD, rank, backend).prepare(ids)
    q, k, v, o = (torch.zeros((T, H // WORLD)) for _ in range(4))
    ops.lora_qkv(0, x_qkv, q, k, v)
    if o_sharded:   # the attention output arrives head-sharded: this rank sees its columns only
        hs = H // WORLD
        ops.lora_o_sharded(0, x_o[:, rank * hs:(rank + 1) * hs].contiguous(), o)
    else:
        ops.lora_o(0, x_o, o)
    torch.save({"q": q, "k": k, "v": v, "o": o, "x_qkv": x_qkv, "x_o": x_o, "ids": ids},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("regroup", [False, True])
def test_two_rank_tp_matches_single_rank(tmp_path, regroup):
    """regroup=False: the expand reads the gathered [N, nproj, T, R/N] buffer; True: all-gather, regroup, plain rows."""
    mp.spawn(_worker, args=(_free_port(), str(tmp_path), regroup), nprocs=WORLD, join=True)
    outs = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(WORLD)]
    ads = _logical_adapters(11)
    ids, x_qkv, x_o = outs[0]["ids"], outs[0]["x_qkv"], outs[0]["x_o"]
    for p, name in enumerate("qkvo"):
        got = torch.cat([o[name] for o in outs], dim=1)
        x = x_o if p == 3 else x_qkv
        want = torch.stack([(x[t] @ ads[int(ids[t])][0][p].T) @ ads[int(ids[t])][1][p].T * (16.0 / RANKS[int(ids[t])])
                            for t in range(T)])
        np.testing.assert_allclose(got.numpy(), want.numpy(), rtol=1e-4, atol=1e-5)


def test_two_rank_tp_with_input_sharded_o_projection(tmp_path):
    """The o projection with a head-sharded input: A cut over its input columns, partial results summed over the ranks
    (all_reduce), B output-sharded as before."""
    mp.spawn(_worker, args=(_free_port(), str(tmp_path), False, True), nprocs=WORLD, join=True)
    outs = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(WORLD)]
    ads = _logical_adapters(11)
    ids, x_o = outs[0]["ids"], outs[0]["x_o"]
    got = torch.cat([o["o"] for o in outs], dim=1)
    want = torch.stack([(x_o[t] @ ads[int(ids[t])][0][3].T) @ ads[int(ids[t])][1][3].T * (16.0 / RANKS[int(ids[t])])
                        for t in range(T)])
    np.testing.assert_allclose(got.numpy(), want.numpy(), rtol=1e-4, atol=1e-5)


def test_shard_adapter_layout():
    A, B = _logical_adapters(3)[1]
    ra, rb = tp.shard_adapter(A, B, 1, 2, H)
    r = RANKS[1]
    assert ra.shape == (4 * r // 2, H) and rb.shape == (4 * r // 2, H)
    assert torch.equal(ra[: r // 2], A[0][r // 2:])
    assert torch.equal(rb[r // 2: r].reshape(-1)[: (H // 2) * r].view(H // 2, r), B[1][H // 2:])
    with pytest.raises(ValueError):
        tp.shard_adapter(A, B, 0, 3, H)
