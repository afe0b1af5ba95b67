"""The q/k/v call with the rotary embedding and the KV-pool scatter in the expand's epilogue
(``LoraBatchOps.lora_get_qkv(..., rope=, kv_dest=)``, C entry ``slora_batch_lora_qkv_rope``) against the CPU oracles:
LoRA delta (``oracle/lora_oracle.py``) on top of a base projection, rounded to fp16 where the reference stores it,
then ``oracle/rope_oracle.py``.  Needs a B200."""
import numpy as np
import pytest
import torch

import slora_b200 as sl
from oracle import rope_oracle as rorc
from slora_b200.workloads import build_workload
from tests.helpers import assert_parity, orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(wl, head_dim, seed=7):
    g = torch.Generator().manual_seed(seed)
    H, K, T = wl.spec.hidden, wl.spec.h_kv, wl.T
    base = [(torch.randn((T, n), generator=g) * 0.5).to(wl.dtype) for n in (H, K, K)]
    pos = torch.randint(0, 4096, (T,), generator=g).float()
    inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))
    fr = torch.outer(pos, inv)
    return base, torch.cos(fr).to(wl.dtype), torch.sin(fr).to(wl.dtype)


def _expected(wl, base, cos, sin):
    """q, k, v as the reference's sequence leaves them: y = fp16(base + delta); q, k rotated."""
    outs = []
    for p in range(3):
        y = orc.lora_delta_grouped(base[p].float().numpy(), wl.x_qkv[0], wl.pools_a[0], wl.pools_b[0], wl.a_start,
                                   wl.a_len, wl.a_loc, wl.ids, p, wl.a_scaling)
        y = y.astype(np.float16 if wl.dtype == torch.float16 else np.float32).astype(np.float32)
        if wl.dtype == torch.bfloat16:
            y = torch.from_numpy(y).to(torch.bfloat16).float().numpy()
        outs.append(rorc.rotary_ref(y, cos.float().numpy(), sin.float().numpy()) if p < 2 else y)
    return outs


def _run(wl, base, cos, sin, head_dim=128, kv_dest=None, **prepare_kw):
    w = wl.to(DEV)
    ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, w.max_rank)
    ops.prepare(w.ids, **prepare_kw)
    q, k, v = (b.clone().to(DEV) for b in base)
    ops.lora_get_qkv(0, w.x_qkv[0], q, k, v, rope=(cos.to(DEV), sin.to(DEV)), kv_dest=kv_dest, head_dim=head_dim)
    torch.cuda.synchronize()
    return q, k, v, ops


@pytest.mark.parametrize("case", ["s1_rank8", "mixed_ranks_gqa", "rank128", "bf16"])
def test_rotary_in_the_expand_epilogue_in_place(case):
    dt = torch.float16
    if case == "s1_rank8":
        wl = build_workload(2, pool_rows=65536)
    elif case == "mixed_ranks_gqa":
        wl = build_workload(5, pool_rows=16384, n_adapters=60, decode_tokens=300, hidden=4096, h_kv=1024,
                            rank_choices=(8, 16, 32, 64))
    elif case == "rank128":
        wl = build_workload(2, pool_rows=8192, n_adapters=6, decode_tokens=40, rank_choices=(128,))
    else:
        dt = torch.bfloat16
        wl = build_workload(3, dtype=dt, pool_rows=16384, n_adapters=40, decode_tokens=150, prefill=None)
    base, cos, sin = _inputs(wl, 128)
    before = sl.launch_counts()
    q, k, v, ops = _run(wl, base, cos, sin)
    after = sl.launch_counts()
    ops.plan.check()
    assert after["pipelined"] - before["pipelined"] == 2 and after["simple"] == before["simple"]   # no pass of its own
    want = _expected(wl, base, cos, sin)
    for name, got, ref in zip("qkv", (q, k, v), want):
        assert_parity(got, ref, dt, what=f"{case} {name} after the rotary epilogue")


def test_kv_rows_go_straight_into_the_pool():
    wl = build_workload(2, pool_rows=65536, decode_tokens=200)
    base, cos, sin = _inputs(wl, 128)
    T, K = wl.T, wl.spec.h_kv
    g = torch.Generator().manual_seed(3)
    rows = torch.randperm(1000, generator=g)[:T].to(torch.int64)
    k_pool = torch.full((1000, 32, 128), 9.0, dtype=wl.dtype, device=DEV)       # key_buffer[layer] of the KV pool
    v_pool = torch.full((1000, 32, 128), 9.0, dtype=wl.dtype, device=DEV)
    q, k, v, ops = _run(wl, base, cos, sin, kv_dest=(rows.to(DEV), k_pool, v_pool))
    ops.plan.check()
    want = _expected(wl, base, cos, sin)
    assert_parity(q, want[0], what="q")
    assert torch.equal(k.cpu(), base[1]) and torch.equal(v.cpu(), base[2])      # the base projections are only read
    assert_parity(k_pool.view(1000, -1)[rows.to(DEV)], want[1], what="k rows in the pool")
    assert_parity(v_pool.view(1000, -1)[rows.to(DEV)], want[2], what="v rows in the pool")
    other = torch.ones(1000, dtype=torch.bool)
    other[rows] = False
    assert bool((k_pool.view(1000, -1)[other.to(DEV)] == 9.0).all()) and bool((v_pool.view(1000, -1)[other.to(DEV)] == 9.0).all())
    # a destination row outside the pool: that token is skipped and reported, the others are written
    bad = rows.clone()
    bad[5] = 5000
    k_pool.fill_(9.0)
    q, k, v, ops = _run(wl, base, cos, sin, kv_dest=(bad.to(DEV), k_pool, v_pool))
    assert ops.plan.status()[0] & 2
    keep = [t for t in range(T) if t != 5]
    assert_parity(k_pool.view(1000, -1)[rows[keep].to(DEV)], want[1][keep], what="k rows beside a bad destination")
    assert bool((k_pool.view(1000, -1)[rows[5]] == 9.0).all())


@pytest.mark.parametrize("case", ["head_dim_64", "big_groups", "narrow_pool_rows"])
def test_rotary_as_a_pass_of_its_own_where_the_epilogue_does_not_apply(case):
    head_dim = 128
    if case == "head_dim_64":
        head_dim = 64
        wl = build_workload(2, pool_rows=8192, n_adapters=12, decode_tokens=50)
    elif case == "big_groups":
        wl = build_workload(3, pool_rows=16384, n_adapters=12, decode_tokens=20, prefill=("seqs", 2, 130, 300))
    else:
        wl = build_workload(2, pool_rows=8192, n_adapters=12, decode_tokens=50, hidden=1024)
    base, cos, sin = _inputs(wl, head_dim)
    T = wl.T
    rows = torch.arange(T, dtype=torch.int64).flip(0)
    k_pool = torch.zeros((T, wl.spec.h_kv), dtype=wl.dtype, device=DEV)
    v_pool = torch.zeros((T, wl.spec.h_kv), dtype=wl.dtype, device=DEV)
    before = sl.launch_counts()
    q, k, v, ops = _run(wl, base, cos, sin, head_dim=head_dim, kv_dest=(rows.to(DEV), k_pool, v_pool))
    after = sl.launch_counts()
    ops.plan.check()
    assert after["simple"] - before["simple"] >= 1          # the rotary / scatter launch (counted with that family)
    want = _expected(wl, base, cos, sin)
    assert_parity(q, want[0], what=f"{case} q")
    assert_parity(k_pool[rows.to(DEV)], want[1], what=f"{case} k")
    assert_parity(v_pool[rows.to(DEV)], want[2], what=f"{case} v")
