"""Parity at the real widths of the S2-, S4- and S6-shaped configurations, through ``LoraBatchOps`` with the flags that
``prepare()`` picks by itself (exact work-item count, 8-row shrink items, the long expand ring, tensor-core routing of
big same-adapter groups, k/v narrower than a pool row).  The adapter count and the pool are cut down so that the host
side of a case stays within seconds; hidden size, ranks, token counts and the batch composition are the
configuration's own.  Checked against the adapter-grouped form of the CPU oracle (same numbers as the per-token
formula, one matrix product per distinct adapter).  Needs a B200."""
import numpy as np
import pytest
import torch

import slora_b200 as sl
from slora_b200 import _lib
from slora_b200.workloads import build_workload
from tests.helpers import assert_parity, orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _grouped_oracle(wl, layer=0):
    outs = []
    for p, (h_in, h_out) in enumerate(wl.proj_dims()):
        x = wl.x_o[layer] if p == 3 else wl.x_qkv[layer]
        outs.append(orc.lora_delta_grouped(np.zeros((wl.T, h_out), dtype=np.float32), x, wl.pools_a[layer],
                                           wl.pools_b[layer], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p, wl.a_scaling))
    return outs


def _run(w, **prepare_kw):
    ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, w.max_rank)
    ops.prepare(w.ids, **prepare_kw)
    H, K = w.spec.hidden, w.spec.h_kv
    q = torch.zeros((w.T, H), dtype=w.dtype, device=DEV)
    k = torch.zeros((w.T, K), dtype=w.dtype, device=DEV)
    v = torch.zeros((w.T, K), dtype=w.dtype, device=DEV)
    o = torch.zeros((w.T, H), dtype=w.dtype, device=DEV)
    ops.lora_get_qkv(0, w.x_qkv[0], q, k, v)
    ops.lora_get_o(0, w.x_o[0], o)
    torch.cuda.synchronize()
    ops.plan.check()
    return [q, k, v, o], ops


def test_s4_shape_hidden_5120_mixed_ranks():
    """Hidden 5120, ranks {64, 32, 16}, 512 tokens = 461 decode tokens Zipf(0.8) + prefill chunks of 16..256 tokens;
    300 resident adapters in a pool of 49152 rows.  prepare() must turn on the exact work-item count."""
    wl = build_workload(4, pool_rows=49152, n_adapters=300)
    assert wl.T == 512 and wl.spec.hidden == 5120 and set(wl.ranks) == {16, 32, 64}
    outs, ops = _run(wl.to(DEV))
    assert ops.flags & _lib.FLAG_EXACT_ITEMS
    ref = _grouped_oracle(wl)
    for p in range(4):
        assert_parity(outs[p], ref[p], what=f"S4 shape proj {p}")
    # the padded enumeration of work items gives the same bits
    plain, _ = _run(wl.to(DEV), mixed_ranks=False, big_groups=False)
    for p in range(4):
        assert torch.equal(plain[p], outs[p])


def test_s6_shape_hidden_8192_gqa_rank_64():
    """Hidden 8192, k/v width 1024 (a B matrix of k or v fills 8 of its slot's 64 pool rows), 200 adapters of rank
    64, 1024 decode tokens with uniform adapter ids."""
    wl = build_workload(5, pool_rows=53248)
    assert wl.T == 1024 and wl.spec.hidden == 8192 and wl.spec.h_kv == 1024 and set(wl.ranks) == {64}
    outs, _ = _run(wl.to(DEV))
    ref = _grouped_oracle(wl)
    for p in range(4):
        assert outs[p].shape[1] == (1024 if p in (1, 2) else 8192)
        assert_parity(outs[p], ref[p], what=f"S6 shape proj {p}")


def test_s2_shape_hidden_4096_prefill_sequences_on_the_tensor_cores():
    """Hidden 4096, ranks {64, 32, 16, 8}, 8 prefill sequences of 8..512 tokens + 248 decode tokens Zipf(1.0): the
    sequences of 128 tokens or more run on the tensor-core kernels (prepare() finds them in the plan), the rest of
    the same call on the CUDA-core kernels."""
    wl = build_workload(3, pool_rows=32768, n_adapters=200)
    assert wl.spec.hidden == 4096 and wl.T >= 248 + 8 * 8
    long_seqs = [n for _, n, _ in wl.segments if n >= 128]
    assert long_seqs, "the seeded batch is expected to hold sequences of 128 tokens or more"
    before = sl.launch_counts()["tensor_core"]
    outs, ops = _run(wl.to(DEV))
    assert ops.flags & _lib.FLAG_BIG_GROUPS and ops.flags & _lib.FLAG_EXACT_ITEMS
    assert sl.launch_counts()["tensor_core"] - before == 4  # shrink + expand, q/k/v call and o call
    ref = _grouped_oracle(wl)
    for p in range(4):
        assert_parity(outs[p], ref[p], what=f"S2 shape proj {p}")
    # the same batch entirely on the CUDA cores
    plain, _ = _run(wl.to(DEV), big_groups=False)
    for p in range(4):
        assert_parity(plain[p], ref[p], what=f"S2 shape, CUDA cores only, proj {p}")


def test_s1_shape_full_pool():
    """Hidden 4096, 1000 adapters of rank 8 scattered over the full [262144, 4096] pool, 256 tokens Zipf(1.0)."""
    wl = build_workload(2)
    assert wl.spec.pool_rows == 262144 and wl.T == 256
    outs, _ = _run(wl.to(DEV))
    ref = _grouped_oracle(wl)
    for p in range(4):
        assert_parity(outs[p], ref[p], what=f"S1 shape proj {p}")
