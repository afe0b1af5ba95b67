"""Parity of the tensor-core (tcgen05) segment kernels with the CPU oracle: long prefill segments through the
reference's ``lora_get_qkvo_fwd_shrink`` / ``lora_get_qkvo_fwd_expand`` API.  Needs a B200."""
import numpy as np
import pytest
import torch

import slora_b200 as sl
from slora_b200.workloads import build_workload
from tests.helpers import assert_parity, orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _segments(wl):
    seg = wl.segments
    b_start = torch.tensor([s for s, _, _ in seg], dtype=torch.int32, device=DEV)
    b_len = torch.tensor([n for _, n, _ in seg], dtype=torch.int32, device=DEV)
    req_bins = torch.tensor([a for _, _, a in seg], dtype=torch.int64, device=DEV)
    return b_start, b_len, req_bins, max(n for _, n, _ in seg)


def _run_segments(wl, w, p, y_init=None, hidden=None):
    hidden = hidden or wl.spec.hidden
    h_out = wl.proj_dims()[p][1]
    b_start, b_len, req_bins, max_len = _segments(wl)
    x = w.x_o[0] if p == 3 else w.x_qkv[0]
    delta = torch.zeros((wl.T, wl.max_rank), dtype=wl.dtype, device=DEV)
    y = torch.zeros((wl.T, h_out), dtype=wl.dtype, device=DEV) if y_init is None else y_init.clone()
    sl.lora_get_qkvo_fwd_shrink(x, w.pools_a[0], delta, w.a_loc, w.a_start, w.a_len, b_start, b_len, req_bins,
                                hidden, p, wl.max_rank, max_len)
    sl.lora_get_qkvo_fwd_expand(delta, w.pools_b[0], y, w.a_scaling, w.a_loc, w.a_start, w.a_len, b_start, b_len,
                                req_bins, h_out, p, wl.max_rank, max_len)
    torch.cuda.synchronize()
    return delta, y


def _oracle(wl, p, y0=None):
    h_out = wl.proj_dims()[p][1]
    x = wl.x_o[0] if p == 3 else wl.x_qkv[0]
    y0 = np.zeros((wl.T, h_out), dtype=np.float32) if y0 is None else y0
    return orc.lora_delta_ref(y0, x, wl.pools_a[0], wl.pools_b[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p,
                              wl.a_scaling)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_long_segments_mixed_ranks(dtype):
    """Sequences of 20..300 tokens (one, two and three 128-token tiles, and short ones that stay on the CUDA cores)
    plus single decode tokens, adapters of rank 8, 16, 32 and 64."""
    wl = build_workload(3, dtype=dtype, pool_rows=8192, n_adapters=24, decode_tokens=9, prefill=("seqs", 9, 20, 300),
                        hidden=1024)
    w = wl.to(DEV)
    before = sl.launch_counts()["tensor_core"]
    for p in range(4):
        _, y = _run_segments(wl, w, p)
        assert_parity(y, _oracle(wl, p), dtype, what=f"long segments {dtype} proj {p}")
    assert sl.launch_counts()["tensor_core"] - before == 8  # one shrink and one expand launch per projection


def test_shrink_output_and_untouched_columns():
    """The shrink alone against the oracle; columns at and beyond an adapter's rank keep their contents."""
    wl = build_workload(3, pool_rows=8192, n_adapters=12, decode_tokens=0, prefill=("seqs", 4, 100, 260), hidden=1024)
    w = wl.to(DEV)
    b_start, b_len, req_bins, max_len = _segments(wl)
    for p in (0, 2):
        delta = torch.full((wl.T, wl.max_rank), 7.0, dtype=wl.dtype, device=DEV)
        sl.lora_get_qkvo_fwd_shrink(w.x_qkv[0], w.pools_a[0], delta, w.a_loc, w.a_start, w.a_len, b_start, b_len,
                                    req_bins, 1024, p, wl.max_rank, max_len)
        torch.cuda.synchronize()
        got = delta.float().cpu().numpy()
        ref = orc.lora_shrink_ref(wl.x_qkv[0], wl.pools_a[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p, wl.max_rank)
        for t in range(wl.T):
            r = wl.ranks[int(wl.ids[t])]
            assert (got[t, r:] == 7.0).all()
        mask = np.zeros_like(got, dtype=bool)
        for t in range(wl.T):
            mask[t, :wl.ranks[int(wl.ids[t])]] = True
        assert_parity(np.where(mask, got, 0.0), np.where(mask, ref, 0.0), what=f"shrink proj {p}")


def test_expand_accumulates_into_y():
    wl = build_workload(3, pool_rows=8192, n_adapters=12, decode_tokens=3, prefill=("seqs", 3, 64, 200), hidden=1024)
    w = wl.to(DEV)
    g = torch.Generator().manual_seed(11)
    y0 = (torch.randn((wl.T, 1024), generator=g) * 0.05).to(wl.dtype)
    _, y = _run_segments(wl, w, 1, y_init=y0.to(DEV))
    ref = _oracle(wl, 1, y0.float().numpy().copy())
    max_rel, mean_rel = orc.error_metrics(y, ref)
    assert max_rel <= 1e-2 and mean_rel <= 2e-3, (max_rel, mean_rel)


def test_full_width_single_adapter_rank_128():
    """hidden 4096, rank 128, one 512-token sequence: the widest tile the kernels take (K = 128 in the expand)."""
    wl = build_workload(3, pool_rows=2048, n_adapters=2, decode_tokens=0, prefill=("seqs", 1, 512, 512),
                        rank_choices=(128,))
    w = wl.to(DEV)
    for p in (0, 3):
        _, y = _run_segments(wl, w, p)
        assert_parity(y, _oracle(wl, p), what=f"rank 128 proj {p}")


def test_gqa_narrow_outputs_and_ragged_tail():
    """k/v width 320 (not a multiple of the 128-output accumulator tile) over pool rows of 1024 elements."""
    wl = build_workload(5, pool_rows=4096, n_adapters=4, decode_tokens=0, prefill=("seqs", 3, 40, 150), hidden=1024,
                        h_kv=320, rank_choices=(16, 64))
    w = wl.to(DEV)
    before = sl.launch_counts()["tensor_core"]
    for p in (1, 2):
        _, y = _run_segments(wl, w, p)
        assert_parity(y, _oracle(wl, p), what=f"gqa proj {p}")
    assert sl.launch_counts()["tensor_core"] > before


def test_out_of_range_pool_row_skips_the_tile():
    """A loc entry beyond the pool: the tile is skipped (y unchanged), nothing is read out of bounds."""
    wl = build_workload(3, pool_rows=4096, n_adapters=2, decode_tokens=0, prefill=("seqs", 1, 128, 128), hidden=1024,
                        rank_choices=(16,))
    w = wl.to(DEV)
    a = int(wl.segments[0][2])
    bad = w.a_loc.clone()
    bad[int(wl.a_start[a]) + 3] = 1 << 40
    w.a_loc = bad
    _, y = _run_segments(wl, w, 0)
    assert float(y.abs().max()) == 0.0


def _planned_layer(wl, w, use_pdl=True):
    ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, w.max_rank, use_pdl)
    ops.prepare(w.ids)
    H, K = wl.spec.hidden, wl.spec.h_kv
    outs = [torch.zeros((wl.T, n), dtype=wl.dtype, device=DEV) for n in (H, K, K, H)]
    ops.lora_get_qkv(0, w.x_qkv[0], outs[0], outs[1], outs[2])
    ops.lora_get_o(0, w.x_o[0], outs[3])
    torch.cuda.synchronize()
    ops.plan.check()
    return outs


@pytest.mark.parametrize("use_pdl", [True, False])
def test_planned_batch_routes_big_groups_to_the_tensor_cores(use_pdl):
    """A mixed batch through LoraBatchOps: sequences of 130..400 tokens (same-adapter groups of 128 tokens or more,
    gathered through the plan's permutation) run on the tensor cores, the decode tokens and short sequences on the
    CUDA cores, in the same calls."""
    wl = build_workload(3, pool_rows=8192, n_adapters=16, decode_tokens=40, prefill=("seqs", 5, 20, 400), hidden=1024)
    assert max(n for _, n, _ in wl.segments) >= 128
    w = wl.to(DEV)
    before = sl.launch_counts()
    outs = _planned_layer(wl, w, use_pdl)
    after = sl.launch_counts()
    assert after["tensor_core"] - before["tensor_core"] == 4    # q,k,v shrink, q,k,v expand, o shrink, o expand
    cuda_core = sum(after[k] - before[k] for k in ("pipelined", "simple"))
    assert cuda_core == 4                                       # the rest of the batch, same four calls
    for p in range(4):
        assert_parity(outs[p], _oracle(wl, p), what=f"planned big groups proj {p}")


def test_planned_batch_bf16_rank_128():
    wl = build_workload(3, dtype=torch.bfloat16, pool_rows=4096, n_adapters=3, decode_tokens=10,
                        prefill=("seqs", 2, 200, 300), hidden=1024, rank_choices=(128,))
    w = wl.to(DEV)
    outs = _planned_layer(wl, w)
    for p in range(4):
        assert_parity(outs[p], _oracle(wl, p), torch.bfloat16, what=f"planned rank 128 proj {p}")


def test_small_batch_below_one_tile():
    """One 40-token sequence: the whole batch is smaller than the 128-row box of the tensor maps."""
    wl = build_workload(3, pool_rows=4096, n_adapters=2, decode_tokens=0, prefill=("seqs", 1, 40, 40), hidden=1024,
                        rank_choices=(16,))
    w = wl.to(DEV)
    for p in (0, 3):
        _, y = _run_segments(wl, w, p)
        assert_parity(y, _oracle(wl, p), what=f"40 tokens proj {p}")


def test_empty_and_out_of_range_segments_are_ignored():
    """Zero-length segments, a segment that runs past the batch and a grid sized for a length no segment has: the
    valid tokens are computed, everything else is left alone."""
    wl = build_workload(3, pool_rows=4096, n_adapters=4, decode_tokens=0, prefill=("seqs", 2, 150, 150), hidden=1024,
                        rank_choices=(16,))
    w = wl.to(DEV)
    T = wl.T                                   # 300 tokens: two sequences of 150
    (s0, n0, a0), (s1, n1, a1) = wl.segments
    b_start = torch.tensor([s0, 0, s1, s1 + 100], dtype=torch.int32, device=DEV)
    b_len = torch.tensor([n0, 0, 100, 50 + 77], dtype=torch.int32, device=DEV)      # the last one runs 77 past T
    req = torch.tensor([a0, a0, a1, a1], dtype=torch.int64, device=DEV)
    delta = torch.zeros((T, wl.max_rank), dtype=wl.dtype, device=DEV)
    y = torch.zeros((T, 1024), dtype=wl.dtype, device=DEV)
    guard = torch.full((64, 1024), 9.0, dtype=wl.dtype, device=DEV)                 # memory right behind nothing we own
    sl.lora_get_qkvo_fwd_shrink(w.x_qkv[0], w.pools_a[0], delta, w.a_loc, w.a_start, w.a_len, b_start, b_len, req,
                                1024, 0, wl.max_rank, 1000)
    sl.lora_get_qkvo_fwd_expand(delta, w.pools_b[0], y, w.a_scaling, w.a_loc, w.a_start, w.a_len, b_start, b_len, req,
                                1024, 0, wl.max_rank, 1000)
    torch.cuda.synchronize()
    assert float(guard.min()) == 9.0
    assert_parity(y, _oracle(wl, 0), what="ragged segment table")


def test_pure_prefill_batch_launches_no_cuda_core_kernel():
    """Every group of the plan is a big group the tensor-core kernels serve (sequences of 128 tokens or more, ranks
    that are powers of two): prepare() finds that in the plan header and the four calls launch the four tensor-core
    kernels only.  One short sequence more and the CUDA-core launches are back."""
    wl = build_workload(3, pool_rows=8192, n_adapters=16, decode_tokens=0, prefill=("seqs", 4, 130, 400), hidden=1024)
    w = wl.to(DEV)
    before = sl.launch_counts()
    outs = _planned_layer(wl, w)
    after = sl.launch_counts()
    assert after["tensor_core"] - before["tensor_core"] == 4
    assert sum(after[k] - before[k] for k in ("pipelined", "simple")) == 0
    for p in range(4):
        assert_parity(outs[p], _oracle(wl, p), what=f"pure prefill proj {p}")
    h = sl.BatchPlan(w.ids, w.a_start, w.a_len, w.a_loc.numel()).header()
    assert h["small_tiles"] == 0 and h["big_tiles"] > 0 and h["big_ranks_pow2"] and h["tokens"] == wl.T
    wl2 = build_workload(3, pool_rows=8192, n_adapters=16, decode_tokens=1, prefill=("seqs", 4, 130, 400), hidden=1024)
    w2 = wl2.to(DEV)
    before = sl.launch_counts()
    outs = _planned_layer(wl2, w2)
    after = sl.launch_counts()
    assert sum(after[k] - before[k] for k in ("pipelined", "simple")) == 4
    for p in range(4):
        assert_parity(outs[p], _oracle(wl2, p), what=f"prefill + one decode token proj {p}")


def test_segment_call_without_short_segments_leaves_its_cuda_core_launch_early():
    """Segments of 32 tokens or more only: the accompanying CUDA-core launch finds nothing to do (its early exit);
    results are those of the tensor-core kernels.  With one short segment added its rows are computed as well."""
    for short in (0, 1):
        wl = build_workload(3, pool_rows=8192, n_adapters=12, decode_tokens=short, prefill=("seqs", 3, 40, 200),
                            hidden=1024)
        w = wl.to(DEV)
        for p in (0, 3):
            _, y = _run_segments(wl, w, p)
            assert_parity(y, _oracle(wl, p), what=f"segments, {short} short, proj {p}")
