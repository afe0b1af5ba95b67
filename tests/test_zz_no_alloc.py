"""The entry point that allocates nothing (``slora_batch_lora_o_noalloc``) against the ordinary one.

Some callers cannot allocate device memory when they need a LoRA delta: their process's own pool already holds the
whole GPU, or they run where ``cudaMalloc`` is off limits.  For them the library carries its scratch (batch plan and
rank-r intermediate) in a built-in device array.  This test calls that entry point through the C ABI twice in a row on
different inputs and checks each result against ``slora_batch_lora_o`` with caller-provided scratch; both run the same
kernels, so the results must be identical.  It lives in a file collected last so that a failure here cannot hide the
outcome of any other test.
"""
import pytest
import torch

import slora_b200 as sl
from slora_b200 import batch_infer
from slora_b200.workloads import build_workload
from tests.helpers import assert_parity, oracle_layer

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _reference_o(w, layer):
    ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, w.max_rank)
    ops.prepare(w.ids)
    o = torch.zeros((w.T, w.spec.hidden), dtype=w.dtype, device=DEV)
    ops.lora_get_o(layer, w.x_o[layer], o)
    torch.cuda.synchronize()
    ops.plan.check()
    return o


def test_no_alloc_entry_point_matches_the_ordinary_one_twice():
    first_cpu = build_workload(3, pool_rows=8192, n_adapters=40, decode_tokens=70, prefill=("seqs", 2, 5, 30),
                               hidden=2048)
    second_cpu = build_workload(2, pool_rows=4096, n_adapters=12, decode_tokens=33, hidden=1024, rank_choices=(8, 16))
    second = second_cpu.to(DEV)
    warm = torch.zeros((second.T, 1024), dtype=second.dtype, device=DEV)
    batch_infer.lora_o_noalloc(second.ids, second.x_o[0], warm, second.pools_a[0], second.pools_b[0], second.a_start,
                               second.a_len, second.a_loc, second.a_scaling, second.max_rank)   # loads the kernels
    torch.cuda.synchronize()
    for wl in (first_cpu, second_cpu):       # two calls in a row share the built-in scratch: the second must not see the first
        w = wl.to(DEV)
        want = _reference_o(w, 0)
        got = torch.zeros_like(want)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        batch_infer.lora_o_noalloc(w.ids, w.x_o[0], got, w.pools_a[0], w.pools_b[0], w.a_start, w.a_len, w.a_loc,
                                   w.a_scaling, w.max_rank)
        assert torch.cuda.memory_allocated() == before      # not even through torch's caching allocator
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before  # nor from the driver, behind torch's back
        assert torch.equal(got, want)
        assert float(got.abs().max()) > 0
        assert batch_infer.noalloc_status() == 0
        assert_parity(got, oracle_layer(wl)[3], what="no-alloc entry point against the oracle")


def test_no_alloc_entry_point_rejects_sizes_beyond_its_scratch():
    w = build_workload(2, pool_rows=4096, n_adapters=4, decode_tokens=8, hidden=1024).to(DEV)
    big_ids = torch.zeros(1025, dtype=torch.int64, device=DEV)
    big_x = torch.zeros((1025, 1024), dtype=w.dtype, device=DEV)
    big_o = torch.zeros_like(big_x)
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        batch_infer.lora_o_noalloc(big_ids, big_x, big_o, w.pools_a[0], w.pools_b[0], w.a_start, w.a_len, w.a_loc,
                                   w.a_scaling, w.max_rank)
    o = torch.zeros((w.T, 1024), dtype=w.dtype, device=DEV)
    with pytest.raises(RuntimeError, match="max_rank"):
        batch_infer.lora_o_noalloc(w.ids, w.x_o[0], o, w.pools_a[0], w.pools_b[0], w.a_start, w.a_len, w.a_loc,
                                   w.a_scaling, 256)


def test_no_alloc_entry_point_reports_what_its_kernels_skipped():
    """A token whose adapter id is outside the tables is skipped; the status word in the built-in scratch says so
    (the caller holds no pointer to that word, hence the accessor), and the wrapper refuses what the C entry would
    index blindly."""
    w = build_workload(2, pool_rows=4096, n_adapters=6, decode_tokens=16, hidden=1024).to(DEV)
    ids = w.ids.clone()
    ids[5] = 77
    o = torch.zeros((w.T, 1024), dtype=w.dtype, device=DEV)
    batch_infer.lora_o_noalloc(ids, w.x_o[0], o, w.pools_a[0], w.pools_b[0], w.a_start, w.a_len, w.a_loc,
                               w.a_scaling, w.max_rank)
    assert batch_infer.noalloc_status() & 1
    assert float(o[5].abs().max()) == 0.0 and float(o[4].abs().max()) > 0
    with pytest.raises(RuntimeError, match="int64"):
        batch_infer.lora_o_noalloc(w.ids.to(torch.int32), w.x_o[0], o, w.pools_a[0], w.pools_b[0], w.a_start, w.a_len,
                                   w.a_loc, w.a_scaling, w.max_rank)
    with pytest.raises(RuntimeError, match="one row per entry"):
        batch_infer.lora_o_noalloc(w.ids[:-1], w.x_o[0], o, w.pools_a[0], w.pools_b[0], w.a_start, w.a_len, w.a_loc,
                                   w.a_scaling, w.max_rank)
    batch_infer.lora_o_noalloc(w.ids, w.x_o[0], o, w.pools_a[0], w.pools_b[0], w.a_start, w.a_len, w.a_loc,
                               w.a_scaling, w.max_rank)
    assert batch_infer.noalloc_status() == 0          # the next call's plan starts from a clean word
