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
    first = build_workload(3, pool_rows=8192, n_adapters=40, decode_tokens=70, prefill=("seqs", 2, 5, 30),
                           hidden=2048).to(DEV)
    second = build_workload(2, pool_rows=4096, n_adapters=12, decode_tokens=33, hidden=1024,
                            rank_choices=(8, 16)).to(DEV)
    for w in (first, second):       # two calls in a row share the built-in scratch: the second must not see the first
        want = _reference_o(w, 0)
        got = torch.zeros_like(want)
        before = torch.cuda.memory_allocated()
        batch_infer.lora_o_noalloc(w.ids, w.x_o[0], got, w.pools_a[0], w.pools_b[0], w.a_start, w.a_len, w.a_loc,
                                   w.a_scaling, w.max_rank)
        assert torch.cuda.memory_allocated() == before      # not even through torch's caching allocator
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert float(got.abs().max()) > 0


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
