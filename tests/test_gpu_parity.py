"""Parity of the CUDA path (through the C ABI) with the CPU oracle on identical seeded inputs.  Needs a B200."""
import numpy as np
import pytest
import torch

import slora_b200 as sl
from slora_b200 import batch_infer
from slora_b200.workloads import build_workload, make_tables
from tests.helpers import assert_parity, oracle_layer, orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dispatch_layer(w, layer=0, y_init=None):
    """q,k,v,o deltas with eight dispatch_bgmv calls, the reference's call pattern
    (lora_unordered_batch_infer.py:254-318,428-448)."""
    outs, deltas = [], []
    R = w.max_rank
    for p, (h_in, h_out) in enumerate(w.proj_dims()):
        x = w.x_o[layer] if p == 3 else w.x_qkv[layer]
        delta = torch.zeros((w.T, R), dtype=w.dtype, device=DEV)
        y = torch.zeros((w.T, h_out), dtype=w.dtype, device=DEV) if y_init is None else y_init[p].clone()
        ka = w.pools_a[layer].view(w.pools_a[layer].shape[0], 1, -1)
        vb = w.pools_b[layer].view(w.pools_b[layer].shape[0], 1, -1)
        sl.dispatch_bgmv(delta, x, ka, w.a_start, w.a_len, w.a_loc, w.ids, p, w.a_scaling)
        sl.dispatch_bgmv(y, delta, vb, w.a_start, w.a_len, w.a_loc, w.ids, p, w.a_scaling)
        outs.append(y)
        deltas.append(delta)
    torch.cuda.synchronize()
    return outs, deltas


def _fused_layer(w, layer=0, use_plan=True, use_pdl=True, max_rank=None, **prepare_kw):
    ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, max_rank or w.max_rank,
                          use_pdl)
    ops.prepare(w.ids, use_plan=use_plan, **prepare_kw)
    H, K = w.spec.hidden, w.spec.h_kv
    q = torch.zeros((w.T, H), dtype=w.dtype, device=DEV)
    k = torch.zeros((w.T, K), dtype=w.dtype, device=DEV)
    v = torch.zeros((w.T, K), dtype=w.dtype, device=DEV)
    o = torch.zeros((w.T, H), dtype=w.dtype, device=DEV)
    ops.lora_get_qkv(layer, w.x_qkv[layer], q, k, v)
    ops.lora_get_o(layer, w.x_o[layer], o)
    torch.cuda.synchronize()
    if ops.plan is not None:
        ops.plan.check()
    return [q, k, v, o]


def test_config1_dispatch_bgmv():
    wl = build_workload(1)
    ref = oracle_layer(wl)
    outs, deltas = _dispatch_layer(wl.to(DEV))
    for p in range(4):
        assert_parity(outs[p], ref[p], what=f"cfg1 proj {p}")
        x = wl.x_o[0] if p == 3 else wl.x_qkv[0]
        dref = orc.lora_shrink_ref(x, wl.pools_a[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p)
        assert_parity(deltas[p], dref, what=f"cfg1 shrink {p}")


def test_config1_against_committed_golden_vectors():
    import json, os
    from tests.helpers import ROOT
    g = np.load(os.path.join(ROOT, "tests", "golden", "cfg1_oracle.npz"))
    cols = json.load(open(os.path.join(ROOT, "tests", "golden", "cfg1_oracle.json")))["columns"]
    outs = _fused_layer(build_workload(1).to(DEV))
    for p in range(4):
        assert_parity(outs[p][:, cols], g[f"delta_p{p}"], what=f"golden proj {p}")


@pytest.mark.parametrize("rank", [8, 16, 32, 64, 128])
@pytest.mark.parametrize("hidden", [1024, 5120])
def test_uniform_rank_dispatch(rank, hidden):
    wl = build_workload(2, pool_rows=4096, n_adapters=6, decode_tokens=37, hidden=hidden, rank_choices=(rank,))
    ref = oracle_layer(wl)
    outs, _ = _dispatch_layer(wl.to(DEV))
    for p in range(4):
        assert_parity(outs[p], ref[p], what=f"r={rank} H={hidden} proj {p}")


@pytest.mark.parametrize("use_plan,use_pdl", [(True, True), (True, False), (False, True)])
def test_mixed_ranks_fused(use_plan, use_pdl):
    wl = build_workload(3, pool_rows=8192, n_adapters=40, decode_tokens=60, prefill=("seqs", 3, 5, 40), hidden=2048)
    ref = oracle_layer(wl)
    outs = _fused_layer(wl.to(DEV), use_plan=use_plan, use_pdl=use_pdl)
    for p in range(4):
        assert_parity(outs[p], ref[p], what=f"mixed proj {p}")


@pytest.mark.parametrize("case", ["mixed", "narrow", "many_tiles", "bf16_gqa"])
def test_exact_item_count_gives_the_same_bits_as_the_padded_enumeration(case):
    """SLORA_FLAG_EXACT_ITEMS only changes which CTA computes which item: outputs are bit-identical with and without
    it, for mixed ranks (running count per tile), one rank below the delta width (closed form), more tiles than the
    running count holds (falls back to the padded enumeration) and k/v narrower than q."""
    kw, dt = dict(hidden=2048), torch.float16
    if case == "mixed":
        wl = build_workload(3, pool_rows=16384, n_adapters=60, decode_tokens=150, prefill=("seqs", 3, 5, 40), **kw)
    elif case == "narrow":
        wl = build_workload(3, pool_rows=8192, n_adapters=30, decode_tokens=140, prefill=None, rank_choices=(16,), **kw)
    elif case == "many_tiles":
        wl = build_workload(3, pool_rows=163840, n_adapters=3000, decode_tokens=3000, prefill=None, hidden=1024,
                            rank_choices=(8, 16))
    else:
        dt = torch.bfloat16
        wl = build_workload(5, dtype=dt, pool_rows=8192, n_adapters=40, decode_tokens=200, hidden=2048, h_kv=512,
                            rank_choices=(8, 32, 64))
    w = wl.to(DEV)
    if case == "many_tiles":
        assert sl.BatchPlan(w.ids, w.a_start, w.a_len, w.a_loc.numel()).info()[0] > 640
    width = 64 if case == "narrow" else None
    plain = _fused_layer(w, mixed_ranks=False, max_rank=width)
    exact = _fused_layer(w, mixed_ranks=True, max_rank=width)
    asked = _fused_layer(w, max_rank=width)          # prepare() reads the plan and decides
    ref = oracle_layer(wl)
    for p in range(4):
        assert torch.equal(plain[p], exact[p]) and torch.equal(plain[p], asked[p]), f"{case} proj {p}"
        assert_parity(exact[p], ref[p], dt, what=f"exact items {case} proj {p}")


def test_plan_info_reports_the_shared_rank():
    wl = build_workload(3, pool_rows=8192, n_adapters=30, decode_tokens=140, prefill=None, hidden=1024,
                        rank_choices=(16,)).to(DEV)
    plan = sl.BatchPlan(wl.ids, wl.a_start, wl.a_len, wl.a_loc.numel())
    tiles, big, uniform = plan.info()
    assert tiles >= len(set(wl.ids.tolist())) and big == 0 and uniform == 16
    wl = build_workload(3, pool_rows=8192, n_adapters=30, decode_tokens=140, prefill=None, hidden=1024).to(DEV)
    assert sl.BatchPlan(wl.ids, wl.a_start, wl.a_len, wl.a_loc.numel()).info()[2] == 0
    ops = sl.LoraBatchOps(wl.a_start, wl.a_len, wl.a_loc, wl.a_scaling, wl.pools_a, wl.pools_b, wl.max_rank)
    assert ops.prepare(wl.ids).flags & 4 and not ops.prepare(wl.ids[:100]).flags & 4    # small batches are not asked


def test_config2_shape_small_pool():
    """S1-shaped decode batch (1000 rank-8 adapters, 256 Zipf tokens, hidden 4096) over a 65536-row pool."""
    wl = build_workload(2, pool_rows=65536)
    ref = oracle_layer(wl)
    w = wl.to(DEV)
    outs = _fused_layer(w)
    for p in range(4):
        assert_parity(outs[p], ref[p], what=f"cfg2 proj {p}")
    outs2, _ = _dispatch_layer(w)
    for p in range(4):
        # planned and per-token paths do the same arithmetic per token: bit-identical results
        assert torch.equal(outs[p], outs2[p])


def test_bf16():
    wl = build_workload(3, dtype=torch.bfloat16, pool_rows=8192, n_adapters=30, decode_tokens=50,
                        prefill=("seqs", 2, 5, 30), hidden=1024)
    ref = oracle_layer(wl)
    outs = _fused_layer(wl.to(DEV))
    for p in range(4):
        assert_parity(outs[p], ref[p], dtype=torch.bfloat16, what=f"bf16 proj {p}")


def test_expand_accumulates_into_y_and_leaves_other_columns():
    wl = build_workload(2, pool_rows=4096, n_adapters=8, decode_tokens=20, hidden=1024, rank_choices=(8, 16))
    w = wl.to(DEV)
    g = torch.Generator().manual_seed(5)
    y0 = [torch.randn((wl.T, ho), generator=g).to(wl.dtype) for _, ho in wl.proj_dims()]
    outs, _ = _dispatch_layer(w, y_init=[y.to(DEV) for y in y0])
    ref = oracle_layer(wl)
    for p in range(4):
        got_delta = outs[p].float().cpu() - y0[p].float()
        # the sum is rounded to fp16 at |y| ~ 1, i.e. absolute error up to 2^-11 per element
        assert (got_delta - torch.from_numpy(ref[p])).abs().max() < 2e-3
    # shrink writes only columns < r of each token's row
    sentinel = torch.full((wl.T, wl.max_rank), 7.0, dtype=wl.dtype, device=DEV)
    ka = w.pools_a[0].view(-1, 1, 1024)
    sl.dispatch_bgmv(sentinel, w.x_qkv[0], ka, w.a_start, w.a_len, w.a_loc, w.ids, 0, w.a_scaling)
    torch.cuda.synchronize()
    for t in range(wl.T):
        r = wl.ranks[int(wl.ids[t])]
        assert (sentinel[t, r:] == 7.0).all()
        assert not (sentinel[t, :r] == 7.0).all()


def test_segment_entry_points():
    """lora_get_qkvo_fwd_shrink / expand (the reference's Triton prefill API) over request segments."""
    wl = build_workload(3, pool_rows=8192, n_adapters=20, decode_tokens=0, prefill=("seqs", 5, 3, 70), hidden=1024)
    w = wl.to(DEV)
    seg = wl.segments
    b_start = torch.tensor([s for s, _, _ in seg], dtype=torch.int32, device=DEV)
    b_len = torch.tensor([n for _, n, _ in seg], dtype=torch.int32, device=DEV)
    req_bins = torch.tensor([a for _, _, a in seg], dtype=torch.int64, device=DEV)
    max_len = max(n for _, n, _ in seg)
    ref = oracle_layer(wl)
    for p in range(4):
        x = w.x_o[0] if p == 3 else w.x_qkv[0]
        delta = torch.zeros((wl.T, wl.max_rank), dtype=wl.dtype, device=DEV)
        y = torch.zeros((wl.T, 1024), dtype=wl.dtype, device=DEV)
        sl.lora_get_qkvo_fwd_shrink(x, w.pools_a[0], delta, w.a_loc, w.a_start, w.a_len, b_start, b_len, req_bins,
                                    1024, p, wl.max_rank, max_len)
        sl.lora_get_qkvo_fwd_expand(delta, w.pools_b[0], y, w.a_scaling, w.a_loc, w.a_start, w.a_len, b_start, b_len,
                                    req_bins, 1024, p, wl.max_rank, max_len)
        torch.cuda.synchronize()
        assert_parity(y, ref[p], what=f"segments proj {p}")


def test_gqa_narrow_kv_over_wide_pool_rows():
    """k/v output width 256 with pool rows of 1024 elements (the GQA case the reference cannot express)."""
    wl = build_workload(5, pool_rows=4096, n_adapters=5, decode_tokens=40, hidden=1024, h_kv=256, rank_choices=(16, 64))
    ref = oracle_layer(wl)
    outs = _fused_layer(wl.to(DEV))
    for p in range(4):
        assert outs[p].shape[1] == (256 if p in (1, 2) else 1024)
        assert_parity(outs[p], ref[p], what=f"gqa proj {p}")


def test_expand_reads_all_gathered_delta_parts():
    """Expand with the delta laid out as the all-gather of an N-way rank-sharded shrink: [N, T, r/N]."""
    wl = build_workload(2, pool_rows=4096, n_adapters=6, decode_tokens=30, hidden=1024, rank_choices=(16, 32))
    w = wl.to(DEV)
    N, R = 4, wl.max_rank
    p = 0
    dref = orc.lora_shrink_ref(wl.x_qkv[0], wl.pools_a[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p)
    parts = torch.zeros((N, wl.T, R // N), dtype=wl.dtype)
    for t in range(wl.T):
        r = wl.ranks[int(wl.ids[t])]
        rs = r // N
        for g in range(N):
            parts[g, t, :rs] = torch.from_numpy(dref[t, g * rs:(g + 1) * rs]).to(wl.dtype)
    parts = parts.to(DEV)
    y = torch.zeros((wl.T, 1024), dtype=wl.dtype, device=DEV)
    plan = batch_infer.BatchPlan(w.ids, w.a_start, w.a_len, w.a_loc.numel())
    batch_infer.expand_multi(plan, w.ids, [p], [y], [parts], w.pools_b[0], w.a_start, w.a_len, w.a_loc, w.a_scaling,
                             delta_stride=R // N, delta_width=R // N, delta_parts=N, delta_part_stride=wl.T * (R // N))
    torch.cuda.synchronize()
    plan.check()
    assert_parity(y, oracle_layer(wl)[p], what="gathered delta")


def test_empty_batch_and_bad_ids():
    wl = build_workload(2, pool_rows=4096, n_adapters=6, decode_tokens=16, hidden=1024)
    w = wl.to(DEV)
    # empty batch: every entry point returns without launching
    e_ids = torch.empty(0, dtype=torch.int64, device=DEV)
    e_x = torch.empty((0, 1024), dtype=wl.dtype, device=DEV)
    e_d = torch.empty((0, 8), dtype=wl.dtype, device=DEV)
    sl.dispatch_bgmv(e_d, e_x, w.pools_a[0].view(-1, 1, 1024), w.a_start, w.a_len, w.a_loc, e_ids, 0, w.a_scaling)
    # a token with an adapter id outside the tables is skipped and reported, the others are computed
    ids = w.ids.clone()
    ids[3] = 99
    ids[7] = -1
    ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, wl.max_rank)
    ops.prepare(ids)
    o = torch.zeros((wl.T, 1024), dtype=wl.dtype, device=DEV)
    ops.lora_get_o(0, w.x_o[0], o)
    torch.cuda.synchronize()
    st, n_tiles = ops.plan.status()
    assert st & 1 and n_tiles > 0
    with pytest.raises(RuntimeError):
        ops.plan.check()
    ref = oracle_layer(wl)[3]
    keep = [t for t in range(wl.T) if t not in (3, 7)]
    assert_parity(o[keep], ref[keep], what="valid tokens")
    assert (o[3] == 0).all() and (o[7] == 0).all()
    assert sl.validate_tables(w.a_start, w.a_len, w.a_loc, ids, 4096)[0] == 2
    assert sl.validate_tables(w.a_start, w.a_len, w.a_loc, w.ids, 4096) == (0, 0, 0)
    bad_loc = w.a_loc.clone()
    bad_loc[5] = 4096
    n_bad, kind, index = sl.validate_tables(w.a_start, w.a_len, bad_loc, w.ids, 4096)
    assert (n_bad, kind, index) == (1, 3, 5)


def test_out_of_range_pool_row_is_skipped_not_read():
    wl = build_workload(2, pool_rows=4096, n_adapters=4, decode_tokens=12, hidden=1024)
    w = wl.to(DEV)
    bad_loc = w.a_loc.clone()
    a = int(wl.ids[0])
    bad_loc[int(wl.a_start[a])] = 1 << 40  # first q row of that adapter
    ops = sl.LoraBatchOps(w.a_start, w.a_len, bad_loc, w.a_scaling, w.pools_a, w.pools_b, wl.max_rank)
    ops.prepare(w.ids)
    o = torch.zeros((wl.T, 1024), dtype=wl.dtype, device=DEV)
    q = torch.zeros((wl.T, 1024), dtype=wl.dtype, device=DEV)
    k, v = torch.zeros_like(q), torch.zeros_like(q)
    ops.lora_get_qkv(0, w.x_qkv[0], q, k, v)
    torch.cuda.synchronize()
    assert ops.plan.status()[0] & 2
    ref = oracle_layer(wl)
    other = [t for t in range(wl.T) if int(wl.ids[t]) != a]
    assert_parity(k[other], ref[1][other], what="unaffected tokens")


def test_unsupported_inputs_raise():
    wl = build_workload(2, pool_rows=4096, n_adapters=4, decode_tokens=8, hidden=1024)
    w = wl.to(DEV)
    ka = w.pools_a[0].view(-1, 1, 1024)
    d = torch.zeros((wl.T, 8), dtype=wl.dtype, device=DEV)
    with pytest.raises(RuntimeError, match="No suitable kernel"):
        sl.dispatch_bgmv(d.float(), w.x_qkv[0].float(), ka.float(), w.a_start, w.a_len, w.a_loc, w.ids, 0,
                         w.a_scaling.float())
    with pytest.raises(RuntimeError, match="contiguous"):
        sl.dispatch_bgmv(d, w.x_qkv[0][:, ::2], ka, w.a_start, w.a_len, w.a_loc, w.ids, 0, w.a_scaling)
    with pytest.raises(RuntimeError, match="CUDA"):
        sl.dispatch_bgmv(d.cpu(), w.x_qkv[0], ka, w.a_start, w.a_len, w.a_loc, w.ids, 0, w.a_scaling)
    with pytest.raises(RuntimeError):
        sl.dispatch_bgmv(d, w.x_qkv[0], ka, w.a_start, w.a_len, w.a_loc, w.ids, 4, w.a_scaling)
    x_odd = torch.zeros((wl.T, 1020), dtype=wl.dtype, device=DEV)
    with pytest.raises(RuntimeError, match="No suitable kernel"):
        sl.dispatch_bgmv(d, x_odd, ka, w.a_start, w.a_len, w.a_loc, w.ids, 0, w.a_scaling)


@pytest.mark.parametrize("exact_items", [False, True])
def test_adapter_wider_than_the_delta_buffers_is_refused_not_overread(exact_items):
    """Delta buffers of 16 columns, one adapter of rank 64 in the batch: its tokens are skipped by the expand and the
    status word says so; nothing is read past a delta row; the other tokens are right (with the padded and with the
    exact enumeration of work items)."""
    wl = build_workload(3, pool_rows=4096, n_adapters=6, decode_tokens=40, prefill=None, hidden=1024,
                        rank_choices=(16, 64))
    assert 64 in [wl.ranks[int(a)] for a in wl.ids] and 16 in [wl.ranks[int(a)] for a in wl.ids]
    w = wl.to(DEV)
    ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, 16)
    ops.prepare(w.ids, mixed_ranks=exact_items)
    assert bool(ops.flags & 4) == exact_items
    q, k, v = (torch.zeros((wl.T, 1024), dtype=wl.dtype, device=DEV) for _ in range(3))
    ops.lora_get_qkv(0, w.x_qkv[0], q, k, v)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="unsupported rank"):
        ops.plan.check()
    ref = oracle_layer(wl)
    narrow = torch.tensor([wl.ranks[int(a)] == 16 for a in wl.ids])
    assert float(q[~narrow.to(DEV)].abs().max()) == 0.0
    assert_parity(q[narrow.to(DEV)], ref[0][narrow.numpy()], what="rank-16 tokens beside a refused adapter")


@pytest.mark.parametrize("T", [24, 200])
def test_tensor_parallel_shards_on_one_gpu(T):
    """The per-rank shard layout of slora_b200.tp through the real kernels: the N ranks are run one after the other on
    one GPU, their intermediates concatenated the way the all-gather would, and the output slices compared with the
    single-rank formula.  (200 tokens: the backend turns on the exact work-item count for the mixed ranks.)"""
    from slora_b200 import tp
    H, N = 1024, 4
    ranks = [8, 16, 32, 8]
    g = torch.Generator().manual_seed(21)
    ads = [([torch.randn((r, H), generator=g) / 32 for _ in range(4)],
            [torch.randn((H, r), generator=g) * 0.02 for _ in range(4)]) for r in ranks]
    x = torch.randn((T, H), generator=g).to(torch.float16)
    ids = torch.randint(0, len(ranks), (T,), generator=g)
    R, Rl = max(ranks), max(ranks) // N
    shards = []
    for rank in range(N):
        a_start, a_len, a_loc = make_tables([r // N for r in ranks], 512, 300 + rank, True)
        pa = torch.zeros((512, H), dtype=torch.float16)
        pb = torch.zeros((512, H), dtype=torch.float16)
        for i, (A, B) in enumerate(ads):
            ra, rb = tp.shard_adapter(A, B, rank, N, H)
            loc = a_loc[a_start[i]: a_start[i] + a_len[i]]
            pa[loc] = ra.to(torch.float16)
            pb[loc] = rb.to(torch.float16)
        t = tp.TpTables(a_start.to(DEV), a_len.to(DEV), a_loc.to(DEV),
                        torch.tensor([16.0 / r for r in ranks], dtype=torch.float16, device=DEV))
        shards.append((t, pa.to(DEV), pb.to(DEV)))
    be = tp.CudaBackend()
    xd, idd = x.to(DEV), ids.to(DEV)
    for p in range(4):
        gathered = torch.zeros((N, 1, T, Rl), dtype=torch.float16, device=DEV)
        for rank, (t, pa, pb) in enumerate(shards):
            plan = be.make_plan(idd, t)
            assert bool(be.flags & 4) == (T >= 128)
            be.shrink(plan, idd, [p], [gathered[rank, 0]], xd, pa, t)
        slices = []
        for rank, (t, pa, pb) in enumerate(shards):
            y = torch.zeros((T, H // N), dtype=torch.float16, device=DEV)
            plan = be.make_plan(idd, t)
            be.expand(plan, idd, [p], [y], [gathered[0, 0]], pb, t, delta_stride=Rl, delta_width=Rl, delta_parts=N,
                      delta_part_stride=T * Rl, rank_mult=N)
            slices.append(y)
        torch.cuda.synchronize()
        got = torch.cat(slices, dim=1)
        want = torch.stack([(x[i].float() @ ads[int(ids[i])][0][p].half().float().T)
                            @ ads[int(ids[i])][1][p].half().float().T * (16.0 / ranks[int(ids[i])]) for i in range(T)])
        assert_parity(got, want.numpy(), what=f"tp proj {p}")


@pytest.mark.parametrize("case", ["cfg1", "mixed", "wide5120"])
def test_against_outputs_of_the_reference_kernels(case):
    """This library against tests/golden/ref_kernels.npz (outputs of the reference's own CUDA kernels on a B200)."""
    import importlib.util, os
    from tests.helpers import ROOT
    gdir = os.path.join(ROOT, "tests", "golden")
    spec = importlib.util.spec_from_file_location("make_ref_golden", os.path.join(gdir, "make_ref_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    g = np.load(os.path.join(gdir, "ref_kernels.npz"))
    wl = build_workload(**mod.CASES[case])
    outs, deltas = _dispatch_layer(wl.to(DEV))
    for p in range(4):
        ref_d = torch.from_numpy(g[f"{case}_delta_p{p}"].astype(np.float32))
        assert (deltas[p].float().cpu() - ref_d).abs().max() <= 2e-3 * ref_d.abs().max()
        assert_parity(outs[p][:, mod.cols_of(wl.spec.hidden)], g[f"{case}_y_p{p}"].astype(np.float32), what=f"ref kernels {case} p{p}")



@pytest.mark.parametrize("case", ["same_rank", "mixed_ranks", "cap_below_some_ranks", "flag_without_tiles", "bf16_gqa"])
def test_resolved_tiles_give_the_same_bits_as_the_table_chase(case):
    """A plan built with the loc table (slora_plan_build_ex) holds every tile's token ids, scale and pool rows where a
    launch fetches them in one round trip; the kernels fall back to perm and the tables per tile (rank above the
    plan's cap) or altogether (the flag says resolved tiles, the plan has none).  Same bits every way."""
    from slora_b200 import _lib
    dt = torch.float16
    if case == "same_rank":
        wl = build_workload(2, pool_rows=16384, n_adapters=300)
    elif case == "bf16_gqa":
        dt = torch.bfloat16
        wl = build_workload(5, dtype=dt, pool_rows=8192, n_adapters=40, decode_tokens=200, hidden=4096, h_kv=1024,
                            rank_choices=(8, 32, 64))
    else:
        wl = build_workload(3, pool_rows=16384, n_adapters=60, decode_tokens=150, prefill=("seqs", 3, 5, 40), hidden=4096)
    w = wl.to(DEV)
    R = w.max_rank
    mask = 0x1f << 8

    def run(plan_kw, flag_rank, exact):
        ops = sl.LoraBatchOps(w.a_start, w.a_len, w.a_loc, w.a_scaling, w.pools_a, w.pools_b, R)
        ops.prepare(w.ids, mixed_ranks=exact, big_groups=False)
        ops.plan = sl.BatchPlan(w.ids, w.a_start, w.a_len, w.a_loc.numel(), **plan_kw)
        ops.flags = (ops.flags & ~mask) | _lib.flag_resolved(flag_rank)
        H, K = w.spec.hidden, w.spec.h_kv
        out = [torch.zeros((w.T, n), dtype=dt, device=DEV) for n in (H, K, K, H)]
        ops.lora_get_qkv(0, w.x_qkv[0], out[0], out[1], out[2])
        ops.lora_get_o(0, w.x_o[0], out[3])
        torch.cuda.synchronize()
        ops.plan.check()
        return out, ops.plan.header()

    tables = dict(a_loc=w.a_loc, a_scaling=w.a_scaling)
    for exact in (False, True):
        chase, _ = run({}, 0, exact)
        if case == "cap_below_some_ranks":
            got, hdr = run(dict(max_rank=16, **tables), 16, exact)
            assert hdr["resolved_cap"] == 16 and max(wl.ranks) > 16
        elif case == "flag_without_tiles":
            n = _lib.lib.slora_plan_workspace_bytes_ex(w.T, w.a_start.numel(), R)
            ws = torch.empty(n // 4 + 1, dtype=torch.int32, device=DEV)
            got, hdr = run(dict(workspace=ws), R, exact)
            assert hdr["resolved_cap"] == 0
        else:
            got, hdr = run(dict(max_rank=R, **tables), R, exact)
            assert hdr["resolved_cap"] == R
        for p in range(4):
            assert torch.equal(chase[p], got[p]), f"{case} exact={exact} proj {p}"
    ref = oracle_layer(wl)
    for p in range(4):
        assert_parity(got[p], ref[p], dt, what=f"resolved tiles {case} proj {p}")
