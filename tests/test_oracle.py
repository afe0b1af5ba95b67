"""The CPU oracle against independent statements of the same math (no GPU needed)."""
import json
import os

import numpy as np
import pytest
import torch

from tests.helpers import ROOT, orc
from slora_b200.workloads import build_workload, make_tables

GOLDEN = os.path.join(ROOT, "tests", "golden")


def _hf_adapters(ranks, H, seed):
    rng = np.random.default_rng(seed)
    out = []
    for r in ranks:
        A = [rng.standard_normal((r, H)).astype(np.float32) / np.sqrt(H) for _ in range(4)]
        B = [rng.standard_normal((H, r)).astype(np.float32) * 0.02 for _ in range(4)]
        out.append((A, B))
    return out


def _pool_from_hf(adapters, ranks, pool_rows, H, permute, seed=7):
    a_start, a_len, a_loc = make_tables(ranks, pool_rows, seed, permute)
    pool_a = np.zeros((pool_rows, H), dtype=np.float32)
    pool_b = np.zeros((pool_rows, H), dtype=np.float32)
    for i, (A, B) in enumerate(adapters):
        rows_a, rows_b = orc.pool_rows_from_hf(A, B)
        loc = a_loc[a_start[i]: a_start[i] + a_len[i]].numpy()
        pool_a[loc] = rows_a
        pool_b[loc] = rows_b
    return a_start, a_len, a_loc, pool_a, pool_b


@pytest.mark.parametrize("permute", [False, True])
def test_oracle_equals_hf_formula(permute):
    """Pool rows laid out as the loader does (lora_layer_weight.py:215-224) reproduce (x A^T) B^T alpha/r."""
    H, ranks = 256, [8, 16, 32, 8]
    adapters = _hf_adapters(ranks, H, 1)
    a_start, a_len, a_loc, pool_a, pool_b = _pool_from_hf(adapters, ranks, 512, H, permute)
    rng = np.random.default_rng(2)
    T = 24
    x = rng.standard_normal((T, H)).astype(np.float32)
    ids = rng.integers(0, len(ranks), T)
    scales = np.array([16.0 / r for r in ranks], dtype=np.float32)
    for p in range(4):
        got = orc.lora_delta_ref(np.zeros((T, H), np.float32), x, pool_a, pool_b, a_start, a_len, a_loc, ids, p, scales)
        want = np.stack([(x[t] @ adapters[ids[t]][0][p].T) @ adapters[ids[t]][1][p].T * scales[ids[t]]
                         for t in range(T)])
        np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-6)


def test_reference_script_structure():
    """Same set-up as the reference's multi-rank kernel script (H=1024, ranks [8,16], identity a_loc, scale 1,
    qkvo=0, tokens split half/half between the two adapters), its torch loop written out on CPU tensors."""
    torch.manual_seed(42)
    H, R, N = 1024, [8, 16], 128
    key_buffer = torch.cat([torch.randn((R[0] * 4, 32, H // 32)), torch.randn((R[1] * 4, 32, H // 32))])
    a_len = torch.tensor([R[0] * 4, R[1] * 4])
    a_start = torch.zeros_like(a_len)
    a_start[1:] = torch.cumsum(a_len[:-1], 0)
    a_loc = torch.arange((R[0] + R[1]) * 4)
    bins = torch.cat([torch.full((N // 2,), i) for i in range(2)])
    scale = torch.ones(2)
    for part in ("A", "B"):
        x = torch.randn((N, H if part == "A" else max(R)))
        rows = []
        for i in range(N):
            a = int(bins[i])
            w = key_buffer[a_start[a]: a_start[a] + R[a]].reshape(-1)
            w = w.reshape(R[a], H).T if part == "A" else w.reshape(H, R[a]).T
            rows.append(torch.nn.functional.pad(x[i:i + 1, :w.shape[0]] @ w, (0, (max(R) if part == "A" else H) - w.shape[1])))
        want = torch.cat(rows).numpy()
        if part == "A":
            got = orc.lora_shrink_ref(x, key_buffer, a_start, a_len, a_loc, bins, 0, out_width=max(R))
        else:
            got = orc.lora_expand_ref(np.zeros((N, H), np.float32), x, key_buffer, a_start, a_len, a_loc, bins, 0, scale)
        np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4)


def test_grouped_equals_per_token():
    wl = build_workload(3, pool_rows=8192, n_adapters=40, decode_tokens=30, prefill=("seqs", 3, 4, 20), hidden=512)
    for p in range(4):
        x = wl.x_o[0] if p == 3 else wl.x_qkv[0]
        y0 = np.zeros((wl.T, 512), np.float32)
        a = orc.lora_delta_ref(y0, x, wl.pools_a[0], wl.pools_b[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p, wl.a_scaling)
        b = orc.lora_delta_grouped(y0, x, wl.pools_a[0], wl.pools_b[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p, wl.a_scaling)
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)


def test_flat_slot_layout_with_other_strides():
    """B of width h_out < pool stride (GQA k/v) and rank_mult > 1 (tensor-parallel shard) read the slot's flat space."""
    S, r, h_out = 256, 8, 64
    rng = np.random.default_rng(3)
    pool = rng.standard_normal((64, S)).astype(np.float32)
    a_start, a_len, a_loc = make_tables([r], 64, 5, True)
    B = orc.adapter_matrix_B(pool, a_start, a_len, a_loc, 0, 2, h_out)
    flat = pool[a_loc[2 * r: 3 * r].numpy()].reshape(-1)[: h_out * r]
    np.testing.assert_array_equal(B, flat.reshape(h_out, r))
    B2 = orc.adapter_matrix_B(pool, a_start, a_len, a_loc, 0, 1, 32, rank_mult=4)
    flat2 = pool[a_loc[r: 2 * r].numpy()].reshape(-1)[: 32 * 32]
    np.testing.assert_array_equal(B2, flat2.reshape(32, 32))


def test_segments_to_token_ids():
    ids = orc.segments_to_token_ids([0, 5, 9], [5, 3, 1], [2, 0, 1], 11)
    assert ids.tolist() == [2] * 5 + [0] * 3 + [-1] + [1] + [-1]


def test_rounding_variant_is_within_the_parity_bar():
    wl = build_workload(1)
    for p in range(4):
        x = wl.x_o[0] if p == 3 else wl.x_qkv[0]
        y0 = np.zeros((wl.T, 4096), np.float32)
        args = (y0, x, wl.pools_a[0], wl.pools_b[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p, wl.a_scaling)
        max_rel, mean_rel = orc.error_metrics(orc.lora_delta_ref_rounding(*args), orc.lora_delta_ref(*args))
        assert max_rel < 2e-3 and mean_rel < 6e-4


def test_golden_config1():
    """Committed known-answer vectors for configuration 1 (made by tests/golden/make_golden.py)."""
    path = os.path.join(GOLDEN, "cfg1_oracle.npz")
    meta = json.load(open(os.path.join(GOLDEN, "cfg1_oracle.json")))
    g = np.load(path)
    wl = build_workload(1)
    assert wl.ids.tolist() == meta["ids"]
    assert wl.a_loc.tolist() == meta["a_loc"]
    for p in range(4):
        x = wl.x_o[0] if p == 3 else wl.x_qkv[0]
        got = orc.lora_delta_ref(np.zeros((wl.T, 4096), np.float32), x, wl.pools_a[0], wl.pools_b[0], wl.a_start,
                                 wl.a_len, wl.a_loc, wl.ids, p, wl.a_scaling)
        sel = np.asarray(meta["columns"])
        np.testing.assert_allclose(got[:, sel], g[f"delta_p{p}"], rtol=2e-5, atol=1e-7)
        np.testing.assert_allclose(np.abs(got).sum(axis=1), g[f"rowabs_p{p}"], rtol=2e-5)


def _ref_cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_ref_golden", os.path.join(GOLDEN, "make_ref_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.CASES, mod.cols_of


@pytest.mark.parametrize("case", ["cfg1", "mixed", "wide5120"])
def test_oracle_against_outputs_of_the_reference_kernels(case):
    """tests/golden/ref_kernels.npz holds what the reference's own BGMV CUDA kernels (compiled from the reference tree,
    run on a B200) produced on these seeded inputs; the oracle must agree within fp16 rounding of the stored values."""
    cases, cols_of = _ref_cases()
    g = np.load(os.path.join(GOLDEN, "ref_kernels.npz"))
    wl = build_workload(**cases[case])
    H = wl.spec.hidden
    cols = cols_of(H)
    for p in range(4):
        x = wl.x_o[0] if p == 3 else wl.x_qkv[0]
        d = orc.lora_shrink_ref(x, wl.pools_a[0], wl.a_start, wl.a_len, wl.a_loc, wl.ids, p, out_width=wl.max_rank)
        ref_d = g[f"{case}_delta_p{p}"].astype(np.float32)
        assert np.abs(d - ref_d).max() <= 1.5e-3 * np.abs(ref_d).max()          # one fp16 rounding of the result
        y = orc.lora_delta_ref(np.zeros((wl.T, H), np.float32), x, wl.pools_a[0], wl.pools_b[0], wl.a_start, wl.a_len,
                               wl.a_loc, wl.ids, p, wl.a_scaling)
        ref_y = g[f"{case}_y_p{p}"].astype(np.float32)
        max_rel, mean_rel = orc.error_metrics(y[:, cols], ref_y)
        assert max_rel <= 3e-3 and mean_rel <= 1e-3, (p, max_rel, mean_rel)
        np.testing.assert_allclose(np.abs(y).sum(axis=1), g[f"{case}_rowabs_p{p}"], rtol=3e-3)
        # untouched columns of the intermediate stay zero in the reference too
        for t in range(wl.T):
            assert not ref_d[t, wl.ranks[int(wl.ids[t])]:].any()
