"""Host-side mirror of the reference interface: pool allocator, adapter tables, workload builders (CPU only)."""
import numpy as np
import pytest
import torch

from slora_b200.infer_adapter import InferAdapter
from slora_b200.mem_allocator import MemoryAllocator
from slora_b200.workloads import SPECS, build_workload, zipf_probs
from tests.helpers import orc


def _mm(tot=64, layers=2, heads=4, hd=8):
    return MemoryAllocator(tot, 0, torch.float16, heads, hd, layers, device="cpu")


def test_alloc_returns_first_free_rows_and_free_returns_them():
    mm = _mm()
    a = mm.alloc(5)
    assert a.tolist() == [0, 1, 2, 3, 4] and mm.can_use_mem_size == 59
    b = mm.alloc(3)
    assert b.tolist() == [5, 6, 7]
    mm.free(a[1:4])
    c = mm.alloc(4)
    assert c.tolist() == [1, 2, 3, 8]
    assert mm.can_use_mem_size == 64 - 5 - 3 + 3 - 4
    with pytest.raises(Exception, match="no enough pool space"):
        mm.alloc(1000)
    mm.free_all()
    assert mm.can_use_mem_size == 64 and bool(mm.mem_state.all())


def test_alloc_contiguous_finds_first_run():
    mm = _mm(tot=32)
    mm.alloc(10)
    mm.free(torch.tensor([2, 3, 4]))
    idx, s, e = mm.alloc_contiguous(3)
    assert (s, e) == (2, 5) and idx.tolist() == [2, 3, 4]
    idx, s, e = mm.alloc_contiguous(6)
    assert (s, e) == (10, 16)
    mm.free(torch.tensor([0]))
    assert mm.alloc_contiguous(17) is None
    assert len(mm.key_buffer) == 2 and mm.key_buffer[0].shape == (32, 4, 8)
    assert mm.get_memory_size() == 2 * 2 * 32 * 32 * 2


class _Layer:
    def __init__(self, w):
        self.w_combined = w


class _Adapter:
    """Stand-in for LoraTpPartAdapter (slora/models/peft/lora_adapter.py:20-65) with HF-shaped weights."""

    def __init__(self, name, r, H, heads, layers, seed):
        rng = np.random.default_rng(seed)
        self.lora_dir, self.r, self.scaling = name, r, 16.0 / r
        self.A = [[rng.standard_normal((r, H)).astype(np.float32) / 8 for _ in range(4)] for _ in range(layers)]
        self.B = [[rng.standard_normal((H, r)).astype(np.float32) / 8 for _ in range(4)] for _ in range(layers)]
        self.layers = []
        for l in range(layers):
            ra, rb = orc.pool_rows_from_hf(self.A[l], self.B[l])
            w = torch.from_numpy(np.stack([ra, rb])).to(torch.float16).reshape(2, 4 * r, heads, H // heads)
            self.layers.append(_Layer(w))


def test_infer_adapter_load_offload_tables_and_pool_content():
    H, heads, L = 32, 4, 2
    mm = _mm(tot=300, layers=L, heads=heads, hd=H // heads)
    ia = InferAdapter.init(mm, None)
    ads = [_Adapter(f"a{i}", r, H, heads, L, i) for i, r in enumerate([8, 16, 8, 32])]
    mm.alloc(3)  # someone else's rows (KV cache) sit at the front of the pool
    ia.load_adapters(ads[:3])
    assert ia.adapter_dirs == ["a0", "a1", "a2"]
    assert ia.a_len.tolist() == [32, 64, 32] and ia.a_start.tolist() == [0, 32, 96]
    assert ia.a_loc.tolist() == list(range(3, 3 + 128))
    assert ia.a_scaling.tolist() == [2.0, 1.0, 2.0]
    ia.load_adapters([ads[1], ads[3]])   # a1 already resident
    assert ia.adapter_dirs == ["a0", "a1", "a2", "a3"] and ia.a_start.tolist() == [0, 32, 96, 128]
    assert mm.can_use_mem_size == 300 - 3 - (32 + 64 + 32 + 128)

    def check(layer):
        rng = np.random.default_rng(9)
        x = rng.standard_normal((6, H)).astype(np.float32)
        ids = np.array([ia.idx_map[n] for n in ["a3", "a0", "a1", "a3", "a2", "a0"] if n in ia.idx_map])
        x = x[:len(ids)]
        by_name = {a.lora_dir: a for a in ads}
        for p in range(4):
            got = orc.lora_delta_ref(np.zeros((len(ids), H), np.float32), x, mm.key_buffer[layer], mm.value_buffer[layer],
                                     ia.a_start, ia.a_len, ia.a_loc, ids, p, ia.a_scaling)
            for t, i in enumerate(ids):
                ad = by_name[ia.adapter_dirs[i]]
                a16 = ad.A[layer][p].astype(np.float16).astype(np.float32)
                b16 = ad.B[layer][p].astype(np.float16).astype(np.float32)
                np.testing.assert_allclose(got[t], (x[t] @ a16.T) @ b16.T * ad.scaling, rtol=1e-4, atol=1e-5)

    check(0)
    check(1)
    ia.offload_adapters(["a0", "a3"])
    assert ia.adapter_dirs == ["a0", "a3"] and ia.idx_map == {"a0": 0, "a3": 1}
    assert ia.a_len.tolist() == [32, 128] and ia.a_start.tolist() == [0, 32]
    assert mm.can_use_mem_size == 300 - 3 - 160
    check(1)
    ia.offload_adapters([])
    assert ia.a_loc.numel() == 0 and mm.can_use_mem_size == 300 - 3


def test_prefetch_stops_at_capacity_and_protects_tagged_adapters():
    H, heads = 32, 4
    mm = _mm(tot=80, layers=1, heads=heads, hd=8)
    ia = InferAdapter.init(mm, None)
    ads = [_Adapter(f"a{i}", 8, H, heads, 1, i) for i in range(4)]
    ia.load_adapters(ads[:1])
    ia.load_adapters(ads[1:], prefetch=True)     # room for one more 32-row adapter only
    assert ia.adapter_dirs == ["a0", "a1"]
    ia.offload_adapters(["a0"])                   # a1 was tagged by the latest prefetch: kept
    assert ia.adapter_dirs == ["a0", "a1"]


def test_workloads_are_deterministic_and_shaped_like_the_configs():
    a, b = build_workload(1), build_workload(1)
    assert torch.equal(a.ids, b.ids) and torch.equal(a.pools_a[0], b.pools_a[0]) and torch.equal(a.x_o[0], b.x_o[0])
    assert a.T == 32 and a.ranks == [8] * 4 and float(a.a_scaling[0]) == 2.0
    w3 = build_workload(3, pool_rows=65536, hidden=64, with_activations=False)
    assert len(w3.segments) == 8 + 248 and w3.T == sum(n for _, n, _ in w3.segments)
    assert set(w3.ranks) <= {8, 16, 32, 64} and all(8 <= n <= 512 for _, n, _ in w3.segments[:8])
    w4 = build_workload(4, pool_rows=SPECS[4].pool_rows, hidden=64, with_activations=False)
    assert w4.T == 512 and len(w4.ranks) == 2000
    w5 = build_workload(5, hidden=64, h_kv=8, with_activations=False)
    assert w5.T == 1024 and w5.proj_dims() == [(64, 64), (64, 8), (64, 8), (64, 64)]
    assert len(torch.unique(w4.a_loc)) == w4.a_loc.numel()
    assert abs(float(zipf_probs(1000, 1.0).sum()) - 1.0) < 1e-12


def test_algorithmic_bytes_of_the_s1_decode_batch():
    w = build_workload(2, pool_rows=65536, hidden=4096, with_activations=False)
    distinct = len(torch.unique(w.ids))
    want = distinct * 4 * 8 * 8192 * 2 + 256 * 2 * 4096 * 2 + 256 * 4 * 2 * 4096 * 2
    assert w.algorithmic_bytes_per_layer() == want
    assert 100 <= distinct <= 170     # Zipf(1.0) over 1000 adapters, 256 draws
    assert w.gathered_bytes_per_layer() > w.algorithmic_bytes_per_layer()


def test_reference_arm_of_the_benchmark_runs_without_the_product_library(tmp_path):
    """``bench.py --impl reference`` times the CPU restatement of the reference's per-token formula and must not need
    the CUDA library: it is run here with the library path pointing nowhere (importing the package would fail).  Its
    line carries the keys the benchmark contract asks of the reference arm."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, SLORA_B200_LIB=str(tmp_path / "no_such_library.so"))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--config", "1",
                          "--steps", "1", "--warmup", "1"], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "lora_delta_tokens_per_s" and line["value"] > 0
    assert line["gpu_launches"] == 0 and line["vs_baseline"] is None
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and "sample" in cb
    assert str(cb["cores"]) in cb["thread_sweep_s_per_layer"]
    assert line["config"]["workload"].startswith("cfg1") and line["config"]["tokens"] == 32
