"""Adapter load into the Unified-Paging pool on the GPU (``slora_pool_scatter_rows``): the same adapters loaded
through ``InferAdapter`` on a CUDA pool and on a CPU pool (the per-layer indexed copies) must leave bit-identical
pools and tables; then the loaded pool feeds the LoRA kernels.  Needs a B200."""
import ctypes

import numpy as np
import pytest
import torch

import slora_b200 as sl
from slora_b200 import _lib
from tests.helpers import assert_parity, orc
from tests.test_host import _Adapter

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _pool(device, tot, L, heads, hd):
    return sl.MemoryAllocator(tot, 0, torch.float16, heads, hd, L, device=device)


def test_load_adapters_on_the_gpu_matches_the_cpu_copies_bit_for_bit():
    H, heads, L = 1024, 8, 5
    ads = [_Adapter(f"a{i}", r, H, heads, L, 40 + i) for i, r in enumerate([8, 64, 16, 32])]
    pools = {}
    for device in ("cpu", DEV):
        mm = _pool(device, 600, L, heads, H // heads)
        for l in range(L):               # rows no adapter owns must stay as they were
            mm.key_buffer[l].fill_(3.0)
            mm.value_buffer[l].fill_(5.0)
        mm.alloc(7)                      # someone else's rows at the front of the pool
        ia = sl.InferAdapter.init(mm, None)
        before = sl.launch_counts()["plan"]
        ia.load_adapters(ads[:2])
        ia.load_adapters(ads[1:])        # a1 is resident already
        if device == DEV:
            torch.cuda.synchronize()
            assert sl.launch_counts()["plan"] - before == 4     # one launch per adapter, whatever the layer count
        pools[device] = (mm, ia)
    (mc, ic), (mg, ig) = pools["cpu"], pools[DEV]
    assert ic.a_loc.tolist() == ig.a_loc.tolist() and ic.a_start.tolist() == ig.a_start.tolist()
    assert ic.a_len.tolist() == ig.a_len.tolist()
    for l in range(L):
        assert torch.equal(mc.key_buffer[l], mg.key_buffer[l].cpu())
        assert torch.equal(mc.value_buffer[l], mg.value_buffer[l].cpu())

    # the freshly loaded pool through the kernels, against the HF formula
    T = 24
    g = torch.Generator().manual_seed(3)
    x = torch.randn((T, H), generator=g).to(torch.float16)
    ids = torch.randint(0, len(ads), (T,), generator=g)
    ops = sl.LoraBatchOps(ig.a_start, ig.a_len, ig.a_loc, ig.a_scaling,
                          [b.view(b.size(0), -1) for b in mg.key_buffer], [b.view(b.size(0), -1) for b in mg.value_buffer],
                          64)
    ops.prepare(ids.to(DEV))
    o = torch.zeros((T, H), dtype=torch.float16, device=DEV)
    ops.lora_get_o(2, x.to(DEV), o)
    torch.cuda.synchronize()
    ops.plan.check()
    want = np.stack([(x[t].float().numpy() @ ads[int(ids[t])].A[2][3].astype(np.float16).astype(np.float32).T)
                     @ ads[int(ids[t])].B[2][3].astype(np.float16).astype(np.float32).T * ads[int(ids[t])].scaling
                     for t in range(T)])
    assert_parity(o, want, what="o projection from a pool loaded on the GPU")


def test_scatter_skips_rows_outside_the_pool():
    L, n, row = 2, 4, 64
    key = [torch.zeros((10, row), dtype=torch.float16, device=DEV) for _ in range(L)]
    val = [torch.zeros((10, row), dtype=torch.float16, device=DEV) for _ in range(L)]
    src = [torch.arange(2 * n * row, dtype=torch.float32).reshape(2, n, row).to(torch.float16).to(DEV) + l for l in range(L)]
    loc = torch.tensor([2, 99, 0, -1], dtype=torch.int64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    arr = ctypes.c_void_p * L
    _lib.check(_lib.lib.slora_pool_scatter_rows(arr(*[k.data_ptr() for k in key]), arr(*[v.data_ptr() for v in val]),
                                                arr(*[s.data_ptr() for s in src]), L, loc.data_ptr(), n, row * 2, 10,
                                                row * 2, status.data_ptr(), _lib.current_stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) & 2          # SLORA_STATUS_BAD_TABLE
    for l in range(L):
        assert torch.equal(key[l][2], src[l][0, 0]) and torch.equal(key[l][0], src[l][0, 2])
        assert torch.equal(val[l][2], src[l][1, 0]) and torch.equal(val[l][0], src[l][1, 2])
        untouched = [r for r in range(10) if r not in (0, 2)]
        assert float(key[l][untouched].abs().max()) == 0.0 and float(val[l][untouched].abs().max()) == 0.0
    with pytest.raises(RuntimeError, match="multiples of 16"):
        _lib.check(_lib.lib.slora_pool_scatter_rows(arr(*[k.data_ptr() for k in key]), arr(*[v.data_ptr() for v in val]),
                                                    arr(*[s.data_ptr() for s in src]), L, loc.data_ptr(), n, 24, 10,
                                                    row * 2, 0, _lib.current_stream_ptr()))
