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
            # per call two launches allocate the rows; then one launch per adapter, whatever the layer count
            assert sl.launch_counts()["plan"] - before == 2 * 2 + 4
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


# ---------------------------------------------------------------------------------------------------------------
# free map and adapter tables on the device, bit-exact against the CPU oracle
# ---------------------------------------------------------------------------------------------------------------
from oracle import pool_oracle as porc  # noqa: E402  (the checker)


def _alloc_rows(state_t, need, status):
    tot = state_t.numel()
    ws = torch.empty((max(_lib.lib.slora_pool_alloc_workspace_bytes(tot), 4),), dtype=torch.uint8, device=DEV)
    out = torch.full((need + 3,), -7, dtype=torch.int64, device=DEV)        # three guard entries behind the result
    _lib.check(_lib.lib.slora_pool_alloc_rows(state_t.data_ptr(), tot, need, out.data_ptr(), ws.data_ptr(), ws.numel(),
                                              status.data_ptr(), _lib.current_stream_ptr()))
    torch.cuda.synchronize()
    assert out[need:].tolist() == [-7, -7, -7]
    return out[:need].cpu().numpy()


@pytest.mark.parametrize("tot", [1, 15, 16, 1000, 16384, 16385, 70001, 262144])
def test_alloc_rows_matches_the_oracle_on_fragmented_maps(tot):
    rng = np.random.default_rng(tot)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for density in (1.0, 0.5, 0.03):
        state = rng.random(tot) < density
        state_t = torch.from_numpy(state).to(DEV)
        free = int(state.sum())
        for pick in (lambda f: 0, lambda f: 1, lambda f: f // 3, lambda f: f - 1, lambda f: f):
            need = max(0, min(free, pick(free)))       # ... and at last every row that is left
            got = _alloc_rows(state_t, need, status)
            want, state = porc.alloc_ref(state, need)
            assert np.array_equal(got, want), (tot, density, need)
            assert np.array_equal(state_t.cpu().numpy(), state)
            free -= need
        assert free <= 1
    assert int(status.item()) == 0


def test_alloc_rows_far_end_of_a_large_map_and_shortfall():
    tot = 1_000_003                                   # 62 segments, the last one ragged
    state = np.zeros(tot, dtype=bool)
    state[[5, 400_000, 999_990, 1_000_002]] = True
    state_t = torch.from_numpy(state).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert _alloc_rows(state_t, 3, status).tolist() == [5, 400_000, 999_990]
    assert int(status.item()) == 0
    # the caller believes four rows are left, the map holds one: it is handed out, the rest are -1, status says so
    assert _alloc_rows(state_t, 4, status).tolist() == [1_000_002, -1, -1, -1]
    assert int(status.item()) & 2
    assert not bool(state_t.any())
    with pytest.raises(RuntimeError, match="bad sizes"):
        _alloc_rows(state_t, tot + 1, status)


def test_free_rows_and_out_of_range_entries():
    state_t = torch.zeros(100, dtype=torch.bool, device=DEV)
    rows = torch.tensor([3, 99, 3, 100, -1, 0], dtype=torch.int64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    _lib.check(_lib.lib.slora_pool_free_rows(state_t.data_ptr(), 100, rows.data_ptr(), rows.numel(), status.data_ptr(),
                                             _lib.current_stream_ptr()))
    torch.cuda.synchronize()
    assert torch.nonzero(state_t).view(-1).tolist() == [0, 3, 99] and int(status.item()) & 2


@pytest.mark.parametrize("n_adapters", [1, 7, 1024, 2500])
def test_tables_compact_matches_the_oracle(n_adapters):
    rng = np.random.default_rng(n_adapters)
    lens = rng.choice([32, 64, 128, 256], size=n_adapters).astype(np.int64)
    order = rng.permutation(n_adapters)               # runs need not lie in adapter order in a_loc
    pos = np.concatenate([[0], np.cumsum(lens[order])[:-1]])
    starts = np.empty(n_adapters, dtype=np.int64)
    starts[order] = pos
    loc_len = int(lens.sum())
    tot = loc_len + 1000
    a_loc = rng.permutation(tot)[:loc_len].astype(np.int64)
    scal = (16.0 / (lens / 4)).astype(np.float16)
    state = np.ones(tot, dtype=bool)
    state[a_loc] = False
    for keep_p in (0.0, 0.5, 1.0):
        keep = (rng.random(n_adapters) < keep_p).astype(np.uint8)
        want = porc.compact_ref(starts, lens, a_loc, scal, keep, state)
        d = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(dt).to(DEV)
        state_t = d(state, torch.bool)
        nk, nr = int(keep.sum()), int(lens[keep.astype(bool)].sum())
        new_start = torch.full((n_adapters + 1,), -7, dtype=torch.int64, device=DEV)
        new_len = torch.full((n_adapters + 1,), -7, dtype=torch.int64, device=DEV)
        new_loc = torch.full((loc_len + 1,), -7, dtype=torch.int64, device=DEV)
        new_scal = torch.full((n_adapters + 1,), -7.0, dtype=torch.float16, device=DEV)
        scratch = torch.empty((n_adapters,), dtype=torch.int64, device=DEV)
        counts = torch.zeros(2, dtype=torch.int64, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        t_start, t_len, t_loc, t_scal, t_keep = (d(starts, torch.int64), d(lens, torch.int64), d(a_loc, torch.int64),
                                                 d(scal, torch.float16), d(keep, torch.uint8))
        _lib.check(_lib.lib.slora_tables_compact(
            t_start.data_ptr(), t_len.data_ptr(), t_loc.data_ptr(), t_scal.data_ptr(), t_keep.data_ptr(), n_adapters,
            loc_len, new_start.data_ptr(), new_len.data_ptr(), new_loc.data_ptr(), new_scal.data_ptr(),
            scratch.data_ptr(), counts.data_ptr(), state_t.data_ptr(), tot, status.data_ptr(),
            _lib.current_stream_ptr()))
        torch.cuda.synchronize()
        assert counts.tolist() == [nk, nr] and int(status.item()) == 0
        assert np.array_equal(new_start[:nk].cpu().numpy(), want[0]) and np.array_equal(new_len[:nk].cpu().numpy(), want[1])
        assert np.array_equal(new_loc[:nr].cpu().numpy(), want[2])
        assert np.array_equal(new_scal[:nk].cpu().numpy(), want[3])
        assert np.array_equal(state_t.cpu().numpy(), want[4])
        assert int(new_start[nk]) == -7 and int(new_len[nk]) == -7 and int(new_loc[nr]) == -7    # nothing past the end


def test_tables_compact_skips_a_run_that_does_not_fit():
    d = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)
    a_start, a_len, a_loc = d([0, 4, 2], torch.int64), d([2, 9, 2], torch.int64), d([5, 6, 7, 8], torch.int64)
    scal, keep = d([1.0, 2.0, 3.0], torch.float16), d([1, 1, 0], torch.uint8)
    state_t = torch.zeros(16, dtype=torch.bool, device=DEV)
    outs = [torch.full((4,), -7, dtype=torch.int64, device=DEV) for _ in range(3)]
    new_scal = torch.zeros(3, dtype=torch.float16, device=DEV)
    scratch, counts = torch.empty(3, dtype=torch.int64, device=DEV), torch.zeros(2, dtype=torch.int64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    _lib.check(_lib.lib.slora_tables_compact(
        a_start.data_ptr(), a_len.data_ptr(), a_loc.data_ptr(), scal.data_ptr(), keep.data_ptr(), 3, 4,
        outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), new_scal.data_ptr(), scratch.data_ptr(),
        counts.data_ptr(), state_t.data_ptr(), 16, status.data_ptr(), _lib.current_stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) & 2 and counts.tolist() == [1, 2]
    assert outs[0][:1].tolist() == [0] and outs[1][:1].tolist() == [2] and outs[2].tolist() == [5, 6, -7, -7]
    assert torch.nonzero(state_t).view(-1).tolist() == [7, 8]


def test_infer_adapter_load_offload_cycles_on_the_gpu_match_the_cpu_pool():
    """The same sequence of loads, prefetches and offloads on a CUDA pool (device allocation, scatter and table
    compaction) and on a CPU pool (torch index ops): identical tables, free maps and counts after every step."""
    H, heads, L = 256, 4, 3
    ads = [_Adapter(f"a{i}", r, H, heads, L, 70 + i) for i, r in enumerate([8, 64, 16, 32, 8, 16, 64, 8])]
    pair = {}
    for device in ("cpu", DEV):
        mm = _pool(device, 1500, L, heads, H // heads)
        mm.alloc(11)
        pair[device] = (mm, sl.InferAdapter.init(mm, None))

    def same():
        (mc, ic), (mg, ig) = pair["cpu"], pair[DEV]
        torch.cuda.synchronize()
        assert ic.adapter_dirs == ig.adapter_dirs and ic.idx_map == ig.idx_map
        for name in ("a_loc", "a_start", "a_len", "a_scaling"):
            assert getattr(ic, name).tolist() == getattr(ig, name).tolist(), name
        assert mc.can_use_mem_size == mg.can_use_mem_size
        assert torch.equal(mc.mem_state, mg.mem_state.cpu())
        assert int(mg.status.item()) == 0 if mg.status is not None else True

    steps = [("load", [0, 1, 2, 3]), ("off", ["a0", "a2"]), ("load", [4, 5]), ("prefetch", [6, 1]),
             ("off", ["a4"]), ("off", ["a4", "a6"]), ("load", [7, 3, 0]), ("off", ["a0"]), ("off", []), ("load", [2])]
    for kind, arg in steps:
        for device in ("cpu", DEV):
            ia = pair[device][1]
            if kind == "off":
                ia.offload_adapters(arg)
            else:
                ia.load_adapters([ads[i] for i in arg], prefetch=(kind == "prefetch"))
        same()
    (mc, ic), (mg, ig) = pair["cpu"], pair[DEV]
    for l in range(L):
        rows = ic.a_loc
        assert torch.equal(mc.key_buffer[l][rows], mg.key_buffer[l].cpu()[rows])
        assert torch.equal(mc.value_buffer[l][rows], mg.value_buffer[l].cpu()[rows])


@pytest.mark.parametrize("name", ["small", "ragged"])
def test_device_pool_reproduces_the_reference_traces(name):
    """Traces of the reference's own MemoryAllocator / InferAdapter (tests/golden/ref_pool.npz) replayed on a CUDA
    pool: row allocation, release, adapter load and table compaction by the library's kernels, bit-exact after every
    step, pool contents included."""
    from tests import pool_replay
    assert pool_replay.replay_host_mirror(name, DEV) >= 40


def test_prefetch_on_a_side_stream_loads_the_same_rows_as_a_synchronous_load():
    """load_adapters(prefetch=True) with a real prefetch stream: the row indices come from kernels on the current
    stream and are consumed on the prefetch stream, which has to wait for them."""
    H, heads, L = 1024, 8, 4
    ads = [_Adapter(f"a{i}", r, H, heads, L, 90 + i) for i, r in enumerate([64, 8, 32, 16, 64])]
    pools = []
    for side in (False, True):
        mm = _pool(DEV, 3000, L, heads, H // heads)
        for l in range(L):
            mm.key_buffer[l].zero_()
            mm.value_buffer[l].zero_()
        stream = torch.cuda.Stream() if side else None
        ia = sl.InferAdapter.init(mm, stream)
        mm.alloc(13)
        # keep the current stream busy so that an unordered prefetch stream would run ahead of the allocation kernels
        busy = torch.empty((8192, 8192), device=DEV)
        for _ in range(4):
            busy.normal_()
        ia.load_adapters(ads, prefetch=side)
        if side:
            torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        pools.append((mm, ia))
    (m0, i0), (m1, i1) = pools
    assert i0.a_loc.tolist() == i1.a_loc.tolist() and i0.a_start.tolist() == i1.a_start.tolist()
    for l in range(L):
        assert torch.equal(m0.key_buffer[l], m1.key_buffer[l]) and torch.equal(m0.value_buffer[l], m1.value_buffer[l])
    assert float(m1.key_buffer[0][i1.a_loc].abs().max()) > 0
