"""The tensor-parallel exchange of the rank-r intermediates: ``slora_tp_regroup`` (after an all-gather) and
``slora_tp_exchange`` (one kernel over peer memory), against the plain formula.

On one GPU the N ranks are emulated inside one process: every rank's buffers are ordinary device tensors (addresses all
valid on the one GPU), the ranks' launches follow each other on one stream, and a rank only waits for flags that
earlier launches have already raised.  With two or more GPUs the real thing runs as one process per GPU over symmetric
memory and is compared with the single-GPU operator.
"""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch

import slora_b200 as sl
from slora_b200 import _lib, tp
from slora_b200.workloads import make_tables
from tests.helpers import assert_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _expected_full(locals_, ids, slot_rows, N, Rl, nproj):
    """out[p, t, g*rs + j] = locals_[g][p, t, j] for j < rs."""
    T = ids.numel()
    out = torch.zeros((3, T, N * Rl), dtype=locals_[0].dtype)
    for t in range(T):
        rs = slot_rows[int(ids[t])]
        for g in range(N):
            out[:nproj, t, g * rs:(g + 1) * rs] = locals_[g][:nproj, t, :rs].cpu()
    return out


@pytest.mark.parametrize("nproj", [3, 1])
def test_regroup_and_exchange_emulated_on_one_gpu(nproj):
    N, T, Rl = 4, 37, 16
    ranks = [16, 64, 32, 64, 8 * N]            # full ranks; a rank's slot holds r / N rows
    slot_rows = [r // N for r in ranks]
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, len(ranks), (T,), generator=g).to(DEV)
    a_len = torch.tensor([4 * s for s in slot_rows], dtype=torch.int64, device=DEV)
    locals_ = [torch.randn((3, T, Rl), generator=g).to(torch.float16).to(DEV) for _ in range(N)]
    want = _expected_full(locals_, ids.cpu(), slot_rows, N, Rl, nproj)

    # all-gather layout + regroup
    gathered = torch.stack(locals_)            # [N, 3, T, Rl]
    out = torch.zeros((3, T, N * Rl), dtype=torch.float16, device=DEV)
    _lib.check(_lib.lib.slora_tp_regroup(out.data_ptr(), gathered.data_ptr(), ids.data_ptr(), a_len.data_ptr(), N,
                                         nproj, T, Rl, 3 * T * Rl, len(ranks), _lib.F16, _lib.current_stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(out.cpu()[:nproj], want[:nproj])

    # exchange: every emulated rank owns a buffer [2, 3, cap, R] and flags [2, N]
    cap = T + 3
    fulls = [torch.zeros((2, 3, cap, N * Rl), dtype=torch.float16, device=DEV) for _ in range(N)]
    flags = [torch.zeros((2, N), dtype=torch.int32, device=DEV) for _ in range(N)]
    counters = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(N)]
    seq_states = [torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(N)]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    full_ptrs = (ctypes.c_void_p * N)(*[f.data_ptr() for f in fulls])
    flag_ptrs = (ctypes.c_void_p * N)(*[f.data_ptr() for f in flags])

    def call(rank, half, mode):
        _lib.check(_lib.lib.slora_tp_exchange(locals_[rank].data_ptr(), full_ptrs, flag_ptrs,
                                              counters[rank].data_ptr(), status.data_ptr(), ids.data_ptr(),
                                              a_len.data_ptr(), rank, N, nproj, T, cap, Rl, len(ranks), half,
                                              seq_states[rank].data_ptr(), mode, _lib.F16, 0,
                                              _lib.current_stream_ptr()))

    for n, half in enumerate((0, 1, 0), start=1):   # three exchanges: both halves, and a half used a second time
        for f in fulls:
            f[half].zero_()
        for rank in range(N - 1):
            call(rank, half, 1)                # write + signal; its wait comes later
        call(N - 1, half, 3)                   # the last rank finds every flag raised
        for rank in range(N - 1):
            call(rank, half, 2)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        done = (n + 1) // 2 if half == 0 else 1
        for rank in range(N):
            got = fulls[rank][half][:nproj, :T].cpu()
            assert torch.equal(got, want[:nproj]), f"rank {rank} exchange {n}"
            assert flags[rank][half].cpu().tolist() == [done] * N
            assert int(seq_states[rank][half]) == done


def test_input_sharded_o_projection_emulated_on_one_gpu():
    """A cut over its input columns (``rank_mult`` rows per slot row), partial shrinks per rank, the all-sum over
    (emulated) peer memory, then the output-sharded expand: concatenated slices against the formula."""
    H, N, T = 1024, 4, 29
    ranks = [8, 32, 16]
    g = torch.Generator().manual_seed(8)
    ads = [([torch.randn((r, H), generator=g) / 32 for _ in range(4)],
            [torch.randn((H, r), generator=g) * 0.02 for _ in range(4)]) for r in ranks]
    x = torch.randn((T, H), generator=g).to(torch.float16)
    ids = torch.randint(0, len(ranks), (T,), generator=g)
    R, hs = max(ranks), H // N
    shards = []
    for rank in range(N):
        a_start, a_len, a_loc = make_tables([r // N for r in ranks], 256, 500 + rank, True)
        pa = torch.zeros((256, H), dtype=torch.float16)
        pb = torch.zeros((256, H), dtype=torch.float16)
        for i, (A, B) in enumerate(ads):
            ra, rb = tp.shard_adapter(A, B, rank, N, H, o_input_sharded=True)
            loc = a_loc[a_start[i]: a_start[i] + a_len[i]]
            pa[loc] = ra.to(torch.float16)
            pb[loc] = rb.to(torch.float16)
        t = tp.TpTables(a_start.to(DEV), a_len.to(DEV), a_loc.to(DEV),
                        torch.tensor([16.0 / r for r in ranks], dtype=torch.float16, device=DEV))
        shards.append((t, pa.to(DEV), pb.to(DEV)))
    be = tp.CudaBackend()
    idd = ids.to(DEV)
    partials = []
    for rank, (t, pa, pb) in enumerate(shards):
        part = torch.zeros((T, R), dtype=torch.float16, device=DEV)
        plan = be.make_plan(idd, t)
        be.shrink(plan, idd, [3], [part], x[:, rank * hs:(rank + 1) * hs].contiguous().to(DEV), pa, t, rank_mult=N)
        partials.append(part)
    torch.cuda.synchronize()
    got_delta = sum(p.float() for p in partials).cpu().numpy()
    for i in range(T):
        A = ads[int(ids[i])][0][3].half().float().numpy()
        ref = x[i].float().numpy() @ A.T
        assert np.abs(got_delta[i, :A.shape[0]] - ref).max() <= 2e-2 * max(np.abs(ref).max(), 1e-3)

    # all-sum over emulated peer memory: every rank owns parts [N, cap, R] and flags [2, N]
    cap = T + 5
    parts = [torch.zeros((N, cap, R), dtype=torch.float16, device=DEV) for _ in range(N)]
    flags = [torch.zeros((2, N), dtype=torch.int32, device=DEV) for _ in range(N)]
    counters = [torch.zeros(1, dtype=torch.int32, device=DEV) for _ in range(N)]
    seq_states = [torch.zeros(2, dtype=torch.int32, device=DEV) for _ in range(N)]
    outs = [torch.zeros((T, R), dtype=torch.float16, device=DEV) for _ in range(N)]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    part_ptrs = (ctypes.c_void_p * N)(*[p.data_ptr() for p in parts])
    flag_ptrs = (ctypes.c_void_p * N)(*[f.data_ptr() for f in flags])

    def call(rank, mode):
        _lib.check(_lib.lib.slora_tp_allsum(partials[rank].data_ptr(), part_ptrs, flag_ptrs, counters[rank].data_ptr(),
                                            status.data_ptr(), outs[rank].data_ptr(), rank, N, T, cap, R, 1,
                                            seq_states[rank].data_ptr(), mode, _lib.F16, 0, _lib.current_stream_ptr()))

    for rank in range(N - 1):
        call(rank, 1)
    call(N - 1, 3)
    for rank in range(N - 1):
        call(rank, 2)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    total = sum(p.float() for p in partials).to(torch.float16)
    for rank in range(N):
        assert torch.equal(outs[rank], total)

    slices = []
    for rank, (t, pa, pb) in enumerate(shards):
        y = torch.zeros((T, H // N), dtype=torch.float16, device=DEV)
        plan = be.make_plan(idd, t)
        be.expand(plan, idd, [3], [y], [outs[rank]], pb, t, delta_stride=R, delta_width=R, delta_parts=1,
                  delta_part_stride=0, rank_mult=N)
        slices.append(y)
    torch.cuda.synchronize()
    got = torch.cat(slices, dim=1)
    want = torch.stack([(x[i].float() @ ads[int(ids[i])][0][3].half().float().T)
                        @ ads[int(ids[i])][1][3].half().float().T * (16.0 / ranks[int(ids[i])]) for i in range(T)])
    assert_parity(got, want.numpy(), what="input-sharded o projection")


class _EmulatedPeers:
    """What CudaBackend reads of a PeerExchange, for N ranks that all live on one GPU (plain device tensors)."""

    def __init__(self, N, cap, R, inband):
        self.fulls = [torch.zeros((3 if inband == 3 else 2, 3, cap, R), dtype=torch.float16, device=DEV)
                      for _ in range(N)]
        if inband:
            for f in self.fulls:
                f.view(torch.int16).fill_(-1)
        self.flagss = [torch.zeros((2, N), dtype=torch.int32, device=DEV) for _ in range(N)]
        self.N, self.inband = N, inband

    def rank(self, r):
        px = type("Px", (), {})()
        N = self.N
        px.full, px.flags = self.fulls[r], self.flagss[r]
        px.full_ptrs = (ctypes.c_void_p * N)(*[f.data_ptr() for f in self.fulls])
        px.flag_ptrs = (ctypes.c_void_p * N)(*[f.data_ptr() for f in self.flagss])
        px.counter = torch.zeros(4, dtype=torch.int32, device=DEV)
        px.seq_state = torch.zeros(2, dtype=torch.int32, device=DEV)
        px.inband_seq = torch.zeros(2, dtype=torch.int32, device=DEV)
        px.rank, px.world, px.inband = r, N, self.inband
        return px


@pytest.mark.parametrize("inband", [3, 2, True, False])
@pytest.mark.parametrize("T", [40, 200])
def test_fused_exchange_emulated_on_one_gpu(T, inband):
    """slora_tp_shrink_push / slora_tp_expand_wait, four ranks emulated on one GPU: every rank's shrink stores its rows
    into every rank's buffer; every rank's expand then finds them there (in-band signalling: none of the values it
    uses is the empty pattern any more, and its last CTA refills the half - or, with rotating thirds (3), the next
    exchange's shrink refills the part; else: every rank's flag is up).  Five exchanges (q,k,v and o alternating, so
    that the thirds wrap around) against the formula."""
    H, N = 4096, 4
    ranks = [8, 16, 32, 8]
    g = torch.Generator().manual_seed(23)
    ads = [([torch.randn((r, H), generator=g) / 64 for _ in range(4)],
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
    peers = _EmulatedPeers(N, T, R, inband)
    pxs = [peers.rank(r) for r in range(N)]
    # (inband >= 2: the expand does not wait for its own GPU's shrink either; chained as programmatic dependents)
    be = tp.CudaBackend(use_pdl=inband in (2, 3), inband=inband)
    xd, idd = x.to(DEV), ids.to(DEV)
    plans = [be.make_plan(idd, t) for t, _, _ in shards]
    want = [torch.stack([(x[i].float() @ ads[int(ids[i])][0][p].half().float().T)
                         @ ads[int(ids[i])][1][p].half().float().T * (16.0 / ranks[int(ids[i])]) for i in range(T)])
            for p in range(4)]
    for n_done, (qkvo, half) in enumerate((([0, 1, 2], 0), ([3], 1), ([0, 1, 2], 0), ([3], 1), ([0, 1, 2], 0))):
        for rank, (t, pa, pb) in enumerate(shards):
            be.shrink_push(pxs[rank], plans[rank], idd, qkvo, xd, pa, t, Rl, half)
        ys = []
        for rank, (t, pa, pb) in enumerate(shards):
            y = [torch.zeros((T, H // N), dtype=torch.float16, device=DEV) for _ in qkvo]
            be.expand_wait(pxs[rank], plans[rank], idd, qkvo, y, pb, t, Rl, half)
            ys.append(y)
        torch.cuda.synchronize()
        for rank in range(N):
            plans[rank].check()
            if inband == 3:    # the sequence words moved on; the part of the exchange before this one is empty again
                assert pxs[rank].inband_seq.tolist() == [n_done + 1, n_done]
                if n_done > 0:
                    assert bool((peers.fulls[rank][(n_done - 1) % 3].view(torch.int16) == -1).all())
            elif inband:       # the consumed half is empty again
                assert bool((peers.fulls[rank][half].view(torch.int16) == -1).all())
        for j, p in enumerate(qkvo):
            got = torch.cat([ys[rank][j] for rank in range(N)], dim=1)
            assert_parity(got, want[p].numpy(), what=f"fused exchange proj {p}")


def test_rotating_thirds_keep_their_place_across_graph_replays():
    """One exchange per CUDA graph (an odd number, so a replay cannot start where the capture did): the part of the
    buffers an exchange works in comes from the sequence words on the device, so replays rotate on through the three
    parts.  Two ranks emulated on one GPU; five exchanges accumulate into the same outputs, against the same five
    exchanges on the flag path."""
    H, N, T = 4096, 2, 48
    ranks = [16, 32, 16]
    g = torch.Generator().manual_seed(29)
    ads = [([torch.randn((r, H), generator=g) / 64 for _ in range(4)],
            [torch.randn((H, r), generator=g) * 0.02 for _ in range(4)]) for r in ranks]
    x = torch.randn((T, H), generator=g).to(torch.float16).to(DEV)
    ids = torch.randint(0, len(ranks), (T,), generator=g).to(DEV)
    R, Rl = max(ranks), max(ranks) // N
    shards = []
    for rank in range(N):
        a_start, a_len, a_loc = make_tables([r // N for r in ranks], 512, 400 + rank, True)
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

    def run(inband, use_graph):
        peers = _EmulatedPeers(N, T, R, inband)
        pxs = [peers.rank(r) for r in range(N)]
        be = tp.CudaBackend(use_pdl=inband == 3, inband=inband)
        plans = [be.make_plan(ids, t) for t, _, _ in shards]
        ys = [[torch.zeros((T, H // N), dtype=torch.float16, device=DEV) for _ in range(3)] for _ in range(N)]

        def exchange():
            for rank, (t, pa, pb) in enumerate(shards):
                be.shrink_push(pxs[rank], plans[rank], ids, [0, 1, 2], x, pa, t, Rl, 0)
            for rank, (t, pa, pb) in enumerate(shards):
                be.expand_wait(pxs[rank], plans[rank], ids, [0, 1, 2], ys[rank], pb, t, Rl, 0)

        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            exchange()
            if use_graph:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=s):
                    exchange()
                for _ in range(4):
                    graph.replay()
            else:
                for _ in range(4):
                    exchange()
        s.synchronize()
        for plan in plans:
            plan.check()
        return ys, pxs

    want, _ = run(False, False)
    got, pxs = run(3, True)
    for rank in range(N):
        assert pxs[rank].inband_seq.tolist() == [5, 4]
        for j in range(3):
            assert torch.equal(got[rank][j], want[rank][j]), f"rank {rank} proj {j}"


def test_in_band_wait_runs_out_without_hanging():
    """An expand whose delta rows nobody writes (no rank has pushed): the consumers' bounded re-reads give up, the
    status word says so, the launch ends and the context stays usable."""
    H, N, T = 4096, 2, 12
    ranks = [16, 16]
    a_start, a_len, a_loc = make_tables([r // N for r in ranks], 128, 7, True)
    t = tp.TpTables(a_start.to(DEV), a_len.to(DEV), a_loc.to(DEV),
                    torch.tensor([1.0, 1.0], dtype=torch.float16, device=DEV))
    pb = torch.zeros((128, H), dtype=torch.float16, device=DEV)
    ids = torch.zeros(T, dtype=torch.int64, device=DEV)
    peers = _EmulatedPeers(N, T, 16, True)
    px = peers.rank(0)
    be = tp.CudaBackend()
    plan = be.make_plan(ids, t)
    y = torch.zeros((T, H // N), dtype=torch.float16, device=DEV)
    be.expand_wait(px, plan, ids, [0], [y], pb, t, 8, 0)
    torch.cuda.synchronize()
    assert plan.status()[0] & 8                # SLORA_STATUS_TIMEOUT
    assert int((y + 1).sum().item()) == y.numel()


def test_exchange_wait_runs_out_without_hanging():
    """A flag that nobody raises: the bounded wait gives up, the status word says so, the context stays usable."""
    N, T, Rl = 2, 8, 8
    ids = torch.zeros(T, dtype=torch.int64, device=DEV)
    a_len = torch.tensor([4 * Rl], dtype=torch.int64, device=DEV)
    local = torch.ones((3, T, Rl), dtype=torch.float16, device=DEV)
    fulls = [torch.zeros((2, 3, T, N * Rl), dtype=torch.float16, device=DEV) for _ in range(N)]
    flags = [torch.zeros((2, N), dtype=torch.int32, device=DEV) for _ in range(N)]
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    seq_state = torch.zeros(2, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    full_ptrs = (ctypes.c_void_p * N)(*[f.data_ptr() for f in fulls])
    flag_ptrs = (ctypes.c_void_p * N)(*[f.data_ptr() for f in flags])
    _lib.check(_lib.lib.slora_tp_exchange(local.data_ptr(), full_ptrs, flag_ptrs, counter.data_ptr(),
                                          status.data_ptr(), ids.data_ptr(), a_len.data_ptr(), 0, N, 1, T, T, Rl, 1, 1,
                                          seq_state.data_ptr(), 3, _lib.F16, 0, _lib.current_stream_ptr()))  # rank 1 is silent
    torch.cuda.synchronize()
    assert int(status.item()) & 8              # SLORA_STATUS_TIMEOUT
    assert float(fulls[1][1, 0, 0, 0]) == 1.0  # the writes went out all the same
    assert int((local + 1).sum().item()) == 2 * local.numel()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    # pool rows of 4096 elements: every kernel of the pipelined family fits; 160 tokens of mixed ranks: the backend
    # asks the plan and turns on the exact work-item count
    H, T = 4096, 160
    ranks = [8, 16, 32, 16]
    g = torch.Generator().manual_seed(33)
    ads = [([torch.randn((r, H), generator=g) / 32 for _ in range(4)],
            [torch.randn((H, r), generator=g) * 0.02 for _ in range(4)]) for r in ranks]
    x = torch.randn((T, H), generator=g).to(torch.float16)
    ids = torch.randint(0, len(ranks), (T,), generator=g)
    a_start, a_len, a_loc = make_tables([r // world for r in ranks], 512, 300 + rank, True)
    pa = torch.zeros((512, H), dtype=torch.float16)
    pb = torch.zeros((512, H), dtype=torch.float16)
    for i, (A, B) in enumerate(ads):
        ra, rb = tp.shard_adapter(A, B, rank, world, H)
        loc = a_loc[a_start[i]: a_start[i] + a_len[i]]
        pa[loc] = ra.to(torch.float16)
        pb[loc] = rb.to(torch.float16)
    t = tp.TpTables(a_start.to(dev), a_len.to(dev), a_loc.to(dev),
                    torch.tensor([16.0 / r for r in ranks], dtype=torch.float16, device=dev))
    outs = {}
    # peer memory from inside the shrink / expand kernels; one exchange kernel; NCCL all-gather + regroup
    # ("fused_early": chained as programmatic dependents, the expand starts without waiting for this GPU's shrink
    # and the delta buffers rotate through three parts - what the benchmark runs)
    kinds = {"fused": (True, True, False), "fused_early": (True, True, True), "kernel": (True, False, False),
             "nccl": (False, False, False)}
    for kind, (peer, fused, pdl) in kinds.items():
        be = tp.CudaBackend(use_pdl=pdl, fused=fused)
        assert be.inband == (3 if pdl else 1)
        ops = tp.TpLoraOps(t, [pa.to(dev)], [pb.to(dev)], max(ranks), world, rank, be,
                           peer_exchange=peer).prepare(ids.to(dev))
        before = sl.launch_counts()
        for rep in range(4):                    # several layers' worth of exchanges on every part of the buffers
            q, k, v, o = (torch.zeros((T, H // world), dtype=torch.float16, device=dev) for _ in range(4))
            ops.lora_qkv(0, x.to(dev), q, k, v)
            ops.lora_o(0, x.to(dev), o)
        torch.cuda.synchronize()
        ops.plan.check()
        outs[kind] = torch.stack([q, k, v, o]).cpu()
        after = sl.launch_counts()
        if kind.startswith("fused"):            # two launches per call and nothing else: no exchange kernel, no fallback
            assert after["pipelined"] - before["pipelined"] == 4 * 4 and after["simple"] == before["simple"]
            assert after["plan"] == before["plan"]
    assert torch.equal(outs["fused"], outs["nccl"]) and torch.equal(outs["kernel"], outs["nccl"])
    assert torch.equal(outs["fused_early"], outs["nccl"])
    np.save(os.path.join(result_dir, f"rank{rank}.npy"), outs["fused"].float().numpy())

    # the o projection with a head-sharded input: partial shrinks summed over peer memory, and by NCCL all_reduce
    pa2 = torch.zeros((512, H), dtype=torch.float16)
    for i, (A, B) in enumerate(ads):
        ra, _ = tp.shard_adapter(A, B, rank, world, H, o_input_sharded=True)
        pa2[a_loc[a_start[i]: a_start[i] + a_len[i]]] = ra.to(torch.float16)
    hs = H // world
    x_g = x[:, rank * hs:(rank + 1) * hs].contiguous().to(dev)
    o_outs = {}
    for peer in (True, False):
        ops = tp.TpLoraOps(t, [pa2.to(dev)], [pb.to(dev)], max(ranks), world, rank, tp.CudaBackend(),
                           peer_exchange=peer).prepare(ids.to(dev))
        for rep in range(3):
            o = torch.zeros((T, H // world), dtype=torch.float16, device=dev)
            ops.lora_o_sharded(0, x_g, o)
        torch.cuda.synchronize()
        ops.plan.check()
        o_outs[peer] = o.cpu()
    # (the two sums round differently: FP32 sum rounded once against a 16-bit all_reduce)
    assert (o_outs[True].float() - o_outs[False].float()).abs().max() <= 2e-2 * o_outs[False].float().abs().max()
    np.save(os.path.join(result_dir, f"o_sharded_rank{rank}.npy"), o_outs[True].float().numpy())
    if rank == 0:
        want = [torch.stack([(x[i].float() @ ads[int(ids[i])][0][p].half().float().T)
                             @ ads[int(ids[i])][1][p].half().float().T * (16.0 / ranks[int(ids[i])])
                             for i in range(T)]).numpy() for p in range(4)]
        np.save(os.path.join(result_dir, "want.npy"), np.stack(want))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_exchange_over_symmetric_memory_on_two_gpus(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    want = np.load(tmp_path / "want.npy")
    got = np.concatenate([np.load(tmp_path / f"rank{r}.npy") for r in range(world)], axis=2)
    for p in range(4):
        assert_parity(got[p], want[p], what=f"tp2 proj {p}")
    got_o = np.concatenate([np.load(tmp_path / f"o_sharded_rank{r}.npy") for r in range(world)], axis=1)
    assert_parity(got_o, want[3], what="tp2 input-sharded o projection")
