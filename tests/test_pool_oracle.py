"""The pool-bookkeeping oracle against hand-worked cases, and the host mirror on a CPU pool against the oracle."""
import numpy as np
import torch

from oracle import pool_oracle as porc
from slora_b200.mem_allocator import MemoryAllocator


def test_alloc_hands_out_the_first_free_rows_in_order():
    state = np.array([0, 1, 1, 0, 1, 0, 0, 1, 1], dtype=bool)
    rows, after = porc.alloc_ref(state, 3)
    assert rows.tolist() == [1, 2, 4]
    assert after.tolist() == [False, False, False, False, False, False, False, True, True]
    rows, after2 = porc.alloc_ref(after, 0)
    assert rows.tolist() == [] and (after2 == after).all()
    rows, after3 = porc.alloc_ref(after, 2)
    assert rows.tolist() == [7, 8] and not after3.any()
    assert porc.free_ref(after3, np.array([3, 8, 3])).tolist() == [False, False, False, True, False, False, False, False,
                                                                   True]


def test_compaction_keeps_order_and_frees_the_dropped_rows():
    a_start = [0, 4, 6, 9]          # runs of 4, 2, 3 and 1 rows
    a_len = [4, 2, 3, 1]
    a_loc = [10, 11, 12, 13, 20, 21, 5, 6, 7, 30]
    scal = np.array([2.0, 1.0, 0.5, 4.0], dtype=np.float16)
    state = np.zeros(32, dtype=bool)
    ns, nl, nloc, nsc, after = porc.compact_ref(a_start, a_len, a_loc, scal, [1, 0, 1, 0], state)
    assert ns.tolist() == [0, 4] and nl.tolist() == [4, 3]
    assert nloc.tolist() == [10, 11, 12, 13, 5, 6, 7]
    assert nsc.tolist() == [2.0, 0.5]
    assert np.nonzero(after)[0].tolist() == [20, 21, 30]
    ns, nl, nloc, nsc, after = porc.compact_ref(a_start, a_len, a_loc, scal, [0, 0, 0, 0], state)
    assert len(ns) == 0 and len(nloc) == 0 and int(after.sum()) == 10


def test_host_allocator_on_a_cpu_pool_follows_the_oracle():
    rng = np.random.default_rng(5)
    mm = MemoryAllocator(1000, 0, torch.float16, 2, 8, 1, device="cpu", allocate_buffers=False)
    state = np.ones(1000, dtype=bool)
    held = []
    for step in range(40):
        if held and rng.random() < 0.4:
            rows = held.pop(int(rng.integers(len(held))))
            mm.free(torch.from_numpy(rows))
            state = porc.free_ref(state, rows)
        else:
            need = int(rng.integers(0, 60))
            got = mm.alloc(need).numpy()
            want, state = porc.alloc_ref(state, need)
            assert got.tolist() == want.tolist()
            held.append(got)
        assert mm.mem_state.numpy().tolist() == state.tolist()
        assert mm.can_use_mem_size == int(state.sum())


# ---------------------------------------------------------------------------------------------------------------
# pinned to the reference: traces of its own MemoryAllocator / InferAdapter (tests/golden/make_pool_golden.py)
# ---------------------------------------------------------------------------------------------------------------
import pytest  # noqa: E402

from tests import pool_replay  # noqa: E402


@pytest.mark.parametrize("name", ["small", "ragged"])
def test_oracle_reproduces_every_step_of_the_reference_traces(name):
    assert pool_replay.replay_oracle(name) >= 20


@pytest.mark.parametrize("name", ["small", "ragged"])
def test_host_mirror_on_a_cpu_pool_reproduces_the_reference_traces(name):
    assert pool_replay.replay_host_mirror(name, "cpu") >= 40
