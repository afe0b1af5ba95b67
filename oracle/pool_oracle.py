"""CPU oracle for the Unified-Paging pool bookkeeping: row allocation, row release and the compaction of the adapter
tables when adapters are dropped.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; the tests call it as the checker.

What it restates, in numpy, step for step (paths inside the S-LoRA reference tree):

* ``MemoryAllocator.alloc`` (``slora/common/mem_allocator.py:30-39``): cumulative sum of the free map, the rows whose
  running count is in ``1..need`` and that are free themselves are handed out (that is: the first ``need`` free rows,
  in increasing order) and marked used;
* ``MemoryAllocator.free`` (``slora/common/mem_allocator.py:185-199``): ``mem_state[rows] = 1``;
* ``InferAdapter.offload_adapters`` (``slora/server/router/model_infer/infer_adapter.py:186-250``): adapters that are
  neither reserved nor tagged by the latest prefetch are dropped; the rest keep their order, ``a_len`` / ``a_scaling``
  are gathered, ``a_start`` is the exclusive prefix sum of the kept lengths, the kept runs of ``a_loc`` are copied back
  to back (the reference's variable-length copy kernel, ``infer_adapter.py:261-280``), and the dropped adapters' rows
  go back to the free map.

Parity pin: integer work, bit-exact.  The reference holds no stored vectors for these steps, so the pin is the
reference itself: ``tests/golden/make_pool_golden.py`` runs the reference's own ``MemoryAllocator`` and
``InferAdapter`` on CPU tensors (its ``device="cuda"`` tensor factories redirected, nothing else changed) through
seeded scenarios of allocations, releases, adapter loads and offloads and records every returned index tensor, the
free map, the four tables and checksums of the pool rows (``tests/golden/ref_pool.npz``);
``tests/test_pool_oracle.py`` replays those traces through this file.
"""
from __future__ import annotations

import numpy as np


def alloc_ref(mem_state: np.ndarray, need: int):
    """Returns (rows handed out, new free map).  ``mem_state``: bool / uint8, non-zero = free."""
    free = mem_state.astype(bool)
    running = np.cumsum(free.astype(np.int64))
    take = (running > 0) & (running <= need) & free
    rows = np.nonzero(take)[0].astype(np.int64)
    after = free.copy()
    after[rows] = False
    return rows, after


def free_ref(mem_state: np.ndarray, rows: np.ndarray):
    after = mem_state.astype(bool).copy()
    after[np.asarray(rows, dtype=np.int64)] = True
    return after


def compact_ref(a_start, a_len, a_loc, a_scaling, keep, mem_state=None):
    """Returns (new_start, new_len, new_loc, new_scaling, new free map or None)."""
    a_start = np.asarray(a_start, dtype=np.int64)
    a_len = np.asarray(a_len, dtype=np.int64)
    a_loc = np.asarray(a_loc, dtype=np.int64)
    keep = np.asarray(keep).astype(bool)
    left = np.nonzero(keep)[0]
    new_len = a_len[left]
    new_start = np.zeros(len(left), dtype=np.int64)
    if len(left) > 1:
        new_start[1:] = np.cumsum(new_len)[:-1]
    new_loc = np.empty(int(new_len.sum()), dtype=np.int64)
    for k, i in enumerate(left):                        # the variable-length copy, one run per kept adapter
        new_loc[new_start[k]: new_start[k] + new_len[k]] = a_loc[a_start[i]: a_start[i] + a_len[i]]
    new_scaling = np.asarray(a_scaling)[left]
    after = None
    if mem_state is not None:
        after = mem_state.astype(bool).copy()
        for i in np.nonzero(~keep)[0]:
            after[a_loc[a_start[i]: a_start[i] + a_len[i]]] = True
    return new_start, new_len, new_loc, new_scaling, after
