"""Replay of the golden pool traces (``tests/golden/ref_pool.npz``: what the reference's own ``MemoryAllocator`` and
``InferAdapter`` left behind after every step of two seeded sequences, see ``tests/golden/make_pool_golden.py``)
through this repository's allocator and adapter tables on a given device, and through the numpy oracle."""
import importlib.util
import json
import os

import numpy as np
import pytest
import torch

from tests.helpers import ROOT

GDIR = os.path.join(ROOT, "tests", "golden")


def load_golden():
    spec = importlib.util.spec_from_file_location("make_pool_golden", os.path.join(GDIR, "make_pool_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    arrays = np.load(os.path.join(GDIR, "ref_pool.npz"))
    meta = json.load(open(os.path.join(GDIR, "ref_pool.json")))["traces"]
    return mod, arrays, meta


def _refused(step):
    return isinstance(step[-1], str) and step[-1].startswith("raised")


def replay_host_mirror(name, device):
    """Every step through ``slora_b200.MemoryAllocator`` / ``InferAdapter`` on ``device``; bit-exact state after each."""
    import slora_b200 as sl
    mod, g, meta = load_golden()
    m = meta[name]
    tot, layers, heads, hd, ranks, seed = m["tot"], m["layers"], m["heads"], m["head_dim"], m["ranks"], m["seed"]
    ads = [mod._Adapter(f"a{i}", r, heads, hd, layers, 1000 * seed + i) for i, r in enumerate(ranks)]
    mm = sl.MemoryAllocator(tot, 0, torch.float16, heads, hd, layers, device=device)
    for l in range(layers):
        mm.key_buffer[l].fill_(3.0)
        mm.value_buffer[l].fill_(5.0)
    ia = sl.InferAdapter.init(mm, None)
    held = []
    for k, step in enumerate(m["steps"]):
        kind, want_rows = step[0], g[f"{name}_s{k}_rows"]
        ctx = pytest.raises(Exception) if _refused(step) else _Null()
        rows = None
        with ctx:
            if kind in ("load", "prefetch"):
                ia.load_adapters([ads[i] for i in step[1]], prefetch=(kind == "prefetch"))
            elif kind == "offload":
                ia.offload_adapters([f"a{i}" for i in step[1]])
            elif kind == "alloc":
                got = mm.alloc(step[1])
                held.append(got)
                rows = got.cpu().numpy()
            elif kind == "free":
                got = held[step[1]]
                part = got[: int(len(got) * step[2])]
                held[step[1]] = got[len(part):]
                mm.free(part.contiguous())
                rows = part.cpu().numpy()
            else:
                got = mm.alloc_contiguous(step[1])
                if got is None:
                    rows = np.array([-1], dtype=np.int64)
                    held.append(torch.empty(0, dtype=torch.long, device=device))
                else:
                    held.append(got[0])
                    rows = np.array([got[1], got[2]], dtype=np.int64)
        if _refused(step) and kind in ("alloc", "alloc_contiguous"):
            held.append(torch.empty(0, dtype=torch.long, device=device))
        if device != "cpu":
            torch.cuda.synchronize()
        what = f"{name} step {k} {step[:2]}"
        if rows is not None and not _refused(step):
            assert np.array_equal(rows, want_rows), what
        assert np.array_equal(mm.mem_state.cpu().numpy().astype(np.uint8), g[f"{name}_s{k}_mem_state"]), what
        assert mm.can_use_mem_size == int(g[f"{name}_s{k}_free"][0]), what
        assert np.array_equal(ia.a_loc.cpu().numpy(), g[f"{name}_s{k}_a_loc"]), what
        assert np.array_equal(ia.a_start.cpu().numpy(), g[f"{name}_s{k}_a_start"]), what
        assert np.array_equal(ia.a_len.cpu().numpy(), g[f"{name}_s{k}_a_len"]), what
        assert np.array_equal(ia.a_scaling.cpu().numpy(), g[f"{name}_s{k}_a_scaling"]), what
        assert [int(d[1:]) for d in ia.adapter_dirs] == g[f"{name}_s{k}_dirs"].tolist(), what
        if getattr(mm, "status", None) is not None:
            assert int(mm.status.item()) == 0, what
    for l in range(layers):
        assert np.array_equal(mm.key_buffer[l].reshape(tot, -1).cpu().numpy(), g[f"{name}_key_l{l}"]), f"{name} key {l}"
        assert np.array_equal(mm.value_buffer[l].reshape(tot, -1).cpu().numpy(), g[f"{name}_value_l{l}"]), f"{name} value {l}"
    return len(m["steps"])


def replay_oracle(name):
    """The numpy oracle step by step: each golden state is derived from the golden state before it."""
    from oracle import pool_oracle as porc
    _, g, meta = load_golden()
    m = meta[name]
    tot, ranks = m["tot"], m["ranks"]
    state = np.ones(tot, dtype=bool)
    tabs = (np.empty(0, np.int64), np.empty(0, np.int64), np.empty(0, np.int64), np.empty(0, np.float16))
    dirs, checked = [], 0
    for k, step in enumerate(m["steps"]):
        kind = step[0]
        after = g[f"{name}_s{k}_mem_state"].astype(bool)
        new_dirs = g[f"{name}_s{k}_dirs"].tolist()
        new_tabs = tuple(g[f"{name}_s{k}_{t}"] for t in ("a_start", "a_len", "a_loc", "a_scaling"))
        if not _refused(step):
            if kind == "alloc":
                rows, want = porc.alloc_ref(state, step[1])
                assert np.array_equal(rows, g[f"{name}_s{k}_rows"]) and np.array_equal(want, after), (name, k)
                checked += 1
            elif kind == "free":
                assert np.array_equal(porc.free_ref(state, g[f"{name}_s{k}_rows"]), after), (name, k)
                checked += 1
            elif kind in ("load", "prefetch"):
                # the rows of the newly resident adapters are the first free rows, in order
                fresh = [i for i in new_dirs if i not in dirs]
                rows, want = porc.alloc_ref(state, sum(4 * ranks[i] for i in fresh))
                assert np.array_equal(want, after), (name, k)
                assert np.array_equal(new_tabs[2][len(tabs[2]):], rows), (name, k)
                checked += 1
            elif kind == "offload" and new_dirs != dirs:
                keep = np.array([d in new_dirs for d in dirs], dtype=np.uint8)
                ns, nl, nloc, nsc, want = porc.compact_ref(tabs[0], tabs[1], tabs[2], tabs[3], keep, state)
                assert np.array_equal(ns, new_tabs[0]) and np.array_equal(nl, new_tabs[1]), (name, k)
                assert np.array_equal(nloc, new_tabs[2]) and np.array_equal(nsc, new_tabs[3]), (name, k)
                assert np.array_equal(want, after), (name, k)
                checked += 1
        state, tabs, dirs = after, new_tabs, new_dirs
    return checked


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
