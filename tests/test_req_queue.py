"""The request queues (batch composition in front of the LoRA path) against decisions recorded from the reference's
own ReqQueue / ClusterReqQueue (tests/golden/ref_queue.json, made by tests/golden/make_queue_golden.py)."""
import importlib.util
import json
import os

import pytest

from slora_b200.req_queue import Batch, ClusterReqQueue, Req, ReqQueue, order_by_adapter
from tests.helpers import ROOT

GDIR = os.path.join(ROOT, "tests", "golden")


def _gen():
    spec = importlib.util.spec_from_file_location("make_queue_golden", os.path.join(GDIR, "make_queue_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _merge(running, new):
    if running is None:
        return new
    running.merge(new)
    return running


@pytest.mark.parametrize("name", ["fifo_small_pool", "cluster_4", "cluster_16_tight", "cluster_1"])
def test_same_admission_decisions_as_the_reference_queues(name):
    mod = _gen()
    golden = json.load(open(os.path.join(GDIR, "ref_queue.json")))[name]
    got = mod.simulate(lambda kind, qa: ReqQueue(**qa) if kind == "fifo" else ClusterReqQueue(**qa),
                       lambda a, k, n_in, n_out: Req(a, k, n_in, n_out), _merge, mod.SCENARIOS[name])
    assert len(got) == len(golden)
    for step, (g, w) in enumerate(zip(got, golden)):
        assert g == w, f"{name}: call {step}"
    assert sum(1 for d in golden if d) >= 10


def test_clustering_cuts_the_adapters_a_batch_touches():
    """Same request stream, arrival order against clustering at 4 adapters: fewer distinct adapters per running batch
    (each one costs the LoRA kernels its rows once per layer and projection)."""
    mod = _gen()
    kind, qargs, n_adapters, alpha, count, per_step, _, seed = mod.SCENARIOS["cluster_4"]
    seen = {}
    for label, make in (("fifo", lambda k, qa: ReqQueue(qa["max_total_tokens"], qa["batch_max_tokens"],
                                                          qa["running_max_req_size"])),
                        ("cluster", lambda k, qa: ClusterReqQueue(**qa))):
        sizes = []

        def merge(running, new):
            out = _merge(running, new)
            sizes.append(len(out.adapter_dirs) / len(out.reqs))
            return out
        mod.simulate(make, lambda a, k, n_in, n_out: Req(a, k, n_in, n_out), merge,
                     (kind, qargs, n_adapters, alpha, count, per_step, 0.0, seed))
        seen[label] = sum(sizes) / len(sizes)
    assert seen["cluster"] < seen["fifo"]


def test_order_by_adapter_groups_requests_and_keeps_arrival_order_inside_a_group():
    reqs = [Req(a, i, 8, 8) for i, a in enumerate(["b", "a", None, "b", "a", "c"])]
    out = order_by_adapter(reqs)
    assert [r.adapter_dir for r in out] == [None, "a", "a", "b", "b", "c"]
    assert [r.request_id for r in out] == [2, 1, 4, 0, 3, 5]
    assert [d["adapter_dir"] for d in order_by_adapter([{"adapter_dir": "z"}, {"adapter_dir": "y"}])] == ["y", "z"]
    b = Batch("x", reqs[:3])
    assert b.adapter_dirs == {"a", "b", None} and b.input_tokens() == 24
