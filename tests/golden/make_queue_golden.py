"""Golden admission decisions of the reference's request queues.

    SLORA_REFERENCE=/path/to/S-LoRA  python tests/golden/make_queue_golden.py

Drives the reference's own ``ReqQueue`` (``slora/server/router/req_queue.py``) and ``ClusterReqQueue``
(``slora/server/router/cluster_req_queue.py``), imported unmodified from the reference tree, through seeded serving
loops and stores which requests every ``generate_new_batch`` call admitted (``tests/golden/ref_queue.json``).
``tests/test_req_queue.py`` drives ``slora_b200.req_queue`` through the same loops (``simulate`` below is shared) and
demands the same decisions, call for call.

The loop stands in for the router (``slora/server/router/manager.py:177-253``): requests arrive, the queue is asked for
a new batch given the running one, the new batch joins the running one, every running request produces a token and
leaves when it has produced ``max_new_tokens``; now and then a waiting request is aborted.  Request streams follow the
reference's trace generator (``benchmarks/trace.py:33-61``): adapter ``floor(power(alpha) * n)``, input and output
lengths uniform in [8, 512).
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (queue kind, constructor arguments, adapters, power-law alpha, requests, arrivals per step, abort rate, seed)
SCENARIOS = {
    "fifo_small_pool": ("fifo", dict(max_total_tokens=14000, batch_max_tokens=2048, running_max_req_size=24),
                        20, 1.0, 120, 3, 0.05, 1),
    "cluster_4": ("cluster", dict(max_total_tokens=20000, batch_max_tokens=4096, running_max_req_size=48,
                                  batch_num_adapters=4), 40, 0.8, 200, 4, 0.04, 2),
    "cluster_16_tight": ("cluster", dict(max_total_tokens=24000, batch_max_tokens=1536, running_max_req_size=64,
                                         batch_num_adapters=16), 100, 0.3, 240, 6, 0.08, 3),
    "cluster_1": ("cluster", dict(max_total_tokens=30000, batch_max_tokens=8192, running_max_req_size=32,
                                  batch_num_adapters=1), 8, 1.0, 100, 2, 0.0, 4),
}


def draw_requests(n_adapters, alpha, count, seed):
    rng = np.random.default_rng(seed)
    ranks = {f"a{i}": int(rng.choice([8, 16, 32, 64])) for i in range(n_adapters)}
    reqs = []
    for k in range(count):
        a = int(np.floor(rng.power(alpha) * n_adapters))
        reqs.append((f"a{a}", k, int(rng.integers(8, 512)), int(rng.integers(8, 512))))
    return ranks, reqs, rng


def simulate(make_queue, make_req, make_batch_merge, scenario):
    """Runs one scenario; returns the list of decisions: per generate_new_batch call the admitted request numbers
    (or None).  ``make_req(adapter, number, input_len, max_new_tokens)`` builds a request object,
    ``make_batch_merge(running, new)`` merges a new batch into the running one and returns it."""
    kind, qargs, n_adapters, alpha, count, per_step, abort_rate, seed = scenario
    ranks, stream, rng = draw_requests(n_adapters, alpha, count, seed)
    q = make_queue(kind, qargs)
    running, decisions, nxt = None, [], 0
    for step in range(4000):
        for _ in range(per_step):
            if nxt < len(stream):
                q.append(make_req(*stream[nxt]))
                nxt += 1
        for r in q.waiting_req_list:                      # the client went away before the request was scheduled
            if rng.random() < abort_rate:
                r.aborted = True
        new = q.generate_new_batch(running, ranks)
        decisions.append(None if new is None else [r.request_id for r in new.reqs])
        if new is not None:
            running = make_batch_merge(running, new)
        if running is not None:
            for r in running.reqs:                        # one decode step
                r.output_ids.append(0)
                if len(r.output_ids) >= r.max_output_len:
                    r.has_generate_finished = True
            running.filter_finished()
            if running.is_clear():
                running = None
        if nxt >= len(stream) and running is None and not any(not r.aborted for r in q.waiting_req_list):
            break
    return decisions


def main():
    ref = os.environ.get("SLORA_REFERENCE")
    if not ref or not os.path.isdir(os.path.join(ref, "slora")):
        raise SystemExit("set SLORA_REFERENCE to the root of the S-LoRA reference tree")
    sys.path.insert(0, ref)
    from slora.server.io_struct import Req
    from slora.server.router.cluster_req_queue import ClusterReqQueue
    from slora.server.router.req_queue import ReqQueue
    from slora.server.sampling_params import SamplingParams

    def make_queue(kind, qargs):
        return ReqQueue(**qargs) if kind == "fifo" else ClusterReqQueue(**qargs)

    def make_req(adapter, number, input_len, max_new):
        return Req(adapter, number, [0] * input_len, SamplingParams(max_new_tokens=max_new))

    def merge(running, new):
        if running is None:
            return new
        running.merge(new)
        return running

    out = {name: simulate(make_queue, make_req, merge, sc) for name, sc in SCENARIOS.items()}
    with open(os.path.join(HERE, "ref_queue.json"), "w") as f:
        json.dump(out, f)
    print({k: (len(v), sum(1 for d in v if d)) for k, v in out.items()})


if __name__ == "__main__":
    main()
