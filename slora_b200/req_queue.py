"""Batch composition in front of the LoRA path: which waiting requests join the running batch.

The size of the same-adapter groups in a batch decides what the shrink / expand kernels have to stream: every
distinct adapter of a batch costs its rows once (``2 * r * (h_in + h_out)`` bytes per projection and layer), however
many tokens share it, and groups of 128 tokens or more run on the tensor cores.  The reference's scheduler has a hook
for this, ``ClusterReqQueue`` (``slora/server/router/cluster_req_queue.py:10-89``): once the running batch holds
``batch_num_adapters`` adapters, waiting requests that use one of those adapters are admitted first, then the queue
falls back to arrival order.  This module provides that queue and the plain arrival-order queue it extends
(``slora/server/router/req_queue.py:9-104``) with the same interface and the same decisions, request for request
(``tests/test_req_queue.py`` replays traces recorded from the reference's own classes), plus the ordering hook the
reference leaves commented out (``slora/server/router/model_infer/infer_batch.py:77-78``).

Mechanism differs: the reference re-sorts and re-sums the whole running set with numpy for every candidate
(``req_queue.py:39-58``); here the set is kept sorted by insertion and the peak is one pass over it.

The admission test (``_can_add_new_req``): with the running requests sorted by the tokens they may still produce,
longest first, request ``i`` (0-based) finishing last among the first ``i + 1`` needs
``left_i * (i + 1) + sum_{j<=i} held_j`` cache rows at its peak; the largest of those must stay below the pool size
minus the rows of the batch's adapters (``4 * r`` per distinct adapter).
"""
from __future__ import annotations

import bisect
import uuid
from typing import Dict, Iterable, List, Optional


class Req:
    """What the queues read of a request (``slora/server/io_struct.py:6-17``)."""

    def __init__(self, adapter_dir, request_id, input_len, max_output_len):
        self.adapter_dir = adapter_dir
        self.request_id = request_id
        self.input_len = int(input_len)
        self.max_output_len = int(max_output_len)
        self.output_ids: List[int] = []
        self.has_generate_finished = False
        self.aborted = False


class Batch:
    """Running or newly formed batch (``slora/server/io_struct.py:66-128``): requests and the set of their adapters."""

    def __init__(self, batch_id, reqs: List[Req]):
        self.batch_id = batch_id
        self.reqs = list(reqs)
        self._reindex()

    def _reindex(self):
        self.id_to_reqs = {r.request_id: r for r in self.reqs}
        self.adapter_dirs = {r.adapter_dir for r in self.reqs}

    def input_tokens(self):
        return sum(r.input_len for r in self.reqs)

    def merge(self, mini_batch: "Batch"):
        self.reqs.extend(mini_batch.reqs)
        self._reindex()

    def filter_finished(self):
        self.reqs = [r for r in self.reqs if not r.has_generate_finished]
        self._reindex()

    def is_clear(self):
        return not self.reqs


class _CacheBudget:
    """Peak cache rows of a set of running requests, kept sorted by remaining output length (longest first; equal
    lengths in insertion order, as a stable re-sort after every append leaves them)."""

    def __init__(self):
        self.neg_left: List[int] = []   # sort keys: minus the tokens a request may still produce
        self.held: List[int] = []       # cache rows the request holds now (after this step)
        self.adapters = set()
        self.adapter_rows = 0

    def add(self, held, left, adapter_dir, lora_ranks):
        at = bisect.bisect_right(self.neg_left, -left)
        self.neg_left.insert(at, -left)
        self.held.insert(at, held)
        if adapter_dir not in self.adapters:
            self.adapter_rows += lora_ranks[adapter_dir] * 4
            self.adapters.add(adapter_dir)

    def peak(self):
        best, run = None, 0
        for i, (nl, h) in enumerate(zip(self.neg_left, self.held)):
            run += h
            need = -nl * (i + 1) + run
            if best is None or need > best:
                best = need
        return best

    def __len__(self):
        return len(self.held)


class ReqQueue:
    """Arrival-order admission (``req_queue.py:9-104``)."""

    def __init__(self, max_total_tokens, batch_max_tokens, running_max_req_size) -> None:
        assert batch_max_tokens is not None
        self.max_total_tokens = max_total_tokens
        self.batch_max_tokens = batch_max_tokens
        self.running_max_req_size = running_max_req_size
        self.waiting_req_list: List[Req] = []
        self._budget = _CacheBudget()

    def append(self, req):
        self.waiting_req_list.append(req)

    def update_counter(self, req):
        pass

    def _init_cache_list(self, current_batch: Optional[Batch], lora_ranks):
        self._budget = _CacheBudget()
        if current_batch is not None:
            for r in current_batch.reqs:
                self._budget.add(r.input_len + len(r.output_ids), r.max_output_len - len(r.output_ids) - 1,
                                 r.adapter_dir, lora_ranks)

    def _can_add_new_req(self, req, lora_ranks):
        # the candidate stays in the set whatever the answer: later candidates of the same call are judged with it
        # there, exactly as the reference does (req_queue.py:40-44 appends before it decides)
        self._budget.add(req.input_len + 1, req.max_output_len - 1, req.adapter_dir, lora_ranks)
        return (self._budget.peak() < self.max_total_tokens - self._budget.adapter_rows and
                len(self._budget) <= self.running_max_req_size)

    def _admit(self, candidates: Iterable[Req], lora_ranks, taken: List[Req], tokens: int):
        """Walk ``candidates`` in order: aborted ones are passed over (and reported), the others are taken until the
        first that does not fit.  Returns (token total, passed-over aborted requests)."""
        aborted = []
        for req in candidates:
            if req.aborted:
                aborted.append(req)
                continue
            if self._can_add_new_req(req, lora_ranks) and tokens + req.input_len <= self.batch_max_tokens:
                taken.append(req)
                tokens += req.input_len
            else:
                break
        return tokens, aborted

    def generate_new_batch(self, current_batch: Optional[Batch], lora_ranks: Dict[str, int]):
        if current_batch is not None and len(current_batch.reqs) >= self.running_max_req_size:
            return None
        self._init_cache_list(current_batch, lora_ranks)
        taken: List[Req] = []
        _, aborted = self._admit(self.waiting_req_list, lora_ranks, taken, 0)
        if not taken:
            return None
        self.waiting_req_list = self.waiting_req_list[len(taken) + len(aborted):]
        return Batch(uuid.uuid4().hex, taken)

    def next_batch(self):
        taken, tokens = [], 0
        for req in self.waiting_req_list:
            if req.aborted:
                continue
            if tokens + req.input_len > self.batch_max_tokens:
                break
            taken.append(req)
            tokens += req.input_len
        return Batch(uuid.uuid4().hex, taken) if taken else None


class ClusterReqQueue(ReqQueue):
    """Admission that keeps the number of distinct adapters in the running batch down
    (``cluster_req_queue.py:10-89``): while the running batch holds fewer than ``batch_num_adapters`` adapters it is
    the arrival-order queue; from then on waiting requests whose adapter is already in the batch go first."""

    def __init__(self, max_total_tokens, batch_max_tokens, running_max_req_size, batch_num_adapters) -> None:
        super().__init__(max_total_tokens, batch_max_tokens, running_max_req_size)
        self.batch_num_adapters = batch_num_adapters

    def generate_new_batch(self, current_batch: Optional[Batch], lora_ranks: Dict[str, int]):
        clustered = current_batch is not None and len(current_batch.adapter_dirs) >= self.batch_num_adapters
        if not clustered:
            return super().generate_new_batch(current_batch, lora_ranks)
        if len(current_batch.reqs) >= self.running_max_req_size:
            return None
        live = next((i for i, r in enumerate(self.waiting_req_list) if not r.aborted), None)
        if live is None:
            return None           # nothing but aborted requests waiting: they stay where they are
        self._init_cache_list(current_batch, lora_ranks)
        # aborted requests ahead of the first live one leave the queue here
        self.waiting_req_list = self.waiting_req_list[live:]
        taken: List[Req] = []
        # first the requests that bring no new adapter, in arrival order, up to the first that does not fit ...
        same = [r for r in self.waiting_req_list if r.adapter_dir in current_batch.adapter_dirs]
        tokens, aborted = self._admit(same, lora_ranks, taken, 0)
        gone = {id(r) for r in taken} | {id(r) for r in aborted}
        self.waiting_req_list = [r for r in self.waiting_req_list if id(r) not in gone]
        # ... then whoever is next in line
        first_pass = len(taken)
        _, aborted = self._admit(self.waiting_req_list, lora_ranks, taken, tokens)
        gone = {id(r) for r in taken[first_pass:]} | {id(r) for r in aborted}
        self.waiting_req_list = [r for r in self.waiting_req_list if id(r) not in gone]
        return Batch(uuid.uuid4().hex, taken) if taken else None


def order_by_adapter(requests: List, key="adapter_dir"):
    """The ordering hook of ``infer_batch.py:77-78`` (commented out there): requests of one adapter next to each
    other, otherwise in arrival order.  ``requests`` are objects with an ``adapter_dir`` attribute or dicts with that
    key.  With this library the order is a matter of locality only: the batch plan groups tokens by adapter whatever
    order they arrive in."""
    def k(r):
        v = r[key] if isinstance(r, dict) else getattr(r, key)
        return "" if v is None else v
    return sorted(requests, key=k)
