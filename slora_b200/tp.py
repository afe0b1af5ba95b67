"""S-LoRA tensor parallelism for the adapter path (one process per GPU, ``torch.distributed``).

The reference describes the scheme only as a figure (``figures/slora_tp.png``, ``README.md:96-100``); its code asserts
``world_size == 1`` for adapters (``slora/models/peft/lora_adapter.py:24``) and has the LoRA all-reduce commented out
(``slora/models/peft/lora_unordered_batch_infer.py:223-224,247-248``).  What is built here is the rule of that figure
for a column-parallel projection, applied to q, k, v and o with replicated activations:

* A is sharded over the rank dimension: GPU ``g`` owns rank rows ``[g*r/N, (g+1)*r/N)`` of every adapter (full
  ``h_in`` each) and computes ``delta_g[T, r/N]``;
* the small intermediates are all-gathered (one collective per call: q, k and v travel together) into
  ``[N, nproj, T, R/N]``;
* B is sharded over the output dimension (rows of its stored ``[h_out, r]`` layout): GPU ``g`` owns outputs
  ``[g*h_out/N, (g+1)*h_out/N)`` and adds ``scale * delta @ B_g^T`` into its ``[T, h_out/N]`` slice of the base
  model's column-parallel output -- for o that slice lands in the partial sum the base model all-reduces anyway.

Per-rank pool layout: rows of ``pool_stride`` elements; an adapter of rank ``r`` takes ``4 * r / N`` rows per buffer
(slot of ``r/N`` rows per projection): the A shard is ``[r/N, h_in]`` and the B shard ``[h_out/N, r]``, both row-major
in the slot's flat space (``h_in == pool_stride``; ``h_out/N * r <= r/N * pool_stride``).  The kernels read the B shard
with ``rank_mult = N`` and the gathered delta with ``delta_parts = N``.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import List, Sequence

import torch


def shard_adapter(A: Sequence[torch.Tensor], B: Sequence[torch.Tensor], rank: int, world: int, pool_stride: int,
                  o_input_sharded: bool = False):
    """Rows one adapter contributes to rank ``rank``'s A pool and B pool.

    ``A[p]``: ``[r, h_in]``, ``B[p]``: ``[h_out_p, r]`` for p = q, k, v, o.  Returns ``(rows_a, rows_b)``, each
    ``[4 * r / world, pool_stride]``.  With ``o_input_sharded`` the o projection's A is cut over its INPUT columns
    instead of its rank rows (the attention output arrives head-sharded): the slot then holds ``A_o[:, g*h/N:(g+1)*h/N]``
    (``[r, h_in / world]``) flat, and the ranks' partial results are summed (see :meth:`TpLoraOps.lora_o_sharded`).
    """
    r = A[0].shape[0]
    if r % world != 0:
        raise ValueError(f"rank {r} is not divisible by the tensor-parallel size {world}")
    rs = r // world
    rows_a, rows_b = [], []
    for p in range(4):
        h_in, h_out = A[p].shape[1], B[p].shape[0]
        if h_in != pool_stride:
            raise ValueError("the A shard needs pool_stride == h_in")
        if h_out % world != 0:
            raise ValueError(f"h_out {h_out} is not divisible by the tensor-parallel size {world}")
        if p == 3 and o_input_sharded:
            if h_in % world != 0:
                raise ValueError(f"h_in {h_in} is not divisible by the tensor-parallel size {world}")
            hs = h_in // world
            rows_a.append(A[p][:, rank * hs:(rank + 1) * hs].reshape(rs, pool_stride))
        else:
            rows_a.append(A[p][rank * rs:(rank + 1) * rs])
        ho = h_out // world
        flat = B[p][rank * ho:(rank + 1) * ho].reshape(-1)
        if flat.numel() > rs * pool_stride:
            raise ValueError("the B shard does not fit its slot")
        slot = torch.zeros(rs * pool_stride, dtype=flat.dtype)
        slot[:flat.numel()] = flat
        rows_b.append(slot.view(rs, pool_stride))
    return torch.cat(rows_a), torch.cat(rows_b)


@dataclass
class TpTables:
    """Per-rank index tables (same meaning as InferAdapter's, with ``a_len = 4 * r / N``)."""
    a_start: torch.Tensor
    a_len: torch.Tensor
    a_loc: torch.Tensor
    a_scaling: torch.Tensor


class PeerExchange:
    """Symmetric-memory buffers of the exchange over peer memory (C entry ``slora_tp_exchange``).

    Every rank owns a delta buffer ``[2, 3, T, R]`` and a flag array ``[2, N]`` that all ranks can address over
    NVLink (``torch.distributed._symmetric_memory``).  One small kernel per exchange writes this rank's columns into
    every rank's buffer, raises its flag everywhere and waits for everybody's flag: it stands where
    ``all_gather_into_tensor`` + regroup stand otherwise.
    """

    def __init__(self, T, R, world, rank, dtype, device, group=None, inband=True):
        import ctypes
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.world, self.rank = world, rank
        # two halves (q,k,v calls / o calls), or three parts that rotate with the exchange's number (inband == 3)
        self.full = symm_mem.empty((3 if inband == 3 else 2, 3, max(T, 1), R), dtype=dtype, device=device)
        self.flags = symm_mem.empty((2, world), dtype=torch.int32, device=device)
        self.parts = symm_mem.empty((world, max(T, 1), R), dtype=dtype, device=device)  # partial sums of the o shrink
        # in-band signalling of the fused exchange: an element that has not arrived yet is the bit pattern 0xffff
        self.inband = inband
        if inband:
            self.full.view(torch.int16).fill_(-1)
        else:
            self.full.zero_()
        self.flags.zero_()
        self.parts.zero_()
        h_full = symm_mem.rendezvous(self.full, group.group_name)
        h_flags = symm_mem.rendezvous(self.flags, group.group_name)
        h_parts = symm_mem.rendezvous(self.parts, group.group_name)
        self.full_ptrs = (ctypes.c_void_p * world)(*[int(p) for p in h_full.buffer_ptrs])
        self.flag_ptrs = (ctypes.c_void_p * world)(*[int(p) for p in h_flags.buffer_ptrs])
        self.parts_ptrs = (ctypes.c_void_p * world)(*[int(p) for p in h_parts.buffer_ptrs])
        self._handles = (h_full, h_flags, h_parts)
        self.counter = torch.zeros(4, dtype=torch.int32, device=device)   # one arrival counter per entry point
        self.seq_state = torch.zeros(2, dtype=torch.int32, device=device)   # exchanges done per half (device-kept)
        # rotating thirds: [0] the next exchange's number (read by its shrink), [1] left by a shrink for its expand
        self.inband_seq = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)   # nobody signals before everybody's flags are zero


class TpLoraOps:
    """Per-rank LoRA operator under S-LoRA tensor parallelism.

    ``backend`` supplies the two local operations (the CUDA kernels in production, see :class:`CudaBackend`);
    ``group`` is the ``torch.distributed`` process group of the N ranks.  ``max_rank`` is the full (unsharded) maximum
    rank of the batch's adapters.
    """

    def __init__(self, tables: TpTables, pools_a: List[torch.Tensor], pools_b: List[torch.Tensor], max_rank: int,
                 world: int, rank: int, backend, group=None, peer_exchange: bool = False):
        if max_rank % world != 0:
            raise ValueError("max_rank must be divisible by the tensor-parallel size")
        self.t, self.pools_a, self.pools_b = tables, pools_a, pools_b
        self.R, self.N, self.rank = max_rank, world, rank
        self.Rl = max_rank // world
        self.backend, self.group = backend, group
        self.peer_exchange = peer_exchange and world > 1 and hasattr(backend, "exchange")
        self.px = None
        self.sum_in = self.sum_out = None
        self.ids = None

    def prepare(self, token_adapter_ids: torch.Tensor):
        self.ids = token_adapter_ids.contiguous()
        T = self.ids.numel()
        dev, dt = self.ids.device, self.pools_a[0].dtype
        self.local = torch.zeros((3, T, self.Rl), dtype=dt, device=dev)
        self.gathered = torch.zeros((self.N, 3, T, self.Rl), dtype=dt, device=dev)
        # plain [nproj, T, R] delta rows for backends that regroup the gathered intermediates (see lora_qkv)
        self.full = torch.zeros((3, T, self.R), dtype=dt, device=dev) if hasattr(self.backend, "regroup") else None
        self.plan = self.backend.make_plan(self.ids, self.t, self.R // self.N)
        if self.peer_exchange and (self.px is None or self.px.full.shape[2] < T):
            fused = getattr(self.backend, "fused", False)
            self.px = PeerExchange(T, self.R, self.N, self.rank, dt, dev, self.group,
                                   inband=fused and getattr(self.backend, "inband", True))
        return self

    def _exchange(self, nproj):
        """All-gather of the rank-sharded intermediates: ``[nproj, T, R/N]`` per rank -> ``[N, 3, T, R/N]``."""
        import torch.distributed as dist
        if nproj == 3:
            dist.all_gather_into_tensor(self.gathered.view(-1), self.local.view(-1), group=self.group)
        else:
            # o uses slot 0 only: gather that slab ([T, R/N] per rank) into a contiguous staging view
            stage = self.gathered.view(-1)[: self.N * self.local[0].numel()].view(self.N, *self.local[0].shape)
            dist.all_gather_into_tensor(stage.view(-1), self.local[0].contiguous().view(-1), group=self.group)
            return stage, self.local[0].numel()
        return self.gathered, self.local.numel()

    def lora_qkv(self, layer, x, q_g, k_g, v_g):
        """``q_g/k_g/v_g``: this rank's ``[T, h_out/N]`` slices, updated in place."""
        t = self.t
        if self.px is not None and getattr(self.backend, "fused", False):
            # no launch for the exchange: the shrink writes into every rank's buffer, the expand waits for the flags
            self.backend.shrink_push(self.px, self.plan, self.ids, [0, 1, 2], x, self.pools_a[layer], t, self.Rl, 0)
            self.backend.expand_wait(self.px, self.plan, self.ids, [0, 1, 2], [q_g, k_g, v_g], self.pools_b[layer], t,
                                     self.Rl, 0)
            return
        if self.px is not None:
            self.backend.shrink(self.plan, self.ids, [0, 1, 2], [self.local[0], self.local[1], self.local[2]], x,
                                self.pools_a[layer], t)
            full = self.backend.exchange(self.px, self.plan, self.local, self.ids, t, 3, self.Rl, half=0)
            self.backend.expand(self.plan, self.ids, [0, 1, 2], [q_g, k_g, v_g], [full[p] for p in range(3)],
                                self.pools_b[layer], t, delta_stride=self.R, delta_width=self.R, delta_parts=1,
                                delta_part_stride=0, rank_mult=self.N)
            return
        self.backend.shrink(self.plan, self.ids, [0, 1, 2], [self.local[0], self.local[1], self.local[2]], x,
                            self.pools_a[layer], t)
        gathered, part_stride = self._exchange(3)
        if self.full is not None:
            # regroup once, then the expand reads ordinary delta rows (and may use the pipelined kernels)
            self.backend.regroup(self.full, gathered, self.ids, t, self.N, 3, self.Rl, part_stride)
            self.backend.expand(self.plan, self.ids, [0, 1, 2], [q_g, k_g, v_g], [self.full[p] for p in range(3)],
                                self.pools_b[layer], t, delta_stride=self.R, delta_width=self.R, delta_parts=1,
                                delta_part_stride=0, rank_mult=self.N)
            return
        deltas = [gathered[0, p] for p in range(3)]
        self.backend.expand(self.plan, self.ids, [0, 1, 2], [q_g, k_g, v_g], deltas, self.pools_b[layer], t,
                            delta_stride=self.Rl, delta_width=self.Rl, delta_parts=self.N,
                            delta_part_stride=part_stride, rank_mult=self.N)

    def lora_o(self, layer, x, o_g):
        t = self.t
        if self.px is not None and getattr(self.backend, "fused", False):
            self.backend.shrink_push(self.px, self.plan, self.ids, [3], x, self.pools_a[layer], t, self.Rl, 1)
            self.backend.expand_wait(self.px, self.plan, self.ids, [3], [o_g], self.pools_b[layer], t, self.Rl, 1)
            return
        self.backend.shrink(self.plan, self.ids, [3], [self.local[0]], x, self.pools_a[layer], t)
        if self.px is not None:
            full = self.backend.exchange(self.px, self.plan, self.local, self.ids, t, 1, self.Rl, half=1)
            self.backend.expand(self.plan, self.ids, [3], [o_g], [full[0]], self.pools_b[layer], t,
                                delta_stride=self.R, delta_width=self.R, delta_parts=1, delta_part_stride=0,
                                rank_mult=self.N)
            return
        stage, part_stride = self._exchange(1)
        if self.full is not None:
            self.backend.regroup(self.full, stage, self.ids, t, self.N, 1, self.Rl, part_stride)
            self.backend.expand(self.plan, self.ids, [3], [o_g], [self.full[0]], self.pools_b[layer], t,
                                delta_stride=self.R, delta_width=self.R, delta_parts=1, delta_part_stride=0,
                                rank_mult=self.N)
            return
        self.backend.expand(self.plan, self.ids, [3], [o_g], [stage[0]], self.pools_b[layer], t,
                            delta_stride=self.Rl, delta_width=self.Rl, delta_parts=self.N,
                            delta_part_stride=part_stride, rank_mult=self.N)


    def lora_o_sharded(self, layer, x_g, o_g):
        """The o projection with a head-sharded input: ``x_g`` is this rank's ``[T, h_in / N]`` slice of the attention
        output, the adapters were sharded with ``o_input_sharded=True``.  Every rank computes a partial ``[T, R]``
        (all rank rows, its input columns), the partials are summed over the ranks (peer memory, or ``all_reduce``),
        and the output-sharded B gives this rank's ``[T, h_out / N]`` slice as in :meth:`lora_o`."""
        import torch.distributed as dist
        t = self.t
        if self.sum_in is None or self.sum_in.shape[0] != self.ids.numel():
            self.sum_in = torch.zeros((self.ids.numel(), self.R), dtype=self.local.dtype, device=self.local.device)
            self.sum_out = torch.zeros_like(self.sum_in)
        self.backend.shrink(self.plan, self.ids, [3], [self.sum_in], x_g, self.pools_a[layer], t, rank_mult=self.N)
        if self.px is not None:
            self.backend.allsum(self.px, self.plan, self.sum_in, self.sum_out, half=1)
            total = self.sum_out
        else:
            dist.all_reduce(self.sum_in, group=self.group)
            total = self.sum_in
        self.backend.expand(self.plan, self.ids, [3], [o_g], [total], self.pools_b[layer], t, delta_stride=self.R,
                            delta_width=self.R, delta_parts=1, delta_part_stride=0, rank_mult=self.N)


class CudaBackend:
    """The local operations of :class:`TpLoraOps` on the CUDA kernels."""

    def __init__(self, use_pdl=False, fused=True, inband=True):
        from . import _lib
        self.base_flags = _lib.FLAG_PDL if use_pdl else 0
        self.flags = self.base_flags
        self.fused = fused   # with a PeerExchange: push from the shrink / wait in the expand, no exchange launch
        # fused exchange without flags: the expand recognises values that have not arrived (1); 2: and it does not
        # wait for this GPU's own shrink either (see TpLink::inband in csrc/lora_common.cuh)
        # 3: early start over rotating thirds (no bookkeeping at the end of an expand)
        if inband is True and use_pdl:
            inband = {"0": 1, "2": 2}.get(os.environ.get("SLORA_TP_EARLY", "3"), 3)
        self.inband = int(inband)

    def make_plan(self, ids, t, local_width=None):
        """``local_width``: the widest share of rank rows a rank holds (``R / N``).  Adapters of different ranks have
        their work items counted exactly, except where a rank's share is at most 8 rows: the padded enumeration is
        nearly exact there (two row blocks per projection at most) and its launches start sooner (measured on a
        13B-shaped batch per layer: 52.3 against 57.7 us at N = 8, but 86.5 against 77.4 at N = 4)."""
        from . import _lib
        from .batch_infer import BatchPlan
        plan = BatchPlan(ids, t.a_start, t.a_len, t.a_loc.numel(), a_loc=t.a_loc, a_scaling=t.a_scaling,
                         max_rank=int(local_width or 0))
        self.flags = self.base_flags | plan.flags
        if ids.numel() >= 128 and (local_width is None or local_width > 8) and plan.info()[2] == 0:
            self.flags |= _lib.FLAG_EXACT_ITEMS
        return plan

    def shrink(self, plan, ids, qkvo, deltas, x, pool_a, t, rank_mult=1):
        from .batch_infer import shrink_multi
        if rank_mult == 1:
            shrink_multi(plan, ids, qkvo, deltas, x, pool_a, t.a_start, t.a_len, t.a_loc, self.flags)
            return
        import ctypes
        from . import _lib
        n = len(qkvo)
        _lib.check(_lib.lib.slora_lora_shrink_rows(
            0 if plan is None else plan.ptr, ids.data_ptr(), n, (ctypes.c_int * n)(*qkvo),
            (ctypes.c_void_p * n)(*[d.data_ptr() for d in deltas]), deltas[0].stride(0), deltas[0].size(1), rank_mult,
            x.data_ptr(), x.stride(0), x.size(1), pool_a.data_ptr(), pool_a.size(0), pool_a.stride(0),
            t.a_start.data_ptr(), t.a_len.data_ptr(), t.a_loc.data_ptr(), t.a_start.numel(), t.a_loc.numel(),
            ids.numel(), _lib.dtype_code(x.dtype), self.flags, _lib.current_stream_ptr()))

    def allsum(self, px, plan, local, out, half):
        """Sum of every rank's ``local [T, R]`` into ``out`` over peer memory (C entry ``slora_tp_allsum``)."""
        from . import _lib
        status = 0 if plan is None else plan.ptr + 8
        _lib.check(_lib.lib.slora_tp_allsum(local.data_ptr(), px.parts_ptrs, px.flag_ptrs, px.counter.data_ptr() + 8,
                                            status, out.data_ptr(), px.rank, px.world, local.size(0), px.parts.shape[1],
                                            local.size(1), half, px.seq_state.data_ptr(), 3, _lib.dtype_code(local.dtype),
                                            self.flags, _lib.current_stream_ptr()))

    def regroup(self, out, gathered, ids, t, n_parts, nproj, part_width, part_stride):
        """``out[p, t, g*rs + j] = gathered[g, p, t, j]`` (C entry ``slora_tp_regroup``)."""
        from . import _lib
        _lib.check(_lib.lib.slora_tp_regroup(out.data_ptr(), gathered.data_ptr(), ids.data_ptr(), t.a_len.data_ptr(),
                                             n_parts, nproj, ids.numel(), part_width, part_stride, t.a_start.numel(),
                                             _lib.dtype_code(out.dtype), _lib.current_stream_ptr()))

    def exchange(self, px, plan, local, ids, t, nproj, part_width, half, mode=3):
        """Write ``local[:nproj]`` into half ``half`` of every rank's delta buffer, signal, wait; returns this rank's
        ``[3, T, R]`` view of that half.  q,k,v calls use half 0 and o calls half 1, strictly alternating."""
        from . import _lib
        status = 0 if plan is None else plan.ptr + 8      # the plan header's status word
        _lib.check(_lib.lib.slora_tp_exchange(local.data_ptr(), px.full_ptrs, px.flag_ptrs, px.counter.data_ptr(),
                                              status, ids.data_ptr(), t.a_len.data_ptr(), px.rank, px.world, nproj,
                                              ids.numel(), px.full.shape[2], part_width, t.a_start.numel(), half,
                                              px.seq_state.data_ptr(), mode, _lib.dtype_code(local.dtype),
                                              self.flags, _lib.current_stream_ptr()))
        return px.full[half][:, :ids.numel()]

    def shrink_push(self, px, plan, ids, qkvo, x, pool_a, t, part_width, half):
        """Shrink whose results land in every rank's delta buffer (C entry ``slora_tp_shrink_push``)."""
        import ctypes
        from . import _lib
        n = len(qkvo)
        _lib.check(_lib.lib.slora_tp_shrink_push(
            0 if plan is None else plan.ptr, ids.data_ptr(), n, (ctypes.c_int * n)(*qkvo), part_width, x.data_ptr(),
            x.stride(0), x.size(1), pool_a.data_ptr(), pool_a.size(0), pool_a.stride(0), t.a_start.data_ptr(),
            t.a_len.data_ptr(), t.a_loc.data_ptr(), t.a_start.numel(), t.a_loc.numel(), ids.numel(), px.full_ptrs,
            px.flag_ptrs, px.counter.data_ptr(), self._seq(px).data_ptr(), px.rank, px.world,
            0 if px.inband == 3 else half, px.full.shape[2], int(px.inband), _lib.dtype_code(x.dtype), self.flags,
            _lib.current_stream_ptr()))

    def expand_wait(self, px, plan, ids, qkvo, ys, pool_b, t, part_width, half):
        """Expand that waits for every rank's flag, then reads this rank's buffer (``slora_tp_expand_wait``)."""
        import ctypes
        from . import _lib
        n = len(qkvo)
        _lib.check(_lib.lib.slora_tp_expand_wait(
            0 if plan is None else plan.ptr, ids.data_ptr(), n, (ctypes.c_int * n)(*qkvo),
            (ctypes.c_void_p * n)(*[y.data_ptr() for y in ys]), (ctypes.c_int64 * n)(*[y.stride(0) for y in ys]),
            (ctypes.c_int * n)(*[y.size(1) for y in ys]), pool_b.data_ptr(), pool_b.size(0), pool_b.stride(0),
            t.a_start.data_ptr(), t.a_len.data_ptr(), t.a_loc.data_ptr(), t.a_scaling.data_ptr(), t.a_start.numel(),
            t.a_loc.numel(), ids.numel(), px.full.data_ptr(), px.flags.data_ptr(), px.counter.data_ptr() + 4,
            self._seq(px).data_ptr(), px.rank, px.world, 0 if px.inband == 3 else half, px.full.shape[2], part_width,
            int(px.inband), _lib.dtype_code(ys[0].dtype), self.flags, _lib.current_stream_ptr()))

    @staticmethod
    def _seq(px):
        """The device-kept sequence words a fused exchange uses (rotating thirds have their own)."""
        return px.inband_seq if px.inband == 3 else px.seq_state

    def expand(self, plan, ids, qkvo, ys, deltas, pool_b, t, **kw):
        from .batch_infer import expand_multi
        expand_multi(plan, ids, qkvo, ys, deltas, pool_b, t.a_start, t.a_len, t.a_loc, t.a_scaling, flags=self.flags,
                     **kw)
