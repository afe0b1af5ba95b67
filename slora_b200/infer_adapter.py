"""Adapter index tables over the Unified-Paging pool.

Same role and public fields as the reference's ``InferAdapter``
(``slora/server/router/model_infer/infer_adapter.py:11-250``): ``a_loc`` lists the pool rows of every loaded
adapter, ``a_start[i]`` / ``a_len[i]`` (= ``4 * r``) delimit adapter ``i``'s run in it, ``a_scaling[i]`` is
``alpha / r``; within a run the rows of projection ``p`` (q, k, v, o) are ``a_loc[a_start + p*r : a_start + (p+1)*r]``.
``load_adapters`` allocates rows and copies each layer's ``w_combined[0]`` (A rows) into ``key_buffer[l]`` and
``w_combined[1]`` (B rows) into ``value_buffer[l]``; ``offload_adapters`` frees rows and compacts the tables.

Mechanism differs from the reference: table entries are assembled on the host and uploaded in one copy per table
(the reference writes them element by element from Python); on a CUDA pool the rows of an adapter go into all layers
with one launch (``slora_pool_scatter_rows``) and dropping adapters is two launches (``slora_tables_compact``: new
tables and the freed rows, where the reference runs index gathers, a cumulative sum, a Triton variable-length copy
and an indexed store) with nothing read back to the host.  A CPU pool does the same with torch index ops.  An adapter object needs ``lora_dir``, ``r``, ``scaling``
and ``layers[l]`` with ``w_combined`` (``[2, 4r, heads, head_dim]``) plus optional ``load_to_gpu`` /
``offload_from_gpu`` (``slora/models/peft/layer_weights/lora_layer_weight.py:230-261``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List

import torch


@dataclass
class InferAdapter:
    adapter_dirs: List[str]
    a_loc: torch.Tensor
    a_start: torch.Tensor
    a_len: torch.Tensor
    a_scaling: torch.Tensor
    mem_manager: Any
    idx_map: Dict[str, int]
    prefetch_tag: Dict[str, int]
    cur_tag: int
    prefetch_stream: Any
    host_lens: List[int] = field(default_factory=list)   # a_len as the host last wrote it (spares a read-back)

    @classmethod
    def init(cls, mem_manager, prefetch_stream=None):
        dev = mem_manager.mem_state.device
        return cls(
            adapter_dirs=[],
            a_loc=torch.empty(0, dtype=torch.long, device=dev),
            a_start=torch.empty(0, dtype=torch.long, device=dev),
            a_len=torch.empty(0, dtype=torch.long, device=dev),
            a_scaling=torch.empty(0, dtype=mem_manager.dtype, device=dev),
            mem_manager=mem_manager,
            idx_map={},
            prefetch_tag={},
            cur_tag=0,
            prefetch_stream=prefetch_stream,
        )

    # -- copy one adapter's rows into the pool ----------------------------------------------------------
    def _copy_rows_cuda(self, adapter, loc, prefetch):
        """All layers and both buffers in one launch (C entry ``slora_pool_scatter_rows``).  Returns False when the
        layout is not one the kernel takes (the caller then copies layer by layer)."""
        import ctypes
        from . import _lib
        mm = self.mem_manager
        L = len(adapter.layers)
        dev, dt = loc.device, mm.key_buffer[0].dtype
        row_bytes = mm.head_num * mm.head_dim * mm.key_buffer[0].element_size()
        n = loc.numel()
        want = 2 * n * mm.head_num * mm.head_dim
        blocks, ptrs = [], []
        ok = row_bytes % 16 == 0
        for layer in adapter.layers:
            if hasattr(layer, "load_to_gpu"):
                layer.load_to_gpu(prefetch=prefetch)
            w = layer.w_combined
            if w.device != dev:
                w = w.to(dev, non_blocking=True)
            if not w.is_contiguous():
                w = w.contiguous()
            ok = ok and w.dtype == dt and w.numel() == want
            blocks.append(w)
            ptrs.append(w.data_ptr())
        # the pool's pointer tables are rebuilt only when the allocator has new buffer lists (reset_all_pool)
        cached = getattr(mm, "_pool_ptr_tables", None)
        if cached is None or cached[0] is not mm.key_buffer or cached[1] is not mm.value_buffer or cached[2] != L:
            arr = ctypes.c_void_p * L
            contiguous = all(mm.key_buffer[l].is_contiguous() and mm.value_buffer[l].is_contiguous() for l in range(L))
            cached = (mm.key_buffer, mm.value_buffer, L, arr(*[b.data_ptr() for b in mm.key_buffer[:L]]),
                      arr(*[b.data_ptr() for b in mm.value_buffer[:L]]), contiguous, arr)
            mm._pool_ptr_tables = cached
        ok = ok and cached[5]
        if ok:
            loc64 = loc if loc.dtype == torch.long and loc.is_contiguous() else loc.to(torch.long).contiguous()
            _lib.check(_lib.lib.slora_pool_scatter_rows(
                cached[3], cached[4], cached[6](*ptrs), L, loc64.data_ptr(), n, row_bytes, mm.key_buffer[0].size(0),
                row_bytes, 0, _lib.current_stream_ptr()))
            stream = torch.cuda.current_stream()
            for b in blocks:     # the copies above are asynchronous: keep the sources alive on this stream
                b.record_stream(stream)
        for layer in adapter.layers:
            if ok and hasattr(layer, "offload_from_gpu"):
                layer.offload_from_gpu()
        return ok

    def _copy_rows(self, adapter, loc, prefetch):
        mm = self.mem_manager
        if loc.is_cuda and self._copy_rows_cuda(adapter, loc, prefetch):
            return
        for layer_id, layer in enumerate(adapter.layers):
            if hasattr(layer, "load_to_gpu"):
                layer.load_to_gpu(prefetch=prefetch)
            w = layer.w_combined
            if w.device != loc.device:
                w = w.to(loc.device, non_blocking=True)
            mm.key_buffer[layer_id][loc] = w[0].reshape(len(loc), mm.head_num, mm.head_dim)
            mm.value_buffer[layer_id][loc] = w[1].reshape(len(loc), mm.head_num, mm.head_dim)
            if hasattr(layer, "offload_from_gpu"):
                layer.offload_from_gpu()

    def load_adapters(self, adapters, prefetch=False):
        """Make every adapter in ``adapters`` resident (``infer_adapter.py:92-171``).

        With ``prefetch=True`` adapters are tagged as wanted by the next batch and loading stops when the pool is
        full instead of raising.
        """
        if len(adapters) == 0:
            return
        new_adapters, tot_size = [], 0
        if prefetch:
            self.cur_tag ^= 1
            capacity = self.mem_manager.can_use_mem_size
        for adapter in adapters:
            if adapter is None:
                continue
            if prefetch:
                self.prefetch_tag[adapter.lora_dir] = self.cur_tag
            if adapter.lora_dir in self.idx_map or any(adapter.lora_dir == a.lora_dir for a in new_adapters):
                continue
            if prefetch and tot_size + adapter.r * 4 > capacity:
                break
            new_adapters.append(adapter)
            tot_size += adapter.r * 4
        if not new_adapters:
            return
        new_loc = self.mem_manager.alloc(tot_size)
        dev = new_loc.device
        loc_offset = self.a_loc.numel()
        starts, lens, cum = [], [], 0
        for adapter in new_adapters:
            self.idx_map[adapter.lora_dir] = len(self.adapter_dirs)
            self.adapter_dirs.append(adapter.lora_dir)
            starts.append(loc_offset + cum)
            lens.append(adapter.r * 4)
            cum += adapter.r * 4
        if len(self.host_lens) == len(self.adapter_dirs) - len(new_adapters):
            self.host_lens = self.host_lens + lens
        self.a_start = torch.cat((self.a_start, torch.tensor(starts, dtype=torch.long, device=dev)))
        self.a_len = torch.cat((self.a_len, torch.tensor(lens, dtype=torch.long, device=dev)))
        self.a_loc = torch.cat((self.a_loc, new_loc.to(torch.long)))
        self.a_scaling = torch.cat((self.a_scaling, torch.tensor([a.scaling for a in new_adapters],
                                                                 dtype=self.a_scaling.dtype, device=dev)))
        use_stream = prefetch and self.prefetch_stream is not None and dev.type == "cuda"
        if use_stream:
            # The row indices were produced by kernels on the current stream (the allocator reads nothing back, so
            # the host does not wait for them the way the reference's boolean indexing does): the prefetch stream
            # must not read them, nor the tables' uploads, before those kernels have run; and the allocator's
            # caching of `new_loc` must know about its second stream.
            self.prefetch_stream.wait_stream(torch.cuda.current_stream())
            new_loc.record_stream(self.prefetch_stream)
        ctx = torch.cuda.stream(self.prefetch_stream) if use_stream else _NullCtx()
        with ctx:
            rows = new_loc.clone() if use_stream else new_loc
            for adapter, s, n in zip(new_adapters, starts, lens):
                self._copy_rows(adapter, rows[s - loc_offset: s - loc_offset + n], prefetch)

    def offload_adapters(self, reserve_adapter_dirs):
        """Drop every adapter not in ``reserve_adapter_dirs`` (and not tagged by the latest prefetch), free its rows
        and compact the tables (``infer_adapter.py:186-250``)."""
        if len(reserve_adapter_dirs) == len(self.adapter_dirs):
            return
        dev = self.a_loc.device
        if len(reserve_adapter_dirs) == 0:
            self.mem_manager.free(self.a_loc)
            self.adapter_dirs = []
            self.a_loc = torch.empty(0, dtype=torch.long, device=dev)
            self.a_start = torch.empty(0, dtype=torch.long, device=dev)
            self.a_len = torch.empty(0, dtype=torch.long, device=dev)
            self.a_scaling = torch.empty(0, dtype=self.a_scaling.dtype, device=dev)
            self.idx_map = {}
            self.host_lens = []
            return
        reserve = set(reserve_adapter_dirs)
        keep = [i for i, d in enumerate(self.adapter_dirs)
                if d in reserve or self.prefetch_tag.get(d, None) == self.cur_tag]
        if len(keep) == len(self.adapter_dirs):
            return
        if len(self.host_lens) != len(self.adapter_dirs):    # tables were replaced behind our back: read them
            self.host_lens = self.a_len.tolist()
        if dev.type == "cuda" and self.a_scaling.element_size() == 2:
            self._compact_cuda(keep)
            return
        starts = self.a_start.tolist()
        lens = self.a_len.tolist()
        keep_set = set(keep)
        drop_rows = [torch.arange(starts[i], starts[i] + lens[i]) for i in range(len(starts)) if i not in keep_set]
        keep_rows = [torch.arange(starts[i], starts[i] + lens[i]) for i in keep]
        self.mem_manager.free(self.a_loc[torch.cat(drop_rows).to(dev)])
        gather = torch.cat(keep_rows).to(dev) if keep_rows else torch.empty(0, dtype=torch.long, device=dev)
        new_lens = [lens[i] for i in keep]
        new_starts, cum = [], 0
        for n in new_lens:
            new_starts.append(cum)
            cum += n
        keep_t = torch.tensor(keep, dtype=torch.long, device=dev)
        self.a_loc = self.a_loc[gather]
        self.a_scaling = self.a_scaling[keep_t]
        self.a_len = torch.tensor(new_lens, dtype=torch.long, device=dev)
        self.a_start = torch.tensor(new_starts, dtype=torch.long, device=dev)
        self.adapter_dirs = [self.adapter_dirs[i] for i in keep]
        self.idx_map = {d: i for i, d in enumerate(self.adapter_dirs)}
        self.host_lens = new_lens

    def _compact_cuda(self, keep):
        """New tables and freed rows in two launches (C entry ``slora_tables_compact``); sizes come from the host's
        copy of the lengths, nothing is read back."""
        from . import _lib
        mm = self.mem_manager
        dev = self.a_loc.device
        n = len(self.adapter_dirs)
        new_lens = [self.host_lens[i] for i in keep]
        kept_rows = sum(new_lens)
        flags = bytearray(n)
        for i in keep:
            flags[i] = 1
        keep_t = torch.frombuffer(flags, dtype=torch.uint8).to(dev, non_blocking=False)
        new_start = torch.empty((len(keep),), dtype=torch.long, device=dev)
        new_len = torch.empty((len(keep),), dtype=torch.long, device=dev)
        new_loc = torch.empty((kept_rows,), dtype=torch.long, device=dev)
        new_scaling = torch.empty((len(keep),), dtype=self.a_scaling.dtype, device=dev)
        scratch = torch.empty((n,), dtype=torch.long, device=dev)
        if getattr(mm, "status", None) is None:
            mm.status = torch.zeros((1,), dtype=torch.int32, device=dev)
        a_start, a_len, a_loc, a_scaling = (t.contiguous() for t in (self.a_start, self.a_len, self.a_loc,
                                                                      self.a_scaling))
        _lib.check(_lib.lib.slora_tables_compact(
            a_start.data_ptr(), a_len.data_ptr(), a_loc.data_ptr(), a_scaling.data_ptr(), keep_t.data_ptr(), n,
            a_loc.numel(), new_start.data_ptr(), new_len.data_ptr(), new_loc.data_ptr(), new_scaling.data_ptr(),
            scratch.data_ptr(), 0, mm.mem_state.data_ptr(), mm.tot_size, mm.status.data_ptr(),
            _lib.current_stream_ptr()))
        mm.can_use_mem_size += sum(self.host_lens) - kept_rows
        self.a_start, self.a_len, self.a_loc, self.a_scaling = new_start, new_len, new_loc, new_scaling
        self.adapter_dirs = [self.adapter_dirs[i] for i in keep]
        self.idx_map = {d: i for i, d in enumerate(self.adapter_dirs)}
        self.host_lens = new_lens


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
