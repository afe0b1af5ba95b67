"""Unified-Paging pool: one free map plus per-layer A ("key") and B ("value") row buffers.

Same public surface as the reference's ``MemoryAllocator`` (``slora/common/mem_allocator.py:10-238``):
``alloc`` returns the first ``need_size`` free row indices (scattered), ``alloc_contiguous`` the first run of
``need_size`` adjacent free rows, ``free`` / ``free_all`` give rows back, ``key_buffer[l]`` / ``value_buffer[l]``
are ``[tot_size, head_num, head_dim]`` tensors shared by KV cache and adapter rows.  The KV-cache-only helpers
``alloc_strip`` / ``alloc_grid`` are not part of the LoRA path and are not provided.

Differences in mechanism, not in results: on a CUDA pool ``alloc`` and ``free`` are the library's own kernels
(``slora_pool_alloc_rows`` / ``slora_pool_free_rows``): two launches over the free map, nothing read back, so an
allocation does not stall the host the way a ``nonzero`` does; the count of free rows is kept on the host, as in the
reference.  ``alloc_contiguous`` searches a windowed prefix sum.  The device is a parameter so that the allocator's
logic can be unit-tested on CPU (the reference hard-codes ``"cuda"``); a CPU pool uses torch index ops.
"""
from __future__ import annotations

import gc

import torch


class MemoryAllocator:
    def __init__(self, tot_size, cache_size, dtype, head_num, head_dim, layer_num, device="cuda",
                 allocate_buffers=True):
        assert tot_size >= cache_size
        self.dtype = dtype
        self.head_num = head_num
        self.head_dim = head_dim
        self.layer_num = layer_num
        self.cell_size = head_num * head_dim
        self.tot_size = tot_size
        self.cache_size = cache_size
        self.device = torch.device(device)
        self._allocate_buffers = allocate_buffers
        self.reset_all_pool()

    def get_memory_size(self):
        dsize = torch.empty((), dtype=self.dtype).element_size()
        return 2 * self.layer_num * self.tot_size * self.cell_size * dsize

    # -- allocation -------------------------------------------------------------------------------------
    def alloc(self, need_size):
        """First ``need_size`` free rows, in increasing order (``mem_allocator.py:30-39``)."""
        if need_size > self.can_use_mem_size:
            raise Exception(f'warn no enough pool space: need_size {need_size} left_size {self.can_use_mem_size}')
        if self.mem_state.is_cuda:
            return self._alloc_cuda(need_size)
        select_index = torch.nonzero(self.mem_state, as_tuple=False).view(-1)[:need_size]
        self.mem_state[select_index] = False
        self.can_use_mem_size -= select_index.numel()
        return select_index

    def _alloc_cuda(self, need_size):
        from . import _lib
        out = torch.empty((need_size,), dtype=torch.long, device=self.device)
        if need_size > 0:
            if self._alloc_ws is None:
                n = _lib.lib.slora_pool_alloc_workspace_bytes(self.tot_size)
                self._alloc_ws = torch.empty((max(n, 4),), dtype=torch.uint8, device=self.device)
                self.status = torch.zeros((1,), dtype=torch.int32, device=self.device)
            _lib.check(_lib.lib.slora_pool_alloc_rows(self.mem_state.data_ptr(), self.tot_size, need_size,
                                                      out.data_ptr(), self._alloc_ws.data_ptr(),
                                                      self._alloc_ws.numel(), self.status.data_ptr(),
                                                      _lib.current_stream_ptr()))
        self.can_use_mem_size -= need_size
        return out

    def alloc_contiguous(self, need_size):
        """First run of ``need_size`` adjacent free rows: ``(indices, start, end)`` or ``None``
        (``mem_allocator.py:42-59``)."""
        if need_size > self.can_use_mem_size:
            raise Exception(f'warn no enough pool space: need_size {need_size} left_size {self.can_use_mem_size}')
        if need_size <= 0 or need_size > self.tot_size:
            return None
        prefix = torch.zeros(self.tot_size + 1, dtype=torch.int32, device=self.device)
        torch.cumsum(self.mem_state, dim=0, dtype=torch.int32, out=prefix[1:])
        window = prefix[need_size:] - prefix[:self.tot_size - need_size + 1]
        hits = torch.nonzero(window == need_size, as_tuple=False).view(-1)
        if hits.numel() == 0:
            return None
        start = int(hits[0].item())
        end = start + need_size
        select_index = torch.arange(start, end, dtype=torch.long, device=self.device)
        self.mem_state[start:end] = False
        self.can_use_mem_size -= need_size
        return select_index, start, end

    def free(self, free_index):
        """Give rows back (``mem_allocator.py:185-199``)."""
        self.can_use_mem_size += free_index.shape[0]
        if self.mem_state.is_cuda and free_index.is_cuda and free_index.dtype == torch.long and free_index.dim() == 1:
            from . import _lib
            rows = free_index.contiguous()
            _lib.check(_lib.lib.slora_pool_free_rows(self.mem_state.data_ptr(), self.tot_size, rows.data_ptr(),
                                                     rows.numel(), 0, _lib.current_stream_ptr()))
            return
        self.mem_state[free_index] = True

    def free_all(self):
        self.mem_state[:] = True
        self.can_use_mem_size = self.tot_size

    # -- lifetime ---------------------------------------------------------------------------------------
    def delete_all_pool(self):
        self.mem_state = None
        self.can_use_mem_size = 0
        self.key_buffer = None
        self.value_buffer = None
        gc.collect()

    def delete_all_cache(self):
        self.delete_all_pool()

    def reset_all_pool(self):
        self.mem_state = torch.ones((self.tot_size,), dtype=torch.bool, device=self.device)
        self.can_use_mem_size = self.tot_size
        self._alloc_ws = None
        self.status = None      # device int32: SLORA_STATUS_BAD_TABLE if the free map ever held fewer rows than counted
        if self._allocate_buffers:
            shape = (self.tot_size, self.head_num, self.head_dim)
            self.key_buffer = [torch.empty(shape, dtype=self.dtype, device=self.device)
                               for _ in range(self.layer_num)]
            self.value_buffer = [torch.empty(shape, dtype=self.dtype, device=self.device)
                                 for _ in range(self.layer_num)]
        else:
            self.key_buffer, self.value_buffer = [], []

    def reset_all_cache(self):
        self.reset_all_pool()
