"""The LoRA half of the reference's batch-infer layer, as two fused calls per transformer layer.

``LoraUnorderedBatchInfer`` (``slora/models/peft/lora_unordered_batch_infer.py:16-483``) issues, per layer,
``torch.mm`` + shrink + expand for q, k and v and later for o: eight ``dispatch_bgmv`` launches per layer.
:class:`LoraBatchOps` keeps that call structure (``lora_get_qkv`` where the reference has
``_batch_lora_get_qkv`` / ``_lora_get_qkv``, ``lora_get_o`` for ``_batch_lora_get_o`` / ``_lora_get_o``) but each
call is one q/k/v-fused shrink launch plus one fused expand launch, working from a :class:`BatchPlan` that groups
the batch's tokens by adapter once per forward instead of per launch.  The base ``torch.mm`` and the rotary
embedding stay with the caller, exactly where the reference has them.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib


class BatchPlan:
    """Tokens of one batch grouped by adapter (device-resident; built by one small kernel).

    Plays the role of ``req_bins`` / ``batch_req_bins`` (``lora_unordered_batch_infer.py:24-38,66``): it is
    derived from the per-token adapter ids once per forward and shared by every layer and projection.
    """

    def __init__(self, token_adapter_ids: torch.Tensor, a_start: torch.Tensor, a_len: torch.Tensor, loc_len: int,
                 workspace: torch.Tensor | None = None, a_loc: torch.Tensor | None = None,
                 a_scaling: torch.Tensor | None = None, max_rank: int = 0):
        """``a_loc`` (and ``a_scaling``) with ``max_rank`` > 0: the plan also holds resolved tiles for adapters of
        rank up to ``max_rank`` (token ids, scale and pool rows of every tile where a launch finds them in one round
        trip; C entry ``slora_plan_build_ex``).  ``self.flags`` then carries ``SLORA_FLAG_RESOLVED(max_rank)`` for the
        calls that use the plan; the plan must be rebuilt when the tables change."""
        _lib.require_cuda(token_adapter_ids, a_start, a_len)
        if token_adapter_ids.dtype != torch.int64 or token_adapter_ids.dim() != 1:
            raise RuntimeError("token_adapter_ids must be a 1-D int64 tensor")
        self.ids = token_adapter_ids.contiguous()
        self.T = self.ids.numel()
        self.n_adapters = a_start.numel()
        cap = 0
        if a_loc is not None and 0 < max_rank <= 128 and os.environ.get("SLORA_RESOLVED_TILES", "1") != "0":
            _lib.require_cuda(a_loc)
            if a_loc.dtype != torch.int64 or not a_loc.is_contiguous() or a_loc.numel() != int(loc_len):
                raise RuntimeError("a_loc must be the contiguous int64 loc table of loc_len entries")
            if a_scaling is not None and (a_scaling.element_size() != 2 or not a_scaling.is_contiguous()
                                          or a_scaling.numel() != self.n_adapters):
                raise RuntimeError("a_scaling must hold one 16-bit value per adapter")
            cap = int(max_rank)
        self.flags = _lib.flag_resolved(cap)
        need = _lib.lib.slora_plan_workspace_bytes_ex(self.T, self.n_adapters, cap)
        if workspace is None:
            workspace = torch.empty((need + 3) // 4, dtype=torch.int32, device=self.ids.device)
        elif workspace.numel() * workspace.element_size() < need:
            raise RuntimeError(f"plan workspace too small: {workspace.numel() * workspace.element_size()} < {need}")
        self.workspace = workspace
        _lib.check(_lib.lib.slora_plan_build_ex(
            workspace.data_ptr(), workspace.numel() * workspace.element_size(), self.ids.data_ptr(), self.T,
            a_start.data_ptr(), a_len.data_ptr(), a_loc.data_ptr() if cap else 0,
            a_scaling.data_ptr() if cap and a_scaling is not None else 0, self.n_adapters, int(loc_len), cap,
            _lib.current_stream_ptr()))

    @property
    def ptr(self) -> int:
        return self.workspace.data_ptr()

    def status(self):
        """``(status_bits, n_tiles)`` -- synchronises the current stream."""
        st, nt = ctypes.c_int(0), ctypes.c_int(0)
        _lib.check(_lib.lib.slora_plan_status(self.ptr, ctypes.byref(st), ctypes.byref(nt),
                                              _lib.current_stream_ptr()))
        return st.value, nt.value

    def big_tiles(self) -> int:
        """Number of 128-token tiles of adapters with 128 or more tokens in the batch -- synchronises the stream."""
        n = ctypes.c_int(0)
        _lib.check(_lib.lib.slora_plan_big_tiles(self.ptr, ctypes.byref(n), _lib.current_stream_ptr()))
        return n.value

    def info(self):
        """``(tiles, big_tiles, uniform_rank)``: 8-token tiles, 128-token tiles of big groups, and the rank shared by
        every adapter of the batch (0 when they differ) -- synchronises the stream."""
        nt, nb, ur = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
        _lib.check(_lib.lib.slora_plan_info(self.ptr, ctypes.byref(nt), ctypes.byref(nb), ctypes.byref(ur),
                                            _lib.current_stream_ptr()))
        return nt.value, nb.value, ur.value

    def header(self):
        """The plan's header as a dict -- synchronises the stream (C entry ``slora_plan_header``)."""
        buf = (ctypes.c_int32 * 16)()
        _lib.check(_lib.lib.slora_plan_header(self.ptr, buf, _lib.current_stream_ptr()))
        return {"tiles": buf[1], "status": buf[2], "tokens": buf[4], "adapters": buf[5], "big_tiles": buf[6],
                "uniform_rank": buf[9], "small_tiles": buf[10], "big_rank_max": buf[11], "big_ranks_pow2": bool(buf[12]),
                "resolved_cap": buf[14] if buf[13] > 0 else 0}

    def check(self):
        st, _ = self.status()
        if st:
            what = ", ".join(v for k, v in _lib.STATUS_BITS.items() if st & k)
            raise RuntimeError(f"slora_b200: device reported: {what} (status {st})")


class LoraBatchOps:
    """Per-forward LoRA operator: shrink+expand for q/k/v and for o of one layer, in place on the base outputs.

    Parameters mirror what ``LoraUnorderedBatchInfer.__init__`` reads from ``infer_adapter``
    (``lora_unordered_batch_infer.py:26-38``): the four tables and the per-layer pool buffers.
    ``max_lora_dim`` is the width of the delta buffers (``self.max_lora_dim`` there).
    """

    def __init__(self, a_start, a_len, a_loc, a_scaling, key_buffer, value_buffer, max_lora_dim, use_pdl=True):
        _lib.require_cuda(a_start, a_len, a_loc, a_scaling)
        self.a_start, self.a_len, self.a_loc, self.a_scaling = a_start, a_len, a_loc, a_scaling
        self.key_buffer, self.value_buffer = key_buffer, value_buffer
        self.max_lora_dim = int(max_lora_dim)
        self.base_flags = _lib.FLAG_PDL if use_pdl else 0
        self.flags = self.base_flags
        self.plan = None
        self.delta = None

    @classmethod
    def from_infer_adapter(cls, infer_adapter, max_lora_dim, use_pdl=True):
        mm = infer_adapter.mem_manager
        return cls(infer_adapter.a_start, infer_adapter.a_len, infer_adapter.a_loc, infer_adapter.a_scaling,
                   mm.key_buffer, mm.value_buffer, max_lora_dim, use_pdl)

    def prepare(self, token_adapter_ids, use_plan=True, big_groups=None, mixed_ranks=None):
        """Start a forward: ``token_adapter_ids`` is ``req_bins`` (decode) or ``batch_req_bins`` (prefill).

        Allocates the three delta buffers the reference allocates in ``forward`` (``:68-69,75-76``) and builds the
        plan.  ``use_plan=False`` keeps every token its own group (the reference's behaviour).

        ``big_groups``: does some adapter have 128 or more tokens in this batch (a prefill batch)?  Such groups run
        on the tensor cores.  The reference decides the same way on the host (``:127-130``: Triton kernels when
        ``max_len_in_batch >= 200``).  ``None`` asks the plan (one 64-byte read-back and a stream synchronisation,
        only for batches of 128 tokens or more); a scheduler that knows its batch passes ``True`` / ``False``.

        ``mixed_ranks``: do the batch's adapters differ in rank, or are all narrower than ``max_lora_dim``?  Then
        the kernels count their work items exactly (``SLORA_FLAG_EXACT_ITEMS``; a matter of speed only).  ``None``
        asks the plan in the same read-back; batches below 128 tokens are not asked and keep the plain enumeration.

        """
        self.ids = token_adapter_ids.contiguous()
        T = self.ids.numel()
        dtype = self.key_buffer[0].dtype
        self.delta = [torch.zeros((T, self.max_lora_dim), dtype=dtype, device=self.ids.device) for _ in range(3)]
        self.plan = BatchPlan(self.ids, self.a_start, self.a_len, self.a_loc.numel(), a_loc=self.a_loc,
                              a_scaling=self.a_scaling, max_rank=self.max_lora_dim) if use_plan else None
        self.flags = self.base_flags | (self.plan.flags if self.plan is not None else 0)
        only_big, n_big_tiles = False, 0
        if self.plan is not None and T >= 128 and (big_groups is None or mixed_ranks is None):
            h = self.plan.header()
            n_big_tiles = h["big_tiles"]
            if big_groups is None:
                big_groups = h["big_tiles"] > 0
                # a pure prefill batch: every group is big and of a rank the tensor-core kernels take
                stride = self.key_buffer[0].stride(0)
                only_big = (big_groups and h["small_tiles"] == 0 and h["big_ranks_pow2"] and
                            8 <= h["big_rank_max"] <= min(self.max_lora_dim, 128) and stride % h["big_rank_max"] == 0)
            if mixed_ranks is None:
                mixed_ranks = h["uniform_rank"] == 0 or h["uniform_rank"] < self.max_lora_dim
        if self.plan is not None and big_groups:
            self.flags |= _lib.FLAG_BIG_GROUPS
            if only_big:
                self.flags |= _lib.FLAG_ONLY_BIG
            if n_big_tiles:
                self.flags |= (min(n_big_tiles, 0xffff) << 16)     # SLORA_FLAG_BIG_TILES: the plan's own count
        if self.plan is not None and mixed_ranks:
            self.flags |= _lib.FLAG_EXACT_ITEMS
        return self

    def _common(self, layer_id):
        kb, vb = self.key_buffer[layer_id], self.value_buffer[layer_id]
        if kb.stride(0) != vb.stride(0):
            raise RuntimeError("A and B pools must share one row stride")
        return kb, vb, kb.size(0), kb.stride(0)

    def lora_get_qkv(self, layer_id, x, q, k, v, rope=None, kv_dest=None, head_dim=128):
        """``q += lora_q(x)``, ``k += lora_k(x)``, ``v += lora_v(x)`` (2-D views ``[T, h]``), in place.

        ``rope=(cos, sin)`` (``[T, head_dim / 2]`` each, ``infer_state.position_cos / position_sin``) also applies the
        rotary embedding to q and k, as ``rotary_emb_fwd`` does right after each expand in the reference
        (``lora_unordered_batch_infer.py:277,298``); ``kv_dest=(rows, k_out, v_out)`` then writes the new k and v rows
        to rows ``rows[t]`` of the KV-pool buffers ``k_out`` / ``v_out`` instead of updating ``k`` / ``v`` in place
        (``destindex_copy_kv``, ``transformer_layer_infer_template.py:50-62``).  Both happen in the expand's epilogue
        where the kernels allow (C entry ``slora_batch_lora_qkv_rope``).
        """
        kb, vb, rows, stride = self._common(layer_id)
        _lib.require_cuda(x, q, k, v)
        if k.size(1) != v.size(1):
            raise RuntimeError("k and v must have the same width")
        d = self.delta
        if rope is not None:
            cos, sin = rope
            _lib.require_cuda(cos, sin)
            if cos.shape != sin.shape or cos.dim() != 2 or cos.size(0) != x.size(0) or cos.size(1) * 2 != head_dim \
                    or cos.dtype != x.dtype or sin.dtype != x.dtype or cos.stride(1) != 1 or sin.stride(1) != 1 \
                    or cos.stride(0) != sin.stride(0):
                raise RuntimeError("cos and sin must be [T, head_dim / 2] tensors of the activations' dtype")
            kv_rows = k_out = v_out = None
            out_stride = out_rows = 0
            if kv_dest is not None:
                kv_rows, k_out, v_out = kv_dest
                _lib.require_cuda(kv_rows, k_out, v_out)
                if kv_rows.dtype != torch.int64 or kv_rows.dim() != 1 or kv_rows.numel() != x.size(0) \
                        or not kv_rows.is_contiguous():
                    raise RuntimeError("kv_dest rows must be a contiguous int64 tensor with one entry per token")
                ko, vo = k_out.view(k_out.size(0), -1), v_out.view(v_out.size(0), -1)
                if ko.shape != vo.shape or ko.stride() != vo.stride() or ko.stride(1) != 1 or ko.size(1) < k.size(1) \
                        or ko.dtype != x.dtype or vo.dtype != x.dtype:
                    raise RuntimeError("k_out and v_out must be row-major buffers of one shape, at least as wide as k")
                out_stride, out_rows = ko.stride(0), ko.size(0)
            _lib.check(_lib.lib.slora_batch_lora_qkv_rope(
                0 if self.plan is None else self.plan.ptr, self.ids.data_ptr(), q.data_ptr(), k.data_ptr(),
                v.data_ptr(), q.stride(0), k.stride(0), v.stride(0), q.size(1), k.size(1), x.data_ptr(), x.stride(0),
                x.size(1), kb.data_ptr(), vb.data_ptr(), rows, stride, self.a_start.data_ptr(), self.a_len.data_ptr(),
                self.a_loc.data_ptr(), self.a_scaling.data_ptr(), self.a_start.numel(), self.a_loc.numel(),
                d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[0].stride(0), self.max_lora_dim, x.size(0),
                _lib.dtype_code(x.dtype), self.flags, _lib.current_stream_ptr(), cos.data_ptr(), sin.data_ptr(),
                cos.stride(0), int(head_dim), _lib.ptr(kv_rows), _lib.ptr(k_out), _lib.ptr(v_out), out_stride, out_rows))
            return q
        if kv_dest is not None:
            raise RuntimeError("kv_dest needs rope=(cos, sin)")
        _lib.check(_lib.lib.slora_batch_lora_qkv(
            0 if self.plan is None else self.plan.ptr, self.ids.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
            q.stride(0), k.stride(0), v.stride(0), q.size(1), k.size(1), x.data_ptr(), x.stride(0), x.size(1),
            kb.data_ptr(), vb.data_ptr(), rows, stride, self.a_start.data_ptr(), self.a_len.data_ptr(),
            self.a_loc.data_ptr(), self.a_scaling.data_ptr(), self.a_start.numel(), self.a_loc.numel(),
            d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[0].stride(0), self.max_lora_dim, x.size(0),
            _lib.dtype_code(x.dtype), self.flags, _lib.current_stream_ptr()))
        return q

    def lora_get_o(self, layer_id, x, o):
        """``o += lora_o(x)`` in place (``x`` is the attention output, ``[T, H]``)."""
        kb, vb, rows, stride = self._common(layer_id)
        _lib.require_cuda(x, o)
        d = self.delta[0]  # the reference reuses delta[0] for o (:438)
        _lib.check(_lib.lib.slora_batch_lora_o(
            0 if self.plan is None else self.plan.ptr, self.ids.data_ptr(), o.data_ptr(), o.stride(0), o.size(1),
            x.data_ptr(), x.stride(0), x.size(1), kb.data_ptr(), vb.data_ptr(), rows, stride,
            self.a_start.data_ptr(), self.a_len.data_ptr(), self.a_loc.data_ptr(), self.a_scaling.data_ptr(),
            self.a_start.numel(), self.a_loc.numel(), d.data_ptr(), d.stride(0), self.max_lora_dim, x.size(0),
            _lib.dtype_code(x.dtype), self.flags, _lib.current_stream_ptr()))
        return o


def shrink_multi(plan, ids, qkvo, deltas, x, pool_a, a_start, a_len, a_loc, flags=0):
    """Planned shrink of up to three projections that share ``x`` (C entry ``slora_lora_shrink_multi``)."""
    n = len(qkvo)
    q_arr = (ctypes.c_int * n)(*qkvo)
    d_arr = (ctypes.c_void_p * n)(*[d.data_ptr() for d in deltas])
    _lib.check(_lib.lib.slora_lora_shrink_multi(
        0 if plan is None else plan.ptr, _lib.ptr(ids), n, q_arr, d_arr, deltas[0].stride(0), deltas[0].size(1),
        x.data_ptr(), x.stride(0), x.size(1), pool_a.data_ptr(), pool_a.size(0), pool_a.stride(0),
        a_start.data_ptr(), a_len.data_ptr(), a_loc.data_ptr(), a_start.numel(), a_loc.numel(), x.size(0),
        _lib.dtype_code(x.dtype), flags, _lib.current_stream_ptr()))


def expand_multi(plan, ids, qkvo, ys, deltas, pool_b, a_start, a_len, a_loc, a_scaling, delta_stride, delta_width,
                 delta_parts=1, delta_part_stride=0, rank_mult=1, flags=0):
    """Planned expand of up to three projections (C entry ``slora_lora_expand_multi``)."""
    n = len(qkvo)
    q_arr = (ctypes.c_int * n)(*qkvo)
    y_arr = (ctypes.c_void_p * n)(*[y.data_ptr() for y in ys])
    ys_arr = (ctypes.c_int64 * n)(*[y.stride(0) for y in ys])
    ho_arr = (ctypes.c_int * n)(*[y.size(1) for y in ys])
    d_arr = (ctypes.c_void_p * n)(*[d.data_ptr() for d in deltas])
    T = ys[0].size(0)
    _lib.check(_lib.lib.slora_lora_expand_multi(
        0 if plan is None else plan.ptr, _lib.ptr(ids), n, q_arr, y_arr, ys_arr, ho_arr, d_arr, delta_stride,
        delta_width, delta_parts, delta_part_stride, rank_mult, pool_b.data_ptr(), pool_b.size(0), pool_b.stride(0),
        a_start.data_ptr(), a_len.data_ptr(), a_loc.data_ptr(), a_scaling.data_ptr(), a_start.numel(),
        a_loc.numel(), T, _lib.dtype_code(ys[0].dtype), flags, _lib.current_stream_ptr()))


def lora_o_noalloc(ids, x, o, pool_a, pool_b, a_start, a_len, a_loc, a_scaling, max_rank, flags=0):
    """``o += lora_o(x)`` through the entry point that allocates nothing (C entry ``slora_batch_lora_o_noalloc``).

    For callers that may not allocate device memory (a serving process whose own pool holds the whole GPU, a path
    where ``cudaMalloc`` is forbidden): the plan and the intermediate live in 320 KB built into the library, so this
    wrapper creates no tensor either.  Limits: 1024 tokens, 4096 adapters, rank up to 128.  Calls on one stream may
    follow each other; calls that could overlap on the GPU would race on the shared scratch.
    """
    _lib.require_cuda(ids, x, o, pool_a, pool_b, a_start, a_len, a_loc, a_scaling)
    # the C entry takes raw pointers: everything it will index is checked here, before anything is launched
    for name, t in (("ids", ids), ("a_start", a_start), ("a_len", a_len), ("a_loc", a_loc)):
        if t.dtype != torch.int64 or t.dim() != 1 or not t.is_contiguous():
            raise RuntimeError(f"{name} must be a contiguous 1-D int64 tensor")
    if x.dim() != 2 or o.dim() != 2 or ids.numel() != x.size(0) or o.size(0) != x.size(0):
        raise RuntimeError("x and o must be 2-D with one row per entry of ids")
    if not (x.dtype == o.dtype == pool_a.dtype == pool_b.dtype == a_scaling.dtype):
        raise RuntimeError("x, o, the pools and a_scaling must share one dtype")
    if x.stride(1) != 1 or o.stride(1) != 1 or x.stride(0) % 8 or o.stride(0) % 8:
        raise RuntimeError("x and o need unit column stride and rows that start on 16-byte boundaries")
    if a_start.numel() != a_len.numel() or a_scaling.numel() != a_start.numel() or not a_scaling.is_contiguous():
        raise RuntimeError("a_start, a_len and a_scaling must have one entry per adapter")
    pa, pb = pool_a.reshape(pool_a.size(0), -1) if pool_a.is_contiguous() else pool_a, \
        pool_b.reshape(pool_b.size(0), -1) if pool_b.is_contiguous() else pool_b
    if pa.dim() != 2 or pb.dim() != 2 or pa.stride(1) != 1 or pb.stride(1) != 1 or pa.stride(0) != pb.stride(0) \
            or pa.size(0) != pb.size(0):
        raise RuntimeError("A and B pools must be 2-D views with one shape and one row stride")
    _lib.check(_lib.lib.slora_batch_lora_o_noalloc(
        ids.data_ptr(), o.data_ptr(), o.stride(0), o.size(1), x.data_ptr(), x.stride(0), x.size(1), pa.data_ptr(),
        pb.data_ptr(), pa.size(0), pa.stride(0), a_start.data_ptr(), a_len.data_ptr(), a_loc.data_ptr(),
        a_scaling.data_ptr(), a_start.numel(), a_loc.numel(), int(max_rank), x.size(0), _lib.dtype_code(x.dtype), flags,
        _lib.current_stream_ptr()))
    return o


def noalloc_status() -> int:
    """Status bits (``_lib.STATUS_BITS``) the latest :func:`lora_o_noalloc` call on the current device left in the
    built-in scratch -- synchronises the current stream (C entry ``slora_noalloc_status``)."""
    st = ctypes.c_int(0)
    _lib.check(_lib.lib.slora_noalloc_status(ctypes.byref(st), _lib.current_stream_ptr()))
    return st.value
