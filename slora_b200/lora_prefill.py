"""Drop-in for ``slora/models/peft/triton_kernel/lora/lora_prefill.py`` (no Triton: CUDA through the C ABI)."""
from __future__ import annotations

import torch

from . import _lib


def _seg(t):
    return t if t.dtype == torch.int32 else t.to(torch.int32)


@torch.inference_mode()
def lora_get_qkvo_fwd_shrink(x, w, o, b_loc, b_lora_start, b_lora_ranks, b_start_loc, b_seq_len, b_indicies,
                             hidden_size, qkvo, max_rank, max_input_len):
    """Segment shrink with the reference's signature (``lora_prefill.py:139-164``).

    ``x [tokens, hidden_size]``, ``w [rows, stride]`` (the A pool viewed 2-D), ``o [tokens, max_rank]``;
    request ``i`` covers tokens ``b_start_loc[i] .. +b_seq_len[i]`` and uses adapter ``b_indicies[i]``;
    ``o[t, :r] = x[t] @ A.T`` (columns ``>= r`` untouched).
    """
    _lib.require_cuda(x, w, o, b_loc, b_lora_start, b_lora_ranks, b_start_loc, b_seq_len, b_indicies)
    if x.stride(1) != 1 or o.stride(1) != 1 or w.stride(1) != 1:
        raise RuntimeError("x, w and o must be contiguous along their last dimension")
    b_start_loc, b_seq_len = _seg(b_start_loc), _seg(b_seq_len)
    _lib.check(_lib.lib.slora_sgmv_shrink(
        o.data_ptr(), x.data_ptr(), w.data_ptr(), b_lora_start.data_ptr(), b_lora_ranks.data_ptr(),
        b_loc.data_ptr(), b_start_loc.data_ptr(), b_seq_len.data_ptr(), b_indicies.data_ptr(), b_seq_len.numel(),
        int(max_input_len), int(qkvo), x.size(0), int(hidden_size), x.stride(0), o.stride(0), o.size(1), w.size(0),
        w.stride(0), b_lora_start.numel(), b_loc.numel(), _lib.dtype_code(x.dtype), _lib.current_stream_ptr()))


@torch.inference_mode()
def lora_get_qkvo_fwd_expand(x, w, o, scale, b_loc, b_lora_start, b_lora_ranks, b_start_loc, b_seq_len, b_indicies,
                             feat_out, qkvo, max_rank, max_input_len):
    """Segment expand with the reference's signature (``lora_prefill.py:105-136``).

    ``x [tokens, max_rank]`` is the shrink output, ``w [rows, stride]`` the B pool viewed 2-D,
    ``o [tokens, feat_out]`` is updated in place: ``o[t] += scale[a] * x[t, :r] @ B.T``.
    """
    _lib.require_cuda(x, w, o, scale, b_loc, b_lora_start, b_lora_ranks, b_start_loc, b_seq_len, b_indicies)
    if x.stride(1) != 1 or o.stride(1) != 1 or w.stride(1) != 1:
        raise RuntimeError("x, w and o must be contiguous along their last dimension")
    b_start_loc, b_seq_len = _seg(b_start_loc), _seg(b_seq_len)
    _lib.check(_lib.lib.slora_sgmv_expand(
        o.data_ptr(), x.data_ptr(), w.data_ptr(), b_lora_start.data_ptr(), b_lora_ranks.data_ptr(),
        b_loc.data_ptr(), b_start_loc.data_ptr(), b_seq_len.data_ptr(), b_indicies.data_ptr(), scale.data_ptr(),
        b_seq_len.numel(), int(max_input_len), int(qkvo), x.size(0), int(feat_out), x.stride(0), x.size(1),
        o.stride(0), w.size(0), w.stride(0), b_lora_start.numel(), b_loc.numel(), _lib.dtype_code(x.dtype),
        _lib.current_stream_ptr()))
