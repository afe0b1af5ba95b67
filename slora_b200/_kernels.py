"""Drop-in for ``slora._kernels`` (the reference's pybind module, ``slora/csrc/lora_ops.cc:134-136``)."""
from __future__ import annotations

import torch

from . import _lib


def _check_input(t, name):
    # CHECK_INPUT of lora_ops.cc:27-36
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _check_index(t, name):
    _check_input(t, name)
    if t.dtype != torch.int64:
        raise RuntimeError(f"{name} must be an int64 tensor")


def dispatch_bgmv(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies, qkvo, lora_scales):
    """Same call, same argument meaning and same in-place effect on ``y`` as the reference's
    ``dispatch_bgmv`` (``slora/csrc/lora_ops.cc:76-126``).

    ``x.size(1) < y.size(1)`` selects the expand (``y += scale * x[:, :r] @ B``), otherwise the shrink
    (``y[:, :r] = x @ A.T``) -- the rule of ``slora/csrc/bgmv/bgmv_impl.cuh:221,232``.  ``w`` is one layer's pool
    buffer ``[rows, heads, head_dim]``; ``lora_ranks`` holds ``4 * r`` per adapter.  Runs on the current stream
    (the reference uses the legacy default stream).  Unsupported shapes or dtypes raise ``RuntimeError`` with the
    reference's "No suitable kernel." wording.
    """
    for t, n in ((y, "y"), (x, "x"), (w, "w")):
        _check_input(t, n)
    for t, n in ((start_indicies, "start_indicies"), (lora_ranks, "lora_ranks"), (loc_indicies, "loc_indicies"),
                 (indicies, "indicies")):
        _check_index(t, n)
    _check_input(lora_scales, "lora_scales")
    if y.dim() != 2:
        raise RuntimeError("y must be a 2D tensor")
    if x.dim() != 2:
        raise RuntimeError("x must be a 2D tensor")
    if w.dim() != 3:
        raise RuntimeError("w must be a 3D tensor")
    if indicies.dim() != 1:
        raise RuntimeError("indicies must be a 1D tensor")
    if indicies.size(0) != x.size(0):
        raise RuntimeError(f"CHECK_EQ(indicies.size(0), x.size(0)) failed. {indicies.size(0)} vs {x.size(0)}")
    if y.size(0) != x.size(0):
        raise RuntimeError(f"CHECK_EQ(y.size(0), x.size(0)) failed. {y.size(0)} vs {x.size(0)}")
    h_in, h_out = x.size(1), y.size(1)
    if not (x.dtype == y.dtype == w.dtype == lora_scales.dtype) or x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype}")
    if h_in >= 65536 or h_out >= 65536:
        raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype}")
    rc = _lib.lib.slora_dispatch_bgmv(
        y.data_ptr(), x.data_ptr(), w.data_ptr(), start_indicies.data_ptr(), lora_ranks.data_ptr(),
        loc_indicies.data_ptr(), indicies.data_ptr(), int(qkvo), lora_scales.data_ptr(), x.size(0), h_in, h_out,
        w.size(0), w.size(1) * w.size(2), start_indicies.numel(), loc_indicies.numel(), _lib.dtype_code(x.dtype),
        _lib.current_stream_ptr())
    if rc != 0:
        msg = _lib.last_error()
        if "No suitable kernel" in msg:
            raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype} ({msg})")
        _lib.check(rc)


def validate_tables(start_indicies, lora_ranks, loc_indicies, indicies, pool_rows):
    """Range-check the adapter tables on the device (debug aid; the reference has no such check).

    Returns ``(n_bad, kind, index)`` where kind is 0 none, 1 ``indicies``, 2 ``start/ranks``, 3 ``loc``.
    Synchronises the current stream.
    """
    _lib.require_cuda(start_indicies, lora_ranks, loc_indicies, indicies)
    report = torch.zeros(4, dtype=torch.int32, device=start_indicies.device)
    _lib.check(_lib.lib.slora_validate_tables(
        start_indicies.data_ptr(), lora_ranks.data_ptr(), loc_indicies.data_ptr(), _lib.ptr(indicies),
        start_indicies.numel(), loc_indicies.numel(), 0 if indicies is None else indicies.numel(), int(pool_rows),
        report.data_ptr(), _lib.current_stream_ptr()))
    n_bad, kind, index, _ = report.tolist()
    return n_bad, kind, index
