"""ctypes binding of ``libslora_b200.so`` (the C ABI declared in ``include/slora_b200.h``).

There is no fallback: if the shared library is missing the import fails with instructions to build it, and
every compute call needs CUDA tensors.  Status codes are turned into ``RuntimeError`` with the library's
message, the way the reference's ``TORCH_CHECK`` failures surface in Python (``slora/csrc/lora_ops.cc:124``).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int32, c_int64, c_size_t, c_uint, c_void_p, c_char_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SLORA_B200_LIB") or os.path.join(_HERE, "libslora_b200.so")   # override: a development build

F16, BF16 = 0, 1
FLAG_PDL = 1
FLAG_BIG_GROUPS = 2
FLAG_EXACT_ITEMS = 4
FLAG_ONLY_BIG = 16


def flag_resolved(max_rank: int) -> int:
    """``SLORA_FLAG_RESOLVED(max_rank)``: the plan holds resolved tiles for adapters of rank up to ``max_rank``."""
    return (((int(max_rank) + 7) >> 3) & 0x1f) << 8 if 0 < max_rank <= 128 else 0

STATUS_BITS = {1: "bad adapter id", 2: "bad table entry", 4: "unsupported rank", 8: "bulk-copy wait timed out"}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python slora_b200/build.py` (needs nvcc, sm_100a). "
            "slora_b200 has no CPU or PyTorch fallback.")
    return ctypes.CDLL(LIB_PATH)


lib = _load()

_P = c_void_p
_tables = [_P, _P, _P]  # start, ranks4, loc

_SIGS = {
    "slora_version": (c_int, []),
    "slora_last_error": (c_char_p, []),
    "slora_dispatch_bgmv": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, _P, c_int64, c_int, c_int, c_int64, c_int64,
                                    c_int64, c_int64, c_int, _P]),
    "slora_bgmv_shrink": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, c_int64, c_int, c_int64, c_int64, c_int,
                                  c_int64, c_int64, c_int64, c_int64, c_int, _P]),
    "slora_bgmv_expand": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int64, c_int, c_int64, c_int, c_int64,
                                  c_int64, c_int64, c_int64, c_int64, c_int, _P]),
    "slora_sgmv_shrink": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int64, c_int, c_int64,
                                  c_int64, c_int, c_int64, c_int64, c_int64, c_int64, c_int, _P]),
    "slora_sgmv_expand": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int64, c_int,
                                  c_int64, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, _P]),
    "slora_plan_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "slora_plan_build": (c_int, [_P, c_size_t, _P, c_int64, _P, _P, c_int64, c_int64, _P]),
    "slora_plan_workspace_bytes_ex": (c_size_t, [c_int64, c_int64, c_int]),
    "slora_plan_build_ex": (c_int, [_P, c_size_t, _P, c_int64, _P, _P, _P, _P, c_int64, c_int64, c_int, _P]),
    "slora_plan_status": (c_int, [_P, POINTER(c_int), POINTER(c_int), _P]),
    "slora_lora_shrink_multi": (c_int, [_P, _P, c_int, POINTER(c_int), POINTER(c_void_p), c_int64, c_int, _P,
                                        c_int64, c_int, _P, c_int64, c_int64, _P, _P, _P, c_int64, c_int64, c_int64,
                                        c_int, c_uint, _P]),
    "slora_lora_expand_multi": (c_int, [_P, _P, c_int, POINTER(c_int), POINTER(c_void_p), POINTER(c_int64),
                                        POINTER(c_int), POINTER(c_void_p), c_int64, c_int, c_int, c_int64, c_int, _P,
                                        c_int64, c_int64, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int, c_uint,
                                        _P]),
    "slora_batch_lora_qkv": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int, c_int, _P, c_int64, c_int,
                                     _P, _P, c_int64, c_int64, _P, _P, _P, _P, c_int64, c_int64, _P, _P, _P, c_int64,
                                     c_int, c_int64, c_int, c_uint, _P]),
    "slora_batch_lora_qkv_rope": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int, c_int, _P, c_int64,
                                          c_int, _P, _P, c_int64, c_int64, _P, _P, _P, _P, c_int64, c_int64, _P, _P, _P,
                                          c_int64, c_int, c_int64, c_int, c_uint, _P, _P, _P, c_int64, c_int, _P, _P,
                                          _P, c_int64, c_int64]),
    "slora_batch_lora_o": (c_int, [_P, _P, _P, c_int64, c_int, _P, c_int64, c_int, _P, _P, c_int64, c_int64, _P, _P,
                                   _P, _P, c_int64, c_int64, _P, c_int64, c_int, c_int64, c_int, c_uint, _P]),
    "slora_batch_lora_o_noalloc": (c_int, [_P, _P, c_int64, c_int, _P, c_int64, c_int, _P, _P, c_int64, c_int64, _P, _P,
                                           _P, _P, c_int64, c_int64, c_int, c_int64, c_int, c_uint, _P]),
    "slora_noalloc_status": (c_int, [POINTER(c_int), _P]),
    "slora_validate_tables": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, _P, _P]),
    "slora_tp_regroup": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int64, c_int, c_int64, c_int64, c_int, _P]),
    "slora_tp_exchange": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int64, c_int64, c_int, c_int64,
                                  c_int, _P, c_int, c_int, c_uint, _P]),
    "slora_tp_shrink_push": (c_int, [_P, _P, c_int, _P, c_int, _P, c_int64, c_int, _P, c_int64, c_int64, _P, _P, _P,
                                     c_int64, c_int64, c_int64, _P, _P, _P, _P, c_int, c_int, c_int, c_int64, c_int,
                                     c_int, c_uint, _P]),
    "slora_tp_expand_wait": (c_int, [_P, _P, c_int, _P, _P, _P, _P, _P, c_int64, c_int64, _P, _P, _P, _P, c_int64,
                                     c_int64, c_int64, _P, _P, _P, _P, c_int, c_int, c_int, c_int64, c_int, c_int,
                                     c_int, c_uint, _P]),
    "slora_pool_scatter_rows": (c_int, [_P, _P, _P, c_int, _P, c_int64, c_int64, c_int64, c_int64, _P, _P]),
    "slora_lora_shrink_rows": (c_int, [_P, _P, c_int, _P, _P, c_int64, c_int, c_int, _P, c_int64, c_int, _P, c_int64,
                                       c_int64, _P, _P, _P, c_int64, c_int64, c_int64, c_int, c_uint, _P]),
    "slora_tp_allsum": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int64, c_int64, c_int, c_int, _P, c_int, c_int,
                                c_uint, _P]),
    "slora_pool_alloc_workspace_bytes": (ctypes.c_size_t, [c_int64]),
    "slora_pool_alloc_rows": (c_int, [_P, c_int64, c_int64, _P, _P, ctypes.c_size_t, _P, _P]),
    "slora_pool_free_rows": (c_int, [_P, c_int64, _P, c_int64, _P, _P]),
    "slora_tables_compact": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int64, _P, _P, _P, _P, _P, _P, _P, c_int64, _P,
                                     _P]),
    "slora_plan_info": (c_int, [_P, _P, _P, _P, _P]),
    "slora_plan_header": (c_int, [_P, _P, _P]),
    "slora_launch_counts": (None, [_P]),
    "slora_plan_big_tiles": (c_int, [_P, _P, _P]),
}

EXPORTS = tuple(_SIGS)

for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)  # AttributeError here means the header and the library disagree
    _fn.restype = _res
    _fn.argtypes = _args


def launch_counts():
    """Kernels launched by the library so far: ``{"simple", "pipelined", "tensor_core", "plan"}`` (growing counters)."""
    import ctypes
    buf = (ctypes.c_int64 * 4)()
    lib.slora_launch_counts(buf)
    return dict(zip(("simple", "pipelined", "tensor_core", "plan"), (int(v) for v in buf)))


def last_error() -> str:
    msg = lib.slora_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"slora_b200: {last_error()} (status {rc})")


def dtype_code(torch_dtype) -> int:
    import torch
    if torch_dtype == torch.float16:
        return F16
    if torch_dtype == torch.bfloat16:
        return BF16
    raise RuntimeError(f"No suitable kernel. dtype={torch_dtype}")


def ptr(t) -> int:
    """Device pointer of a CUDA tensor (or 0 for None)."""
    return 0 if t is None else t.data_ptr()


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("slora_b200 runs on CUDA tensors only (there is no CPU path)")


def current_stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream
