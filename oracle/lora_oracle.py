"""CPU oracle for the multi-adapter LoRA shrink / expand path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; only the
tests, the smoke check and the CPU-baseline leg of the benchmark call it, and only as the
checker (or as the thing whose CPU time is reported), never as the product path.

What it restates (all paths are inside the S-LoRA reference tree):

* the per-token torch formula that the reference's kernel scripts print their deltas against:
  ``test/kernel/test_kernel_correctness_multi_rank.py:97-106`` and
  ``test/kernel/test_kernel_correctness.py:87-95``
  (rows of adapter ``a`` for projection ``qkvo`` are ``buf[a_start[a] + qkvo*r : a_start[a] + (qkvo+1)*r]``;
  part A is ``rows.reshape(r, H).T``, part B is ``rows.reshape(H, r).T``, result ``x[i:i+1, :r] @ a_w``);
* the indirection through the location table exactly as the CUDA kernels do it:
  ``slora/csrc/bgmv/bgmv_impl.cuh:34-38`` (shrink) and ``:164-179,191`` (expand);
  the permuted-cell fixtures of ``slora/models/peft/triton_kernel/tests/bench_ops.py:118-124,158-165``
  are the model for a non-identity table;
* the scale is applied in the expand only (``bgmv_impl.cuh:180,197``), ``scale = alpha / r``
  (``slora/models/peft/lora_adapter.py:34``);
* the pool row content written by the loader (``slora/models/peft/layer_weights/lora_layer_weight.py:215-224``):
  A rows are ``lora_A.weight[j, :]``; the B rows are ``lora_B.weight`` (``[h_out, r]`` row-major) flattened
  and cut into ``r`` rows.  :func:`pool_rows_from_hf` builds rows that way and the tests check that the oracle
  equals ``(x @ A.T) @ B.T * alpha / r``.

Parity pin: the reference stores no golden values for this path (its kernel scripts draw CUDA random numbers
and only print a max delta).  The oracle is therefore pinned (1) by formula against the HF-layout identity above
and (2) by outputs of the reference's own CUDA kernels compiled from the reference tree by ``oracle/Makefile``
and run on a B200 (``tests/golden/ref_kernels.npz``, made by ``tests/golden/make_ref_golden.py``).

Arithmetic: inputs are taken as given (fp16/bf16 values upcast), everything is accumulated in float32 with no
intermediate rounding; :func:`lora_delta_ref_rounding` additionally mimics the reference kernels' fp16 rounding of
the intermediate and of ``y`` (``bgmv_impl.cuh:147,206``).

Generalisation beyond the reference (used for GQA and tensor-parallel shards): the reference kernels assume that
the pool row stride equals the wide feature size.  Here a projection's slot is the concatenation ("flat space") of
its ``slot_rows`` pool rows of ``pool_stride`` elements each; A is ``[r_a, h_in]`` row-major in that flat space and
B is ``[h_out, r_b]`` row-major in it, with ``r_a = slot_rows`` and ``r_b = slot_rows * rank_mult``.
With ``pool_stride == h_in`` / ``== h_out`` and ``rank_mult == 1`` this is exactly the reference layout.
"""
from __future__ import annotations

import numpy as np


def _f32(a):
    """Return a float32 numpy view/copy of a numpy array or torch tensor (fp16/bf16/fp32)."""
    if hasattr(a, "detach"):  # torch tensor
        return a.detach().to("cpu").float().numpy()
    return np.asarray(a, dtype=np.float32)


def _i64(a):
    if hasattr(a, "detach"):
        return a.detach().to("cpu").long().numpy()
    return np.asarray(a, dtype=np.int64)


def _slot_flat(pool, loc, base, slot_rows, count):
    """First ``count`` elements (float32) of the flat space of the slot ``loc[base : base+slot_rows]``.

    Only the slot's rows are converted, so a multi-gigabyte pool costs nothing beyond the gather."""
    pool2d = pool.reshape(pool.shape[0], -1)
    stride = pool2d.shape[1]
    need_rows = -(-count // stride)
    assert need_rows <= slot_rows, "matrix does not fit in its slot"
    rows = loc[base: base + need_rows]
    if hasattr(pool2d, "detach"):
        import torch
        got = pool2d[torch.as_tensor(rows, device=pool2d.device)]
    else:
        got = pool2d[rows]
    return _f32(got).reshape(-1)[:count]


def adapter_matrix_A(pool, a_start, a_len, a_loc, adapter, qkvo, h_in, rank_mult=1):
    """``[r, h_in]`` float32 shrink matrix of one adapter/projection, gathered through the tables.

    Follows ``bgmv_impl.cuh:34-38``: ``r = a_len[a] / 4``, ``mem_pos = a_start[a] + r * qkvo``,
    row ``j`` lives in pool row ``a_loc[mem_pos + j]``.  ``rank_mult`` > 1 (no counterpart in the reference): the slot
    holds ``rank_mult`` rows of ``h_in`` elements per pool row (an input-sharded A under tensor parallelism).
    """
    a_start, a_len, a_loc = _i64(a_start), _i64(a_len), _i64(a_loc)
    slot = int(a_len[adapter]) // 4
    r = slot * rank_mult
    base = int(a_start[adapter]) + slot * qkvo
    return _slot_flat(pool, a_loc, base, slot, r * h_in).reshape(r, h_in)


def adapter_matrix_B(pool, a_start, a_len, a_loc, adapter, qkvo, h_out, rank_mult=1):
    """``[h_out, r]`` float32 expand matrix (``lora_B.weight`` orientation), gathered through the tables.

    Follows ``bgmv_impl.cuh:174-179,191``: flat index ``f = o * r + k`` lives in pool row
    ``a_loc[mem_pos + f // stride]`` at column ``f % stride``.
    """
    a_start, a_len, a_loc = _i64(a_start), _i64(a_len), _i64(a_loc)
    slot = int(a_len[adapter]) // 4
    r = slot * rank_mult
    base = int(a_start[adapter]) + slot * qkvo
    return _slot_flat(pool, a_loc, base, slot, h_out * r).reshape(h_out, r)


def lora_shrink_ref(x, pool, a_start, a_len, a_loc, ids, qkvo, out_width=None, rank_mult=1):
    """Per-token shrink: ``delta[t, :r] = x[t] @ A_{ids[t], qkvo}.T``; columns ``>= r`` stay zero.

    The loop is the reference's own (``test_kernel_correctness_multi_rank.py:97-106``, part "A").
    """
    xf = _f32(x)
    ids = _i64(ids)
    a_len_i = _i64(a_len)
    T, h_in = xf.shape
    if out_width is None:
        out_width = int(a_len_i.max()) // 4 * rank_mult if a_len_i.size else 0
    out = np.zeros((T, out_width), dtype=np.float32)
    cache = {}
    for t in range(T):
        a = int(ids[t])
        if a not in cache:
            cache[a] = adapter_matrix_A(pool, a_start, a_len, a_loc, a, qkvo, h_in, rank_mult)
        A = cache[a]
        r = A.shape[0]
        out[t, :r] = xf[t:t + 1] @ A.T
    return out


def lora_expand_ref(y, delta, pool, a_start, a_len, a_loc, ids, qkvo, scales, rank_mult=1):
    """Per-token expand: ``y[t] + scale_a * delta[t, :r] @ B_{a, qkvo}.T`` (returns a new float32 array).

    The loop is the reference's own (``test_kernel_correctness_multi_rank.py:97-106``, part "B") plus the
    per-adapter scale of ``bgmv_impl.cuh:180,197``.
    """
    yf = _f32(y).copy()
    df = _f32(delta)
    sc = _f32(scales)
    ids = _i64(ids)
    T, h_out = yf.shape
    cache = {}
    for t in range(T):
        a = int(ids[t])
        if a not in cache:
            cache[a] = adapter_matrix_B(pool, a_start, a_len, a_loc, a, qkvo, h_out, rank_mult)
        B = cache[a]
        r = B.shape[1]
        yf[t] += (df[t:t + 1, :r] @ B.T)[0] * sc[a]
    return yf


def lora_delta_ref(y, x, pool_a, pool_b, a_start, a_len, a_loc, ids, qkvo, scales, h_out=None):
    """Shrink followed by expand, float32 throughout, no intermediate rounding (the parity oracle)."""
    if h_out is None:
        h_out = _f32(y).shape[1]
    d = lora_shrink_ref(x, pool_a, a_start, a_len, a_loc, ids, qkvo)
    return lora_expand_ref(y, d, pool_b, a_start, a_len, a_loc, ids, qkvo, scales)


def lora_delta_ref_rounding(y, x, pool_a, pool_b, a_start, a_len, a_loc, ids, qkvo, scales, dtype=np.float16):
    """As :func:`lora_delta_ref` but rounding the intermediate and the result to ``dtype`` the way the
    reference kernels do (``bgmv_impl.cuh:147`` stores the shrink result as T, ``:206`` does ``y(T) += float``)."""
    d = lora_shrink_ref(x, pool_a, a_start, a_len, a_loc, ids, qkvo).astype(dtype).astype(np.float32)
    out = lora_expand_ref(y, d, pool_b, a_start, a_len, a_loc, ids, qkvo, scales)
    return out.astype(dtype).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# Grouped (vectorised) restatement: same numbers, one matmul per distinct adapter instead of per token.
# Used where the per-token loop would take minutes (larger parity cases) and as a second CPU timing.
# ----------------------------------------------------------------------------------------------

def lora_delta_grouped(y, x, pool_a, pool_b, a_start, a_len, a_loc, ids, qkvo, scales):
    xf = _f32(x)
    yf = _f32(y).copy()
    sc = _f32(scales)
    ids = _i64(ids)
    h_in = xf.shape[1]
    h_out = yf.shape[1]
    for a in np.unique(ids):
        sel = np.nonzero(ids == a)[0]
        A = adapter_matrix_A(pool_a, a_start, a_len, a_loc, int(a), qkvo, h_in)
        B = adapter_matrix_B(pool_b, a_start, a_len, a_loc, int(a), qkvo, h_out)
        yf[sel] += (xf[sel] @ A.T) @ B.T * sc[a]
    return yf


def segments_to_token_ids(seg_start, seg_len, seg_adapter, total_tokens):
    """Per-token adapter ids of a batch given as request segments.

    Mirrors ``torch.repeat_interleave(req_bins, b_seq_len)`` in
    ``slora/models/peft/lora_unordered_batch_infer.py:66`` but honours explicit segment starts the way the
    prefill kernels index (``lora_prefill.py:31,77``).  Tokens covered by no segment get id -1.
    """
    ids = np.full((total_tokens,), -1, dtype=np.int64)
    for s, n, a in zip(_i64(seg_start), _i64(seg_len), _i64(seg_adapter)):
        ids[int(s): int(s) + int(n)] = int(a)
    return ids


# ----------------------------------------------------------------------------------------------
# Pool row content as the reference's loader writes it
# ----------------------------------------------------------------------------------------------

def pool_rows_from_hf(lora_A_weights, lora_B_weights):
    """Rows an adapter contributes to the A pool and the B pool, from HF-PEFT-shaped weights.

    ``lora_A_weights``: four arrays ``[r, h_in]`` (q, k, v, o); ``lora_B_weights``: four arrays ``[h_out, r]``.
    Returns ``(rows_a [4r, H], rows_b [4r, H])`` as ``lora_layer_weight.py:215-224`` lays them out
    (``w_combined_home`` reshaped to ``[2, 4r, heads, head_dim]``); requires ``h_in == h_out == H``.
    """
    r = lora_A_weights[0].shape[0]
    rows_a = np.concatenate([np.asarray(w, dtype=np.float32).reshape(r, -1) for w in lora_A_weights], axis=0)
    rows_b = np.concatenate([np.asarray(w, dtype=np.float32).reshape(-1).reshape(r, -1) for w in lora_B_weights],
                            axis=0)
    return rows_a, rows_b


def error_metrics(y, ref):
    """The two normalised errors the parity bar is stated in: ``max|y-ref| / max|ref|`` and
    ``mean|y-ref| / mean|ref|`` (element-wise relative error is unbounded near zeros of ``ref``)."""
    y = _f32(y).astype(np.float64)
    ref = _f32(ref).astype(np.float64)
    diff = np.abs(y - ref)
    max_ref = np.abs(ref).max()
    mean_ref = np.abs(ref).mean()
    max_rel = float(diff.max() / max_ref) if max_ref > 0 else float(diff.max())
    mean_rel = float(diff.mean() / mean_ref) if mean_ref > 0 else float(diff.mean())
    return max_rel, mean_rel
