"""CPU oracle for the two steps that follow the q/k/v expand in the reference's layer: the rotary embedding of q and k
and the scatter of the new k / v rows into the KV pool.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; the tests call it as the checker.

What it restates, in numpy (paths inside the S-LoRA reference tree):

* ``rotary_emb_fwd`` (``slora/models/llama/triton_kernel/rotary_emb.py:8-71``; the same arithmetic as the file's own
  torch statement ``torch_rotary_emb``, ``:74-82``): for every token and head, with ``x0`` the first half of the head
  and ``x1`` the second half, ``out0 = x0 * cos - x1 * sin`` and ``out1 = x0 * sin + x1 * cos``, ``cos`` / ``sin``
  being ``[tokens, head_dim / 2]`` (``infer_state.position_cos / position_sin``).  Applied to q and k right after their
  LoRA expand (``slora/models/peft/lora_unordered_batch_infer.py:277,298``).
* ``destindex_copy_kv`` (``slora/common/basemodel/triton_kernel/destindex_copy_kv.py:8-50``): row ``t`` of ``K``
  goes to row ``dest[t]`` of ``Out`` (``transformer_layer_infer_template.py:50-62``).

Parity pin: ``tests/golden/ref_rope.npz`` holds outputs of the reference's own two Triton kernels (run unmodified under
Triton's interpreter on the host by ``tests/golden/make_rope_golden.py``); ``tests/test_rope_oracle.py`` holds this
file to them.  Arithmetic here is float32 throughout; the reference computes in the tensors' 16-bit type, so the
comparison carries one 16-bit rounding per operation.
"""
from __future__ import annotations

import numpy as np


def rotary_ref(x, cos, sin):
    """``x``: ``[T, heads, head_dim]`` (or ``[T, heads * head_dim]`` with ``head_dim = 2 * cos.shape[1]``); returns
    float32 of the same shape."""
    x = np.asarray(x, dtype=np.float32)
    cos = np.asarray(cos, dtype=np.float32)
    sin = np.asarray(sin, dtype=np.float32)
    shape = x.shape
    T, half = cos.shape
    x3 = x.reshape(T, -1, 2 * half)
    x0, x1 = x3[:, :, :half], x3[:, :, half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate((x0 * c - x1 * s, x0 * s + x1 * c), axis=-1).reshape(shape)


def destindex_copy_ref(k, dest, out):
    """Returns a copy of ``out`` with ``out[dest[t]] = k[t]``."""
    res = np.array(out, copy=True)
    res[np.asarray(dest, dtype=np.int64)] = np.asarray(k).astype(res.dtype)
    return res
