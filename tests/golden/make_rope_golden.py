"""Golden vectors of the rotary embedding and the KV-pool scatter, produced by the reference's own Triton kernels.

    SLORA_REFERENCE=/path/to/S-LoRA  python tests/golden/make_rope_golden.py

Runs ``rotary_emb_fwd`` (``slora/models/llama/triton_kernel/rotary_emb.py``) and ``destindex_copy_kv``
(``slora/common/basemodel/triton_kernel/destindex_copy_kv.py``), imported unmodified from the reference tree, under
Triton's interpreter on the host (``TRITON_INTERPRET=1``) on seeded fp16 inputs and stores inputs and outputs in
``tests/golden/ref_rope.npz``.  ``tests/test_rope_oracle.py`` holds ``oracle/rope_oracle.py`` to them; the GPU tests
hold the CUDA epilogue to the oracle.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = os.environ.get("SLORA_REFERENCE")
    if not ref or not os.path.isdir(os.path.join(ref, "slora")):
        raise SystemExit("set SLORA_REFERENCE to the root of the S-LoRA reference tree")
    sys.path.insert(0, ref)
    from slora.common.basemodel.triton_kernel.destindex_copy_kv import destindex_copy_kv
    from slora.models.llama.triton_kernel.rotary_emb import rotary_emb_fwd
    g = torch.Generator().manual_seed(91)
    out = {}
    for name, (T, heads, D) in {"a": (37, 4, 128), "b": (5, 3, 64)}.items():
        x = torch.randn((T, heads, D), generator=g).to(torch.float16)
        pos = torch.randint(0, 2048, (T,), generator=g).float()
        inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))       # slora/models/llama/model.py:110-120
        freqs = torch.outer(pos, inv)
        cos, sin = torch.cos(freqs).to(torch.float16), torch.sin(freqs).to(torch.float16)
        out[f"{name}_x"], out[f"{name}_cos"], out[f"{name}_sin"] = x.numpy().copy(), cos.numpy(), sin.numpy()
        y = x.clone()
        rotary_emb_fwd(y, cos, sin)
        out[f"{name}_rotary"] = y.numpy()
        dest = torch.randperm(3 * T, generator=g)[:T]
        pool = torch.full((3 * T, heads, D), 9.0, dtype=torch.float16)
        destindex_copy_kv(y, dest, pool)
        out[f"{name}_dest"], out[f"{name}_pool"] = dest.numpy(), pool.numpy()
    np.savez_compressed(os.path.join(HERE, "ref_rope.npz"), **out)
    print("wrote ref_rope.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
