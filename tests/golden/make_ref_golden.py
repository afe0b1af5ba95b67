"""Writes reference-produced golden vectors: outputs of the REFERENCE's own BGMV CUDA kernels on seeded inputs.

Needs a GPU and oracle/_ref/libref_bgmv.so (built by `make -C oracle` where the reference tree is present).
Run from the repository root:  python tests/golden/make_ref_golden.py <output.npz>
The committed copy is tests/golden/ref_kernels.npz; tests/test_oracle.py checks the CPU oracle against it and
tests/test_gpu_parity.py checks this library against it.
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from slora_b200.workloads import build_workload  # noqa: E402

CASES = {
    # name: build_workload keyword arguments (pool row width == hidden, which the reference kernels need)
    "cfg1": dict(cfg=1),
    "mixed": dict(cfg=3, pool_rows=4096, n_adapters=6, decode_tokens=24, prefill=None, rank_choices=(16, 64)),
    # hidden 5120 (the S4 shape; 5120 x 64 is in the reference's shape list, bgmv_config.h:21), ranks 16 / 32 / 64
    "wide5120": dict(cfg=4, pool_rows=4096, n_adapters=6, decode_tokens=24, prefill=None, rank_choices=(16, 32, 64)),
}
COLS = list(range(0, 4096, 64))


def cols_of(hidden):
    """Output columns kept in the fixture (every 64th)."""
    return list(range(0, hidden, 64))


def ref_lib():
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_bgmv.so"))
    lib.ref_dispatch_bgmv.restype = ctypes.c_int
    lib.ref_dispatch_bgmv.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                                             ctypes.c_int, ctypes.c_void_p]
    return lib


def run_reference(lib, w, p):
    """The reference's two dispatch_bgmv calls for projection p (lora_unordered_batch_infer.py:266-274)."""
    R, H = w.max_rank, w.spec.hidden
    x = w.x_o[0] if p == 3 else w.x_qkv[0]
    delta = torch.zeros((w.T, R), dtype=torch.float16, device="cuda")
    y = torch.zeros((w.T, H), dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    for out, inp, pool, hi, ho in ((delta, x, w.pools_a[0], H, R), (y, delta, w.pools_b[0], R, H)):
        rc = lib.ref_dispatch_bgmv(out.data_ptr(), inp.data_ptr(), pool.data_ptr(), w.a_start.data_ptr(),
                                   w.a_len.data_ptr(), w.a_loc.data_ptr(), w.ids.data_ptr(), p, w.T, hi, ho,
                                   w.a_scaling.data_ptr())
        assert rc == 0, rc
    torch.cuda.synchronize()
    return delta, y


def main(out_path):
    lib = ref_lib()
    out = {}
    for name, kw in CASES.items():
        w = build_workload(**kw).to("cuda")
        for p in range(4):
            delta, y = run_reference(lib, w, p)
            out[f"{name}_delta_p{p}"] = delta.cpu().numpy()
            out[f"{name}_y_p{p}"] = y[:, cols_of(w.spec.hidden)].cpu().numpy()
            out[f"{name}_rowabs_p{p}"] = y.float().abs().sum(dim=1).cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "ref_kernels.npz")
