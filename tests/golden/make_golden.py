"""Writes tests/golden/cfg1_oracle.{npz,json}: known-answer vectors of the CPU oracle for configuration 1.

Run from the repository root:  python tests/golden/make_golden.py
The full [32, 4096] outputs are not stored; a fixed set of 64 columns of every projection plus each row's
absolute sum are (a few tens of KB), which pins both individual values and every element's contribution.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import lora_oracle as orc  # noqa: E402
from slora_b200.workloads import build_workload  # noqa: E402


def main():
    wl = build_workload(1)
    cols = list(range(0, 4096, 64))
    out = {}
    for p in range(4):
        x = wl.x_o[0] if p == 3 else wl.x_qkv[0]
        d = orc.lora_delta_ref(np.zeros((wl.T, 4096), np.float32), x, wl.pools_a[0], wl.pools_b[0], wl.a_start,
                               wl.a_len, wl.a_loc, wl.ids, p, wl.a_scaling)
        out[f"delta_p{p}"] = d[:, cols]
        out[f"rowabs_p{p}"] = np.abs(d).sum(axis=1)
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "cfg1_oracle.npz"), **out)
    json.dump({"ids": wl.ids.tolist(), "a_loc": wl.a_loc.tolist(), "columns": cols},
              open(os.path.join(here, "cfg1_oracle.json"), "w"))


if __name__ == "__main__":
    main()
