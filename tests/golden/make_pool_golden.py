"""Golden traces of the pool bookkeeping, produced by the reference's own Python code.

    SLORA_REFERENCE=/path/to/S-LoRA  python tests/golden/make_pool_golden.py

Runs the reference's ``MemoryAllocator`` (``slora/common/mem_allocator.py``: ``alloc`` :30-39, ``alloc_contiguous``
:42-59, ``free`` :185-199) and ``InferAdapter`` (``slora/server/router/model_infer/infer_adapter.py``:
``load_adapters`` :92-171, ``offload_adapters`` :186-250 with its Triton variable-length copy :261-280) UNMODIFIED,
imported from the reference tree, on seeded sequences of steps, and stores what they leave behind after every step
(row lists handed out, free map, tables, free-row count) and the pool buffers at the end in
``tests/golden/ref_pool.npz``.  ``tests/test_pool_oracle.py`` holds ``oracle/pool_oracle.py`` and the host mirror to
these traces on CPU; ``tests/test_gpu_pool.py`` holds the CUDA kernels to them.

The reference hard-codes ``device="cuda"``; here it runs on the host: a ``TorchFunctionMode`` rewrites that one keyword
to ``"cpu"`` on the way into torch, and the Triton copy kernel runs under Triton's interpreter
(``TRITON_INTERPRET=1``).  Integer and byte work only, so the device does not change a single bit of the results.
Needs the reference tree (not shipped with this repository) and nothing else.
"""
import json
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np  # noqa: E402
import torch  # noqa: E402
from torch.overrides import TorchFunctionMode  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# Traces: name -> (pool rows, layers, heads, head_dim, adapter ranks, seed, number of steps)
TRACES = {
    "small": (1500, 2, 2, 16, [8, 64, 16, 32, 8, 16, 64, 8], 11, 40),
    "ragged": (20000, 1, 1, 8, [8, 16, 32, 64, 128, 8, 8, 16, 32, 64, 16, 8], 12, 60),
}


class CudaToCpu(TorchFunctionMode):
    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = dict(kwargs or {})
        if "device" in kwargs and str(kwargs["device"]).startswith("cuda"):
            kwargs["device"] = "cpu"
        return func(*args, **kwargs)


class _Layer:
    def __init__(self, w):
        self.w_combined = w

    def load_to_gpu(self, prefetch=False):
        pass

    def offload_from_gpu(self):
        pass


class _Adapter:
    """What ``InferAdapter`` reads of a ``LoraTpPartAdapter`` (``slora/models/peft/lora_adapter.py:20-65``)."""

    def __init__(self, name, r, heads, hd, layers, seed):
        g = torch.Generator().manual_seed(seed)
        self.lora_dir, self.r, self.scaling = name, r, 16.0 / r
        self.network_config = {"hidden_size": heads * hd, "num_attention_heads": heads, "num_hidden_layers": layers}
        self.layers = [_Layer(torch.randn((2, 4 * r, heads, hd), generator=g).to(torch.float16)) for _ in range(layers)]


def draw_steps(n_adapters, tot, seed, count):
    """A seeded sequence of steps.  A step the reference refuses (it raises when the pool is short) is recorded as
    refused by the replay below; sizes are drawn so that most steps go through."""
    rng = np.random.default_rng(seed)
    steps, held = [], 0
    for _ in range(count):
        kind = rng.choice(["load", "prefetch", "offload", "alloc", "free", "alloc_contiguous"],
                          p=[0.25, 0.1, 0.25, 0.2, 0.15, 0.05])
        if kind in ("load", "prefetch"):
            steps.append([str(kind), sorted(set(rng.integers(0, n_adapters, size=int(rng.integers(1, 5))).tolist()))])
        elif kind == "offload":
            steps.append(["offload", [i for i in range(n_adapters) if rng.random() < 0.4]])
        elif kind == "alloc":
            steps.append(["alloc", int(rng.integers(0, tot // 6 + 1))])
            held += 1
        elif kind == "free":
            if held:
                steps.append(["free", int(rng.integers(0, held)), float(rng.random())])
        else:
            steps.append(["alloc_contiguous", int(rng.integers(1, 40))])
            held += 1
    return steps


def run_trace(MemoryAllocator, InferAdapter, name):
    tot, layers, heads, hd, ranks, seed, count = TRACES[name]
    ads = [_Adapter(f"a{i}", r, heads, hd, layers, 1000 * seed + i) for i, r in enumerate(ranks)]
    mm = MemoryAllocator(tot, 0, torch.float16, heads, hd, layers)
    for l in range(layers):
        mm.key_buffer[l].fill_(3.0)
        mm.value_buffer[l].fill_(5.0)
    ia = InferAdapter.init(mm, None)
    steps = draw_steps(len(ranks), tot, seed, count)
    out, held, done = {}, [], []
    for k, step in enumerate(steps):
        kind = step[0]
        rows = np.empty(0, dtype=np.int64)
        try:
            if kind in ("load", "prefetch"):
                ia.load_adapters([ads[i] for i in step[1]], prefetch=(kind == "prefetch"))
            elif kind == "offload":
                ia.offload_adapters([f"a{i}" for i in step[1]])
            elif kind == "alloc":
                got = mm.alloc(step[1])
                held.append(got)
                rows = got.numpy().copy()
            elif kind == "free":
                got = held[step[1]]
                part = got[: int(len(got) * step[2])]
                held[step[1]] = got[len(part):]
                mm.free(part)
                rows = part.numpy().copy()
            else:
                got = mm.alloc_contiguous(step[1])
                if got is None:
                    rows = np.array([-1], dtype=np.int64)
                    held.append(torch.empty(0, dtype=torch.long))
                else:
                    held.append(got[0])
                    rows = np.array([got[1], got[2]], dtype=np.int64)
        except Exception as e:  # the reference raises when the pool is short: the step is recorded as refused
            rows = np.array([-2], dtype=np.int64)
            if kind in ("alloc", "alloc_contiguous"):
                held.append(torch.empty(0, dtype=torch.long))
            step = step + [f"raised: {type(e).__name__}: {str(e)[:80]}"]
        done.append(step)
        out[f"{name}_s{k}_rows"] = rows
        out[f"{name}_s{k}_mem_state"] = mm.mem_state.numpy().astype(np.uint8).copy()
        out[f"{name}_s{k}_free"] = np.array([int(mm.can_use_mem_size)], dtype=np.int64)
        out[f"{name}_s{k}_a_loc"] = ia.a_loc.numpy().copy()
        out[f"{name}_s{k}_a_start"] = ia.a_start.numpy().copy()
        out[f"{name}_s{k}_a_len"] = ia.a_len.numpy().copy()
        out[f"{name}_s{k}_a_scaling"] = ia.a_scaling.numpy().copy()
        out[f"{name}_s{k}_dirs"] = np.array([int(d[1:]) for d in ia.adapter_dirs], dtype=np.int64)
    # pool contents of the rows adapters own at the end (the other rows keep the fill values)
    for l in range(layers):
        out[f"{name}_key_l{l}"] = mm.key_buffer[l].reshape(tot, -1).numpy().copy()
        out[f"{name}_value_l{l}"] = mm.value_buffer[l].reshape(tot, -1).numpy().copy()
    return out, done


def main():
    ref = os.environ.get("SLORA_REFERENCE")
    if not ref or not os.path.isdir(os.path.join(ref, "slora")):
        raise SystemExit("set SLORA_REFERENCE to the root of the S-LoRA reference tree")
    sys.path.insert(0, ref)
    arrays, meta = {}, {"traces": {}}
    with CudaToCpu():
        from slora.common.mem_allocator import MemoryAllocator
        from slora.server.router.model_infer.infer_adapter import InferAdapter
        import contextlib
        import io
        for name in TRACES:
            with contextlib.redirect_stdout(io.StringIO()):       # the reference prints a line per call
                out, steps = run_trace(MemoryAllocator, InferAdapter, name)
            arrays.update(out)
            tot, layers, heads, hd, ranks, seed, _ = TRACES[name]
            meta["traces"][name] = {"tot": tot, "layers": layers, "heads": heads, "head_dim": hd, "ranks": ranks,
                                    "seed": seed, "steps": steps}
    np.savez_compressed(os.path.join(HERE, "ref_pool.npz"), **arrays)
    with open(os.path.join(HERE, "ref_pool.json"), "w") as f:
        json.dump(meta, f)
    print("wrote ref_pool.npz / ref_pool.json:", {k: len(v["steps"]) for k, v in meta["traces"].items()})


if __name__ == "__main__":
    main()
