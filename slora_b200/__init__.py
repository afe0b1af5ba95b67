"""slora_b200 -- B200-native multi-adapter LoRA shrink/expand behind S-LoRA's operator API.

Importing the package loads the CUDA shared library (``libslora_b200.so``); a missing library is an
ImportError, never a silent fallback.

Public surface (each item names the reference symbol it stands in for):

* ``dispatch_bgmv``                               -- ``slora._kernels.dispatch_bgmv``
* ``lora_get_qkvo_fwd_shrink`` / ``_expand``      -- ``slora.models.peft.triton_kernel.lora.lora_prefill``
* ``LoraBatchOps``                                -- the LoRA half of ``LoraUnorderedBatchInfer._batch_lora_get_qkv`` /
                                                     ``_batch_lora_get_o`` / ``_lora_get_qkv`` / ``_lora_get_o``
* ``MemoryAllocator``                             -- ``slora.common.mem_allocator.MemoryAllocator``
* ``InferAdapter``                                -- ``slora.server.router.model_infer.infer_adapter.InferAdapter``
* ``tp``                                          -- S-LoRA tensor parallelism for the adapter path
"""
from ._lib import EXPORTS, LIB_PATH, launch_counts, lib  # noqa: F401  (fails loudly when the library is not built)
from ._kernels import dispatch_bgmv, validate_tables  # noqa: F401
from .lora_prefill import lora_get_qkvo_fwd_expand, lora_get_qkvo_fwd_shrink  # noqa: F401
from .batch_infer import BatchPlan, LoraBatchOps  # noqa: F401
from .mem_allocator import MemoryAllocator  # noqa: F401
from .infer_adapter import InferAdapter  # noqa: F401

__version__ = "0.1.0"
