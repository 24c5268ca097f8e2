"""B200 (sm_100a) Qwen3 greedy decode step behind ``decode_backend="megakernel"``.

Importing this package never touches CUDA; the native library is loaded when a
decoder is built (``native.lib()``), and that fails loudly if it is missing.
"""

from .backend import (
    Compatibility,
    MegakernelBackend,
    QWEN3_CONTRACT,
    cuda_arch_for_capability,
    is_megakernel_backend,
    qwen3_contract_mismatch,
)
from .contracts import PagedKVCacheSpec, row_active_mask
from .decoder import TG_MAX_BATCH, TaskGraphCompatibility, taskgraph_compatibility
from .dispatch import DecodeDispatch
from .geometry import QWEN3_06B, ModelGeometry

__all__ = [
    "Compatibility", "DecodeDispatch", "MegakernelBackend", "ModelGeometry", "PagedKVCacheSpec",
    "QWEN3_06B", "QWEN3_CONTRACT", "TG_MAX_BATCH", "TaskGraphCompatibility",
    "cuda_arch_for_capability", "is_megakernel_backend", "qwen3_contract_mismatch",
    "row_active_mask", "taskgraph_compatibility",
]
