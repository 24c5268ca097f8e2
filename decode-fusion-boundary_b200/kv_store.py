"""``store_kvcache`` of the reference (layers/attention.py:33-40) on the CUDA
library: the K / V rows of the prompt tokens of a prefill go to their slots of
the shared paged cache.  Same signature and the same checks; the work is done
by ``dfb_store_kvcache`` (no Triton, no CPU fallback)."""

from __future__ import annotations


def store_kvcache(key, value, k_cache, v_cache, slot_mapping, status=None) -> None:
    """``key`` / ``value``: ``[N, kv_heads, head_dim]`` bf16 CUDA tensors (any row
    stride); ``k_cache`` / ``v_cache``: one layer's ``[num_blocks, block_size,
    kv_heads, head_dim]`` views; ``slot_mapping``: int32 ``[N]``, -1 = skip.
    ``status``: optional int32 CUDA tensor ``[4]`` that receives a bad slot."""
    import torch

    from . import native

    n, num_heads, head_dim = key.shape
    d = num_heads * head_dim
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == head_dim and value.stride(1) == head_dim
    assert k_cache.stride(1) == d and v_cache.stride(1) == d
    assert slot_mapping.numel() == n
    if key.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise TypeError("store_kvcache moves bf16 rows")
    if slot_mapping.dtype != torch.int32 or not slot_mapping.is_cuda:
        raise TypeError("slot_mapping must be an int32 CUDA tensor")
    if n == 0:
        return
    num_slots = k_cache.shape[0] * k_cache.shape[1]
    native.check(native.lib().dfb_store_kvcache(
        key.data_ptr(), value.data_ptr(), key.stride(0), value.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        slot_mapping.data_ptr(), n, d, num_slots, status.data_ptr() if status is not None else None,
        torch.cuda.current_stream().cuda_stream), "dfb_store_kvcache")
