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


def prefill_attention(q, k, v, cu_seqlens_q, max_seqlen_q: int, softmax_scale: float, cu_seqlens_k=None,
                      block_table=None, status=None):
    """The reference's ``flash_attn_varlen_func(q, k, v, cu_seqlens_q=…, cu_seqlens_k=…, max_seqlen_q=…,
    softmax_scale=s, causal=True, block_table=…)`` of ``layers/attention.py:64-70``.  ``q`` ``[N, q_heads, 128]``
    bf16 (any row stride), ``cu_seqlens_*`` int32 CUDA ``[batch + 1]``.  Without ``block_table``: ``k`` / ``v``
    ``[N, kv_heads, 128]``, the projections of the same tokens.  With it (prefix cache): ``k`` / ``v`` are one
    layer's cache ``[num_blocks, block_size, kv_heads, 128]`` and ``block_table`` the int32 CUDA
    ``[batch, columns]`` table.  Returns ``[N, q_heads, 128]`` bf16."""
    import torch

    from . import native

    n, q_heads, head_dim = q.shape
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and q.stride(1) == head_dim
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("prefill_attention takes bf16 tensors")
    if cu_seqlens_q.dtype != torch.int32 or not cu_seqlens_q.is_cuda:
        raise TypeError("cu_seqlens_q must be an int32 CUDA tensor")
    if block_table is not None:
        num_blocks, block_size, kv_heads = k.shape[0], k.shape[1], k.shape[2]
        assert k.stride(2) == head_dim and v.stride(2) == head_dim and k.stride(0) == block_size * k.stride(1)
        if block_table.dtype != torch.int32 or block_table.stride(-1) != 1 or cu_seqlens_k is None:
            raise TypeError("the prefix-cache case needs an int32 block table and cu_seqlens_k")
        k_stride, v_stride = k.stride(1), v.stride(1)
        bt_ptr, bt_stride = block_table.data_ptr(), block_table.stride(0)
    else:
        kv_heads = k.shape[1]
        assert k.stride(1) == head_dim and v.stride(1) == head_dim
        num_blocks = block_size = 0
        k_stride, v_stride = k.stride(0), v.stride(0)
        bt_ptr, bt_stride = None, 0
    out = torch.empty(n, q_heads, head_dim, dtype=torch.bfloat16, device=q.device)
    if n == 0:
        return out
    native.check(native.lib().dfb_prefill_attention(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), cu_seqlens_q.data_ptr(),
        cu_seqlens_k.data_ptr() if cu_seqlens_k is not None else None, cu_seqlens_q.numel() - 1, int(max_seqlen_q),
        q.stride(0), k_stride, v_stride, out.stride(0), q_heads, kv_heads, head_dim, float(softmax_scale),
        bt_ptr, bt_stride, block_size, num_blocks, status.data_ptr() if status is not None else None,
        torch.cuda.current_stream().cuda_stream), "dfb_prefill_attention")
    return out
