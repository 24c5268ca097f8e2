"""Torch-free host contracts the decode step relies on.

Restated from three small reference modules so the backend and its tests have
one place to look:

* paged KV layout and offsets  -- backends/megakernel/cache.py:16-119
* per-row activation mask      -- backends/megakernel/row_contract.py:32-52
* decode position / slot rules -- engine/kv_layout.py:132-197

(paths under ``src/nanovllm/`` of the reference).  Names and error behaviour
match the reference so its contract tests read the same here.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence


@dataclass(frozen=True)
class PagedKVCacheSpec:
    """Shape and strides (in elements) of one K or V view
    ``[layers, blocks, block_size, kv_heads, head_dim]`` of the engine's cache
    tensor ``[2, layers, blocks, block_size, kv_heads, head_dim]``."""

    num_layers: int
    num_blocks: int
    block_size: int
    num_kv_heads: int
    head_dim: int
    dtype_itemsize: int

    def __post_init__(self) -> None:
        for name in ("num_layers", "num_blocks", "block_size", "num_kv_heads", "head_dim", "dtype_itemsize"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")

    @property
    def shape(self) -> tuple[int, ...]:
        return (2, self.num_layers, self.num_blocks, self.block_size, self.num_kv_heads, self.head_dim)

    @property
    def head_stride(self) -> int:
        return self.head_dim

    @property
    def token_stride(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def block_stride(self) -> int:
        return self.block_size * self.token_stride

    @property
    def layer_stride(self) -> int:
        return self.num_blocks * self.block_stride

    @property
    def total_elements(self) -> int:
        return self.num_layers * self.layer_stride

    @property
    def total_bytes(self) -> int:
        return 2 * self.total_elements * self.dtype_itemsize

    def physical_slot(self, block_table: Sequence[int], logical_position: int) -> tuple[int, int]:
        """``(physical block, offset in block)`` of a logical token position."""
        if logical_position < 0:
            raise IndexError("position must be non-negative")
        if not block_table:
            raise ValueError("block table must not be empty")
        page, offset = divmod(logical_position, self.block_size)
        if page >= len(block_table):
            raise IndexError("position is outside the block table")
        block = int(block_table[page])
        if block < 0 or block >= self.num_blocks:
            raise ValueError("block table contains an invalid physical block")
        return block, offset

    def element_offset(self, layer: int, block_table: Sequence[int], logical_position: int,
                       kv_head: int, head_dim_index: int) -> int:
        """Flat element offset inside one K or V view (what the kernel computes)."""
        if not 0 <= layer < self.num_layers:
            raise IndexError("layer is outside the cache")
        if not 0 <= kv_head < self.num_kv_heads:
            raise IndexError("kv_head is outside the cache")
        if not 0 <= head_dim_index < self.head_dim:
            raise IndexError("head dimension is outside the cache")
        block, offset = self.physical_slot(block_table, logical_position)
        return (layer * self.layer_stride + block * self.block_stride + offset * self.token_stride
                + kv_head * self.head_stride + head_dim_index)


def row_active_mask(active_rows: Iterable[object] | None, batch_size: int) -> list[int]:
    """0/1 mask for a launch of ``batch_size`` rows.  ``None`` activates every
    row.  An inactive row skips its KV-cache write and nothing else; a mask of
    the wrong length, or one with no active row, is a caller bug."""
    if batch_size < 1:
        raise ValueError(f"batch_size must be >= 1; got {batch_size}")
    if active_rows is None:
        return [1] * batch_size
    mask = [int(bool(v)) for v in active_rows]
    if len(mask) != batch_size:
        raise ValueError(f"active_rows has {len(mask)} entries for a {batch_size}-row launch")
    if sum(mask) == 0:
        raise ValueError("active_rows activates no row; there is nothing to launch")
    return mask


def decode_position(num_tokens: int) -> int:
    """RoPE position (= pre-decode KV length) of the token a decode step
    computes, for a sequence that already counts that token."""
    if num_tokens < 1:
        raise ValueError(f"num_tokens must be at least 1; got {num_tokens}")
    return num_tokens - 1


def decode_cache_seqlens(num_tokens: int) -> int:
    return decode_position(num_tokens)


def decode_cache_len(num_tokens: int) -> int:
    """KV entries attended by the step (the new token included)."""
    if num_tokens < 1:
        raise ValueError(f"num_tokens must be at least 1; got {num_tokens}")
    return num_tokens


def decode_slot_mapping(block_table: Sequence[int], num_tokens: int, block_size: int) -> int:
    """Flat slot ``block * block_size + offset`` the step's K/V is written to.
    The table must hold exactly the blocks ``num_tokens`` tokens need."""
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    if num_tokens < 1:
        raise ValueError(f"num_tokens must be at least 1; got {num_tokens}")
    need = -(-num_tokens // block_size)
    if len(block_table) != need:
        raise RuntimeError(
            f"decode of {num_tokens} tokens needs {need} blocks but the block table has {len(block_table)}; "
            "BlockManager.may_append() must run before the model call")
    return block_table[-1] * block_size + (num_tokens - 1) % block_size


def pad_block_table(block_table: Iterable[int], max_pages: int) -> list[int]:
    """Right-pad with physical block 0 (never -1: the kernel forms addresses
    from every entry it is told to read)."""
    table = list(block_table)
    if len(table) > max_pages:
        raise ValueError(f"block table has {len(table)} pages but the stride is {max_pages}")
    return table + [0] * (max_pages - len(table))


def max_pages_per_seq(max_model_len: int, block_size: int) -> int:
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    return max(1, -(-max_model_len // block_size))
