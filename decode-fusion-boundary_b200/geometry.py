"""Model geometry of the decode step and the byte accounting derived from it."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ModelGeometry:
    """Shape contract of the compiled kernels.  The defaults are Qwen3-0.6B
    (reference: backends/megakernel/backend.py:35-45, QWEN3_CONTRACT)."""

    hidden: int = 1024
    layers: int = 28
    q_heads: int = 16
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 3072
    vocab: int = 151936
    eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    max_model_len: int = 2048
    block_size: int = 256

    @property
    def q_size(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def qkv_rows(self) -> int:
        return self.q_size + 2 * self.kv_size

    @property
    def max_pages(self) -> int:
        return max(1, -(-self.max_model_len // self.block_size))

    def layer_weight_bytes(self) -> int:
        """bf16 bytes of one layer: four matrices plus its four norm vectors
        (reference: model_spec.py:214-233)."""
        h, i = self.hidden, self.intermediate
        return 2 * (self.qkv_rows * h + h * self.q_size + 2 * i * h + h * i + 2 * h + 2 * self.head_dim)

    def lm_head_bytes(self) -> int:
        return 2 * self.vocab * self.hidden

    def weight_bytes_per_step(self) -> int:
        """Weight bytes one decode step must stream: 1,192,099,840 for
        Qwen3-0.6B (reference: roofline.py:471-487).  The tied embedding is
        counted once, as the LM head; the rows gathered per token are not."""
        return self.layers * self.layer_weight_bytes() + 2 * self.hidden + self.lm_head_bytes()

    def kv_bytes_per_token(self) -> int:
        """KV bytes read per attended context token per step: 114,688
        (reference: roofline.py:540-548)."""
        return 2 * self.layers * self.kv_size * 2

    def step_bytes(self, contexts) -> int:
        """Algorithmic HBM bytes of one step for rows attending ``contexts``
        tokens each (the new token included)."""
        return self.weight_bytes_per_step() + self.kv_bytes_per_token() * int(sum(contexts))


QWEN3_06B = ModelGeometry()
