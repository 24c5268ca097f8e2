"""Weight views handed to the CUDA decoder.

Replaces backends/megakernel/weights.py:120-183 of the reference: the tensors
are taken from the live nano-vLLM module (no second copy), but nano-vLLM's
fused ``qkv_proj`` / ``gate_up_proj`` matrices are kept fused (the kernels
stream them as one matrix) and the RoPE table stays fp32 like the torch path's
``cos_sin_cache`` (layers/rotary_embedding.py:27-35) instead of being rounded to
bf16.
"""

from __future__ import annotations

from dataclasses import dataclass, fields

import torch

from .geometry import ModelGeometry


@dataclass
class LayerTensors:
    ln_in: torch.Tensor
    wqkv: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    wo: torch.Tensor
    ln_post: torch.Tensor
    wgu: torch.Tensor
    wd: torch.Tensor


LAYER_FIELDS = tuple(f.name for f in fields(LayerTensors))


@dataclass
class DecoderWeights:
    geom: ModelGeometry
    embed: torch.Tensor          # [vocab, hidden] bf16, also the LM head
    layers: list[LayerTensors]
    final_norm: torch.Tensor
    cos_sin: torch.Tensor        # [max_model_len, head_dim] fp32
    # tensor-parallel shard (tensor_parallel.shard_weights): `geom` then holds the per-rank sizes, `embed`
    # stays the whole table of `embed_rows` rows and the rank's LM head starts at row `vocab_offset`
    embed_rows: int | None = None
    vocab_offset: int = 0

    def validate(self) -> None:
        g = self.geom
        expect = dict(ln_in=(g.hidden,), wqkv=(g.qkv_rows, g.hidden), q_norm=(g.head_dim,), k_norm=(g.head_dim,),
                      wo=(g.hidden, g.q_size), ln_post=(g.hidden,), wgu=(2 * g.intermediate, g.hidden),
                      wd=(g.hidden, g.intermediate))
        tensors = [("embed", self.embed, (self.embed_rows or g.vocab, g.hidden)), ("final_norm", self.final_norm, (g.hidden,))]
        if len(self.layers) != g.layers:
            raise RuntimeError(f"expected {g.layers} layers, got {len(self.layers)}")
        for i, layer in enumerate(self.layers):
            tensors += [(f"layers[{i}].{n}", getattr(layer, n), expect[n]) for n in LAYER_FIELDS]
        for name, t, shape in tensors:
            if t.dtype != torch.bfloat16:
                raise RuntimeError("Qwen Megakernel requires BF16 model weights")
            if tuple(t.shape) != shape:
                raise RuntimeError(f"{name} has shape {tuple(t.shape)}, expected {shape}")
            if not t.is_cuda or not t.is_contiguous() or t.data_ptr() % 16:
                raise RuntimeError(f"{name} must be a contiguous, 16-byte aligned CUDA tensor")
        if self.cos_sin.dtype != torch.float32 or tuple(self.cos_sin.shape) != (g.max_model_len, g.head_dim):
            raise RuntimeError("cos_sin must be fp32 [max_model_len, head_dim]")
        if not self.cos_sin.is_cuda or not self.cos_sin.is_contiguous():
            raise RuntimeError("cos_sin must be a contiguous CUDA tensor")


def rope_cos_sin_table(geom: ModelGeometry) -> torch.Tensor:
    """fp32 ``[max_model_len, head_dim]``, cos in the first half of each row
    and sin in the second, built with the reference's formula
    (layers/rotary_embedding.py:27-35)."""
    d = geom.head_dim
    inv_freq = 1.0 / (geom.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float, device="cpu") / d))
    t = torch.arange(geom.max_model_len, dtype=torch.float, device="cpu")
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous()


def geometry_from_hf_config(hf_config, max_model_len: int, block_size: int, rope_theta: float) -> ModelGeometry:
    head_dim = getattr(hf_config, "head_dim", None) or hf_config.hidden_size // hf_config.num_attention_heads
    return ModelGeometry(
        hidden=hf_config.hidden_size, layers=hf_config.num_hidden_layers, q_heads=hf_config.num_attention_heads,
        kv_heads=hf_config.num_key_value_heads, head_dim=head_dim, intermediate=hf_config.intermediate_size,
        vocab=hf_config.vocab_size, eps=float(hf_config.rms_norm_eps), rope_theta=float(rope_theta),
        max_model_len=int(max_model_len), block_size=int(block_size))


def _resolve_rope_theta(hf_config, default: float = 1_000_000.0) -> float:
    """Same precedence as the reference's rope_config.py:38-60: top-level
    ``rope_theta``, then one nested in ``rope_scaling`` / ``rope_parameters``,
    then Qwen3's 1e6."""
    def num(v):
        return float(v) if isinstance(v, (int, float)) and not isinstance(v, bool) else None
    for key in ("rope_theta", "rope_parameters"):
        v = num(getattr(hf_config, key, None))
        if v is not None:
            return v
    nested = getattr(hf_config, "rope_scaling", None) or getattr(hf_config, "rope_parameters", None)
    if isinstance(nested, dict):
        for key in ("rope_theta", "rope_parameters"):
            v = num(nested.get(key))
            if v is not None:
                return v
    return float(default)


def weights_from_nano_model(model, hf_config, max_model_len: int = 2048, block_size: int = 256) -> DecoderWeights:
    """Views of a loaded nano-vLLM ``Qwen3ForCausalLM`` (models/qwen3.py:190-220).
    Same checks and messages as the reference's weights.py:120-131."""
    qwen = model.model
    if qwen.embed_tokens.weight.dtype != torch.bfloat16:
        raise RuntimeError("Qwen Megakernel requires BF16 model weights")
    if getattr(hf_config, "attention_bias", False):
        raise RuntimeError("Qwen Megakernel requires Qwen QK normalization")
    if model.lm_head.weight.data_ptr() != qwen.embed_tokens.weight.data_ptr():
        raise RuntimeError("Qwen Megakernel requires tied lm_head and embed_tokens storage")
    geom = geometry_from_hf_config(hf_config, max_model_len, block_size, _resolve_rope_theta(hf_config))
    layers = []
    for layer in qwen.layers:
        attn = layer.self_attn
        layers.append(LayerTensors(
            ln_in=layer.input_layernorm.weight.data, wqkv=attn.qkv_proj.weight.data,
            q_norm=attn.q_norm.weight.data, k_norm=attn.k_norm.weight.data, wo=attn.o_proj.weight.data,
            ln_post=layer.post_attention_layernorm.weight.data, wgu=layer.mlp.gate_up_proj.weight.data,
            wd=layer.mlp.down_proj.weight.data))
    device = qwen.embed_tokens.weight.device
    # The model's own cos/sin cache when it has one (layers/rotary_embedding.py:27-35 builds it on whatever
    # device the engine constructs the model on, so its last bits can differ from a table computed elsewhere):
    # the decode kernels then rotate with exactly the values the torch path uses.
    cos_sin = None
    rotary = getattr(getattr(qwen.layers[0], "self_attn", None), "rotary_emb", None) if len(qwen.layers) else None
    cache = getattr(rotary, "cos_sin_cache", None)
    if torch.is_tensor(cache) and cache.dtype == torch.float32 and cache.numel() >= geom.max_model_len * geom.head_dim \
            and cache.shape[-1] == geom.head_dim:
        cos_sin = cache.reshape(-1, geom.head_dim)[: geom.max_model_len].to(device).contiguous()
    if cos_sin is None:
        cos_sin = rope_cos_sin_table(geom).to(device)
    return DecoderWeights(geom, qwen.embed_tokens.weight.data, layers, qwen.norm.weight.data, cos_sin)
