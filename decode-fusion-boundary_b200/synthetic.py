"""Seeded random-init weights of a given geometry, for benchmarks and smoke
runs without a checkpoint (the reference's own benchmarks use seeded synthetic
inputs: benchmarks/compare.py:69-71)."""

from __future__ import annotations

import numpy as np
import torch

from .geometry import ModelGeometry
from .weights import DecoderWeights, LayerTensors, rope_cos_sin_table


def random_init_weights(geom: ModelGeometry, seed: int = 0, std: float = 0.02, norm: str = "ones",
                        device: str = "cuda") -> DecoderWeights:
    """Every matrix N(0, std) from numpy's Philox stream (platform independent),
    drawn in the order embed, then per layer ln_in, wqkv, q_norm, k_norm, wo,
    ln_post, wgu, wd, then the final norm; cast to bf16.  RMSNorm weights are
    1.0 (``norm="ones"``) or 1 + 0.1 N(0, 1) (``norm="random"``)."""
    rng = np.random.Generator(np.random.Philox(key=seed))

    def mat(rows: int, cols: int) -> torch.Tensor:
        a = rng.standard_normal((rows, cols), dtype=np.float32)
        a *= np.float32(std)
        return torch.from_numpy(a).to(torch.bfloat16).to(device)

    def vec(n: int) -> torch.Tensor:
        if norm == "ones":
            return torch.ones(n, dtype=torch.bfloat16, device=device)
        a = rng.standard_normal(n, dtype=np.float32)
        return torch.from_numpy(1.0 + 0.1 * a).float().to(torch.bfloat16).to(device)

    embed = mat(geom.vocab, geom.hidden)
    layers = []
    for _ in range(geom.layers):
        layers.append(LayerTensors(
            ln_in=vec(geom.hidden), wqkv=mat(geom.qkv_rows, geom.hidden), q_norm=vec(geom.head_dim),
            k_norm=vec(geom.head_dim), wo=mat(geom.hidden, geom.q_size), ln_post=vec(geom.hidden),
            wgu=mat(2 * geom.intermediate, geom.hidden), wd=mat(geom.hidden, geom.intermediate)))
    return DecoderWeights(geom, embed, layers, vec(geom.hidden), rope_cos_sin_table(geom).to(device))


class _Holder:
    """Attribute bag standing in for an ``nn.Module`` (only ``.weight`` /
    ``.data`` style access is needed by ``weights_from_nano_model``)."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


def nano_model_view(w: DecoderWeights):
    """An object tree with nano-vLLM's ``Qwen3ForCausalLM`` attribute layout
    (reference: models/qwen3.py:122-207) over the tensors of ``w``, so the
    backend can be driven exactly like it is by ``ModelRunner`` without loading
    a checkpoint.  Returns ``(model, hf_config)``."""
    g = w.geom
    P = lambda t: _Holder(weight=_Holder(data=t, dtype=t.dtype, device=t.device, data_ptr=t.data_ptr))
    layers = []
    for l in w.layers:
        attn = _Holder(qkv_proj=P(l.wqkv), q_norm=P(l.q_norm), k_norm=P(l.k_norm), o_proj=P(l.wo),
                       q_size=g.q_size, kv_size=g.kv_size)
        mlp = _Holder(gate_up_proj=P(l.wgu), down_proj=P(l.wd))
        layers.append(_Holder(self_attn=attn, mlp=mlp, input_layernorm=P(l.ln_in),
                              post_attention_layernorm=P(l.ln_post)))
    embed = P(w.embed)
    model = _Holder(model=_Holder(embed_tokens=embed, layers=layers, norm=P(w.final_norm)), lm_head=embed)
    hf_config = _Holder(model_type="qwen3", hidden_size=g.hidden, intermediate_size=g.intermediate,
                        num_hidden_layers=g.layers, num_attention_heads=g.q_heads,
                        num_key_value_heads=g.kv_heads, vocab_size=g.vocab, head_dim=g.head_dim,
                        rms_norm_eps=g.eps, rope_theta=g.rope_theta, tie_word_embeddings=True,
                        attention_bias=False)
    return model, hf_config
