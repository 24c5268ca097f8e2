"""``MegakernelBackend``: the adapter nano-vLLM's ``ModelRunner`` talks to.

Drop-in for the reference class of the same name
(backends/megakernel/backend.py:104-258): same constructor, attributes
(``decoder``, ``kv_cache``, ``disabled_reason``), methods and error behaviour;
the internals build a :class:`StreamDecoder` over the native sm_100a library
instead of JIT-compiling the cooperative task-graph kernel.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .contracts import PagedKVCacheSpec, decode_position
from .decoder import taskgraph_compatibility

MAX_BATCH_SIZE = 8
MEGAKERNEL_BACKENDS = ("megakernel",)
# Architectures this build's kernels are compiled for (the reference lists
# sm_70..sm_90 and sm_120, backend.py:18).
VALID_CUDA_ARCHES = {"sm_100"}

# Fixed shape contract of the compiled kernels (backend.py:35-45).
QWEN3_CONTRACT = {
    "model_type": "qwen3",
    "hidden_size": 1024,
    "intermediate_size": 3072,
    "num_hidden_layers": 28,
    "num_attention_heads": 16,
    "num_key_value_heads": 8,
    "vocab_size": 151936,
    "max_model_len": 2048,
    "head_dim": 128,
}


def is_megakernel_backend(value: Any) -> bool:
    """Whether ``value`` selects the megakernel decode path (backend.py:25-28)."""
    return value in MEGAKERNEL_BACKENDS


def _get_attr(obj: Any, name: str, default: Any = None) -> Any:
    return getattr(obj, name, default)


def qwen3_contract_mismatch(config) -> str | None:
    """Name of the first contract field ``config`` violates, else ``None``
    (backend.py:48-75: tie_word_embeddings, attention_bias, then the table)."""
    hf = _get_attr(config, "hf_config")
    if _get_attr(hf, "tie_word_embeddings", True) is not True:
        return "tie_word_embeddings"
    if _get_attr(hf, "attention_bias", False) is not False:
        return "attention_bias"
    for name, expected in QWEN3_CONTRACT.items():
        if name == "max_model_len":
            actual = _get_attr(config, "max_model_len", 2048)
        elif name == "head_dim":
            actual = _get_attr(hf, "head_dim", None)
            if actual is None:
                actual = hf.hidden_size // hf.num_attention_heads
        else:
            actual = _get_attr(hf, name)
        if actual != expected:
            return name
    return None


@dataclass(frozen=True)
class Compatibility:
    supported: bool
    reason: str = ""


def cuda_arch_for_capability(capability: tuple[int, int]) -> str:
    """``-arch`` name for a device capability; raises ``ValueError`` for one the
    kernels are not built for (backend.py:84-97)."""
    major, minor = capability
    arch = f"sm_{major}{minor}"
    if arch not in VALID_CUDA_ARCHES:
        raise ValueError(f"unsupported CUDA capability: {major}.{minor}")
    return arch


class MegakernelBackend:
    """Lazy adapter around the native single-step decoder."""

    def __init__(self, config, model):
        self.config = config
        self.model = model
        self.decoder = None
        self.kv_cache = None
        self.disabled_reason = None

    @staticmethod
    def compatibility(config, seqs, is_prefill: bool) -> Compatibility:
        decision = taskgraph_compatibility(config, seqs, is_prefill)
        if not decision.supported:
            return Compatibility(False, decision.reason)
        mismatch = qwen3_contract_mismatch(config)
        if mismatch is not None:
            return Compatibility(False, f"unsupported Qwen config: {mismatch}")
        return Compatibility(True)

    def set_kv_cache(self, kv_cache) -> None:
        """Attach the engine-owned ``[K/V, layer, block, token, head, dim]`` cache."""
        if kv_cache is None or kv_cache.dim() != 6 or kv_cache.shape[0] != 2:
            raise ValueError("kv_cache must have shape [2, layers, blocks, tokens, heads, dim]")
        self.kv_cache = kv_cache

    def disable(self, reason: str) -> None:
        self.disabled_reason = reason

    @property
    def ready(self) -> bool:
        return self.decoder is not None

    def ensure_ready(self) -> None:
        """Build the decoder eagerly (called at ModelRunner start-up, after the
        KV cache is attached).  Raises on any failure; the caller then calls
        :meth:`disable` and stays on the torch path."""
        self._ensure_decoder()

    def _validate_cache_layout(self) -> None:
        """The kernels index one contiguous ``[layers, blocks, block_size,
        kv_heads, head_dim]`` view per K and V (backend.py:148-190)."""
        kv = self.kv_cache
        hf = self.config.hf_config
        head_dim = getattr(hf, "head_dim", None) or (hf.hidden_size // hf.num_attention_heads)
        spec = PagedKVCacheSpec(
            num_layers=hf.num_hidden_layers, num_blocks=kv.shape[2], block_size=self.config.kvcache_block_size,
            num_kv_heads=kv.shape[4], head_dim=kv.shape[5], dtype_itemsize=kv.element_size())
        if tuple(kv.shape) != spec.shape:
            raise RuntimeError(
                f"paged KV cache shape {tuple(kv.shape)} does not match the megakernel contract {spec.shape}")
        if not (kv[0].is_contiguous() and kv[1].is_contiguous()):
            raise RuntimeError(
                "paged KV cache views must be contiguous for the megakernel layer-stride offset math")
        if kv[0].size(0) * spec.layer_stride != kv[0].numel():
            raise RuntimeError("paged KV cache layer stride does not match the megakernel offset contract")
        if head_dim != QWEN3_CONTRACT["head_dim"]:
            raise RuntimeError("Qwen head_dim differs from the megakernel contract")

    def _ensure_decoder(self):
        if self.disabled_reason:
            raise RuntimeError(self.disabled_reason)
        if self.decoder is not None:
            return
        if self.kv_cache is None:
            raise RuntimeError("nano-vLLM KV cache has not been attached")

        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("Megakernel requires a CUDA device")
        capability = torch.cuda.get_device_capability()
        if capability[0] != 10:
            raise RuntimeError(
                "this megakernel build targets B200 (sm_100a); "
                f"detected sm_{capability[0]}{capability[1]}")
        self._validate_cache_layout()

        from . import native
        from .decoder import StreamDecoder
        from .weights import weights_from_nano_model

        native.lib()  # loud failure when the CUDA library is missing
        max_model_len = _get_attr(self.config, "max_model_len", 2048)
        weights = weights_from_nano_model(
            self.model, self.config.hf_config, max_model_len=max_model_len,
            block_size=self.config.kvcache_block_size)
        # Tensor parallel (this build's extension of the reference's tensor_parallel_size == 1 rule,
        # taskgraph.py:119-122): the rank's nano-vLLM modules already hold its shards of the projections and
        # of the vocabulary (layers/linear.py:54-153, layers/embed_head.py); the decoder needs the local
        # shapes plus the whole embedding table for the token gather, collected once here.
        group = _get_attr(self.config, "megakernel_tensor_parallel", None)
        if group is not None and getattr(group, "size", 1) > 1:
            from .tensor_parallel import localize_nano_weights

            weights = localize_nano_weights(weights, group)
        else:
            group = None
        self.decoder = StreamDecoder(
            weights,
            k_cache=self.kv_cache[0],
            v_cache=self.kv_cache[1],
            block_size=self.config.kvcache_block_size,
            num_cache_blocks=self.kv_cache.shape[2],
            max_model_len=max_model_len,
            attn_splits=int(_get_attr(self.config, "megakernel_attn_splits", 1)),
            fusion_groups=int(_get_attr(self.config, "fusion_groups", 1)),
            verbose=bool(_get_attr(self.config, "megakernel_verbose", False)),
            debug_bounds=bool(_get_attr(self.config, "megakernel_debug_bounds", False)),
            tensor_parallel=group,
        )
        seed = _get_attr(self.config, "megakernel_seed", None)
        if seed is not None:
            self.decoder.set_seed(int(seed))
        if _get_attr(self.config, "megakernel_warm", True) and group is None:   # sharded decoders capture lazily
            # every step geometry this engine can ask for is captured now, as ModelRunner.capture_cudagraph does
            # for the torch path (engine/model_runner.py:379-416): 160 graphs, about 0.1 s and 70 MB at 8 rows
            rows = min(int(_get_attr(self.config, "max_num_seqs", 8) or 8), 8)
            kinds = self.decoder.WARM_HOST | self.decoder.WARM_DEVICE_TOKENS
            if _get_attr(self.config, "megakernel_sampling", False):
                kinds |= self.decoder.WARM_SAMPLING
            self.decoder.warm(max_rows=max(rows, 1), max_context=max_model_len, kinds=kinds)

    def decode_batch(self, input_ids, positions, block_tables, temperatures=None) -> list[int]:
        """Decode one token for each scheduler-selected sequence.  ``temperatures``
        (not passed by the stock ``ModelRunner.run``): the float32 CUDA tensor of
        ``ModelRunner.prepare_sample``; rows above 1e-10 are sampled."""
        self._ensure_decoder()
        if temperatures is not None:
            return self.decoder.decode_rows(input_ids, positions, block_tables, temperatures=temperatures)
        return self.decoder.decode_rows(input_ids, positions, block_tables)

    def decode(self, seq, block_table) -> list[int]:
        """Decode one token for one sequence and return a one-element list.  The
        new K/V goes into the scheduler-owned paged cache; earlier positions are
        read from that same cache (no prompt replay, no private cache)."""
        self._ensure_decoder()
        temperature = 0.0
        if _get_attr(self.config, "megakernel_sampling", False):
            # admitted by the opt-in of ``taskgraph_compatibility``; a greedy row stays on the plain argmax
            temperature = float(getattr(seq, "temperature", 0.0) or 0.0)
        if temperature > 1e-10:
            return [int(self.decoder.step(seq.last_token, position=decode_position(len(seq)),
                                          block_table=block_table, temperature=temperature))]
        return [int(self.decoder.step(seq.last_token, position=decode_position(len(seq)), block_table=block_table))]
