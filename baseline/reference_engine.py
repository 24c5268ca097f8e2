#!/usr/bin/env python
"""Drives the UNMODIFIED reference engine (nano-vLLM fork, installed by
``baseline/install_reference.sh`` into ``baseline/_ref``) on a GPU:

* ``write_model_dir``: a synthetic model directory the reference loads offline
  (config.json of the Qwen3-0.6B geometry, a dummy tokenizer, safetensors with
  the HF parameter names and the seeded N(0, 0.02) bf16 weights the rest of this
  repository uses);
* ``time_decode``: the reference's torch decode path with CUDA graphs
  (``LLM(dir, decode_backend="torch", enforce_eager=False)``, the
  "torch-cudagraph" arm of benchmarks/compare.py:34-47,198-203) on seeded
  token-id prompts, timed three ways per decode step: the reference's own
  CUDA-event span around ``ModelRunner.run`` (metrics.py:120-157, which includes
  the host's staging gaps), the wall clock, and the sum of the GPU kernel
  durations from ``torch.profiler`` (graph replay + the LM-head GEMM + the
  sampler that run outside the graph, engine/model_runner.py:292-313,374) --
  the last one is the number most favourable to the reference;
* ``install_backend_switch``: the one-line import switch a maintainer would make
  in ``engine/model_runner.py:10-13``, applied to the loaded reference modules, after which ``decode_backend="megakernel"``
  builds THIS repository's backend inside the reference's ``ModelRunner``.

This file is benchmark / test infrastructure: nothing in the product package
imports it.  Run as a script it prints one JSON object:

    python baseline/reference_engine.py --points 1:1,1:512,8:512 --steps 64
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
REF_DIR = HERE / "_ref"


def available() -> bool:
    return (REF_DIR / "nanovllm" / "__init__.py").exists()


def import_reference():
    """Put ``baseline/_ref`` on the path and import the reference package."""
    if not available():
        raise RuntimeError(f"{REF_DIR} is missing: run `sh baseline/install_reference.sh` where the checkout exists")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import nanovllm

    return nanovllm


def write_model_dir(path, seed: int = 0, layers: int = 28, vocab: int = 151936, norm: str = "ones") -> Path:
    """A model directory for the reference's loader (utils/loader.py:12-28,
    models/qwen3.py:191-197: q/k/v and gate/up are separate tensors that it packs;
    a tied checkpoint has no ``lm_head.weight``).  Weights come from the same
    Philox stream, in the same order, as ``synthetic.random_init_weights``."""
    import numpy as np
    import torch
    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    hidden, q_heads, kv_heads, head_dim, inter = 1024, 16, 8, 128, 3072
    config = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": hidden,
        "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": q_heads,
        "num_key_value_heads": kv_heads, "head_dim": head_dim, "vocab_size": vocab, "hidden_act": "silu",
        "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"}, "rope_scaling": None,
        "tie_word_embeddings": True, "attention_bias": False, "dtype": "bfloat16", "torch_dtype": "bfloat16",
        "bos_token_id": 1, "eos_token_id": 2, "use_cache": True,
    }
    (path / "config.json").write_text(json.dumps(config, indent=1))
    # dummy tokenizer: prompts are passed as token-id lists, only eos_token_id is read
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    words = {"<unk>": 0, "<s>": 1, "</s>": 2}
    words.update({f"w{i}": i for i in range(3, 64)})
    tok = Tokenizer(WordLevel(words, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(path / "tokenizer.json"))
    (path / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "bos_token": "<s>", "eos_token": "</s>"}))
    (path / "special_tokens_map.json").write_text(json.dumps(
        {"unk_token": "<unk>", "bos_token": "<s>", "eos_token": "</s>"}))

    rng = np.random.Generator(np.random.Philox(key=seed))

    def mat(rows, cols):
        a = rng.standard_normal((rows, cols), dtype=np.float32)
        a *= np.float32(0.02)
        return torch.from_numpy(a).to(torch.bfloat16)

    def vec(n):
        if norm == "ones":
            return torch.ones(n, dtype=torch.bfloat16)
        return torch.from_numpy(1.0 + 0.1 * rng.standard_normal(n, dtype=np.float32)).float().to(torch.bfloat16)

    q_size, kv_size = q_heads * head_dim, kv_heads * head_dim
    tensors = {"model.embed_tokens.weight": mat(vocab, hidden)}
    for i in range(layers):
        p = f"model.layers.{i}."
        tensors[p + "input_layernorm.weight"] = vec(hidden)
        wqkv = mat(q_size + 2 * kv_size, hidden)
        tensors[p + "self_attn.q_proj.weight"] = wqkv[:q_size].contiguous()
        tensors[p + "self_attn.k_proj.weight"] = wqkv[q_size:q_size + kv_size].contiguous()
        tensors[p + "self_attn.v_proj.weight"] = wqkv[q_size + kv_size:].contiguous()
        tensors[p + "self_attn.q_norm.weight"] = vec(head_dim)
        tensors[p + "self_attn.k_norm.weight"] = vec(head_dim)
        tensors[p + "self_attn.o_proj.weight"] = mat(hidden, q_size)
        tensors[p + "post_attention_layernorm.weight"] = vec(hidden)
        wgu = mat(2 * inter, hidden)
        tensors[p + "mlp.gate_proj.weight"] = wgu[:inter].contiguous()
        tensors[p + "mlp.up_proj.weight"] = wgu[inter:].contiguous()
        tensors[p + "mlp.down_proj.weight"] = mat(hidden, inter)
    tensors["model.norm.weight"] = vec(hidden)
    save_file(tensors, str(path / "model.safetensors"))
    return path


STORE_KVCACHE_CALLS = [0]   # calls of this repository's store_kvcache made by the reference's Attention.forward
PREFILL_ATTENTION_CALLS = [0]   # ... and of its prefill attention


def install_backend_switch(store_kvcache: bool = True):
    """The import switch of ``engine/model_runner.py:10-13`` applied at run time: the reference's
    ``ModelRunner`` (engine/model_runner.py:10-13,80-95,315-376) then builds this
    repository's ``MegakernelBackend`` for ``decode_backend="megakernel"``.  With ``store_kvcache`` the
    reference's ``Attention.forward`` (layers/attention.py:59-64) also writes the prompt tokens' K / V into the
    shared paged cache through this repository's kernel instead of its Triton kernel, and runs the causal
    attention of every prefill (with or without a prefix cache) on this repository's kernel instead of FlashAttention."""
    import_reference()
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    import __graft_entry__  # noqa: F401  (registers the package as dfb_b200)
    import dfb_b200
    from nanovllm.engine import model_runner

    model_runner.MegakernelBackend = dfb_b200.MegakernelBackend
    model_runner.is_megakernel_backend = dfb_b200.is_megakernel_backend
    if store_kvcache:
        from dfb_b200 import kv_store
        from nanovllm.layers import attention

        def counted_store(key, value, k_cache, v_cache, slot_mapping):
            STORE_KVCACHE_CALLS[0] += 1
            kv_store.store_kvcache(key, value, k_cache, v_cache, slot_mapping)

        attention.store_kvcache = counted_store
        library_attention = attention.flash_attn_varlen_func

        def prefill_attention(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k, softmax_scale,
                              causal, block_table=None):
            # both cases of the reference's call: K / V as the projections of the same tokens, or (prefix cache)
            # as the layer's cache read through the block table
            if causal:
                PREFILL_ATTENTION_CALLS[0] += 1
                return kv_store.prefill_attention(q, k, v, cu_seqlens_q, max_seqlen_q, softmax_scale,
                                                  cu_seqlens_k=cu_seqlens_k, block_table=block_table)
            return library_attention(q, k, v, max_seqlen_q=max_seqlen_q, cu_seqlens_q=cu_seqlens_q,
                                     max_seqlen_k=max_seqlen_k, cu_seqlens_k=cu_seqlens_k,
                                     softmax_scale=softmax_scale, causal=causal, block_table=block_table)

        attention.flash_attn_varlen_func = prefill_attention
    return model_runner


def seeded_prompts(batch: int, prompt_len: int, vocab: int, seed: int):
    import numpy as np

    rng = np.random.Generator(np.random.Philox(key=seed))
    return [rng.integers(3, vocab, prompt_len).tolist() for _ in range(batch)]


def make_llm(model_dir, backend: str = "torch", max_num_seqs: int = 8, enforce_eager: bool = False,
             gpu_memory_utilization: float = 0.25):
    nanovllm = import_reference()
    return nanovllm.LLM(str(model_dir), decode_backend=backend, enforce_eager=enforce_eager,
                        max_num_seqs=max_num_seqs, max_model_len=2048,
                        gpu_memory_utilization=gpu_memory_utilization)


def generate(llm, prompts, max_tokens: int):
    """Greedy generation through the reference's public API; returns the token
    id lists and the reference's own metrics report."""
    from nanovllm import SamplingParams

    sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
    result = llm.generate_with_metrics(prompts, sp, use_tqdm=False)
    return [o["token_ids"] for o in result["outputs"]], result["metrics"]


def time_decode(llm, batch: int, prompt_len: int, steps: int, vocab: int = 151936, warmup_runs: int = 2,
                runs: int = 3):
    """One point of the torch-cudagraph arm: ``batch`` seeded prompts of
    ``prompt_len`` ids, ``steps`` greedy tokens each (the first comes from the
    prefill, so ``steps - 1`` decode steps)."""
    import torch

    for w in range(warmup_runs):
        generate(llm, seeded_prompts(batch, prompt_len, vocab, 1000 + w), min(steps, 16))
    ev, wall, backend = [], [], None
    for r in range(runs):
        prompts = seeded_prompts(batch, prompt_len, vocab, 2000 + r)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        _, report = generate(llm, prompts, steps)
        torch.cuda.synchronize()
        s = report["summary"]
        n = max(int(s["decode_steps"]), 1)
        ev.append(1e3 * s["cuda_decode_time_ms_total"] / n)
        wall.append(1e3 * s["decode_time_ms_total"] / n)
        backend = report["requests"][0]["backend_actual"]
        del t0
    # GPU-busy time per decode step: every kernel the reference launches (graph replay, LM head, sampler,
    # the staging copies), prefill excluded by profiling a run whose prompt was already timed above
    busy_us = None
    try:
        from torch.profiler import ProfilerActivity, profile

        prompts = seeded_prompts(batch, prompt_len, vocab, 3000)
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            _, report = generate(llm, prompts, steps)
            torch.cuda.synchronize()
        n = max(int(report["summary"]["decode_steps"]), 1)
        total = sum(e.device_time_total for e in prof.key_averages() if e.device_time_total)
        # subtract the prefill's share, measured by its own CUDA-event span (one prefill step, dense kernels)
        prefill_us = 1e3 * report["summary"]["cuda_prefill_time_ms_total"]
        busy_us = max(total - prefill_us, 0.0) / n
    except Exception as exc:  # profiler problems must not lose the event numbers
        busy_us = f"unavailable: {type(exc).__name__}: {exc}"[:160]
    ev.sort(); wall.sort()
    return {"batch": batch, "prompt": prompt_len, "decode_steps": steps - 1, "backend_actual": backend,
            "cuda_event_us_per_step": ev[len(ev) // 2], "cuda_event_us_min": ev[0], "cuda_event_us_max": ev[-1],
            "host_wall_us_per_step": wall[len(wall) // 2], "gpu_busy_us_per_step": busy_us, "runs": runs}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--points", default="1:1,1:512,2:512,4:512,8:512,8:1920",
                    help="comma-separated batch:prompt_len pairs")
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    out = {"arm": "reference torch-cudagraph (unmodified nanovllm from baseline/_ref)", "points": []}
    if not available():
        out["unavailable"] = f"{REF_DIR} missing"
        print(json.dumps(out), flush=True)
        return
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    tmp = None
    model_dir = args.model_dir
    if not model_dir:
        tmp = tempfile.TemporaryDirectory(prefix="dfb_model_")
        model_dir = write_model_dir(tmp.name, seed=args.seed)
    try:
        import torch

        llm = make_llm(model_dir, "torch", max_num_seqs=8)
        out["gpu"] = torch.cuda.get_device_name()
        for item in args.points.split(","):
            b, p = (int(x) for x in item.split(":"))
            steps = min(args.steps, 2048 - p)
            try:
                out["points"].append(time_decode(llm, b, p, steps))
            except Exception as exc:
                out["points"].append({"batch": b, "prompt": p, "unavailable": f"{type(exc).__name__}: {exc}"[:200]})
        llm.exit()
    except Exception as exc:
        out["unavailable"] = f"{type(exc).__name__}: {exc}"[:300]
    print(json.dumps(out), flush=True)
    if tmp is not None:
        tmp.cleanup()


if __name__ == "__main__":
    main()
