"""Generate the golden fixtures in this directory from the REFERENCE project.

Run once, in a container that has the reference checkout (it is read-only and
is never copied):

    python tests/golden/make_golden.py --reference /path/to/reference

What runs is the reference's own code, imported unmodified from
``<reference>/src``: ``nanovllm.models.qwen3.Qwen3ForCausalLM`` (and through it
every layer in ``nanovllm/layers``), ``nanovllm.layers.sampler.Sampler``,
``nanovllm.utils.context`` and the position / slot helpers of
``nanovllm.engine.kv_layout``.  Only ``Attention.forward``
(layers/attention.py:59-75) is replaced, because it hard-calls FlashAttention
and a Triton kernel that need a GPU; the replacement follows that method line
by line on the CPU (slot write by ``slot_mapping``, causal attention for
prefill, block-table gather for decode).  ``TORCHDYNAMO_DISABLE=1`` turns the
``@torch.compile`` decorators into plain Python.

The weights come from ``oracle.qwen3_decode.make_weights`` (numpy Philox, so the
test-suite can re-draw the identical tensors on any machine); only reference
OUTPUTS are stored here: token ids and logits.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]
sys.path.insert(0, str(REPO))

from oracle import qwen3_decode as O  # noqa: E402


def _import_reference(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import torch.distributed as dist

    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29611", rank=0, world_size=1)
    from nanovllm.models.qwen3 import Qwen3ForCausalLM
    from nanovllm.layers import attention as ref_attention
    from nanovllm.layers.sampler import Sampler
    from nanovllm.utils import context as ref_context
    from nanovllm.engine import kv_layout

    def cpu_attention_forward(self, q, k, v):
        # layers/attention.py:59-75 on the CPU.
        ctx = ref_context.get_context()
        k_cache, v_cache = self.k_cache, self.v_cache
        D = self.num_kv_heads * self.head_dim
        slots = ctx.slot_mapping.long()
        keep = slots >= 0  # store_kvcache_kernel skips slot -1 (:22)
        k_cache.view(-1, D)[slots[keep]] = k.reshape(-1, D)[keep]
        v_cache.view(-1, D)[slots[keep]] = v.reshape(-1, D)[keep]
        group = self.num_heads // self.num_kv_heads
        outs = []
        if ctx.is_prefill:
            cu = ctx.cu_seqlens_q.tolist()
            for a, b in zip(cu[:-1], cu[1:]):
                n = b - a
                qf = q[a:b].float().reshape(n, self.num_kv_heads, group, self.head_dim)
                s = torch.einsum("qhgd,thd->hgqt", qf, k[a:b].float()) * self.scale
                mask = torch.ones(n, n, dtype=torch.bool).tril()
                p = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)
                o = torch.einsum("hgqt,thd->qhgd", p, v[a:b].float())
                outs.append(o.reshape(n, self.num_heads, self.head_dim).to(q.dtype))
            return torch.cat(outs, 0)
        for r in range(q.shape[0]):
            n = int(ctx.context_lens[r])
            bs = k_cache.shape[1]
            nblk = (n + bs - 1) // bs
            idx = ctx.block_tables[r, :nblk].long()
            kk = k_cache[idx].reshape(-1, self.num_kv_heads, self.head_dim)[:n].float()
            vv = v_cache[idx].reshape(-1, self.num_kv_heads, self.head_dim)[:n].float()
            qf = q[r].float().reshape(self.num_kv_heads, group, self.head_dim)
            p = torch.softmax(torch.einsum("hgd,thd->hgt", qf, kk) * self.scale, dim=-1)
            o = torch.einsum("hgt,thd->hgd", p, vv)
            outs.append(o.reshape(1, self.num_heads, self.head_dim).to(q.dtype))
        return torch.cat(outs, 0)

    ref_attention.Attention.forward = cpu_attention_forward
    return Qwen3ForCausalLM, Sampler, ref_context, kv_layout


def _build_reference_model(Qwen3ForCausalLM, geom: O.Geometry, w: O.Weights, dtype):
    from transformers import Qwen3Config

    cfg = Qwen3Config(
        vocab_size=geom.vocab, hidden_size=geom.hidden, intermediate_size=geom.intermediate,
        num_hidden_layers=geom.layers, num_attention_heads=geom.q_heads,
        num_key_value_heads=geom.kv_heads, head_dim=geom.head_dim, hidden_act="silu",
        max_position_embeddings=geom.max_pos, rms_norm_eps=geom.eps, tie_word_embeddings=True,
        attention_bias=False,
        rope_parameters={"rope_theta": geom.rope_theta, "rope_type": "default"},
    )
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        model = Qwen3ForCausalLM(cfg)
    finally:
        torch.set_default_dtype(old)
    with torch.no_grad():
        model.model.embed_tokens.weight.copy_(w.embed)
        for layer, lw in zip(model.model.layers, w.layers):
            layer.input_layernorm.weight.copy_(lw.ln_in)
            layer.self_attn.qkv_proj.weight.copy_(lw.wqkv)
            layer.self_attn.q_norm.weight.copy_(lw.q_norm)
            layer.self_attn.k_norm.weight.copy_(lw.k_norm)
            layer.self_attn.o_proj.weight.copy_(lw.wo)
            layer.post_attention_layernorm.weight.copy_(lw.ln_post)
            layer.mlp.gate_up_proj.weight.copy_(lw.wgu)
            layer.mlp.down_proj.weight.copy_(lw.wd)
        model.model.norm.weight.copy_(w.final_norm)
    assert model.lm_head.weight.data_ptr() == model.model.embed_tokens.weight.data_ptr()
    return model.eval()


@torch.inference_mode()
def run_reference(ref, geom, w, dtype, prompts, steps, block_permutation=None, forced_inputs=None):
    """Prefill each prompt, then batched greedy decode, exactly the way
    engine/model_runner.py:227-289 prepares the inputs (positions, slot mapping,
    context lens, padded block tables)."""
    Qwen3ForCausalLM, Sampler, C, L = ref
    model = _build_reference_model(Qwen3ForCausalLM, geom, w, dtype)
    sampler = Sampler()
    bs = geom.block_size
    lengths = [len(p) + steps for p in prompts]
    tables, nblocks = O.allocate_blocks(lengths, bs, block_permutation)
    pool = nblocks if block_permutation is None else len(block_permutation)
    kv = torch.zeros(2, geom.layers, pool, bs, geom.kv_heads, geom.head_dim, dtype=dtype)
    for i, layer in enumerate(model.model.layers):
        layer.self_attn.attn.k_cache = kv[0, i]
        layer.self_attn.attn.v_cache = kv[1, i]
    zero_t = torch.zeros(1)
    cur, lens = [], []
    for p, table in zip(prompts, tables):
        n = len(p)
        ids = torch.tensor(list(p), dtype=torch.int64)
        pos = torch.tensor(list(L.prefill_positions(0, n)), dtype=torch.int64)
        cu = torch.tensor([0, n], dtype=torch.int32)
        slots = torch.tensor(L.prefill_slot_mapping(table[: (n + bs - 1) // bs], 0, n, bs), dtype=torch.int32)
        C.set_context(True, cu, cu, n, n, slots, None, None)
        logits = model.compute_logits(model(ids, pos))
        cur.append(int(sampler(logits, zero_t)[0]))
        lens.append(n + 1)
        C.reset_context()
    toks, all_logits = [list(cur)], []
    for step in range(steps):
        if forced_inputs is not None:
            cur = [int(t) for t in forced_inputs[step]]
        nblk = [(n + bs - 1) // bs for n in lens]
        width = max(nblk)
        bt = torch.tensor([L.pad_block_table(t[:k], width) for t, k in zip(tables, nblk)], dtype=torch.int32)
        ids = torch.tensor(cur, dtype=torch.int64)
        pos = torch.tensor([L.decode_position(n) for n in lens], dtype=torch.int64)
        slots = torch.tensor([L.decode_slot_mapping(t[:k], n, bs) for t, k, n in zip(tables, nblk, lens)], dtype=torch.int32)
        clen = torch.tensor([L.decode_cache_len(n) for n in lens], dtype=torch.int32)
        C.set_context(False, slot_mapping=slots, context_lens=clen, block_tables=bt)
        logits = model.compute_logits(model(ids, pos))
        nxt = sampler(logits, torch.zeros(len(cur))).tolist()
        C.reset_context()
        all_logits.append(logits.float().clone())
        cur = [int(t) for t in nxt]
        lens = [n + 1 for n in lens]
        toks.append(list(cur))
    return np.asarray(toks, dtype=np.int64), torch.stack(all_logits).numpy()


def config1_prompt(geom: O.Geometry) -> list[int]:
    """Prompt of BASELINE config 1: 32 ids uniform in [0, vocab), seed 0."""
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, geom.vocab, (32,), generator=g).tolist()


SMALL = O.Geometry(layers=2, vocab=2048)
SMALL_PROMPT_LENS = (5, 255, 300)
SMALL_STEPS = 6


def small_prompts() -> list[list[int]]:
    rng = np.random.Generator(np.random.Philox(key=7))
    return [rng.integers(0, SMALL.vocab, n).tolist() for n in SMALL_PROMPT_LENS]


FORCED_PROMPT_LENS = (20, 250)
FORCED_STEPS = 8


def forced_case(geom: O.Geometry):
    """Teacher-forced case at the full geometry: two rows, the second crossing
    the 256-token block boundary while decoding; every decode input is a seeded
    random token so the trajectory is not the degenerate repeated-token one."""
    rng = np.random.Generator(np.random.Philox(key=5))
    prompts = [rng.integers(0, geom.vocab, n).tolist() for n in FORCED_PROMPT_LENS]
    forced = rng.integers(0, geom.vocab, (FORCED_STEPS, len(prompts))).tolist()
    return prompts, forced


def _summarise(logits, probe):
    """Per (step, row): logits at the probe indices and the top-8 entries."""
    top = np.argsort(-logits, axis=-1, kind="stable")[..., :8]
    return dict(probe_logits=logits[..., probe].astype(np.float32), top_index=top,
                top_logits=np.take_along_axis(logits, top, -1).astype(np.float32))


def sampler_fixture(ref) -> None:
    """The reference's ``Sampler.forward`` (layers/sampler.py:7-16) on seeded
    logits with greedy and sampled rows.  The exponential noise it draws is
    stored too: the generator is re-seeded, the same-shaped fp32 draw is taken
    once outside and once (after re-seeding again) inside the sampler."""
    Sampler = ref[1]
    rows, vocab = 6, 1024
    torch.manual_seed(1234)
    logits = (torch.randn(rows, vocab) * 3.0).to(torch.bfloat16)
    temps = torch.tensor([0.0, 1e-12, 0.5, 0.7, 1.0, 1.6], dtype=torch.float32)
    tokens, noises = [], []
    for draw in range(8):
        torch.manual_seed(9000 + draw)
        noises.append(torch.empty(rows, vocab, dtype=torch.float32).exponential_(1))
        torch.manual_seed(9000 + draw)
        tokens.append(Sampler()(logits, temps))
    np.savez_compressed(HERE / "sampler_rows6_vocab1024.npz", logits=logits.float().numpy(), temperatures=temps.numpy(),
                        noise=torch.stack(noises).numpy(), tokens=torch.stack(tokens).numpy().astype(np.int64))
    print("sampler tokens", torch.stack(tokens).tolist())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (the directory holding src/nanovllm)")
    ap.add_argument("--skip-full", action="store_true")
    ap.add_argument("--only-sampler", action="store_true", help="write only the sampler fixture")
    args = ap.parse_args()
    ref = _import_reference(args.reference)
    sampler_fixture(ref)
    if args.only_sampler:
        return

    # (B) small geometry, three rows crossing the 256-token block boundary,
    # blocks scattered by a permutation; fp32 and bf16 activations.
    w32 = O.make_weights(SMALL, seed=1, norm="random")
    perm = np.random.Generator(np.random.Philox(key=3)).permutation(8).tolist()
    for name, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        w = w32 if dtype == torch.float32 else w32.to(dtype)
        toks, logits = run_reference(ref, SMALL, w, dtype, small_prompts(), SMALL_STEPS, perm)
        np.savez_compressed(HERE / f"small_l2_v2048_{name}.npz", tokens=toks, logits=logits.astype(np.float32),
                            perm=np.asarray(perm))
        print(name, "small tokens", toks.tolist())

    if args.skip_full:
        return
    # (A) BASELINE config 1: full geometry, fp32, prompt 32, 64 greedy tokens.
    geom = O.QWEN3_06B
    w = O.make_weights(geom, seed=0, norm="ones")
    toks, logits = run_reference(ref, geom, w, torch.float32, [config1_prompt(geom)], 64)
    probe = np.random.Generator(np.random.Philox(key=11)).choice(geom.vocab, 256, replace=False)
    probe.sort()
    # (C) full geometry, bf16 (the dtype the CUDA backend runs), teacher forced.
    prompts, forced = forced_case(geom)
    ftoks, flogits = run_reference(ref, geom, w.to(torch.bfloat16), torch.bfloat16, prompts, FORCED_STEPS,
                                   forced_inputs=forced)
    np.savez_compressed(HERE / "qwen3_06b_bf16_forced8.npz", tokens=ftoks, probe_index=probe,
                        **_summarise(flogits, probe))
    print("forced bf16 tokens", ftoks.tolist())
    lg = logits[:, 0, :]
    top = np.argsort(-lg, axis=-1, kind="stable")[:, :8]
    np.savez_compressed(
        HERE / "qwen3_06b_fp32_prompt32_greedy64.npz",
        prompt=np.asarray(config1_prompt(geom)), tokens=toks[:, 0],
        probe_index=probe, probe_logits=lg[:, probe].astype(np.float32),
        top_index=top, top_logits=np.take_along_axis(lg, top, -1).astype(np.float32),
    )
    print("config1 tokens", toks[:, 0].tolist())


if __name__ == "__main__":
    main()
