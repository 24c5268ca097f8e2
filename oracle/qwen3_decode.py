"""CPU restatement of the reference torch path for one Qwen3 decode step.

TEST INFRASTRUCTURE: the checker for the CUDA decode backend, never part of it.

Every function cites the reference file:line (paths inside the reference
project, under ``src/nanovllm/``) whose arithmetic and rounding points it
follows.  All math is done in fp32 on the CPU; ``act_dtype`` selects where the
reference would round: ``torch.float32`` reproduces the fp32 reference run,
``torch.bfloat16`` reproduces every bf16 rounding point of the bf16 run
(residual stream, norm output, each GEMM output, RoPE output, attention output,
SwiGLU output, logits).

Weight layout follows the reference's fused modules: ``wqkv`` is ``[q|k|v]``
rows (``layers/linear.py`` QKVParallelLinear), ``wgu`` is ``[gate|up]`` rows
(MergedColumnParallelLinear), every matrix is ``[out, in]`` row-major.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class Geometry:
    """Model shape.  Defaults are the Qwen3-0.6B contract
    (backends/megakernel/backend.py:35-45)."""

    hidden: int = 1024
    layers: int = 28
    q_heads: int = 16
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 3072
    vocab: int = 151936
    eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    max_pos: int = 2048
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

    def weight_bytes_per_step(self, itemsize: int = 2) -> int:
        """Bytes of weights one decode step streams (tied embedding counted
        once, as the LM head): roofline.py:471-487, model_spec.py:214-243."""
        per_layer = (
            self.qkv_rows * self.hidden
            + self.hidden * self.q_size
            + 2 * self.intermediate * self.hidden
            + self.hidden * self.intermediate
            + 2 * self.hidden
            + 2 * self.head_dim
        )
        return itemsize * (self.layers * per_layer + self.hidden + self.vocab * self.hidden)

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        """KV bytes read per attended token per step: roofline.py:540-548."""
        return 2 * self.layers * self.kv_size * itemsize


QWEN3_06B = Geometry()


@dataclass
class LayerWeights:
    ln_in: torch.Tensor
    wqkv: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    wo: torch.Tensor
    ln_post: torch.Tensor
    wgu: torch.Tensor
    wd: torch.Tensor


@dataclass
class Weights:
    geom: Geometry
    embed: torch.Tensor
    layers: list[LayerWeights]
    final_norm: torch.Tensor
    dtype: torch.dtype = torch.float32
    _f32: dict = field(default_factory=dict, repr=False)

    def f32(self, t: torch.Tensor) -> torch.Tensor:
        """fp32 view of a (possibly bf16) weight, cached so the matmuls below
        run at fp32 BLAS speed while holding exactly the stored values."""
        if t.dtype == torch.float32:
            return t
        key = t.data_ptr()
        got = self._f32.get(key)
        if got is None:
            got = t.float()
            self._f32[key] = got
        return got

    def to(self, dtype: torch.dtype) -> "Weights":
        """Cast (not re-draw) every tensor, e.g. the bf16 copy of fp32 weights."""
        c = lambda t: t.to(dtype)
        return Weights(
            self.geom,
            c(self.embed),
            [LayerWeights(*(c(getattr(l, f)) for f in LayerWeights.__dataclass_fields__)) for l in self.layers],
            c(self.final_norm),
            dtype,
        )


def make_weights(geom: Geometry, seed: int = 0, std: float = 0.02, norm: str = "ones") -> Weights:
    """Seeded random-init fp32 weights: every linear / embedding matrix drawn
    N(0, std); RMSNorm weights 1.0 (``norm="ones"``) or 1 + 0.1 N(0,1)
    (``norm="random"``, used by kernel tests so the weight multiply is
    exercised).  numpy's Philox bit generator is used because its stream does
    not depend on the host CPU, so fixtures made on one machine can be checked
    on another."""

    rng = np.random.Generator(np.random.Philox(key=seed))

    def mat(rows: int, cols: int) -> torch.Tensor:
        a = rng.standard_normal((rows, cols), dtype=np.float32)
        a *= np.float32(std)
        return torch.from_numpy(a)

    def vec(n: int) -> torch.Tensor:
        if norm == "ones":
            return torch.ones(n, dtype=torch.float32)
        a = rng.standard_normal(n, dtype=np.float32)
        return torch.from_numpy(1.0 + 0.1 * a).float()

    embed = mat(geom.vocab, geom.hidden)
    layers = []
    for _ in range(geom.layers):
        layers.append(
            LayerWeights(
                ln_in=vec(geom.hidden),
                wqkv=mat(geom.qkv_rows, geom.hidden),
                q_norm=vec(geom.head_dim),
                k_norm=vec(geom.head_dim),
                wo=mat(geom.hidden, geom.q_size),
                ln_post=vec(geom.hidden),
                wgu=mat(2 * geom.intermediate, geom.hidden),
                wd=mat(geom.hidden, geom.intermediate),
            )
        )
    return Weights(geom, embed, layers, vec(geom.hidden))


def rope_cos_sin_table(geom: Geometry) -> torch.Tensor:
    """fp32 ``[max_pos, head_dim]`` table, ``cos`` in the first half and ``sin``
    in the second: layers/rotary_embedding.py:27-35."""
    d = geom.head_dim
    inv_freq = 1.0 / (geom.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float) / d))
    t = torch.arange(geom.max_pos, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous()


def new_kv_cache(geom: Geometry, num_blocks: int, dtype: torch.dtype) -> torch.Tensor:
    """``[2, layers, blocks, block_size, kv_heads, head_dim]``:
    engine/model_runner.py:203."""
    return torch.zeros(2, geom.layers, num_blocks, geom.block_size, geom.kv_heads, geom.head_dim, dtype=dtype)


# ----------------------------------------------------------------------------
# Per-op restatements (each is also the checker of one CUDA kernel).
# ----------------------------------------------------------------------------

def rms_forward(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """layers/layernorm.py:16-26.  Two rounding points: the normalised value is
    rounded to the activation dtype, then multiplied by the weight and rounded
    again."""
    orig = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return (xf.to(orig).float() * w.float()).to(orig)


def add_rms_forward(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float):
    """layers/layernorm.py:28-40.  The new residual is the sum rounded to the
    activation dtype; the variance uses the unrounded fp32 sum.

    fp32 quirk, reproduced on purpose: the reference writes this with in-place
    ops on ``x.float()`` / ``x.to(orig_dtype)``.  When the activations already
    are fp32 those casts return the same tensor, so ``residual`` aliases ``x``
    and ends up holding the *normalised, weighted output* instead of the sum
    (layernorm.py:34-39).  In bf16 the casts copy and no aliasing happens."""
    orig = x.dtype
    xf = x.float() + residual.float()
    new_residual = xf.to(orig)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    out = (xf.to(orig).float() * w.float()).to(orig)
    if orig == torch.float32:
        new_residual = out
    return out, new_residual


def linear(x: torch.Tensor, w_f32: torch.Tensor) -> torch.Tensor:
    """layers/linear.py:51,73,153 (``F.linear``): fp32 accumulate, one rounding
    of the output to the activation dtype."""
    return F.linear(x.float(), w_f32).to(x.dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """layers/rotary_embedding.py:6-14 (NeoX half split, fp32 math, one
    rounding).  ``x`` is ``[rows, heads, head_dim]``; ``cos``/``sin`` are
    ``[rows, 1, head_dim/2]`` fp32."""
    x1, x2 = torch.chunk(x.float(), 2, dim=-1)
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((y1, y2), dim=-1).to(x.dtype)


def silu_and_mul(gate_up: torch.Tensor, fused_rounding: bool = True) -> torch.Tensor:
    """layers/activation.py:8-11.  The GPU arms of the reference run this under
    ``torch.compile``, which evaluates ``silu(gate) * up`` in fp32 and rounds
    once (``fused_rounding=True``); the uncompiled module rounds ``silu(gate)``
    to the activation dtype first (``fused_rounding=False``).  In fp32 the two
    coincide."""
    gate, up = gate_up.chunk(2, -1)
    if fused_rounding:
        return (F.silu(gate.float()) * up.float()).to(gate_up.dtype)
    return F.silu(gate) * up


def op_rmsnorm_qkv(h, residual, lw: LayerWeights, w: Weights):
    """Input norm + fused QKV projection of one layer: models/qwen3.py:153-156
    then :79.  ``residual=None`` is the first layer, where the residual becomes
    the embedding itself."""
    eps = w.geom.eps
    if residual is None:
        x = rms_forward(h, lw.ln_in, eps)
        # fp32 quirk (see add_rms_forward): rms_forward normalises its fp32
        # input in place (layernorm.py:21-25), and models/qwen3.py:154 keeps that
        # same tensor as the residual.
        residual = x if h.dtype == torch.float32 else h
    else:
        x, residual = add_rms_forward(h, residual, lw.ln_in, eps)
    return linear(x, w.f32(lw.wqkv)), residual


def op_qknorm_rope(qkv, positions, lw: LayerWeights, w: Weights, cos_sin):
    """models/qwen3.py:80-87: split, per-head q/k RMSNorm, RoPE."""
    g = w.geom
    q, k, v = qkv.split([g.q_size, g.kv_size, g.kv_size], dim=-1)
    q = q.reshape(-1, g.q_heads, g.head_dim)
    k = k.reshape(-1, g.kv_heads, g.head_dim)
    v = v.reshape(-1, g.kv_heads, g.head_dim)
    q = rms_forward(q, lw.q_norm, g.eps)
    k = rms_forward(k, lw.k_norm, g.eps)
    cs = cos_sin[positions].unsqueeze(1)
    cos, sin = cs.chunk(2, dim=-1)
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin), v


def op_paged_attention_decode(q, k_new, v_new, kv_cache, layer, positions, block_tables, geom, row_active=None):
    """KV write + decode attention: layers/attention.py:33-40 (slot write) and
    :72-74 (``flash_attn_with_kvcache`` semantics: bf16 inputs, fp32 softmax and
    accumulation, output rounded once).  The new token is written at
    ``position`` (= len-1, engine/kv_layout.py:132-151) and attention covers
    ``[0, position]``.  Rows with ``row_active == 0`` skip the write only
    (backends/megakernel/row_contract.py:1-24)."""
    rows = q.shape[0]
    bs = geom.block_size
    scale = geom.head_dim ** -0.5
    group = geom.q_heads // geom.kv_heads
    out = torch.empty(rows, geom.q_size, dtype=q.dtype)
    for r in range(rows):
        pos = int(positions[r])
        table = block_tables[r]
        blk, off = int(table[pos // bs]), pos % bs
        if row_active is None or row_active[r]:
            kv_cache[0, layer, blk, off] = k_new[r]
            kv_cache[1, layer, blk, off] = v_new[r]
        ctx = pos + 1
        nblk = (ctx + bs - 1) // bs
        idx = torch.as_tensor([int(b) for b in table[:nblk]], dtype=torch.long)
        k = kv_cache[0, layer, idx].reshape(-1, geom.kv_heads, geom.head_dim)[:ctx].float()
        v = kv_cache[1, layer, idx].reshape(-1, geom.kv_heads, geom.head_dim)[:ctx].float()
        if row_active is not None and not row_active[r]:
            k = k.clone(); v = v.clone()
            k[pos] = k_new[r].float(); v[pos] = v_new[r].float()
        qr = q[r].float().reshape(geom.kv_heads, group, geom.head_dim)
        s = torch.einsum("hgd,thd->hgt", qr, k) * scale
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgt,thd->hgd", p, v)
        out[r] = o.reshape(-1).to(q.dtype)
    return out


def op_oproj(attn_out, lw: LayerWeights, w: Weights):
    """models/qwen3.py:89."""
    return linear(attn_out, w.f32(lw.wo))


def op_rmsnorm_gateup_swiglu(h, residual, lw: LayerWeights, w: Weights, fused_rounding=True):
    """models/qwen3.py:158 then :115-117."""
    x, residual = add_rms_forward(h, residual, lw.ln_post, w.geom.eps)
    return silu_and_mul(linear(x, w.f32(lw.wgu)), fused_rounding), residual


def op_down(act, lw: LayerWeights, w: Weights):
    """models/qwen3.py:118."""
    return linear(act, w.f32(lw.wd))


def op_final_norm_lmhead(h, residual, w: Weights):
    """models/qwen3.py:186 then :216-220 / layers/embed_head.py:61: final
    add+RMSNorm, tied LM head, logits rounded to the activation dtype."""
    x, _ = add_rms_forward(h, residual, w.final_norm, w.geom.eps)
    return linear(x, w.f32(w.embed))


def greedy(logits: torch.Tensor) -> torch.Tensor:
    """layers/sampler.py:9,15: argmax over the fp32 view of the (already
    rounded) logits; ties resolve to the lowest index."""
    return logits.float().argmax(dim=-1)


def sample(logits: torch.Tensor, temperatures: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """layers/sampler.py:7-16 with the exponential draw passed in (``noise``,
    fp32 ``[rows, vocab]``, what ``torch.empty_like(probs).exponential_(1)``
    returned): softmax of logits / T, divided by the clamped noise, argmax;
    rows with T <= 1e-10 take the plain argmax."""
    logits = logits.float()
    greedy_rows = temperatures <= 1e-10
    safe = temperatures.clamp_min(1e-10).unsqueeze(1)
    probs = torch.softmax(logits / safe, dim=-1)
    sampled = (probs / noise.clamp_min(1e-10)).argmax(dim=-1)
    return torch.where(greedy_rows, logits.argmax(dim=-1), sampled)


def sample_keys(logits: torch.Tensor, temperatures: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """The same draw in log space: argmax(probs / E) = argmax(logit / T - log E),
    since the softmax divides a row by one positive number.  Used to judge how
    close a second candidate was (fp32 ``[rows, vocab]``; greedy rows: the logits)."""
    logits = logits.float()
    safe = temperatures.clamp_min(1e-10).unsqueeze(1)
    keys = logits / safe - torch.log(noise.clamp_min(1e-10))
    return torch.where((temperatures <= 1e-10).unsqueeze(1), logits, keys)


def counter_noise(seed: int, step: int, rows: int, vocab: int, index_offset: int = 0) -> torch.Tensor:
    """The exponential noise of the CUDA backend's fused sampler, as its
    interface documents it (include/dfb_decode.h, dfb_set_seed): for row r and
    vocabulary index i the 64-bit counter c = ((step * 8 + r) << 32) | i, the
    splitmix64 finaliser of seed + c * 0x9E3779B97F4A7C15, its top 23 bits + 0.5
    over 2^23 as the uniform u, and E = max(-log u, 1e-10).  (The reference
    draws from torch's generator instead; only the distribution is shared.)"""
    mask = (1 << 64) - 1
    r = np.arange(rows, dtype=np.uint64)[:, None]
    i = (np.arange(vocab, dtype=np.uint64) + np.uint64(index_offset))[None, :]
    with np.errstate(over="ignore"):
        ctr = ((np.uint64(step * 8) + r) << np.uint64(32)) | i
        z = np.uint64(seed & mask) + ctr * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = ((z >> np.uint64(41)).astype(np.float32) + np.float32(0.5)) * np.float32(2.0 ** -23)
    e = np.maximum(-np.log(u, dtype=np.float32), np.float32(1e-10))
    return torch.from_numpy(e.astype(np.float32))


# ----------------------------------------------------------------------------
# Whole-step and whole-sequence drivers.
# ----------------------------------------------------------------------------

def decode_step(w: Weights, kv_cache, cos_sin, input_ids, positions, block_tables,
                row_active=None, fused_rounding=True, trace: dict | None = None):
    """One decode step for ``rows`` sequences (models/qwen3.py:174-187,209-220).
    ``positions[r]`` is the pre-decode length; ``block_tables[r]`` lists the
    physical blocks of row ``r``.  Returns ``(logits[rows, vocab], tokens[rows])``.
    ``trace`` (a dict) receives the per-layer intermediates."""
    g = w.geom
    ids = torch.as_tensor(input_ids, dtype=torch.long)
    pos = torch.as_tensor(positions, dtype=torch.long)
    h = w.embed[ids]
    residual = None
    for li, lw in enumerate(w.layers):
        qkv, residual = op_rmsnorm_qkv(h, residual, lw, w)
        q, k, v = op_qknorm_rope(qkv, pos, lw, w, cos_sin)
        attn = op_paged_attention_decode(q, k, v, kv_cache, li, pos, block_tables, g, row_active)
        h_attn = op_oproj(attn, lw, w)
        act, residual = op_rmsnorm_gateup_swiglu(h_attn, residual, lw, w, fused_rounding)
        h = op_down(act, lw, w)
        if trace is not None:
            trace[li] = dict(qkv=qkv, q=q, k=k, attn=attn, h_attn=h_attn, act=act, h=h, residual=residual)
    logits = op_final_norm_lmhead(h, residual, w)
    return logits, greedy(logits)


def prefill(w: Weights, kv_cache, cos_sin, token_ids: Sequence[int], block_table: Sequence[int],
            fused_rounding=True):
    """Causal prefill of one fresh prompt, filling the paged cache the decode
    step later reads (models/qwen3.py:174-187 with layers/attention.py:64-70;
    slots from engine/kv_layout.py:86-129).  Returns the last token's logits."""
    g = w.geom
    n = len(token_ids)
    ids = torch.as_tensor(list(token_ids), dtype=torch.long)
    pos = torch.arange(n)
    bs = g.block_size
    blocks = torch.as_tensor([int(block_table[p // bs]) for p in range(n)], dtype=torch.long)
    offs = pos % bs
    scale = g.head_dim ** -0.5
    group = g.q_heads // g.kv_heads
    causal = torch.ones(n, n, dtype=torch.bool).tril()
    h = w.embed[ids]
    residual = None
    for li, lw in enumerate(w.layers):
        qkv, residual = op_rmsnorm_qkv(h, residual, lw, w)
        q, k, v = op_qknorm_rope(qkv, pos, lw, w, cos_sin)
        kv_cache[0, li, blocks, offs] = k
        kv_cache[1, li, blocks, offs] = v
        qf = q.float().reshape(n, g.kv_heads, group, g.head_dim)
        s = torch.einsum("qhgd,thd->hgqt", qf, k.float()) * scale
        s = s.masked_fill(~causal, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgqt,thd->qhgd", p, v.float()).reshape(n, g.q_size).to(q.dtype)
        h_attn = op_oproj(o, lw, w)
        act, residual = op_rmsnorm_gateup_swiglu(h_attn, residual, lw, w, fused_rounding)
        h = op_down(act, lw, w)
    return op_final_norm_lmhead(h[-1:], residual[-1:], w)[0]


def allocate_blocks(lengths: Sequence[int], block_size: int, permutation: Sequence[int] | None = None):
    """Block tables for sequences that will grow to ``lengths`` tokens, blocks
    handed out in order (or through ``permutation`` of the physical pool)."""
    tables, nxt = [], 0
    for n in lengths:
        need = (n + block_size - 1) // block_size
        ids = list(range(nxt, nxt + need))
        nxt += need
        tables.append([int(permutation[i]) for i in ids] if permutation is not None else ids)
    return tables, nxt


def greedy_generate(w: Weights, prompts: Sequence[Sequence[int]], steps: int, act_dtype=None,
                    keep_logits: bool = False, fused_rounding=True, block_permutation=None,
                    forced_inputs=None):
    """Prefill every prompt, then ``steps`` batched greedy decode steps through
    the paged cache.  Returns ``(tokens[steps + 1, rows], logits list or None)``;
    ``tokens[0]`` is the token chosen from the prefill logits and is the input
    of the first decode step (engine/llm_engine.py:92-127 loop).  With
    ``forced_inputs[step][row]`` the input of every decode step is taken from
    that table instead of the previous argmax (teacher forcing), which keeps
    two implementations on the same trajectory when comparing logits."""
    g = w.geom
    dtype = act_dtype or w.dtype
    cos_sin = rope_cos_sin_table(g)
    lengths = [len(p) + steps for p in prompts]
    tables, nblocks = allocate_blocks(lengths, g.block_size, block_permutation)
    pool = nblocks if block_permutation is None else len(block_permutation)
    kv = new_kv_cache(g, pool, dtype)
    cur, lens = [], []
    for p, t in zip(prompts, tables):
        lg = prefill(w, kv, cos_sin, p, t, fused_rounding)
        cur.append(int(greedy(lg)))
        lens.append(len(p) + 1)
    toks = [list(cur)]
    all_logits = []
    for step in range(steps):
        positions = [n - 1 for n in lens]
        if forced_inputs is not None:
            cur = [int(t) for t in forced_inputs[step]]
        logits, nxt = decode_step(w, kv, cos_sin, cur, positions, tables, fused_rounding=fused_rounding)
        if keep_logits:
            all_logits.append(logits.float().clone())
        cur = [int(t) for t in nxt]
        lens = [n + 1 for n in lens]
        toks.append(list(cur))
    return torch.tensor(toks), (all_logits if keep_logits else None)
