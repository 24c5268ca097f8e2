"""Shared parity harness: drives the CUDA decoder and the CPU oracle on the same
seeded inputs.  The oracle is the checker here, never the thing under test."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__  # noqa: E402,F401
from oracle import qwen3_decode as O  # noqa: E402

# Stated tolerances of the bf16 path against the oracle.  Logits of the seeded
# N(0, 0.02) models stay below 8 in magnitude, where one bf16 step is 2**-5 at
# most; two valid bf16 implementations that sum in a different order differ by a
# few such steps after 28 layers.
LOGIT_ATOL = 6.25e-2        # max |logit difference|
LOGIT_MEAN_ATOL = 1.0e-2    # mean |logit difference|
HIDDEN_ATOL = 6.25e-2
# A greedy token may differ from the oracle's only if the oracle itself scores
# the two candidates closer than this (a tie within rounding noise).
TOKEN_GAP_ATOL = LOGIT_ATOL


def oracle_geometry(layers=28, vocab=151936, max_pos=2048, block_size=256) -> O.Geometry:
    return O.Geometry(layers=layers, vocab=vocab, max_pos=max_pos, block_size=block_size)


def to_model_geometry(g: O.Geometry):
    from dfb_b200.geometry import ModelGeometry

    return ModelGeometry(hidden=g.hidden, layers=g.layers, q_heads=g.q_heads, kv_heads=g.kv_heads,
                         head_dim=g.head_dim, intermediate=g.intermediate, vocab=g.vocab, eps=g.eps,
                         rope_theta=g.rope_theta, max_model_len=g.max_pos, block_size=g.block_size)


def to_decoder_weights(w: O.Weights, device="cuda"):
    """The oracle's bf16 weights as CUDA tensors for the decoder."""
    from dfb_b200.weights import DecoderWeights, LayerTensors, LAYER_FIELDS

    assert w.dtype == torch.bfloat16
    dev = lambda t: t.to(device).contiguous()
    layers = [LayerTensors(**{f: dev(getattr(l, f)) for f in LAYER_FIELDS}) for l in w.layers]
    return DecoderWeights(to_model_geometry(w.geom), dev(w.embed), layers, dev(w.final_norm),
                          dev(O.rope_cos_sin_table(w.geom)))


def make_decoder(w: O.Weights, kv_cache_gpu, **kw):
    from dfb_b200.decoder import StreamDecoder

    g = w.geom
    return StreamDecoder(to_decoder_weights(w), kv_cache_gpu[0], kv_cache_gpu[1], block_size=g.block_size,
                         num_cache_blocks=kv_cache_gpu.shape[2], max_model_len=g.max_pos, **kw)


def padded_tables(tables, lens, block_size, device="cuda"):
    need = [-(-n // block_size) for n in lens]
    width = max(need)
    rows = [list(t[:k]) + [0] * (width - k) for t, k in zip(tables, need)]
    return torch.tensor(rows, dtype=torch.int32, device=device)


def token_gap_ok(oracle_logits: torch.Tensor, got: int, want: int, atol=TOKEN_GAP_ATOL) -> bool:
    return got == want or float(oracle_logits[want] - oracle_logits[got]) <= atol


def run_parity_case(layers=2, vocab=4096, prompt_lens=(3, 70, 250), steps=4, seed=3, norm="random",
                    block_permutation=None, use_graph=True, use_pdl=True, host_path=False, max_pos=2048,
                    check_kv=True, persistent=False, options=None):
    """Prefill by the oracle, then ``steps`` teacher-forced decode steps on both
    sides; returns the worst differences seen."""
    g = oracle_geometry(layers=layers, vocab=vocab, max_pos=max_pos)
    w = O.make_weights(g, seed=seed, norm=norm).to(torch.bfloat16)
    cos_sin = O.rope_cos_sin_table(g)
    rng = np.random.Generator(np.random.Philox(key=seed + 100))
    prompts = [rng.integers(0, g.vocab, n).tolist() for n in prompt_lens]
    lengths = [n + steps for n in prompt_lens]
    tables, nblocks = O.allocate_blocks(lengths, g.block_size, block_permutation)
    pool = nblocks if block_permutation is None else len(block_permutation)
    kv = O.new_kv_cache(g, pool, torch.bfloat16)
    cur = []
    for p, t in zip(prompts, tables):
        cur.append(int(O.greedy(O.prefill(w, kv, cos_sin, p, t))))
    kv_gpu = kv.cuda()
    dec = make_decoder(w, kv_gpu, use_graph=use_graph, use_pdl=use_pdl, persistent=persistent)
    for opt, value in (options or {}).items():
        dec.set_option(opt, value)
    rows = len(prompts)
    lens = [n + 1 for n in prompt_lens]
    logits_gpu = torch.zeros(rows, g.vocab, dtype=torch.float32, device="cuda")
    worst, mean_worst, flips, bad_flips = 0.0, 0.0, 0, 0
    for _ in range(steps):
        positions = [n - 1 for n in lens]
        want_logits, want_tok = O.decode_step(w, kv, cos_sin, cur, positions, tables)
        ids = torch.tensor(cur, dtype=torch.int64, device="cuda")
        pos = torch.tensor(positions, dtype=torch.int64, device="cuda")
        bt = padded_tables(tables, lens, g.block_size)
        if host_path:
            got_tok = dec.decode_host(cur, positions, [t[: -(-n // g.block_size)] for t, n in zip(tables, lens)])
            got_logits = None
        else:
            dec.enqueue_rows(ids, pos, bt, out_logits=logits_gpu)
            torch.cuda.synchronize()
            got_tok = dec.tokens_device()[:rows].tolist()
            got_logits = logits_gpu.cpu()
            d = (got_logits - want_logits.float()).abs()
            worst = max(worst, float(d.max()))
            mean_worst = max(mean_worst, float(d.mean()))
            # the kernel's argmax must agree with an argmax over its own logits
            assert got_tok == got_logits.argmax(-1).tolist(), (got_tok, got_logits.argmax(-1).tolist())
        for r in range(rows):
            if got_tok[r] != int(want_tok[r]):
                flips += 1
                if not token_gap_ok(want_logits[r].float(), got_tok[r], int(want_tok[r])):
                    bad_flips += 1
        cur = [int(t) for t in want_tok]  # teacher forcing keeps both on the oracle's trajectory
        lens = [n + 1 for n in lens]
    code, st = dec.status()
    report = dict(max_abs_logit_diff=worst, mean_abs_logit_diff=mean_worst, token_flips=flips,
                  tokens_match_or_tie=bad_flips == 0, device_status=int(st.device_status),
                  kernels_per_step=int(st.kernels_per_step))
    if check_kv:
        report["max_abs_kv_diff"] = float((kv_gpu.cpu().float() - kv.float()).abs().max())
    dec.close()
    return report
