"""Full Qwen3-0.6B geometry on the GPU: against the golden fixture produced by
the reference's torch model (bf16, teacher forced), against the oracle over 64
greedy steps (BASELINE config 1 in bf16), and size-independent properties at the
benchmark's sizes."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import qwen3_decode as O
from tests import harness as H

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden as G  # noqa: E402  (case definitions only)


@pytest.fixture(scope="module")
def full(cuda_device):
    w = O.make_weights(O.QWEN3_06B, seed=0, norm="ones").to(torch.bfloat16)
    return w, H.to_decoder_weights(w)


def _decoder(dw, kv_gpu, g):
    from dfb_b200.decoder import StreamDecoder
    return StreamDecoder(dw, kv_gpu[0], kv_gpu[1], block_size=g.block_size, num_cache_blocks=kv_gpu.shape[2],
                         max_model_len=g.max_pos)


def test_golden_bf16_teacher_forced(full):
    """The CUDA step against logits the REFERENCE model produced (fixture)."""
    w, dw = full
    g = w.geom
    z = np.load(GOLDEN / "qwen3_06b_bf16_forced8.npz")
    prompts, forced = G.forced_case(g)
    cos_sin = O.rope_cos_sin_table(g)
    lengths = [len(p) + G.FORCED_STEPS for p in prompts]
    tables, nblocks = O.allocate_blocks(lengths, g.block_size)
    kv = O.new_kv_cache(g, nblocks, torch.bfloat16)
    for p, t in zip(prompts, tables):
        O.prefill(w, kv, cos_sin, p, t, fused_rounding=False)      # prefill stays off the CUDA path
    kv_gpu = kv.cuda()
    dec = _decoder(dw, kv_gpu, g)
    logits = torch.zeros(2, g.vocab, device="cuda")
    lens = [len(p) + 1 for p in prompts]
    probe = torch.from_numpy(z["probe_index"]).long()
    worst = 0.0
    for s in range(G.FORCED_STEPS):
        dec.enqueue_rows(torch.tensor(forced[s], device="cuda"), torch.tensor([n - 1 for n in lens], device="cuda"),
                         H.padded_tables(tables, lens, g.block_size), out_logits=logits)
        torch.cuda.synchronize()
        got = logits.cpu()
        worst = max(worst, float((got[:, probe] - torch.from_numpy(z["probe_logits"][s])).abs().max()))
        toks = dec.tokens_device()[:2].tolist()
        for r in range(2):
            ref_tok = int(z["tokens"][s + 1, r])
            top_i, top_v = z["top_index"][s, r], z["top_logits"][s, r]
            if toks[r] != ref_tok:   # only a tie within rounding may differ
                assert toks[r] in top_i.tolist(), (s, r, toks[r], top_i)
                gap = float(top_v[0] - top_v[top_i.tolist().index(toks[r])])
                assert gap <= H.TOKEN_GAP_ATOL, (s, r, gap)
        lens = [n + 1 for n in lens]
    assert worst <= H.LOGIT_ATOL, worst
    dec.close()


def test_config1_bf16_greedy64_vs_oracle(full):
    """Prompt of 32 ids, 64 greedy decode steps, batch 1, block 256: tokens equal
    to the oracle's (up to ties within rounding, which are then teacher-forced
    to the oracle's choice) and logits within tolerance at every step."""
    w, dw = full
    g = w.geom
    prompt = G.config1_prompt(g)
    cos_sin = O.rope_cos_sin_table(g)
    tables, nblocks = O.allocate_blocks([len(prompt) + 65], g.block_size)
    kv = O.new_kv_cache(g, nblocks, torch.bfloat16)
    cur = [int(O.greedy(O.prefill(w, kv, cos_sin, prompt, tables[0])))]
    kv_gpu = kv.cuda()
    dec = _decoder(dw, kv_gpu, g)
    logits = torch.zeros(1, g.vocab, device="cuda")
    n = len(prompt) + 1
    worst, mean_worst, identical = 0.0, 0.0, 0
    for s in range(64):
        want_logits, want_tok = O.decode_step(w, kv, cos_sin, cur, [n - 1], tables)
        dec.enqueue_rows(torch.tensor(cur, device="cuda"), torch.tensor([n - 1], device="cuda"),
                         H.padded_tables(tables, [n], g.block_size), out_logits=logits)
        torch.cuda.synchronize()
        d = (logits.cpu() - want_logits.float()).abs()
        worst, mean_worst = max(worst, float(d.max())), max(mean_worst, float(d.mean()))
        got = int(dec.tokens_device()[0])
        identical += got == int(want_tok[0])
        assert H.token_gap_ok(want_logits[0].float(), got, int(want_tok[0])), (s, got, int(want_tok[0]))
        cur, n = [int(want_tok[0])], n + 1
    print(f"config1 bf16: max|dlogit|={worst:.4f} mean={mean_worst:.5f} identical tokens {identical}/64")
    assert worst <= H.LOGIT_ATOL and mean_worst <= H.LOGIT_MEAN_ATOL
    assert float((kv_gpu.cpu().float() - kv.float()).abs().max()) <= 2.0 ** -4
    dec.close()


# Tolerance of the full-depth runs on a RANDOM long history.  The seeded N(0, 0.02) network is chaotic on
# such inputs: the oracle's own two admissible roundings of SwiGLU (one rounding, as the compiled torch path
# does, or two, as the uncompiled one does: layers/activation.py:8-11) already differ by about 0.11 in the
# logits there (0.06 at context 1), more than harness.LOGIT_ATOL, which was stated for model-generated
# histories.  So these tests measure that spread on the same inputs and require the CUDA path to stay within
# NOISE_FACTOR of it, with an absolute cap that a real defect (a wrong block, a dropped position) exceeds by far.
NOISE_FACTOR = 1.5
LOGIT_CAP = 0.25


def _oracle_spread(w, kv, cos_sin, cur, positions, tables):
    """Logits of the oracle (its KV write lands in ``kv``) and the spread between its two rounding variants."""
    scratch = kv.clone()
    want_logits, want_tok = O.decode_step(w, kv, cos_sin, cur, positions, tables)
    other, _ = O.decode_step(w, scratch, cos_sin, cur, positions, tables, fused_rounding=False)
    d = (want_logits.float() - other.float()).abs()
    return want_logits, want_tok, float(d.max()), float(d.mean())


def _history_like_real_kv(g, blocks, seed):
    """A random bf16 KV history with the scale of real entries: K is RMS-normalised per head (unit RMS
    with the seeded norm weights of 1.0), V is a projection of a unit-RMS vector through N(0, 0.02)
    weights, i.e. std 0.02 * sqrt(1024) = 0.64."""
    gen = torch.Generator().manual_seed(seed)
    kv = torch.empty(2, g.layers, blocks, g.block_size, g.kv_heads, g.head_dim, dtype=torch.float32)
    kv[0].normal_(0, 1.0, generator=gen)
    kv[1].normal_(0, 0.64, generator=gen)
    return kv.to(torch.bfloat16)


@pytest.mark.parametrize("rows", [2, 4, 8])
def test_full_depth_long_context_vs_oracle(full, rows):
    """BASELINE config 4 as written, against the ORACLE at all 28 layers: per-row contexts drawn uniformly in
    [256, 2048), block tables scattered by a seeded permutation, the same random KV history on both sides,
    three teacher-forced steps.  Rows 4 and 8 run the tensor-core chain, 2 rows the FP32 kernels."""
    w, dw = full
    g = w.geom
    steps = 3
    rng = np.random.Generator(np.random.Philox(key=900 + rows))
    ctx = rng.integers(256, 2048 - steps, rows).tolist()
    perm = rng.permutation(8 * rows).tolist()
    tables, _ = O.allocate_blocks([2048] * rows, g.block_size, perm)
    kv = _history_like_real_kv(g, 8 * rows, seed=rows)
    kv_gpu = kv.cuda()
    cos_sin = O.rope_cos_sin_table(g)
    dec = _decoder(dw, kv_gpu, g)
    logits = torch.zeros(rows, g.vocab, device="cuda")
    cur = rng.integers(0, g.vocab, rows).tolist()
    lens = [c + 1 for c in ctx]                     # length after the step's token is appended
    worst, mean_worst, identical, floor, floor_mean = 0.0, 0.0, 0, 0.0, 0.0
    for s in range(steps):
        positions = [n - 1 for n in lens]
        want_logits, want_tok, spread_max, spread_mean = _oracle_spread(w, kv, cos_sin, cur, positions, tables)
        floor, floor_mean = max(floor, spread_max), max(floor_mean, spread_mean)
        dec.enqueue_rows(torch.tensor(cur, device="cuda"), torch.tensor(positions, device="cuda"),
                         H.padded_tables(tables, lens, g.block_size), out_logits=logits)
        torch.cuda.synchronize()
        got = logits.cpu()
        d = (got - want_logits.float()).abs()
        worst, mean_worst = max(worst, float(d.max())), max(mean_worst, float(d.mean()))
        toks = dec.tokens_device()[:rows].tolist()
        assert toks == got.argmax(-1).tolist()
        for r in range(rows):
            identical += toks[r] == int(want_tok[r])
            assert H.token_gap_ok(want_logits[r].float(), toks[r], int(want_tok[r]),
                                  atol=max(H.TOKEN_GAP_ATOL, NOISE_FACTOR * spread_max)), (s, r)
            # the new K/V rows: layer 0 sees identical inputs on both sides, so one bf16 step at most; the
            # deeper layers inherit the rounding differences of the residual stream (K is normalised to
            # unit RMS with entries up to about 5, so a 2 % difference of the stream is 0.1 there)
            blk, off = tables[r][positions[r] // g.block_size], positions[r] % g.block_size
            a, b = kv_gpu[:, :, blk, off].cpu().float(), kv[:, :, blk, off].float()
            assert float(((a[:, 0] - b[:, 0]).abs() / b[:, 0].abs().clamp(min=1.0)).max()) <= 2.0 ** -7, (s, r)
            assert float((a - b).abs().max()) <= 0.25 and float((a - b).abs().mean()) <= 2.5e-2, (s, r)
        cur = [int(t) for t in want_tok]
        lens = [n + 1 for n in lens]
    print(f"rows {rows}: max|dlogit|={worst:.4f} mean={mean_worst:.5f} (oracle's own rounding spread: max "
          f"{floor:.4f} mean {floor_mean:.5f}) identical tokens {identical}/{rows * steps}")
    assert worst <= min(LOGIT_CAP, NOISE_FACTOR * max(floor, H.LOGIT_ATOL)), (worst, floor)
    assert mean_worst <= NOISE_FACTOR * max(floor_mean, H.LOGIT_MEAN_ATOL), (mean_worst, floor_mean)
    code, st = dec.status()
    assert code == 0
    dec.close()


@pytest.mark.parametrize("rows", [4, 8])
def test_full_depth_batch_equals_single_rows_at_prompt_512(full, rows):
    """BASELINE config 3 shape (prompt 512) at full depth: every row of a batch of 4 / 8 (tensor-core
    chain) against the oracle AND against the same row decoded alone (FP32 kernels)."""
    w, dw = full
    g = w.geom
    rng = np.random.Generator(np.random.Philox(key=950 + rows))
    ctx = [512] * rows
    tables, nblocks = O.allocate_blocks([520] * rows, g.block_size)
    kv = _history_like_real_kv(g, nblocks, seed=50 + rows)
    kv_gpu = kv.cuda()
    kv0 = kv_gpu.clone()
    cos_sin = O.rope_cos_sin_table(g)
    cur = rng.integers(0, g.vocab, rows).tolist()
    positions = list(ctx)
    lens = [c + 1 for c in ctx]
    want_logits, want_tok, floor, floor_mean = _oracle_spread(w, kv, cos_sin, cur, positions, tables)
    bound = min(LOGIT_CAP, NOISE_FACTOR * max(floor, H.LOGIT_ATOL))
    dec = _decoder(dw, kv_gpu, g)
    la, lb = torch.zeros(rows, g.vocab, device="cuda"), torch.zeros(1, g.vocab, device="cuda")
    bt = H.padded_tables(tables, lens, g.block_size)
    dec.enqueue_rows(torch.tensor(cur, device="cuda"), torch.tensor(positions, device="cuda"), bt, out_logits=la)
    torch.cuda.synchronize()
    print(f"rows {rows} prompt 512: max|dlogit|={float((la.cpu() - want_logits.float()).abs().max()):.4f} "
          f"(oracle's own rounding spread {floor:.4f})")
    assert float((la.cpu() - want_logits.float()).abs().max()) <= bound
    for r in range(rows):
        assert H.token_gap_ok(want_logits[r].float(), int(dec.tokens_device()[r]), int(want_tok[r]), atol=bound)
    for r in (0, rows - 1):
        kv_gpu.copy_(kv0)
        dec.enqueue_rows(torch.tensor(cur[r:r + 1], device="cuda"), torch.tensor(positions[r:r + 1], device="cuda"),
                         bt[r:r + 1].contiguous(), out_logits=lb)
        torch.cuda.synchronize()
        assert float((lb[0].cpu() - want_logits[r].float()).abs().max()) <= bound
    dec.close()


def test_full_size_properties_batch8_long_context(full):
    """BASELINE config 4 sizes (batch 8, contexts in [256, 2048], scattered
    blocks): properties that need no oracle run -- determinism, batch ==
    independent rows, and each row's logits depend only on its own KV blocks."""
    w, dw = full
    g = w.geom
    rng = np.random.Generator(np.random.Philox(key=77))
    ctx = rng.integers(256, 2048, 8).tolist()
    perm = rng.permutation(64).tolist()
    tables, _ = O.allocate_blocks([2048] * 8, g.block_size, perm)
    kv = torch.empty(2, g.layers, 64, g.block_size, g.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    kv.normal_(0, 1, generator=torch.Generator(device="cuda").manual_seed(5))
    kv0 = kv.clone()
    ids = torch.from_numpy(rng.integers(0, g.vocab, 8)).cuda()
    pos = torch.tensor([c - 1 for c in ctx], device="cuda")
    bt = H.padded_tables(tables, ctx, g.block_size)
    dec = _decoder(dw, kv, g)
    la, lb = torch.zeros(8, g.vocab, device="cuda"), torch.zeros(8, g.vocab, device="cuda")
    dec.enqueue_rows(ids, pos, bt, out_logits=la)
    torch.cuda.synchronize()
    tok_a = dec.tokens_device()[:8].tolist()
    kv_after = kv.clone()
    kv.copy_(kv0)
    dec.enqueue_rows(ids, pos, bt)              # graph path, no logits
    torch.cuda.synchronize()
    assert dec.tokens_device()[:8].tolist() == tok_a
    assert torch.equal(kv, kv_after)
    # only the 8 new (row, position) slots changed
    changed = (kv_after != kv0).any(dim=-1).any(dim=-1).any(dim=0).any(dim=0)   # [blocks, block_size]
    want = torch.zeros_like(changed)
    for r in range(8):
        p = ctx[r] - 1
        want[tables[r][p // g.block_size], p % g.block_size] = True
    assert torch.equal(changed, want)
    # rows one at a time (single rows run on the FP32 pipe, the batch of 8 on the
    # tensor cores: agreement to bf16 rounding, same KV slot written)
    for r in (0, 3, 7):
        kv.copy_(kv0)
        dec.enqueue_rows(ids[r:r + 1], pos[r:r + 1], bt[r:r + 1].contiguous(), out_logits=lb)
        torch.cuda.synchronize()
        # two CUDA paths that are each within LOGIT_ATOL of the exact result
        assert float((lb[0] - la[r]).abs().max()) <= 2 * H.LOGIT_ATOL
        p = ctx[r] - 1
        blk, off = tables[r][p // g.block_size], p % g.block_size
        # the history here is N(0,1) noise, far larger than real K/V, so late layers amplify the
        # rounding differences of the two paths; this only checks that the same slot was written
        assert float((kv[:, :, blk, off].float() - kv_after[:, :, blk, off].float()).abs().max()) <= 0.25
    code, st = dec.status()
    assert code == 0
    dec.close()
