"""The whole decode step through the C ABI against the oracle, on small models
with the Qwen3-0.6B layer shape (the oracle finishes these in seconds)."""

import numpy as np
import pytest
import torch

from oracle import qwen3_decode as O
from tests import harness as H

pytestmark = pytest.mark.gpu


def _check(report):
    assert report["device_status"] == 0, report
    assert report["tokens_match_or_tie"], report
    assert report["max_abs_logit_diff"] <= H.LOGIT_ATOL, report
    assert report["mean_abs_logit_diff"] <= H.LOGIT_MEAN_ATOL, report
    assert report["max_abs_kv_diff"] <= 2.0 ** -5, report


@pytest.mark.parametrize("persistent", [True, False])
@pytest.mark.parametrize("rows", [1, 2, 3, 4, 5, 6, 7, 8])
def test_step_matches_oracle_for_every_batch_size(cuda_device, rows, persistent):
    """Both step implementations: the chain of per-op kernels (default) and the
    persistent kernel."""
    lens = [3, 70, 250, 129, 64, 1, 300, 17][:rows]
    r = H.run_parity_case(layers=2, vocab=4096, prompt_lens=lens, steps=3, seed=rows, persistent=persistent)
    _check(r)
    assert r["kernels_per_step"] == (1 if persistent else 2 * 5 + 1)


@pytest.mark.parametrize("mask", [0, 1, 2, 4, 7])
@pytest.mark.parametrize("rows", [3, 4, 5, 8])
def test_tcgen05_projections_match_oracle(cuda_device, rows, mask):
    """The K = 1024 projections on tcgen05.mma (bit mask: 1 = QKV, 2 = gate/up, 4 = LM head) and on the
    mma.sync kernels (0), each against the oracle; the vocabulary of 4,160 rows ends in a partial tile of
    the LM head (64 rows per tile)."""
    from dfb_b200 import native
    lens = [3, 70, 250, 129, 64, 1, 300, 17][:rows]
    r = H.run_parity_case(layers=2, vocab=4160, prompt_lens=lens, steps=3, seed=30 + rows,
                          options={native.DFB_OPT_TCGEN05: mask})
    _check(r)


@pytest.mark.parametrize("mask", [1, 2, 7, 15])
@pytest.mark.parametrize("rows", [2, 5, 8])
def test_register_resident_projections_match_oracle(cuda_device, rows, mask):
    """The mma.sync kernels that keep their weights in registers instead of shared-memory stages (bit mask:
    1 = QKV and gate/up, 2 = o_proj and down_proj, 4 = LM head, 8 = up to two CTAs per SM), with tcgen05 off
    so that the LM head bit takes effect."""
    from dfb_b200 import native
    lens = [3, 70, 250, 129, 64, 1, 300, 17][:rows]
    r = H.run_parity_case(layers=2, vocab=4096, prompt_lens=lens, steps=3, seed=40 + rows,
                          options={native.DFB_OPT_TCGEN05: 0, native.DFB_OPT_REG_WEIGHTS: mask})
    _check(r)


@pytest.mark.parametrize("prompt", [254, 255, 256, 257])
def test_block_boundary(cuda_device, prompt):
    """Decode across the 256-token block boundary (the reference's
    tests/test_kv_block_boundary.py cases, on the device)."""
    _check(H.run_parity_case(layers=2, vocab=2048, prompt_lens=[prompt], steps=4, seed=11))


def test_scattered_block_tables(cuda_device):
    perm = np.random.Generator(np.random.Philox(key=4)).permutation(16).tolist()
    _check(H.run_parity_case(layers=2, vocab=2048, prompt_lens=[600, 40, 257], steps=3, seed=12,
                             block_permutation=perm))


def test_max_context(cuda_device):
    """The last admissible position: context 2048 after the step."""
    _check(H.run_parity_case(layers=1, vocab=1024, prompt_lens=[2044, 1], steps=3, seed=13))


@pytest.mark.parametrize("use_graph,use_pdl,persistent", [
    (False, False, False), (False, True, False), (True, False, False), (True, True, False), (False, False, True)])
def test_launch_modes_agree(cuda_device, use_graph, use_pdl, persistent):
    """Plain launches, PDL launches, graph replay and the persistent kernel
    outside a graph must all give the same result."""
    _check(H.run_parity_case(layers=3, vocab=2048, prompt_lens=[5, 130], steps=3, seed=14,
                             use_graph=use_graph, use_pdl=use_pdl, persistent=persistent))


def test_persistent_and_chained_steps_agree(cuda_device):
    """The two step implementations split K differently across warps for o_proj
    and down_proj (another summation order), so they agree to bf16 rounding, not
    bit for bit."""
    lens = [40, 300, 7, 64]
    g, w, kv, tables, first = _setup(lens, seed=21, layers=3)
    outs = []
    for persistent in (True, False):
        kvg = kv.cuda()
        dec = H.make_decoder(w, kvg, persistent=persistent)
        logits = torch.zeros(4, g.vocab, device="cuda")
        cur, cl, seen = list(first), [n + 1 for n in lens], []
        for _ in range(3):
            dec.enqueue_rows(torch.tensor(cur, device="cuda"), torch.tensor([n - 1 for n in cl], device="cuda"),
                             H.padded_tables(tables, cl, g.block_size), out_logits=logits)
            torch.cuda.synchronize()
            seen.append(logits.clone())
            cur, cl = dec.tokens_device()[:4].tolist(), [n + 1 for n in cl]
        outs.append((seen, kvg.clone()))
        dec.close()
    for a, b in zip(outs[0][0], outs[1][0]):
        assert float((a - b).abs().max()) <= H.LOGIT_ATOL
    assert float((outs[0][1].float() - outs[1][1].float()).abs().max()) <= 2.0 ** -5


@pytest.mark.parametrize("ctas", [1, 7, 64, 147])
def test_persistent_kernel_with_fewer_ctas(cuda_device, ctas):
    """The persistent kernel is correct for any grid size (the CTA-count sweep
    of the reference's TG_NUM_SMS diagnostic relies on it)."""
    from dfb_b200 import native
    lens = [130, 9]
    g, w, kv, tables, first = _setup(lens, seed=22, layers=2)
    res = []
    for n in (0, ctas):
        kvg = kv.cuda()
        dec = H.make_decoder(w, kvg, persistent=True)
        dec.set_option(native.DFB_OPT_PERSIST_CTAS, n)
        logits = torch.zeros(2, g.vocab, device="cuda")
        dec.enqueue_rows(torch.tensor(first, device="cuda"), torch.tensor(lens, device="cuda"),
                         H.padded_tables(tables, [n_ + 1 for n_ in lens], g.block_size), out_logits=logits)
        torch.cuda.synchronize()
        code, st = dec.status()
        assert code == 0
        res.append((logits.clone(), dec.tokens_device()[:2].tolist()))
        dec.close()
    assert torch.equal(res[0][0], res[1][0]) and res[0][1] == res[1][1]


def test_host_buffer_step(cuda_device):
    """dfb_decode_step_host: H2D + step + D2H inside the call."""
    r = H.run_parity_case(layers=2, vocab=2048, prompt_lens=[9, 300, 64], steps=4, seed=15, host_path=True)
    assert r["device_status"] == 0 and r["tokens_match_or_tie"], r
    assert r["max_abs_kv_diff"] <= 2.0 ** -5, r


def _setup(rows_lens, seed, layers=2, vocab=2048, steps=4):
    g = H.oracle_geometry(layers=layers, vocab=vocab)
    w = O.make_weights(g, seed=seed, norm="random").to(torch.bfloat16)
    cos_sin = O.rope_cos_sin_table(g)
    rng = np.random.Generator(np.random.Philox(key=seed))
    prompts = [rng.integers(0, g.vocab, n).tolist() for n in rows_lens]
    tables, nblocks = O.allocate_blocks([n + steps for n in rows_lens], g.block_size)
    kv = O.new_kv_cache(g, nblocks, torch.bfloat16)
    first = [int(O.greedy(O.prefill(w, kv, cos_sin, p, t))) for p, t in zip(prompts, tables)]
    return g, w, kv, tables, first


@pytest.mark.parametrize("persistent", [False, True])
def test_batch_equals_independent_rows(cuda_device, persistent):
    """B rows in one launch == B single-row launches (the reference's
    tests/test_taskgraph_bs2.py:235-248).  One- and two-row batches are
    multiplied on the FP32 pipe and larger ones on the tensor cores (another
    summation order), so a 3-row launch agrees with single-row launches to bf16
    rounding; with the FP32 kernels and the 128-position attention chunks (chosen
    by the launch's longest row) switched off the arithmetic is the same for
    every batch size and the agreement is bit for bit."""
    from dfb_b200 import native
    lens = [40, 300, 7]
    g, w, kv, tables, first = _setup(lens, seed=16)
    kv_a, kv_b = kv.cuda(), kv.cuda()
    dec_a, dec_b = H.make_decoder(w, kv_a, persistent=persistent), H.make_decoder(w, kv_b, persistent=persistent)
    exact = not persistent
    if exact:
        for dec in (dec_a, dec_b):                      # options belong to the decoder they are set on
            dec.set_option(native.DFB_OPT_ROW_GEMV, 0)
            dec.set_option(native.DFB_OPT_ATTN_CHUNK128, 0)
    la = torch.zeros(3, g.vocab, device="cuda")
    lb = torch.zeros(1, g.vocab, device="cuda")
    cur = list(first)
    cl = [n + 1 for n in lens]
    for _ in range(3):
        pos = [n - 1 for n in cl]
        dec_a.enqueue_rows(torch.tensor(cur, device="cuda"), torch.tensor(pos, device="cuda"),
                           H.padded_tables(tables, cl, g.block_size), out_logits=la)
        torch.cuda.synchronize()
        tok_a = dec_a.tokens_device()[:3].tolist()
        for r in range(3):
            dec_b.enqueue_rows(torch.tensor([cur[r]], device="cuda"), torch.tensor([pos[r]], device="cuda"),
                               H.padded_tables([tables[r]], [cl[r]], g.block_size), out_logits=lb)
            torch.cuda.synchronize()
            if not exact:
                assert float((la[r] - lb[0]).abs().max()) <= H.LOGIT_ATOL
            else:
                assert torch.equal(la[r], lb[0])
                assert dec_b.tokens_device()[0].item() == tok_a[r]
        cur, cl = tok_a, [n + 1 for n in cl]
    if not exact:
        assert float((kv_a.float() - kv_b.float()).abs().max()) <= 2.0 ** -5
    else:
        assert torch.equal(kv_a, kv_b)
    dec_a.close(); dec_b.close()


def test_deterministic_and_feedback(cuda_device):
    """Same inputs twice -> identical tokens; device-side token feedback
    (input_ids=None) follows the same trajectory as passing the ids."""
    lens = [33, 100]
    g, w, kv, tables, first = _setup(lens, seed=17, steps=8)
    runs = []
    for feedback in (False, False, True):
        kvg = kv.cuda()
        dec = H.make_decoder(w, kvg)
        cur, cl, out = list(first), [n + 1 for n in lens], []
        for s in range(8):
            ids = torch.tensor(cur, device="cuda") if (s == 0 or not feedback) else None
            toks = None
            dec.enqueue_rows(ids, torch.tensor([n - 1 for n in cl], device="cuda"),
                             H.padded_tables(tables, cl, g.block_size))
            torch.cuda.synchronize()
            cur = dec.tokens_device()[:2].tolist()
            out.append(cur)
            cl = [n + 1 for n in cl]
        runs.append((out, kvg.cpu()))
        dec.close()
    assert runs[0][0] == runs[1][0] == runs[2][0]
    assert torch.equal(runs[0][1], runs[1][1]) and torch.equal(runs[0][1], runs[2][1])


def test_bad_block_id_is_reported_not_followed(cuda_device):
    """An out-of-range block id sets the status word; the kernel substitutes
    block 0 instead of forming an address from it."""
    g, w, kv, tables, first = _setup([10], seed=18)
    dec = H.make_decoder(w, kv.cuda())
    with pytest.raises(RuntimeError, match="device status 2"):
        dec.decode_host([first[0]], [10], [[999999]])
    # the decoder stays usable and the word was cleared
    assert dec.decode_host([first[0]], [10], [tables[0]])
    code, st = dec.status()
    assert code == 0
    dec.close()


def test_options_are_per_decoder(cuda_device):
    """An option set on one decoder leaves another decoder of the same process alone: with other kernels
    chosen on A only (8 instead of 16 weight rows per MMA, no tcgen05, no FP32 kernels), a two-row step of B
    still equals a fresh decoder's."""
    from dfb_b200 import native
    lens = [40, 300]
    g, w, kv, tables, first = _setup(lens, seed=24)
    outs = []
    for touch_other in (False, True):
        other = H.make_decoder(w, kv.cuda())
        if touch_other:
            other.set_option(native.DFB_OPT_ROW_GEMV, 0)
            other.set_option(native.DFB_OPT_PAIR_GEMV, 0)
            other.set_option(native.DFB_OPT_TCGEN05, 0)
            other.set_option(native.DFB_OPT_LOOK_AHEAD, 0)
        dec = H.make_decoder(w, kv.cuda())
        logits = torch.zeros(2, g.vocab, device="cuda")
        dec.enqueue_rows(torch.tensor(first, device="cuda"), torch.tensor(lens, device="cuda"),
                         H.padded_tables(tables, [n + 1 for n in lens], g.block_size), out_logits=logits)
        torch.cuda.synchronize()
        outs.append(logits.clone())
        dec.close(); other.close()
    assert torch.equal(outs[0], outs[1])


def test_look_ahead_prefetch_changes_nothing(cuda_device):
    """The L2 look-ahead only moves bytes early: results are bit-identical with it on and off."""
    from dfb_b200 import native
    lens = [40, 300, 7, 64, 129]
    g, w, kv, tables, first = _setup(lens, seed=25, layers=3)
    outs = []
    for ahead in (31, 0):
        kvg = kv.cuda()
        dec = H.make_decoder(w, kvg)
        dec.set_option(native.DFB_OPT_LOOK_AHEAD, ahead)
        for rows in (5, 2, 1):
            logits = torch.zeros(rows, g.vocab, device="cuda")
            dec.enqueue_rows(torch.tensor(first[:rows], device="cuda"), torch.tensor(lens[:rows], device="cuda"),
                             H.padded_tables(tables[:rows], [n + 1 for n in lens[:rows]], g.block_size),
                             out_logits=logits)
            dec.enqueue_rows(torch.tensor(first[:rows], device="cuda"), torch.tensor(lens[:rows], device="cuda"),
                             H.padded_tables(tables[:rows], [n + 1 for n in lens[:rows]], g.block_size))   # graph path
            torch.cuda.synchronize()
            outs.append((logits.clone(), dec.tokens_device()[:rows].tolist()))
        code, st = dec.status()
        assert code == 0
        dec.close()
    for a, b in zip(outs[:3], outs[3:]):
        assert torch.equal(a[0], b[0]) and a[1] == b[1]


def test_bad_token_id_is_reported_not_followed(cuda_device):
    """A token id outside the embedding table, arriving on the DEVICE path (the host path refuses it before the
    launch), sets status 5 in the staging kernel and row 0 of the table is used instead: no address is formed
    from the id.  The decoder stays usable."""
    g, w, kv, tables, first = _setup([10, 20], seed=26)
    dec = H.make_decoder(w, kv.cuda())
    pos = torch.tensor([10, 20], device="cuda")
    bt = H.padded_tables(tables, [11, 21], g.block_size)
    for bad in (g.vocab, -1, 2 ** 40):
        dec.enqueue_rows(torch.tensor([first[0], bad], device="cuda"), pos, bt)
        torch.cuda.synchronize()
        code, st = dec.status()
        assert code == -4 and st.device_status == 5 and st.detail[1] == 1, (bad, code, st.device_status, list(st.detail))
    with pytest.raises(RuntimeError, match="bad argument"):
        dec.decode_host([g.vocab], [10], [tables[0][:1]])
    assert len(dec.decode_host([first[0]], [10], [tables[0][:1]])) == 1
    code, st = dec.status()
    assert code == 0
    dec.close()


def test_context_bound_too_small_is_reported(cuda_device):
    """``max_context`` below a row's real context would leave the chunk with the new token without a CTA:
    the kernel reports status 6, writes no K/V for that row and the merge tickets still balance (the next
    correct step matches the oracle).  A position beyond the block-table columns given is caught the same
    way (the grid never covers more than the given columns), so a stale table entry is never read."""
    lens = [200]
    g, w, kv, tables, first = _setup(lens, seed=27)
    kvg = kv.cuda()
    before = kvg.clone()
    dec = H.make_decoder(w, kvg)
    ids, pos = torch.tensor(first, device="cuda"), torch.tensor(lens, device="cuda")
    bt = H.padded_tables(tables, [201], g.block_size)
    dec.enqueue_rows(ids, pos, bt, max_context=10)
    torch.cuda.synchronize()
    code, st = dec.status()
    assert code == -4 and st.device_status == 6 and st.detail[0] == 2 and st.detail[2] == 200
    assert torch.equal(kvg, before)
    dec.enqueue_rows(ids, torch.tensor([300], device="cuda"), bt)      # position 300 needs a second column
    torch.cuda.synchronize()
    code, st = dec.status()
    assert code == -4 and st.device_status == 6 and st.detail[2] == 300
    assert torch.equal(kvg, before)
    # and a correct step afterwards is still right
    cos_sin = O.rope_cos_sin_table(g)
    want_logits, want_tok = O.decode_step(w, kv, cos_sin, first, lens, tables)
    logits = torch.zeros(1, g.vocab, device="cuda")
    dec.enqueue_rows(ids, pos, bt, out_logits=logits)
    torch.cuda.synchronize()
    assert float((logits.cpu() - want_logits.float()).abs().max()) <= H.LOGIT_ATOL
    dec.close()


def test_capacity_errors(cuda_device):
    g, w, kv, tables, first = _setup([10], seed=19)
    dec = H.make_decoder(w, kv.cuda())
    with pytest.raises(RuntimeError, match="sized for 8"):
        dec.decode_host([1] * 9, [1] * 9, [[0]] * 9)
    with pytest.raises(ValueError, match="page_table stride is 8"):
        dec.decode_host([1], [1], [[0] * 9])
    with pytest.raises(RuntimeError, match="bad argument"):
        dec.decode_host([1], [5000], [[0]])          # position beyond max_model_len
    assert dec.decode_rows(torch.zeros(0, dtype=torch.int64, device="cuda"), None, None) == []
    dec.close()


def test_option_and_tensor_parallel_argument_errors(cuda_device):
    """Bad option values and tensor-parallel misuse are refused with an error code, not acted on."""
    import ctypes as C

    from dfb_b200 import native

    g, w, kv, tables, first = _setup([10], seed=23)
    dec = H.make_decoder(w, kv.cuda())
    lib, h = native.lib(), dec._handle
    for opt, bad in ((native.DFB_OPT_ROW_GEMV, 9), (native.DFB_OPT_STEP_MODE, 2), (native.DFB_OPT_SMEM_CARVEOUT, 101),
                     (native.DFB_OPT_SMEM_CARVEOUT_MMA, -2), (native.DFB_OPT_LATE_TRIGGER, 2),
                     (native.DFB_OPT_PAIR_GEMV, 5), (native.DFB_OPT_BULK_X, -1), (native.DFB_OPT_TP_FUSED, 3),
                     (native.DFB_OPT_ATTN_WIDE, -1), (native.DFB_OPT_LOOK_AHEAD, 64),
                     (native.DFB_OPT_LMHEAD_AHEAD_MB, 101), (native.DFB_OPT_PEER_WAIT_US, 0), (99, 0)):
        assert lib.dfb_set_option(h, opt, bad) == -1, (opt, bad)          # DFB_E_BAD_ARG
    # a single-GPU decoder has no exchange window, and a tensor-parallel group needs 2, 4 or 8 ranks
    buf = C.create_string_buffer(native.DFB_TP_HANDLE_BYTES)
    assert lib.dfb_tp_window_handle(h, buf) == -1
    assert lib.dfb_tp_open_peers(h, buf) == -1
    assert lib.dfb_tp_open_loopback(h) == -1
    for size, rank in ((3, 0), (1, 0), (2, 2), (2, -1)):
        tp = native.DfbTensorParallel(size=size, rank=rank, vocab_offset=0, dtype_bf16=9, dtype_int8=0, op_sum=0)
        assert lib.dfb_set_tensor_parallel(h, C.byref(tp)) == -1, (size, rank)
    assert lib.dfb_set_tensor_parallel(h, None) == -1
    # the decoder still works after the refused calls
    assert len(dec.decode_host([first[0]], [10], [tables[0][:1]])) == 1
    dec.close()


def test_warm_captures_every_geometry_ahead_of_time(cuda_device):
    """After ``warm`` no step of the prepared kinds captures a graph any more: rows 1..3, contexts across the
    chunk (64, 128) and block (256, 512) boundaries, through the host-buffer and the device-pointer entries."""
    import time
    g = H.oracle_geometry(layers=2, vocab=2048)
    w = O.make_weights(g, seed=61, norm="random").to(torch.bfloat16)
    kv = O.new_kv_cache(g, 12, torch.bfloat16).cuda()
    dec = H.make_decoder(w, kv)
    t0 = time.perf_counter()
    held = dec.warm(max_rows=3, max_context=700)
    warm_s = time.perf_counter() - t0
    assert held > 0
    for rows in (1, 2, 3):
        tables = [[3 * r, 3 * r + 1, 3 * r + 2] for r in range(rows)]
        for ctx in (1, 64, 65, 128, 129, 256, 257, 511, 512, 513, 699):
            cols = -(-(ctx + 1) // g.block_size)
            ids, pos = [5] * rows, [ctx] * rows
            dec.decode_host(ids, pos, [t[:cols] for t in tables])
            bt = torch.tensor([t[:cols] for t in tables], dtype=torch.int32, device="cuda")
            dec.decode_rows(torch.tensor(ids, device="cuda"), torch.tensor(pos, device="cuda"), bt)
    assert dec.warm(max_rows=3, max_context=700) == held, "a step captured a graph that warm() had not prepared"
    assert warm_s < 30.0
    dec.close()
