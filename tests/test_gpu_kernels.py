"""Each CUDA kernel, launched alone through the C ABI, against the oracle's
restatement of the same step of the reference torch path."""

import ctypes as C

import numpy as np
import pytest
import torch

from oracle import qwen3_decode as O
from tests import harness as H

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _rand(shape, seed, scale=1.0):
    rng = np.random.Generator(np.random.Philox(key=seed))
    return torch.from_numpy((rng.standard_normal(shape, dtype=np.float32) * scale)).to(BF)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return t.data_ptr() if t is not None else None


@pytest.fixture(scope="module")
def small(cuda_device):
    g = H.oracle_geometry(layers=1, vocab=1024)
    w = O.make_weights(g, seed=21, norm="random").to(BF)
    return g, w


def _close(a, b, atol):
    d = (a.float().cpu() - b.float()).abs()
    return float(d.max()) <= atol, float(d.max())


@pytest.mark.parametrize("rows", [1, 2, 3, 5, 8])
def test_rmsnorm_qkv(small, rows):
    from dfb_b200 import native
    g, w = small
    lw = w.layers[0]
    h, res = _rand((rows, g.hidden), 1), _rand((rows, g.hidden), 2)
    want_qkv, want_res = O.op_rmsnorm_qkv(h, res, lw, w)
    out = torch.zeros(rows, g.qkv_rows, dtype=BF, device="cuda")
    res_out = torch.zeros(rows, g.hidden, dtype=BF, device="cuda")
    hd, rd, ln, wq = h.cuda(), res.cuda(), lw.ln_in.cuda(), lw.wqkv.cuda()
    native.check(native.lib().dfb_launch_rmsnorm_qkv(_ptr(hd), None, _ptr(rd), _ptr(res_out), _ptr(ln), _ptr(wq),
                                                     _ptr(out), rows, g.hidden, g.qkv_rows, g.eps, _stream()), "qkv")
    torch.cuda.synchronize()
    assert torch.equal(res_out.cpu(), want_res)            # the residual sum is rounded once: exact
    ok, d = _close(out, want_qkv, 2.0 ** -6)                # |qkv| < 4: at most one bf16 step
    assert ok, d


def test_rmsnorm_qkv_embedding_gather(small):
    from dfb_b200 import native
    g, w = small
    lw = w.layers[0]
    ids = [5, 1023, 0]
    want_qkv, want_res = O.op_rmsnorm_qkv(w.embed[torch.tensor(ids)], None, lw, w)
    out = torch.zeros(3, g.qkv_rows, dtype=BF, device="cuda")
    res_out = torch.zeros(3, g.hidden, dtype=BF, device="cuda")
    emb, ln, wq = w.embed.cuda(), lw.ln_in.cuda(), lw.wqkv.cuda()
    idt = torch.tensor(ids, dtype=torch.int32, device="cuda")
    native.check(native.lib().dfb_launch_rmsnorm_qkv(_ptr(emb), _ptr(idt), None, _ptr(res_out), _ptr(ln), _ptr(wq),
                                                     _ptr(out), 3, g.hidden, g.qkv_rows, g.eps, _stream()), "qkv")
    torch.cuda.synchronize()
    assert torch.equal(res_out.cpu(), want_res)
    ok, d = _close(out, want_qkv, 2.0 ** -8)
    assert ok, d


@pytest.mark.parametrize("n,k", [(1024, 2048), (1024, 3072), (4096, 1024),
                                 # o_proj / down_proj of the tensor-parallel shards (1/2, 1/4, 1/8 of 2048 and 3072)
                                 (1024, 1024), (1024, 512), (1024, 256), (1024, 1536), (1024, 768), (1024, 384)])
@pytest.mark.parametrize("rows", [1, 2, 4, 8])
def test_linear(cuda_device, n, k, rows):
    from dfb_b200 import native
    x, wt = _rand((rows, k), 3), _rand((n, k), 4, 0.02)
    want = O.linear(x, wt.float())
    out = torch.zeros(rows, n, dtype=BF, device="cuda")
    xd, wd = x.cuda(), wt.cuda()
    native.check(native.lib().dfb_launch_linear(_ptr(xd), _ptr(wd), _ptr(out), rows, n, k, _stream()), "linear")
    torch.cuda.synchronize()
    ok, d = _close(out, want, 2.0 ** -6)
    assert ok, d
    # an exact fp64 dot product rounded once must be within one bf16 step too
    exact = (x.double() @ wt.double().T).to(BF)
    ok, d = _close(out, exact, 2.0 ** -6)
    assert ok, d


def test_linear_rejects_unsupported_k(cuda_device):
    from dfb_b200 import native
    t = torch.zeros(8, 4096, dtype=BF, device="cuda")
    assert native.lib().dfb_launch_linear(_ptr(t), _ptr(t), _ptr(t), 1, 8, 4096, _stream()) == -2
    assert native.lib().dfb_launch_linear(_ptr(t), _ptr(t), _ptr(t), 9, 8, 1024, _stream()) == -1


@pytest.mark.parametrize("rows", [1, 8])
def test_rmsnorm_gateup_swiglu(small, rows):
    from dfb_b200 import native
    g, w = small
    lw = w.layers[0]
    h, res = _rand((rows, g.hidden), 5), _rand((rows, g.hidden), 6)
    want_act, want_res = O.op_rmsnorm_gateup_swiglu(h, res, lw, w, fused_rounding=True)
    act = torch.zeros(rows, g.intermediate, dtype=BF, device="cuda")
    res_out = torch.zeros(rows, g.hidden, dtype=BF, device="cuda")
    hd, rd, ln, wg = h.cuda(), res.cuda(), lw.ln_post.cuda(), lw.wgu.cuda()
    native.check(native.lib().dfb_launch_rmsnorm_gateup_swiglu(
        _ptr(hd), _ptr(rd), _ptr(res_out), _ptr(ln), _ptr(wg), _ptr(act), rows, g.hidden, g.intermediate, g.eps,
        _stream()), "gateup")
    torch.cuda.synchronize()
    assert torch.equal(res_out.cpu(), want_res)
    ok, d = _close(act, want_act, 2.0 ** -6)
    assert ok, d


def _attention_case(g, w, rows, ctx_lens, seed, perm=None, row_active=None, ring=None, options=None):
    """Random KV history in a paged cache; one new token per row.  ``ring``: True forces the streaming
    kernel (dfb_attnring.cuh) for every grid size, False the register-resident one, None the default rule.
    ``options``: further ``{option name: value}`` of the decoder."""
    from dfb_b200 import native
    lw = w.layers[0]
    tables, nblocks = O.allocate_blocks(ctx_lens, g.block_size, perm)
    pool = nblocks if perm is None else len(perm)
    kv = _rand((2, g.layers, pool, g.block_size, g.kv_heads, g.head_dim), seed)
    qkv = _rand((rows, g.qkv_rows), seed + 1)
    positions = torch.tensor([n - 1 for n in ctx_lens])
    cos_sin = O.rope_cos_sin_table(g)
    kv_want = kv.clone()
    q, k, v = O.op_qknorm_rope(qkv, positions, lw, w, cos_sin)
    want = O.op_paged_attention_decode(q, k, v, kv_want, 0, positions, tables, g, row_active)
    kv_gpu = kv.cuda()
    dec = H.make_decoder(w, kv_gpu)
    if ring is not None:
        dec.set_option(native.DFB_OPT_ATTN_RING, 1 if ring else 0)
        dec.set_option(native.DFB_OPT_ATTN_RING32, 0)
    for name, value in (options or {}).items():
        dec.set_option(getattr(native, name), value)
    out = torch.zeros(rows, g.q_size, dtype=BF, device="cuda")
    bt = H.padded_tables(tables, ctx_lens, g.block_size)
    pos32 = positions.to(torch.int32).cuda()
    act = torch.tensor(row_active, dtype=torch.int32, device="cuda") if row_active is not None else None
    qd = qkv.cuda()
    native.check(native.lib().dfb_launch_attention(dec._handle, 0, _ptr(qd), _ptr(pos32), _ptr(bt), bt.stride(0),
                                                   _ptr(act), _ptr(out), rows, max(ctx_lens), _stream()), "attn")
    torch.cuda.synchronize()
    code, st = dec.status()
    assert code == 0, (st.device_status, list(st.detail))
    dec.close()
    return out.cpu(), want, kv_gpu.cpu(), kv_want, kv


@pytest.mark.parametrize("ring", [False, True])
@pytest.mark.parametrize("ctx_lens", [(1,), (2,), (8,), (9,), (63,), (64,), (65,), (72,), (73,), (255, 256, 257),
                                      (1, 700, 2048), (300, 17, 1025, 64, 128, 129, 2047, 512)])
def test_paged_attention(small, ctx_lens, ring):
    g, w = small
    out, want, kv_got, kv_want, _ = _attention_case(g, w, len(ctx_lens), list(ctx_lens), seed=31, ring=ring)
    d = (out.float() - want.float()).abs().max()
    assert float(d) <= 2.0 ** -6, float(d)          # |out| < 4
    assert torch.equal(kv_got, kv_want)            # new K/V rows written bit-exactly, nothing else touched


# How the register-resident kernel splits a row and merges the chunks: 64-position chunks merged through global
# partials and a ticket, the same merged inside a thread-block cluster (distributed shared memory), and both
# with 128-position chunks.  The limits are raised so that every grid of the list takes the variant.
ATTENTION_VARIANTS = {
    "ticket": {"DFB_OPT_ATTN_CLUSTER": 0, "DFB_OPT_ATTN_CHUNK128": 0},
    "cluster": {"DFB_OPT_ATTN_CLUSTER": 1 << 20, "DFB_OPT_ATTN_CHUNK128": 0},
    "chunk128_ticket": {"DFB_OPT_ATTN_CLUSTER": 0, "DFB_OPT_ATTN_CHUNK128": 1 << 20},
    "chunk128_cluster": {"DFB_OPT_ATTN_CLUSTER": 1 << 20, "DFB_OPT_ATTN_CHUNK128": 1 << 20},
    # the streaming kernel with 32 positions per CTA for every bound up to 1024 tokens
    "ring32": {"DFB_OPT_ATTN_RING32": 1},
}


@pytest.mark.parametrize("variant", sorted(ATTENTION_VARIANTS))
@pytest.mark.parametrize("ctx_lens", [(65,), (128,), (129,), (1, 100), (64, 65, 300), (1000, 3, 513, 1024),
                                      (255, 256, 257, 1, 2, 130, 700, 1024), (2048, 5)])
def test_paged_attention_split_variants(small, ctx_lens, variant):
    """Rows of one launch with different chunk counts (a cluster whose row has a single chunk passes no cluster
    barrier; CTAs beyond a row's last chunk pass both), up to the largest cluster (16 chunks) and beyond it."""
    g, w = small
    out, want, kv_got, kv_want, _ = _attention_case(g, w, len(ctx_lens), list(ctx_lens), seed=61, ring=False,
                                                    options=ATTENTION_VARIANTS[variant])
    assert float((out.float() - want.float()).abs().max()) <= 2.0 ** -6
    assert torch.equal(kv_got, kv_want)


@pytest.mark.parametrize("ring", [False, True])
def test_paged_attention_scattered_blocks(small, ring):
    g, w = small
    perm = np.random.Generator(np.random.Philox(key=9)).permutation(24).tolist()
    out, want, kv_got, kv_want, _ = _attention_case(g, w, 3, [1000, 2048, 513], seed=41, perm=perm, ring=ring)
    assert float((out.float() - want.float()).abs().max()) <= 2.0 ** -6
    assert torch.equal(kv_got, kv_want)


@pytest.mark.parametrize("ring", [False, True])
def test_inactive_row_leaves_kv_untouched(small, ring):
    """row_active == 0 skips the KV write and nothing else (the reference's
    tests/test_taskgraph_bs2.py:211-233)."""
    g, w = small
    out, want, kv_got, kv_want, kv_before = _attention_case(g, w, 2, [300, 40], seed=51, row_active=[1, 0], ring=ring)
    assert torch.equal(kv_got, kv_want)
    # row 1's slot is unchanged, row 0's slot changed
    assert torch.equal(kv_got[:, 0, 2, 39], kv_before[:, 0, 2, 39])
    assert not torch.equal(kv_got[:, 0, 1, 299 - 256], kv_before[:, 0, 1, 299 - 256])
    assert float((out.float() - want.float()).abs().max()) <= 2.0 ** -6


@pytest.mark.parametrize("rows", [1, 8])
def test_lmhead_argmax(small, rows):
    from dfb_b200 import native
    g, w = small
    h, res = _rand((rows, g.hidden), 7), _rand((rows, g.hidden), 8)
    want = O.op_final_norm_lmhead(h, res, w)
    kv = O.new_kv_cache(g, 1, BF).cuda()
    dec = H.make_decoder(w, kv)
    toks = torch.zeros(12, dtype=torch.int32, device="cuda")
    logits = torch.zeros(rows, g.vocab, dtype=torch.float32, device="cuda")
    hd, rd = h.cuda(), res.cuda()
    for _ in range(2):  # twice: the arrival ticket must reset itself
        native.check(native.lib().dfb_launch_lmhead_argmax(dec._handle, _ptr(hd), _ptr(rd), _ptr(toks), _ptr(logits),
                                                           rows, _stream()), "lmhead")
        torch.cuda.synchronize()
        got = logits.cpu()
        assert float((got - want.float()).abs().max()) <= 2.0 ** -5
        assert torch.equal(got, got.to(BF).float())                    # logits are bf16-rounded values
        assert toks[:rows].tolist() == got.argmax(-1).tolist()         # lowest index wins ties, like torch
    dec.close()


def test_argmax_tie_takes_lowest_index(cuda_device):
    """Duplicate embedding rows give exactly equal logits; the lower index must win."""
    from dfb_b200 import native
    g = H.oracle_geometry(layers=1, vocab=1024)
    w = O.make_weights(g, seed=22, norm="ones").to(BF)
    h, res = _rand((2, g.hidden), 9), _rand((2, g.hidden), 10)
    first = O.op_final_norm_lmhead(h, res, w)
    top = int(first[0].float().argmax())
    lo, hi = (3, 900) if top not in (3, 900) else (4, 901)
    w.embed[lo] = w.embed[top]
    w.embed[hi] = w.embed[top]
    w._f32.clear()
    want = O.op_final_norm_lmhead(h, res, w)
    kv = O.new_kv_cache(g, 1, BF).cuda()
    dec = H.make_decoder(w, kv)
    toks = torch.zeros(12, dtype=torch.int32, device="cuda")
    hd, rd = h.cuda(), res.cuda()
    native.check(native.lib().dfb_launch_lmhead_argmax(dec._handle, _ptr(hd), _ptr(rd), _ptr(toks), None, 2,
                                                       _stream()), "lmhead")
    torch.cuda.synchronize()
    assert int(toks[0]) == min(lo, top) == int(want[0].float().argmax())
    dec.close()
