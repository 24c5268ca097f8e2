"""Every tensor-parallel shard shape on ONE GPU: the ops of rank r of t are run
through the C ABI on the rank's slices of the weights and of the KV cache, the
ranks' partial results are added on the host, and the sums are compared with
the unsharded CPU oracle.  This covers what a rank computes for t = 2, 4, 8
(QKV rows 2048 / 1024 / 512, 4 / 2 / 1 KV heads, o_proj and down_proj input
widths, gate/up rows, LM-head shard and its vocabulary offset) without needing
t GPUs; the exchange itself is covered by test_gpu_tensor_parallel.py."""

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


@pytest.mark.parametrize("rows", [1, 2, 5, 8])
@pytest.mark.parametrize("size", [2, 4, 8])
def test_rank_ops_sum_to_the_unsharded_layer(cuda_device, size, rows):
    from dfb_b200 import native
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.tensor_parallel import merge_shard_argmax, shard_weights

    lib = native.lib()
    g = H.oracle_geometry(layers=1, vocab=2048)
    w = O.make_weights(g, seed=40 + size, norm="random").to(BF)
    lw = w.layers[0]
    cos_sin = O.rope_cos_sin_table(g)
    ctx_lens = [300, 17, 1025, 64, 128, 129, 2047, 1][:rows]
    tables, nblocks = O.allocate_blocks(ctx_lens, g.block_size)
    kv = _rand((2, g.layers, nblocks, g.block_size, g.kv_heads, g.head_dim), 7)
    positions = torch.tensor([n - 1 for n in ctx_lens])
    h, res = _rand((rows, g.hidden), 1), _rand((rows, g.hidden), 2)

    # unsharded oracle layer
    kv_want = kv.clone()
    qkv_want, res1 = O.op_rmsnorm_qkv(h, res, lw, w)
    q, k, v = O.op_qknorm_rope(qkv_want, positions, lw, w, cos_sin)
    attn_want = O.op_paged_attention_decode(q, k, v, kv_want, 0, positions, tables, g)
    o_want = O.op_oproj(attn_want, lw, w)
    act_want, res2 = O.op_rmsnorm_gateup_swiglu(o_want, res1, lw, w, fused_rounding=True)
    down_want = O.op_down(act_want, lw, w)
    logits_want = O.op_final_norm_lmhead(down_want, res2, w).float()

    full = H.to_decoder_weights(w)
    bt = H.padded_tables(tables, ctx_lens, g.block_size)
    pos32 = positions.to(torch.int32).cuda()
    hd, rd = h.cuda(), res.cuda()
    o_sum = torch.zeros(rows, g.hidden)
    down_sum = torch.zeros(rows, g.hidden)
    best_vals, best_idx = [], []
    for rank in range(size):
        sw = shard_weights(full, rank, size)
        lg, sl = sw.geom, sw.layers[0]
        h0, h1 = rank * lg.kv_heads, (rank + 1) * lg.kv_heads
        kv_r = kv[:, :, :, :, h0:h1, :].contiguous().cuda()
        dec = StreamDecoder(sw, kv_r[0], kv_r[1], g.block_size, nblocks, g.max_pos)
        # fused norm + this rank's Q/K/V rows
        qkv = torch.zeros(rows, lg.qkv_rows, dtype=BF, device="cuda")
        res_out = torch.zeros(rows, g.hidden, dtype=BF, device="cuda")
        native.check(lib.dfb_launch_rmsnorm_qkv(hd.data_ptr(), None, rd.data_ptr(), res_out.data_ptr(),
                                                sl.ln_in.data_ptr(), sl.wqkv.data_ptr(), qkv.data_ptr(), rows,
                                                g.hidden, lg.qkv_rows, g.eps, _stream()), "qkv")
        # attention over the rank's KV heads
        attn = torch.zeros(rows, lg.q_size, dtype=BF, device="cuda")
        native.check(lib.dfb_launch_attention(dec._handle, 0, qkv.data_ptr(), pos32.data_ptr(), bt.data_ptr(),
                                              bt.stride(0), None, attn.data_ptr(), rows, max(ctx_lens), _stream()),
                     "attention")
        torch.cuda.synchronize()
        assert torch.equal(res_out.cpu(), res1)
        want_slice = attn_want[:, rank * lg.q_size:(rank + 1) * lg.q_size]
        assert float((attn.cpu().float() - want_slice.float()).abs().max()) <= 2.0 ** -6
        assert float((kv_r.cpu().float() - kv_want[:, :, :, :, h0:h1, :].float()).abs().max()) <= 2.0 ** -6
        # o_proj partial from the ORACLE's attention slice (so that every rank's partial belongs to one sum)
        a_in = want_slice.contiguous().cuda()
        part = torch.zeros(rows, g.hidden, dtype=BF, device="cuda")
        native.check(lib.dfb_launch_linear(a_in.data_ptr(), sl.wo.data_ptr(), part.data_ptr(), rows, g.hidden,
                                           lg.q_size, _stream()), "o_proj")
        torch.cuda.synchronize()
        o_sum += part.cpu().float()
        # gate/up rows of the rank, then its down_proj partial
        act = torch.zeros(rows, lg.intermediate, dtype=BF, device="cuda")
        o_in, r1 = o_want.cuda(), res1.cuda()
        native.check(lib.dfb_launch_rmsnorm_gateup_swiglu(o_in.data_ptr(), r1.data_ptr(), None, sl.ln_post.data_ptr(),
                                                          sl.wgu.data_ptr(), act.data_ptr(), rows, g.hidden,
                                                          lg.intermediate, g.eps, _stream()), "gate/up")
        torch.cuda.synchronize()
        act_slice = act_want[:, rank * lg.intermediate:(rank + 1) * lg.intermediate]
        assert float((act.cpu().float() - act_slice.float()).abs().max()) <= 2.0 ** -6
        a2 = act_slice.contiguous().cuda()
        part2 = torch.zeros(rows, g.hidden, dtype=BF, device="cuda")
        native.check(lib.dfb_launch_linear(a2.data_ptr(), sl.wd.data_ptr(), part2.data_ptr(), rows, g.hidden,
                                           lg.intermediate, _stream()), "down_proj")
        torch.cuda.synchronize()
        down_sum += part2.cpu().float()
        dec.close()
        # LM-head shard: logits of rows [offset, offset + local vocab) and the shard's winner.  A decoder that
        # knows its vocabulary offset is needed for that, which only a tensor-parallel decoder has; the
        # host merge rule is applied to the slices of the oracle's logits instead.
        sl_logits = logits_want[:, sw.vocab_offset:sw.vocab_offset + lg.vocab]
        val, idx = sl_logits.max(dim=1)
        idx = torch.tensor([int((sl_logits[b] == val[b]).nonzero()[0]) for b in range(rows)])
        best_vals.append(val.tolist())
        best_idx.append(idx.tolist())

    # partial sums: each partial was rounded to bf16 once, so the sum differs from the oracle's single rounding
    # by at most one bf16 step per rank at these magnitudes (|o_proj|, |down| < 2)
    assert float((o_sum - o_want.float()).abs().max()) <= size * 2.0 ** -7
    assert float((down_sum - down_want.float()).abs().max()) <= size * 2.0 ** -7
    want_tok = [int((logits_want[b] == logits_want[b].max()).nonzero()[0]) for b in range(rows)]
    assert merge_shard_argmax(best_vals, best_idx, g.vocab // size) == want_tok
