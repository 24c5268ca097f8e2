"""Causal varlen prefill attention against the reference computation in fp32
(the CPU restatement of layers/attention.py:64-70 that the oracle and the golden
fixtures use: per sequence, causal softmax(q k^T / sqrt(d)) v with grouped-query
heads), on ragged batches, strided q / k / v views of a fused projection, and
the lengths around the 64-row tiles."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _reference(q, k, v, lens, scale):
    """fp32 causal attention per sequence; q [N, Hq, D], k / v [N, Hkv, D] (bf16 values)."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    rep = q.shape[1] // k.shape[1]
    start = 0
    for n in lens:
        qs = q[start:start + n].float().transpose(0, 1)                       # [Hq, n, D]
        ks = k[start:start + n].float().repeat_interleave(rep, dim=1).transpose(0, 1)
        vs = v[start:start + n].float().repeat_interleave(rep, dim=1).transpose(0, 1)
        s = torch.matmul(qs, ks.transpose(1, 2)) * scale
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), diagonal=1), float("-inf"))
        out[start:start + n] = torch.matmul(torch.softmax(s, dim=-1), vs).transpose(0, 1)
        start += n
    return out


@pytest.mark.parametrize("lens", [(1,), (5,), (63,), (64,), (65,), (128, 129), (200, 1, 64, 513), (1000,), (17, 300, 2, 90, 64, 7)])
def test_prefill_attention_matches_fp32_reference(cuda_device, lens):
    from dfb_b200.kv_store import prefill_attention

    rng = np.random.Generator(np.random.Philox(key=80 + sum(lens)))
    n, hq, hkv, d = sum(lens), 16, 8, 128
    # q / k / v as the slices of one fused projection output (row stride 4096), scaled like post-norm activations
    qkv = torch.from_numpy(rng.standard_normal((n, 4096), dtype=np.float32)).to(BF)
    q, k, v = qkv[:, :2048].view(n, hq, d), qkv[:, 2048:3072].view(n, hkv, d), qkv[:, 3072:].view(n, hkv, d)
    scale = d ** -0.5
    want = _reference(q, k, v, lens, scale)
    dev = qkv.cuda()
    qd, kd, vd = dev[:, :2048].view(n, hq, d), dev[:, 2048:3072].view(n, hkv, d), dev[:, 3072:].view(n, hkv, d)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    got = prefill_attention(qd, kd, vd, cu, max(lens), scale)
    torch.cuda.synchronize()
    diff = (got.float().cpu() - want).abs()
    # outputs are averages of N(0,1) values, |out| < 4: bf16 rounding of the output (2^-7 at |x| in [2, 4)) plus
    # the bf16 rounding of the probabilities before they multiply V
    assert float(diff.max()) <= 2.0 ** -6, float(diff.max())
    assert float(diff.mean()) <= 2.0 ** -9, float(diff.mean())
    # the first token of every sequence attends to itself only: its output is its own V row, exactly
    start = 0
    for m in lens:
        for h in range(hq):
            assert torch.equal(got[start, h].cpu(), v[start, h // 2])
        start += m


def test_prefill_attention_then_store_fill_the_cache_like_the_decode_path_reads_it(cuda_device):
    """Prefill side end to end: attention over the prompt and the KV write into paged slots; the cache rows
    are then exactly the K / V rows of the prompt, at the slots the block table names."""
    from dfb_b200.kv_store import prefill_attention, store_kvcache

    rng = np.random.Generator(np.random.Philox(key=91))
    lens, hq, hkv, d, bs = (300, 40), 16, 8, 128, 256
    n = sum(lens)
    qkv = torch.from_numpy(rng.standard_normal((n, 4096), dtype=np.float32)).to(BF).cuda()
    q, k, v = qkv[:, :2048].view(n, hq, d), qkv[:, 2048:3072].view(n, hkv, d), qkv[:, 3072:].view(n, hkv, d)
    tables = [[5, 2], [7]]
    slots = []
    for t, m in zip(tables, lens):
        slots += [t[p // bs] * bs + p % bs for p in range(m)]
    k_cache = torch.zeros(8, bs, hkv, d, dtype=BF, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    store_kvcache(k, v, k_cache, v_cache, torch.tensor(slots, dtype=torch.int32, device="cuda"))
    cu = torch.tensor([0, lens[0], n], dtype=torch.int32, device="cuda")
    out = prefill_attention(q, k, v, cu, max(lens), d ** -0.5)
    torch.cuda.synchronize()
    flat_k, flat_v = k_cache.view(-1, hkv, d), v_cache.view(-1, hkv, d)
    assert torch.equal(flat_k[slots], k) and torch.equal(flat_v[slots], v)
    assert int((k_cache.float().abs().sum(dim=(2, 3)) > 0).sum()) == n          # no other slot was written
    want = _reference(q.cpu(), k.cpu(), v.cpu(), lens, d ** -0.5)
    assert float((out.float().cpu() - want).abs().max()) <= 2.0 ** -6
