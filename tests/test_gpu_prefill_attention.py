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


@pytest.mark.parametrize("case", [((300, 44),), ((513, 1), (256, 256)), ((70, 70), (1000, 300), (64, 3))])
def test_prefill_attention_with_prefix_cache(cuda_device, case):
    """Keys read back from the paged cache through scattered block tables, fewer queries than keys: query i of a
    sequence attends to keys 0 .. i + (keys - queries), like the last `queries` rows of a full causal pass."""
    from dfb_b200 import native
    from dfb_b200.kv_store import prefill_attention, store_kvcache

    rng = np.random.Generator(np.random.Philox(key=95 + len(case)))
    hq, hkv, d, bs = 16, 8, 128, 256
    k_lens, q_lens = [c[0] for c in case], [c[1] for c in case]
    n_k = sum(k_lens)
    qkv = torch.from_numpy(rng.standard_normal((n_k, 4096), dtype=np.float32)).to(BF)
    q_all, k_all, v_all = qkv[:, :2048].view(n_k, hq, d), qkv[:, 2048:3072].view(n_k, hkv, d), qkv[:, 3072:].view(n_k, hkv, d)
    want_all = _reference(q_all, k_all, v_all, k_lens, d ** -0.5)          # full causal pass over every sequence
    # scattered physical blocks, the whole of every sequence's K / V written through store_kvcache
    need = [-(-n // bs) for n in k_lens]
    pool = rng.permutation(sum(need) + 3).tolist()
    tables, slots = [], []
    for n, nb in zip(k_lens, need):
        t = [pool.pop() for _ in range(nb)]
        tables.append(t)
        slots += [t[p // bs] * bs + p % bs for p in range(n)]
    dev = qkv.cuda()
    kd, vd = dev[:, 2048:3072].view(n_k, hkv, d), dev[:, 3072:].view(n_k, hkv, d)
    k_cache = torch.zeros(sum(need) + 3, bs, hkv, d, dtype=BF, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    store_kvcache(kd, vd, k_cache, v_cache, torch.tensor(slots, dtype=torch.int32, device="cuda"))
    # the queries: only the last q_len tokens of every sequence
    rows, start = [], 0
    for n, m in zip(k_lens, q_lens):
        rows += list(range(start + n - m, start + n))
        start += n
    qd = dev[rows][:, :2048].contiguous().view(len(rows), hq, d)
    cu_q = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor(np.concatenate([[0], np.cumsum(k_lens)]), dtype=torch.int32, device="cuda")
    width = max(need)
    bt = torch.tensor([t + [0] * (width - len(t)) for t in tables], dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    got = prefill_attention(qd, k_cache, v_cache, cu_q, max(q_lens), d ** -0.5, cu_seqlens_k=cu_k, block_table=bt,
                            status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    diff = (got.float().cpu() - want_all[rows]).abs()
    assert float(diff.max()) <= 2.0 ** -6, float(diff.max())
    # a block id outside the cache is recorded, not followed
    bad = bt.clone()
    bad[0, 0] = k_cache.shape[0] + 5
    prefill_attention(qd, k_cache, v_cache, cu_q, max(q_lens), d ** -0.5, cu_seqlens_k=cu_k, block_table=bad, status=status)
    torch.cuda.synchronize()
    st = status.tolist()
    assert st[0] == native.DFB_STATUS_BAD_BLOCK and st[2] == 0 and st[3] == k_cache.shape[0] + 5
