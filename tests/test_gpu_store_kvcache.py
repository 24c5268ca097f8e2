"""``store_kvcache`` (the prefill side of the shared paged cache) against the
reference semantics (layers/attention.py:10-40): row i of key / value lands in
row slot_mapping[i] of the cache, slot -1 is skipped, nothing else changes."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _reference(key, value, k_cache, v_cache, slots):
    """The Triton kernel of the reference restated with torch indexing."""
    d = key.shape[1] * key.shape[2]
    kc, vc = k_cache.clone().view(-1, d), v_cache.clone().view(-1, d)
    for i, s in enumerate(slots.tolist()):
        if s == -1:
            continue
        kc[s] = key[i].reshape(-1)
        vc[s] = value[i].reshape(-1)
    return kc.view_as(k_cache), vc.view_as(v_cache)


@pytest.mark.parametrize("n_tokens", [0, 1, 7, 300, 4096])
def test_store_kvcache_matches_reference_semantics(cuda_device, n_tokens):
    from dfb_b200.kv_store import store_kvcache

    rng = np.random.Generator(np.random.Philox(key=70 + n_tokens))
    blocks, bs, heads, dim = 20, 256, 8, 128
    k_cache = torch.from_numpy(rng.standard_normal((blocks, bs, heads, dim), dtype=np.float32)).to(BF).cuda()
    v_cache = torch.from_numpy(rng.standard_normal((blocks, bs, heads, dim), dtype=np.float32)).to(BF).cuda()
    # key / value as slices of a fused qkv projection output: row stride larger than the row (as in the model)
    qkv = torch.from_numpy(rng.standard_normal((max(n_tokens, 1), 4096), dtype=np.float32)).to(BF).cuda()
    key = qkv[:n_tokens, 2048:3072].view(n_tokens, heads, dim)
    value = qkv[:n_tokens, 3072:4096].view(n_tokens, heads, dim)
    slots = rng.permutation(blocks * bs)[:n_tokens].astype(np.int32)
    slots[::5] = -1                                           # padding entries of a captured batch
    slots_t = torch.from_numpy(slots).cuda()
    want_k, want_v = _reference(key.cpu(), value.cpu(), k_cache.cpu(), v_cache.cpu(), torch.from_numpy(slots))
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    store_kvcache(key, value, k_cache, v_cache, slots_t, status)
    torch.cuda.synchronize()
    assert torch.equal(k_cache.cpu(), want_k) and torch.equal(v_cache.cpu(), want_v)   # bit-exact, nothing else touched
    assert status.tolist() == [0, 0, 0, 0]


def test_store_kvcache_skips_and_reports_a_bad_slot(cuda_device):
    from dfb_b200 import native
    from dfb_b200.kv_store import store_kvcache

    blocks, bs, heads, dim = 2, 256, 8, 128
    k_cache = torch.zeros(blocks, bs, heads, dim, dtype=BF, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    key = torch.ones(3, heads, dim, dtype=BF, device="cuda")
    value = torch.full((3, heads, dim), 2.0, dtype=BF, device="cuda")
    slots = torch.tensor([5, blocks * bs + 40, 7], dtype=torch.int32, device="cuda")   # the second is out of range
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    store_kvcache(key, value, k_cache, v_cache, slots, status)
    torch.cuda.synchronize()
    st = status.tolist()
    assert st[0] == native.DFB_STATUS_BAD_SLOT and st[2] == 1 and st[3] == blocks * bs + 40
    flat = k_cache.view(-1, heads * dim)
    assert float(flat[5].float().sum()) == heads * dim and float(flat[7].float().sum()) == heads * dim
    assert float(k_cache.float().sum()) == 2 * heads * dim              # only the two valid rows were written
    assert float(v_cache.float().sum()) == 2 * 2.0 * heads * dim
