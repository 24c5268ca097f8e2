"""The sampler fused after the LM head (temperature rows) against the oracle's
restatement of the reference sampler (layers/sampler.py:7-16), with the noise
the kernels document (``oracle.counter_noise``), and against the softmax
distribution itself."""

import numpy as np
import pytest
import torch

from oracle import qwen3_decode as O
from tests import harness as H

pytestmark = pytest.mark.gpu

BF = torch.bfloat16
# A sampled token may differ from the oracle's only if the oracle's own keys (logit / T - log E) of the two
# candidates are closer than this: logf on the device and in numpy differ in the last bits.
KEY_GAP_ATOL = 1e-3


def _rand(shape, seed, scale=1.0):
    rng = np.random.Generator(np.random.Philox(key=seed))
    return torch.from_numpy((rng.standard_normal(shape, dtype=np.float32) * scale)).to(BF)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _lmhead(dec, hd, rd, temps, toks, logits, rows):
    from dfb_b200 import native

    native.check(native.lib().dfb_launch_lmhead_sample(
        dec._handle, hd.data_ptr(), rd.data_ptr(), temps.data_ptr() if temps is not None else None,
        toks.data_ptr(), logits.data_ptr() if logits is not None else None, rows, _stream()), "lmhead_sample")


def _check_tokens(got_tokens, logits, temps, seed, step):
    """Every token equals the oracle sampler's on the same logits and noise, or was a near tie of its keys."""
    rows, vocab = logits.shape
    noise = O.counter_noise(seed, step, rows, vocab)
    want = O.sample(logits, temps, noise)
    keys = O.sample_keys(logits, temps, noise)
    for r in range(rows):
        g, w = int(got_tokens[r]), int(want[r])
        assert g == w or float(keys[r, w] - keys[r, g]) <= KEY_GAP_ATOL, (r, g, w, float(keys[r, w] - keys[r, g]))


# (rows, options): the FP32 kernel (1-2 rows), tcgen05 (default for 3-8 rows), mma.sync with 16 rows per MMA,
# mma.sync with 8 rows per MMA
@pytest.mark.parametrize("rows,options", [(1, {}), (2, {}), (4, {}), (8, {}), (8, {"DFB_OPT_TCGEN05": 0}),
                                          (5, {"DFB_OPT_TCGEN05": 0, "DFB_OPT_PAIR_GEMV": 0})])
def test_sampled_lmhead_matches_oracle_sampler(cuda_device, rows, options):
    from dfb_b200 import native

    g = H.oracle_geometry(layers=1, vocab=4096)
    w = O.make_weights(g, seed=31, norm="random").to(BF)
    dec = H.make_decoder(w, O.new_kv_cache(g, 1, BF).cuda())
    for name, value in options.items():
        dec.set_option(getattr(native, name), value)
    seed = 0x1234_5678_9ABC_DEF0
    dec.set_seed(seed)
    h, res = _rand((rows, g.hidden), 41, 4.0), _rand((rows, g.hidden), 42, 4.0)
    temps_host = torch.tensor([0.7, 0.0, 1.0, 1.5, 0.3, 1e-12, 2.0, 0.9][:rows], dtype=torch.float32)
    hd, rd, temps = h.cuda(), res.cuda(), temps_host.cuda()
    toks = torch.zeros(12, dtype=torch.int32, device="cuda")
    logits = torch.zeros(rows, g.vocab, dtype=torch.float32, device="cuda")
    seen = []
    for step in range(3):   # the noise stream advances by one per sampled launch
        _lmhead(dec, hd, rd, temps, toks, logits, rows)
        torch.cuda.synchronize()
        got_logits = logits.cpu()
        assert float((got_logits - O.op_final_norm_lmhead(h, res, w).float()).abs().max()) <= 2.0 ** -4
        _check_tokens(toks[:rows].tolist(), got_logits, temps_host, seed, step)
        for r in range(rows):   # rows at or below 1e-10 stay greedy
            if temps_host[r] <= 1e-10:
                assert int(toks[r]) == int(got_logits[r].argmax())
        seen.append(toks[:rows].tolist())
    assert seen[0] != seen[1] or seen[1] != seen[2]       # fresh noise each step
    # a greedy launch in between neither draws nor advances the stream
    _lmhead(dec, hd, rd, None, toks, logits, rows)
    torch.cuda.synchronize()
    assert toks[:rows].tolist() == logits.cpu().argmax(-1).tolist()
    _lmhead(dec, hd, rd, temps, toks, logits, rows)
    torch.cuda.synchronize()
    _check_tokens(toks[:rows].tolist(), logits.cpu(), temps_host, seed, 3)
    # the same seed again restarts the stream
    dec.set_seed(seed)
    _lmhead(dec, hd, rd, temps, toks, logits, rows)
    torch.cuda.synchronize()
    assert toks[:rows].tolist() == seen[0]
    dec.close()


@pytest.mark.parametrize("rows", [1, 8])
def test_sampled_tokens_follow_the_softmax(cuda_device, rows):
    """Frequencies of the sampled tokens over many draws against softmax(logits / T): a chi-square test over
    the most likely tokens and the rest (the noise differs per row and step, so all rows of a launch with the
    same hidden state are independent draws from one distribution)."""
    g = H.oracle_geometry(layers=1, vocab=1024)
    w = O.make_weights(g, seed=32, norm="random").to(BF)
    dec = H.make_decoder(w, O.new_kv_cache(g, 1, BF).cuda())
    dec.set_seed(77)
    h1, r1 = _rand((1, g.hidden), 43, 6.0), _rand((1, g.hidden), 44, 6.0)
    h, res = h1.repeat(rows, 1).contiguous(), r1.repeat(rows, 1).contiguous()
    temperature = 0.8
    hd, rd = h.cuda(), res.cuda()
    temps = torch.full((rows,), temperature, dtype=torch.float32, device="cuda")
    launches = 16000 // rows
    toks = torch.zeros(launches, 12, dtype=torch.int32, device="cuda")
    logits = torch.zeros(rows, g.vocab, dtype=torch.float32, device="cuda")
    _lmhead(dec, hd, rd, None, toks[0], logits, rows)
    for i in range(launches):
        _lmhead(dec, hd, rd, temps, toks[i], None, rows)
    torch.cuda.synchronize()
    draws = toks[:, :rows].reshape(-1).cpu().numpy()
    probs = torch.softmax(logits[0].cpu().double() / temperature, dim=-1).numpy()
    order = np.argsort(-probs)
    top = order[:24]
    assert probs[top[0]] < 0.8                      # the case is not a degenerate one-token distribution
    counts = np.bincount(draws, minlength=g.vocab).astype(np.float64)
    n = float(len(draws))
    observed = np.append(counts[top], n - counts[top].sum())
    expected = np.append(probs[top], 1.0 - probs[top].sum()) * n
    keep = expected >= 5.0
    chi2 = float((((observed - expected) ** 2) / expected)[keep].sum())
    dof = int(keep.sum()) - 1
    # 99.9th percentile of chi-square (Wilson-Hilferty): a correct sampler fails this once in a thousand seeds,
    # and the seed is fixed
    limit = dof * (1.0 - 2.0 / (9.0 * dof) + 3.09 * (2.0 / (9.0 * dof)) ** 0.5) ** 3
    assert chi2 <= limit, (chi2, limit, dof)
    dec.close()


def test_sampled_decode_step_through_the_decoder(cuda_device):
    """Whole steps from host data with per-row temperatures: greedy rows of a mixed batch are untouched, the
    sampled rows follow the oracle sampler on the step's own logits, and the seed makes the run repeatable."""
    g = H.oracle_geometry(layers=2, vocab=4096)
    w = O.make_weights(g, seed=33, norm="random").to(BF)
    rows, lens = 4, [5, 17, 40, 3]
    temps = [0.0, 0.9, 1.3, 0.0]
    history = torch.from_numpy(np.random.Generator(np.random.Philox(key=45)).standard_normal(
        tuple(O.new_kv_cache(g, 8, BF).shape), dtype=np.float32) * 0.5).to(BF).cuda()

    def run(seed, temperatures, use_graph=True):
        kv = O.new_kv_cache(g, 8, BF).cuda()
        kv.copy_(history)
        dec = H.make_decoder(w, kv, use_graph=use_graph)
        dec.set_seed(seed)
        tables = [[r] for r in range(rows)]
        out = []
        ids = [11, 22, 33, 44]
        for step in range(3):
            ids = dec.decode_host(ids, [n + step for n in lens], tables, temperatures=temperatures)
            out.append(list(ids))
        dec.close()
        return out

    greedy = run(1, None)
    a, b, c = run(1, temps), run(1, temps), run(2, temps)
    assert a == b                                   # same seed: same draws
    assert a == run(1, temps, use_graph=False)      # the captured step draws what the plain launches draw
    assert a != c                                   # another seed: other draws
    assert [t[0] for t in a][0] == greedy[0][0] and a[0][3] == greedy[0][3]   # first step: greedy rows unchanged
    assert a[0][1] != greedy[0][1] or a[0][2] != greedy[0][2] or a[1] != greedy[1]

    # device-pointer path with out_logits: the sampled tokens against the oracle sampler on the same logits
    kv = O.new_kv_cache(g, 8, BF).cuda()
    kv.copy_(history)
    dec = H.make_decoder(w, kv)
    dec.set_seed(5)
    ids = torch.tensor([11, 22, 33, 44], dtype=torch.int64, device="cuda")
    tables = torch.arange(rows, dtype=torch.int32, device="cuda").reshape(rows, 1).contiguous()
    t_dev = torch.tensor(temps, dtype=torch.float32, device="cuda")
    logits = torch.zeros(rows, g.vocab, dtype=torch.float32, device="cuda")
    for step in range(2):
        pos = torch.tensor([n + step for n in lens], dtype=torch.int64, device="cuda")
        dec.enqueue_rows(ids if step == 0 else None, pos, tables, out_logits=logits, temperatures=t_dev)
        torch.cuda.synchronize()
        _check_tokens(dec.tokens_device()[:rows].tolist(), logits.cpu(), torch.tensor(temps), 5, step)
    code, st = dec.status()
    assert code == 0 and st.device_status == 0
    dec.close()
