"""The CPU oracle against the golden fixtures produced by the reference's own
torch model (tests/golden/make_golden.py).  Runs without a GPU."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import qwen3_decode as O

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden as G  # noqa: E402  (only its case definitions are used; the reference is not imported)


@pytest.fixture(scope="module")
def small_weights():
    return O.make_weights(G.SMALL, seed=1, norm="random")


def _run_small(w, z):
    toks, logits = O.greedy_generate(w, G.small_prompts(), G.SMALL_STEPS, keep_logits=True,
                                     fused_rounding=False, block_permutation=z["perm"].tolist())
    return toks.numpy(), torch.stack(logits).numpy()


def test_small_fp32_is_bit_exact(small_weights):
    z = np.load(GOLDEN / "small_l2_v2048_fp32.npz")
    toks, logits = _run_small(small_weights, z)
    assert np.array_equal(toks, z["tokens"])
    assert np.array_equal(logits, z["logits"])


def test_small_bf16_within_rounding(small_weights):
    """bf16: the reference's CPU GEMMs round the same sums in a different order,
    so equality is up to a couple of bf16 steps (2**-6 for |logit| in [2, 4))."""
    z = np.load(GOLDEN / "small_l2_v2048_bf16.npz")
    toks, logits = _run_small(small_weights.to(torch.bfloat16), z)
    assert np.array_equal(toks, z["tokens"])
    d = np.abs(logits - z["logits"])
    assert d.max() <= 2 * 2.0 ** -6 + 1e-6
    assert d.mean() <= 5e-3


@pytest.fixture(scope="module")
def full_weights():
    return O.make_weights(O.QWEN3_06B, seed=0, norm="ones")


def test_config1_fp32_greedy64(full_weights):
    """BASELINE config 1: fp32, prompt of 32 ids, 64 greedy tokens, block 256."""
    z = np.load(GOLDEN / "qwen3_06b_fp32_prompt32_greedy64.npz")
    assert z["prompt"].tolist() == G.config1_prompt(O.QWEN3_06B)
    toks, logits = O.greedy_generate(full_weights, [z["prompt"].tolist()], 64, keep_logits=True)
    assert toks[:, 0].tolist() == z["tokens"].tolist()
    lg = torch.stack(logits)[:, 0, :].numpy()
    assert np.abs(lg[:, z["probe_index"]] - z["probe_logits"]).max() <= 1e-4
    top = np.argsort(-lg, axis=-1, kind="stable")[:, :8]
    assert np.array_equal(top[:, 0], z["top_index"][:, 0])
    assert np.abs(np.take_along_axis(lg, z["top_index"], -1) - z["top_logits"]).max() <= 1e-4


def test_full_bf16_teacher_forced(full_weights):
    """Full geometry in bf16 (the dtype the CUDA path runs), two rows, the second
    crossing the 256-token block boundary, teacher-forced random inputs."""
    z = np.load(GOLDEN / "qwen3_06b_bf16_forced8.npz")
    prompts, forced = G.forced_case(O.QWEN3_06B)
    toks, logits = O.greedy_generate(full_weights.to(torch.bfloat16), prompts, G.FORCED_STEPS, keep_logits=True,
                                     fused_rounding=False, forced_inputs=forced)
    lg = torch.stack(logits).numpy()
    d = np.abs(lg[..., z["probe_index"]] - z["probe_logits"])
    assert d.max() <= 6.25e-2, d.max()
    assert d.mean() <= 1e-2, d.mean()
    want = z["tokens"]
    for s in range(G.FORCED_STEPS):
        for r in range(len(prompts)):
            got, ref = int(toks[s + 1, r]), int(want[s + 1, r])
            # a different argmax is accepted only when the two candidates tie within rounding
            assert got == ref or abs(lg[s, r, got] - lg[s, r, ref]) <= 6.25e-2


def test_byte_accounting():
    g = O.QWEN3_06B
    assert g.weight_bytes_per_step() == 1_192_099_840
    assert g.kv_bytes_per_token() == 114_688


def test_sampler_matches_reference_sampler():
    """``O.sample`` against the reference's ``Sampler.forward`` (layers/sampler.py:7-16) run by
    ``tests/golden/make_golden.py`` on the same logits, temperatures and exponential noise; the log-space
    form the CUDA kernels use picks the same tokens."""
    d = np.load(GOLDEN / "sampler_rows6_vocab1024.npz")
    logits, temps = torch.from_numpy(d["logits"]), torch.from_numpy(d["temperatures"])
    for k in range(d["noise"].shape[0]):
        noise = torch.from_numpy(d["noise"][k])
        assert O.sample(logits, temps, noise).tolist() == d["tokens"][k].tolist()
        assert O.sample_keys(logits, temps, noise).argmax(-1).tolist() == d["tokens"][k].tolist()
    assert len({tuple(t) for t in d["tokens"].tolist()}) > 1          # the draws differ: the fixture samples


def test_counter_noise_is_exponential():
    """The documented counter-based noise: Exp(1) moments and tail, no repeats across rows, steps or seeds."""
    e = O.counter_noise(seed=5, step=3, rows=8, vocab=151936).double()
    n = e.numel()
    assert abs(float(e.mean()) - 1.0) < 5e-3 and abs(float(e.var()) - 1.0) < 2e-2
    for x in (0.1, 1.0, 3.0):
        assert abs(float((e > x).double().mean()) - float(np.exp(-x))) < 4.0 * (np.exp(-x) / n) ** 0.5 + 1e-3
    assert float(e.min()) > 0.0
    assert not torch.equal(e[0], e[1])
    assert not torch.equal(e, O.counter_noise(5, 4, 8, 151936).double())
    assert not torch.equal(e, O.counter_noise(6, 3, 8, 151936).double())
    # a shard sees the noise of its global indices
    part = O.counter_noise(5, 3, 8, 1000, index_offset=4000).double()
    assert torch.equal(part, e[:, 4000:5000])
