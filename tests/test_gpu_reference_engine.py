"""The drop-in claim, exercised through the REFERENCE's own engine.

The unmodified reference package (installed by ``baseline/install_reference.sh``
into the git-ignored ``baseline/_ref``) is driven through its public API,
``LLM(dir, decode_backend=...)``, once with its torch decode path and once with
``decode_backend="megakernel"`` after the backend import switch
(``baseline/reference_engine.install_backend_switch``), so that the reference's
``ModelRunner`` builds and calls THIS repository's ``MegakernelBackend``:
scheduler, block manager, paged KV cache and prefill are the reference's.

Token streams are classified the reference's way (tools/correctness_smoke.py:
318-362): PASS = identical; CASCADE = every divergence starts at a decode token
(>= 1) and lengths agree -- the documented bf16 reduction-order cascade; FAIL =
a divergence at token 0 (the prefill output) or a length mismatch.
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "baseline"))
import reference_engine as R  # noqa: E402

pytestmark = pytest.mark.gpu


def classify(reference, actual):
    details, real_fail = [], False
    for i, (want, got) in enumerate(zip(reference, actual)):
        if want == got:
            continue
        if len(want) != len(got):
            real_fail = True
            details.append({"seq": i, "kind": "length"})
            continue
        first = next(j for j, (a, b) in enumerate(zip(want, got)) if a != b)
        real_fail |= first == 0
        details.append({"seq": i, "kind": "token", "first": first})
    if len(reference) != len(actual):
        real_fail = True
    return ("FAIL" if real_fail else "CASCADE" if details else "PASS"), details


@pytest.fixture(scope="module")
def model_dir(cuda_device, tmp_path_factory):
    if not R.available():
        pytest.skip("baseline/_ref is not installed (sh baseline/install_reference.sh)")
    return R.write_model_dir(tmp_path_factory.mktemp("qwen3_06b_seed0"), seed=0)


def test_megakernel_switch_inside_the_reference_engine(model_dir):
    R.import_reference()
    from nanovllm import SamplingParams

    steps = 64
    single = R.seeded_prompts(1, 32, 151936, 11)
    batch = R.seeded_prompts(4, 48, 151936, 12) + R.seeded_prompts(1, 300, 151936, 13)
    # the reference's own torch path (eager: the oracle arm of benchmarks/compare.py)
    llm = R.make_llm(model_dir, "torch", max_num_seqs=8, enforce_eager=True)
    want_single, _ = R.generate(llm, single, steps)
    want_batch, _ = R.generate(llm, batch, steps)
    llm.exit()

    runner_mod = R.install_backend_switch()
    llm = R.make_llm(model_dir, "megakernel", max_num_seqs=8)
    runner = llm.model_runner
    assert type(runner.megakernel).__module__.startswith("dfb_b200"), type(runner.megakernel)
    assert runner.megakernel.disabled_reason is None and runner.megakernel.ready
    got_single, rep_single = R.generate(llm, single, steps)
    assert runner.last_backend_used == "megakernel" and runner.last_fallback_reason is None
    got_batch, rep_batch = R.generate(llm, batch, steps)
    assert runner.last_backend_used == "megakernel"
    # every prefill wrote its K / V rows through this repository's store_kvcache (28 layers per prefill pass)
    assert R.STORE_KVCACHE_CALLS[0] >= 2 * 28, R.STORE_KVCACHE_CALLS
    # ... and attended over its prompt with this repository's prefill attention
    assert R.PREFILL_ATTENTION_CALLS[0] >= 2 * 28, R.PREFILL_ATTENTION_CALLS
    for rep in (rep_single, rep_batch):
        for req in rep["requests"]:
            # prefill ran on the torch path, every decode step on this repository's kernels
            assert req["backend_actual"] in ("torch+megakernel", "megakernel"), req["backend_actual"]
            assert req["fallback_reason"] is None
    for name, want, got in (("single", want_single, got_single), ("batch", want_batch, got_batch)):
        status, details = classify(want, got)
        print(f"{name}: {status} {details}")
        assert status in ("PASS", "CASCADE"), (name, details)
    # a sampled row is not admitted: explicit reason, torch path, no exception
    sp = SamplingParams(temperature=0.7, max_tokens=4, ignore_eos=True)
    out = llm.generate(R.seeded_prompts(1, 16, 151936, 14), sp, use_tqdm=False)
    assert len(out[0]["token_ids"]) == 4
    assert runner.last_backend_used == "torch"
    assert runner.last_fallback_reason == "Task-graph megakernel supports greedy sampling only"
    llm.exit()
    assert runner_mod.MegakernelBackend.__module__.startswith("dfb_b200")
