"""Admission policy, shape contract, KV-cache attachment and the fallback
contract of the dispatch -- all on CPU with fakes, the way the reference tests
them (tests/test_megakernel_backend.py, tests/test_taskgraph_backend.py)."""

import warnings
from types import SimpleNamespace

import pytest
import torch

import dfb_b200 as P
from dfb_b200.backend import MegakernelBackend, qwen3_contract_mismatch


def hf(**kw):
    base = dict(model_type="qwen3", hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                num_attention_heads=16, num_key_value_heads=8, vocab_size=151936, head_dim=128,
                tie_word_embeddings=True, attention_bias=False)
    base.update(kw)
    return SimpleNamespace(**base)


def cfg(**kw):
    base = dict(hf_config=hf(), max_model_len=2048, max_num_seqs=8, tensor_parallel_size=1,
                kvcache_block_size=256, decode_backend="megakernel")
    base.update(kw)
    return SimpleNamespace(**base)


class Seq:
    def __init__(self, temperature=0.0, n=5, block_table=(0,)):
        self.temperature, self._n, self.block_table, self.last_token = temperature, n, list(block_table), 11

    def __len__(self):
        return self._n


def test_selector():
    assert P.is_megakernel_backend("megakernel")
    assert not P.is_megakernel_backend("torch")
    assert not P.is_megakernel_backend(None)


def test_admission_reasons_in_order():
    c = cfg()
    f = MegakernelBackend.compatibility
    assert f(c, [Seq()], True) == P.Compatibility(False, "Task-graph megakernel is decode-only; use the prefill backend")
    assert f(c, [], False).reason == "Task-graph megakernel needs at least one sequence"
    assert "batch sizes 1..8" in f(c, [Seq()] * 9, False).reason
    assert f(cfg(max_num_seqs=2), [Seq()] * 3, False).reason == "batch 3 exceeds max_num_seqs=2"
    # tensor parallelism: the reference admits size 1 only (taskgraph.py:119-122); this build admits 2, 4 and 8
    # once a group of that size is attached, and says what is missing otherwise
    assert f(cfg(tensor_parallel_size=3), [Seq()], False).reason == \
        "Task-graph megakernel requires tensor_parallel_size in (1, 2, 4, 8)"
    assert "needs a tensor-parallel group" in f(cfg(tensor_parallel_size=2), [Seq()], False).reason
    group = SimpleNamespace(size=4, rank=0)
    assert "has 4 ranks but tensor_parallel_size=2" in \
        f(cfg(tensor_parallel_size=2, megakernel_tensor_parallel=group), [Seq()], False).reason
    assert f(cfg(tensor_parallel_size=4, megakernel_tensor_parallel=group), [Seq()], False).supported
    assert f(c, [Seq(), Seq(temperature=0.7)], False).reason == "Task-graph megakernel supports greedy sampling only"
    assert f(c, [Seq(temperature=None)], False).supported is False
    ok = f(c, [Seq() for _ in range(8)], False)
    assert ok.supported and ok.reason == ""


def test_sampling_is_admitted_only_on_request():
    """Default: the reference's answer for every sampled row (taskgraph.py:123-130).  With
    ``megakernel_sampling`` a sampled single row is taken (its temperature comes from the sequence); batches
    need the value "batch", because the stock ModelRunner.run passes no temperatures to decode_batch."""
    f = MegakernelBackend.compatibility
    only = "Task-graph megakernel supports greedy sampling only"
    assert f(cfg(), [Seq(temperature=0.7)], False).reason == only
    on = cfg(megakernel_sampling=True)
    assert f(on, [Seq(temperature=0.7)], False).supported
    assert f(on, [Seq(temperature=None)], False).reason == only
    assert f(on, [Seq(), Seq()], False).supported                      # greedy batches as before
    assert "passes temperatures to decode_batch" in f(on, [Seq(), Seq(temperature=0.7)], False).reason
    assert f(cfg(megakernel_sampling="batch"), [Seq(), Seq(temperature=0.7)], False).supported


def test_is_greedy_flag_short_circuits_temperature():
    s = Seq(temperature=0.9)
    s.is_greedy = True
    assert MegakernelBackend.compatibility(cfg(), [s], False).supported


@pytest.mark.parametrize("field,value", [
    ("hidden_size", 2048), ("intermediate_size", 4096), ("num_hidden_layers", 12), ("num_attention_heads", 32),
    ("num_key_value_heads", 4), ("vocab_size", 32000), ("model_type", "llama"), ("head_dim", 64)])
def test_contract_mismatch_names_the_field(field, value):
    c = cfg(hf_config=hf(**{field: value}))
    assert qwen3_contract_mismatch(c) == field
    assert MegakernelBackend.compatibility(c, [Seq()], False).reason == f"unsupported Qwen config: {field}"


def test_contract_flags_and_max_len():
    assert qwen3_contract_mismatch(cfg(hf_config=hf(tie_word_embeddings=False))) == "tie_word_embeddings"
    assert qwen3_contract_mismatch(cfg(hf_config=hf(attention_bias=True))) == "attention_bias"
    assert qwen3_contract_mismatch(cfg(max_model_len=4096)) == "max_model_len"
    assert qwen3_contract_mismatch(cfg(max_model_len=1024)) == "max_model_len"   # compared for equality
    # without an explicit head_dim it is derived as hidden // heads = 64, which violates the contract
    h = hf()
    del h.head_dim
    assert qwen3_contract_mismatch(cfg(hf_config=h)) == "head_dim"


def test_set_kv_cache_validation():
    b = MegakernelBackend(cfg(), model=None)
    assert not b.ready and b.decoder is None and b.kv_cache is None and b.disabled_reason is None
    with pytest.raises(ValueError):
        b.set_kv_cache(None)
    with pytest.raises(ValueError):
        b.set_kv_cache(torch.zeros(2, 3, 4))
    with pytest.raises(ValueError):
        b.set_kv_cache(torch.zeros(3, 1, 1, 1, 1, 1))
    kv = torch.zeros(2, 1, 1, 4, 2, 8)
    b.set_kv_cache(kv)
    assert b.kv_cache is kv


def test_ensure_ready_errors():
    b = MegakernelBackend(cfg(), model=None)
    with pytest.raises(RuntimeError, match="KV cache has not been attached"):
        b.ensure_ready()
    b.disable("switched off")
    with pytest.raises(RuntimeError, match="switched off"):
        b.ensure_ready()
    if not torch.cuda.is_available():
        b2 = MegakernelBackend(cfg(), model=None)
        b2.set_kv_cache(torch.zeros(2, 28, 1, 256, 8, 128, dtype=torch.bfloat16))
        with pytest.raises(RuntimeError, match="requires a CUDA device"):
            b2.ensure_ready()


def test_cache_layout_validation():
    b = MegakernelBackend(cfg(), model=None)
    b.set_kv_cache(torch.zeros(2, 27, 1, 256, 8, 128, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="does not match the megakernel contract"):
        b._validate_cache_layout()
    b.set_kv_cache(torch.zeros(2, 28, 2, 256, 8, 128, dtype=torch.bfloat16))
    b._validate_cache_layout()
    b.set_kv_cache(torch.zeros(28, 2, 2, 256, 8, 128, dtype=torch.bfloat16).transpose(0, 1))
    with pytest.raises(RuntimeError, match="must be contiguous"):
        b._validate_cache_layout()


def test_arch_mapping():
    assert P.cuda_arch_for_capability((10, 0)) == "sm_100"
    with pytest.raises(ValueError):
        P.cuda_arch_for_capability((8, 0))


class FakeDecoder:
    def __init__(self, fail=False):
        self.calls, self.fail = [], fail

    def step(self, token, position=None, block_table=None, **sampling):
        if self.fail:
            raise RuntimeError("boom")
        self.calls.append(("step", token, position, list(block_table), *sampling.values()))
        return 42

    def decode_rows(self, ids, positions, tables):
        self.calls.append(("rows", ids, positions, tables))
        return [1, 2]


def test_decode_passes_pre_decode_length_as_position():
    b = MegakernelBackend(cfg(), model=None)
    b.kv_cache = object()
    b.decoder = FakeDecoder()
    s = Seq(n=300, block_table=(4, 9))
    assert b.decode(s, s.block_table) == [42]
    assert b.decoder.calls == [("step", 11, 299, [4, 9])]
    assert b.decode_batch("i", "p", "t") == [1, 2]
    # a sampled row reaches the decoder with its temperature only when sampling was asked for
    hot = Seq(temperature=0.8, n=300, block_table=(4, 9))
    assert b.decode(hot, hot.block_table) == [42] and b.decoder.calls[-1] == ("step", 11, 299, [4, 9])
    b2 = MegakernelBackend(cfg(megakernel_sampling=True), model=None)
    b2.kv_cache = object()
    b2.decoder = FakeDecoder()
    assert b2.decode(hot, hot.block_table) == [42] and b2.decoder.calls[-1] == ("step", 11, 299, [4, 9], 0.8)
    assert b2.decode(s, s.block_table) == [42] and b2.decoder.calls[-1] == ("step", 11, 299, [4, 9])


def test_dispatch_fallback_contract():
    c = cfg()
    b = MegakernelBackend(c, model=None)
    b.kv_cache = object()
    b.decoder = FakeDecoder()
    d = P.DecodeDispatch(c, b, prepare_decode=lambda seqs: ("i", "p", "t"))
    torch_path = lambda seqs, is_prefill: ["torch"] * len(seqs)
    # supported -> megakernel
    assert d.run([Seq()], False, torch_path) == [42]
    assert d.last_backend_used == "megakernel" and d.last_fallback_reason is None
    assert d.run([Seq(), Seq()], False, torch_path) == [1, 2]
    # prefill -> torch, no fallback reason recorded for prefill
    assert d.run([Seq()], True, torch_path) == ["torch"]
    assert d.last_backend_used == "torch" and d.last_fallback_reason is None
    # unsupported decode -> torch with the explicit reason
    assert d.run([Seq(temperature=1.0)], False, torch_path) == ["torch"]
    assert d.last_fallback_reason == "Task-graph megakernel supports greedy sampling only"
    # failure after the decoder exists -> poisoned, never a silent fallback
    b.decoder = FakeDecoder(fail=True)
    with pytest.raises(RuntimeError, match='restart with decode_backend="torch"'):
        d.run([Seq()], False, torch_path)
    assert d._cuda_poisoned


def test_dispatch_disables_backend_when_startup_fails():
    c = cfg()
    b = MegakernelBackend(c, model=None)      # no KV cache attached: decode raises before a decoder exists
    d = P.DecodeDispatch(c, b)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        assert d.run([Seq()], False, lambda s, p: ["torch"]) == ["torch"]
    assert any(issubclass(w.category, RuntimeWarning) for w in caught)
    assert b.disabled_reason and "KV cache has not been attached" in d.last_fallback_reason
    # once disabled the backend is skipped without a reason being recorded
    assert d.run([Seq()], False, lambda s, p: ["torch"]) == ["torch"]
    assert d.last_fallback_reason is None
