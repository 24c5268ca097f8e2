"""The fixed-slot runtime: sequences admitted and retired between steps, more
live slots than one launch holds, a slot waiting for a block, against the same
sequences decoded alone."""

import numpy as np
import pytest
import torch

from oracle import qwen3_decode as O
from tests import harness as H

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _exact_options(dec):
    """One arithmetic for every batch size (see test_batch_equals_independent_rows)."""
    from dfb_b200 import native
    dec.set_option(native.DFB_OPT_ROW_GEMV, 0)
    dec.set_option(native.DFB_OPT_ATTN_CHUNK128, 0)


def _alone(w, history, first, length, table, steps):
    kv = torch.empty_like(history)
    kv.copy_(history)
    dec = H.make_decoder(w, kv)
    _exact_options(dec)
    out, tok = [], first
    for s in range(steps):
        tok = dec.decode_host([tok], [length + s], [table])[0]
        out.append(tok)
    dec.close()
    return out


def test_slots_join_leave_and_exceed_one_launch(cuda_device):
    from dfb_b200.slots import SlotRuntime

    g = H.oracle_geometry(layers=2, vocab=4096)
    w = O.make_weights(g, seed=71, norm="random").to(BF)
    n_seq = 12                                             # more than the 8 rows of one launch
    blocks = 2 * n_seq
    history = torch.from_numpy(np.random.Generator(np.random.Philox(key=72)).standard_normal(
        tuple(O.new_kv_cache(g, blocks, BF).shape), dtype=np.float32) * 0.5).to(BF).cuda()
    lens = [3, 70, 250, 129, 64, 1, 255, 17, 40, 200, 5, 90]
    firsts = [100 + i for i in range(n_seq)]
    tables = [[2 * i, 2 * i + 1] for i in range(n_seq)]
    budget = [9, 4, 12, 6, 9, 3, 10, 5, 7, 8, 2, 11]       # tokens each sequence generates before it retires
    want = [_alone(w, history, firsts[i], lens[i], tables[i], budget[i]) for i in range(n_seq)]

    kv = torch.empty_like(history)
    kv.copy_(history)
    dec = H.make_decoder(w, kv)
    _exact_options(dec)
    rt = SlotRuntime(dec)
    # sequences 0..9 start at once in scattered slots; 10 and 11 are admitted later into slots that were freed
    slot_of = {i: s for i, s in zip(range(10), [0, 3, 4, 7, 9, 12, 13, 20, 30, 31])}
    for i, s in slot_of.items():
        # sequence 6 (length 255) first gets only its first block: it emits one token, then waits for the second
        rt.admit(s, firsts[i], lens[i], tables[i][:1] if i == 6 else tables[i])
    got = {i: [] for i in range(n_seq)}
    waiting, steps_seen, waited_once = [10, 11], [0], [False]

    def on_tokens(tokens):
        steps_seen[0] += 1
        seq_of = {s: i for i, s in slot_of.items()}
        for s, tok in tokens.items():
            i = seq_of[s]
            got[i].append(tok)
            if len(got[i]) == budget[i]:
                rt.retire(s)
                del slot_of[i]
                if waiting:                                    # the freed slot goes to the next waiting sequence
                    j = waiting.pop(0)
                    slot_of[j] = s
                    rt.admit(s, firsts[j], lens[j], tables[j])
        if 6 in slot_of and slot_of[6] not in tokens and len(got[6]) < budget[6]:
            waited_once[0] = True                              # the slot sat a step out: hand it its second block
            rt.extend(slot_of[6], tables[6])
        return not slot_of                                     # stop when every sequence is done

    rt.run(200, on_tokens)
    assert not slot_of and not waiting
    assert waited_once[0], "the slot without room was stepped anyway"
    for i in range(n_seq):
        assert got[i] == want[i], (i, got[i], want[i])
    assert steps_seen[0] >= max(budget)
    # nothing live: a step emits nothing and launches nothing
    assert rt.step() == {}
    code, st = dec.status()
    assert code == 0 and st.device_status == 0
    dec.close()


def test_slot_argument_checks(cuda_device):
    from dfb_b200.slots import SlotRuntime

    g = H.oracle_geometry(layers=1, vocab=1024)
    w = O.make_weights(g, seed=73, norm="random").to(BF)
    dec = H.make_decoder(w, O.new_kv_cache(g, 4, BF).cuda())
    rt = SlotRuntime(dec)
    with pytest.raises(RuntimeError, match="bad argument"):
        rt.admit(32, 1, 0, [0])                    # slot out of range
    with pytest.raises(RuntimeError, match="bad argument"):
        rt.admit(0, 1, 0, [7])                     # block outside the cache
    with pytest.raises(RuntimeError, match="bad argument"):
        rt.admit(0, 5000, 0, [0])                  # token outside the embedding table
    rt.admit(1, 5, 0, [2], temperature=0.7)
    assert rt.state(1) == (True, 5, 0)
    out = rt.step()
    assert set(out) == {1} and rt.state(1) == (True, out[1], 1)
    rt.retire(1)
    assert rt.state(1)[0] is False and rt.step() == {}

    def boom(tokens):
        raise KeyError("from the callback")

    rt.admit(2, 5, 0, [1])
    with pytest.raises(KeyError):
        rt.run(5, boom)
    dec.close()
