"""Bursts: several decode steps enqueued at once (tokens fed back on the device,
published in pinned host memory by the device) against the same steps issued
one by one from the host."""

import time

import numpy as np
import pytest
import torch

from oracle import qwen3_decode as O
from tests import harness as H

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _setup(rows, lens, layers=2, vocab=4096, blocks=16):
    g = H.oracle_geometry(layers=layers, vocab=vocab)
    w = O.make_weights(g, seed=51, norm="random").to(BF)
    history = torch.from_numpy(np.random.Generator(np.random.Philox(key=52)).standard_normal(
        tuple(O.new_kv_cache(g, blocks, BF).shape), dtype=np.float32) * 0.5).to(BF).cuda()
    # two blocks per row: every row may grow across the 256-token block boundary during the burst
    tables = [[2 * r + 1, 2 * r] for r in range(rows)]
    return g, w, history, tables


def _decoder(w, history, **kw):
    kv = torch.empty_like(history)
    kv.copy_(history)
    return H.make_decoder(w, kv, **kw), kv


@pytest.mark.parametrize("rows,lens,steps", [(1, [7], 12), (4, [250, 3, 64, 255], 10), (8, [5, 9, 13, 17, 21, 25, 29, 33], 6)])
def test_burst_equals_step_by_step(cuda_device, rows, lens, steps):
    g, w, history, tables = _setup(rows, lens)
    first = [100 + r for r in range(rows)]
    dec, kv_a = _decoder(w, history)
    want, ids = [], first
    for s in range(steps):
        ids = dec.decode_host(ids, [n + s for n in lens], tables)
        want.append(list(ids))
    dec.close()
    dec, kv_b = _decoder(w, history)
    got = dec.decode_burst(first, lens, tables, steps)
    assert got == want
    assert torch.equal(kv_a, kv_b)                      # the same K/V rows were written
    # a second burst on the same decoder continues where the first ended
    more = dec.decode_burst(got[-1], [n + steps for n in lens], tables, 2)
    dec.close()
    dec, _ = _decoder(w, history, use_graph=False)      # and the plain-launch path agrees
    assert dec.decode_burst(first, lens, tables, steps) == want
    assert dec.decode_burst(want[-1], [n + steps for n in lens], tables, 2) == more
    dec.close()


def test_burst_with_sampling_and_inactive_row(cuda_device):
    rows, lens, steps = 3, [10, 20, 30], 5
    g, w, history, tables = _setup(rows, lens)
    temps = [0.0, 0.8, 1.2]
    first = [1, 2, 3]
    dec, kv_a = _decoder(w, history)
    dec.set_seed(9)
    want, ids = [], first
    for s in range(steps):
        ids = dec.decode_host(ids, [n + s for n in lens], tables, active_rows=[1, 0, 1], temperatures=temps)
        want.append(list(ids))
    dec.close()
    dec, kv_b = _decoder(w, history)
    dec.set_seed(9)
    assert dec.decode_burst(first, lens, tables, steps, active_rows=[1, 0, 1], temperatures=temps) == want
    assert torch.equal(kv_a, kv_b)
    # the inactive row's cache slots were left alone
    assert torch.equal(kv_b[:, :, tables[1][0]], history[:, :, tables[1][0]])
    dec.close()


def test_burst_tokens_arrive_while_it_runs(cuda_device):
    """Non-blocking collection: finished steps are readable from the pinned ring before the burst ends."""
    rows, lens, steps = 2, [4, 8], 200
    g, w, history, tables = _setup(rows, lens, layers=8)
    dec, _ = _decoder(w, history)
    want = dec.decode_burst([5, 6], lens, tables, steps)
    dec.burst_enqueue([5, 6], lens, tables, steps)
    seen, polls = [], 0
    deadline = time.time() + 30.0
    while time.time() < deadline:
        part = dec.burst_collect(wait=False)
        polls += 1
        seen.append(len(part))
        assert part == want[:len(part)]
        if len(part) == steps:
            break
    assert seen[-1] == steps
    assert seen == sorted(seen)
    assert any(0 < n < steps for n in seen), seen[:10]   # some steps were read while others were still running
    dec.close()


def test_burst_argument_checks(cuda_device):
    from dfb_b200 import native

    rows, lens = 1, [500]
    g, w, history, tables = _setup(rows, lens)
    dec, _ = _decoder(w, history)
    with pytest.raises(RuntimeError, match="bad argument"):
        dec.decode_burst([1], lens, tables, 13)            # 500 + 13 - 1 = 512: beyond the two blocks given
    assert len(dec.decode_burst([1], lens, tables, 12)) == 12
    with pytest.raises(RuntimeError, match="fixed capacity"):
        dec.decode_burst([1], [0], tables, native.DFB_MAX_BURST + 1)
    dec.burst_enqueue([1], [0], tables, 3)
    with pytest.raises(RuntimeError, match="bad argument"):
        dec.decode_host([1], [0], tables)                  # a burst is in flight
    assert len(dec.burst_collect()) == 3
    assert dec.decode_host([1], [0], tables)
    dec.close()
