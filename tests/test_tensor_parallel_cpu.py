"""Host side of tensor parallelism on CPU: the weight partition reproduces the
unsharded projections, and the cross-rank greedy merge picks the token of the
unsharded argmax (gloo, world size 2)."""

import socket

import pytest
import torch

from tests import harness as H
from tests.harness import O


def _small_weights():
    g = H.oracle_geometry(layers=1, vocab=2048)
    return g, O.make_weights(g, seed=11, norm="random").to(torch.bfloat16)


def _decoder_weights_cpu(w):
    return H.to_decoder_weights(w, device="cpu")


@pytest.mark.parametrize("size", [2, 4, 8])
def test_shards_reassemble_the_projections(size):
    from dfb_b200.tensor_parallel import shard_geometry, shard_weights

    g, w = _small_weights()
    full = _decoder_weights_cpu(w)
    lg = shard_geometry(full.geom, size)
    assert (lg.q_heads, lg.kv_heads, lg.intermediate, lg.vocab) == (16 // size, 8 // size, 3072 // size, 2048 // size)
    x = torch.randn(3, g.hidden, dtype=torch.float64)
    a = torch.randn(3, full.geom.q_size, dtype=torch.float64)
    m = torch.randn(3, g.intermediate, dtype=torch.float64)
    layer = full.layers[0]
    q_parts, k_parts, v_parts, o_sum, gate_parts, up_parts, d_sum = [], [], [], 0, [], [], 0
    for r in range(size):
        s = shard_weights(full, r, size)
        assert s.vocab_offset == r * lg.vocab and s.embed is full.embed
        l = s.layers[0]
        qkv = x @ l.wqkv.double().T
        q_parts.append(qkv[:, : lg.q_size]); k_parts.append(qkv[:, lg.q_size: lg.q_size + lg.kv_size])
        v_parts.append(qkv[:, lg.q_size + lg.kv_size:])
        o_sum = o_sum + a[:, r * lg.q_size:(r + 1) * lg.q_size] @ l.wo.double().T
        gu = x @ l.wgu.double().T
        gate_parts.append(gu[:, : lg.intermediate]); up_parts.append(gu[:, lg.intermediate:])
        d_sum = d_sum + m[:, r * lg.intermediate:(r + 1) * lg.intermediate] @ l.wd.double().T
    want_qkv = x @ layer.wqkv.double().T
    got_qkv = torch.cat(q_parts + k_parts + v_parts, dim=1)
    assert torch.equal(got_qkv, want_qkv)
    assert torch.allclose(o_sum, a @ layer.wo.double().T, atol=1e-9)
    assert torch.equal(torch.cat(gate_parts + up_parts, dim=1), x @ layer.wgu.double().T)
    assert torch.allclose(d_sum, m @ layer.wd.double().T, atol=1e-9)


def test_shard_geometry_rejects_bad_sizes():
    from dfb_b200.geometry import ModelGeometry
    from dfb_b200.tensor_parallel import shard_geometry

    with pytest.raises(ValueError, match="must be 1, 2, 4 or 8"):
        shard_geometry(ModelGeometry(), 3)
    with pytest.raises(ValueError, match="vocab=100 is not divisible"):
        shard_geometry(ModelGeometry(vocab=100), 8)


def test_merge_prefers_value_then_lowest_global_index():
    from dfb_b200.tensor_parallel import merge_shard_argmax

    # row 0: rank 1 wins by value; row 1: equal values, the lower global index (rank 0) wins;
    # row 2: equal values inside one rank are already resolved to the lower index by that rank
    values = [[1.0, 2.0, 0.5], [3.0, 2.0, 0.25]]
    indices = [[5, 7, 1], [0, 0, 9]]
    assert merge_shard_argmax(values, indices, shard_rows=10) == [10, 7, 1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _merge_worker(rank, world, port, out_dir):
    import json
    from pathlib import Path

    import torch.distributed as dist

    from dfb_b200.tensor_parallel import merge_shard_argmax, shard_weights

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    g, w = _small_weights()
    full = _decoder_weights_cpu(w)
    s = shard_weights(full, rank, world)
    torch.manual_seed(0)
    hidden = torch.randn(4, g.hidden).to(torch.bfloat16)
    # this rank's slice of the LM head, rounded like the kernel's logits
    head = s.embed[s.vocab_offset:s.vocab_offset + s.geom.vocab]
    logits = (hidden.float() @ head.float().T).to(torch.bfloat16).float()
    logits[2, :] = 1.0                                   # a row of exact ties: global index 0 must win
    val, idx = logits.max(dim=1)
    idx = torch.tensor([int((logits[b] == val[b]).nonzero()[0]) for b in range(4)])  # lowest index among equals
    pairs = [None] * world
    dist.all_gather_object(pairs, (val.tolist(), idx.tolist()))
    tokens = merge_shard_argmax([p[0] for p in pairs], [p[1] for p in pairs], s.geom.vocab)
    full_logits = (hidden.float() @ full.embed.float().T).to(torch.bfloat16).float()
    full_logits[2, :] = 1.0
    want = [int((full_logits[b] == full_logits[b].max()).nonzero()[0]) for b in range(4)]
    Path(out_dir, f"merge{rank}.json").write_text(json.dumps(dict(tokens=tokens, want=want)))
    dist.barrier()
    dist.destroy_process_group()


def test_greedy_merge_over_gloo_ranks(tmp_path):
    import json

    import torch.multiprocessing as mp

    mp.spawn(_merge_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        rep = json.loads((tmp_path / f"merge{r}.json").read_text())
        assert rep["tokens"] == rep["want"], rep
        assert rep["tokens"][2] == 0
