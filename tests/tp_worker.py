"""One rank of the tensor-parallel parity test (spawned by test_gpu_tensor_parallel.py).

Every rank builds the same seeded model, lets the CPU oracle prefill the same
prompts, keeps its own shard of the weights and of the KV cache on its GPU and
runs the decode steps through the C library; its slice of the logits and the
merged greedy tokens are compared with the oracle's unsharded step.
"""

from __future__ import annotations

import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def tp_parity_worker(rank: int, world: int, port: int, out_dir: str, layers: int, vocab: int, prompt_lens, steps: int,
                     use_graph: bool, transport: str):
    import numpy as np
    import torch
    import torch.distributed as dist

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from tests import harness as H
    from tests.harness import O
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.tensor_parallel import TensorParallelGroup, shard_weights

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    group = TensorParallelGroup.create(dist, rank, transport="nccl" if transport == "nccl" else "direct")
    seed = 5
    g = H.oracle_geometry(layers=layers, vocab=vocab)
    w = O.make_weights(g, seed=seed, norm="random").to(torch.bfloat16)
    cos_sin = O.rope_cos_sin_table(g)
    rng = np.random.Generator(np.random.Philox(key=seed + 100))
    prompts = [rng.integers(0, g.vocab, n).tolist() for n in prompt_lens]
    tables, nblocks = O.allocate_blocks([n + steps for n in prompt_lens], g.block_size)
    kv = O.new_kv_cache(g, nblocks, torch.bfloat16)
    cur = [int(O.greedy(O.prefill(w, kv, cos_sin, p, t))) for p, t in zip(prompts, tables)]

    local = shard_weights(H.to_decoder_weights(w), rank, world)
    lg = local.geom
    h0, h1 = rank * lg.kv_heads, (rank + 1) * lg.kv_heads
    kv_gpu = kv[:, :, :, :, h0:h1, :].contiguous().cuda()
    dec = StreamDecoder(local, kv_gpu[0], kv_gpu[1], block_size=g.block_size, num_cache_blocks=nblocks,
                        max_model_len=g.max_pos, use_graph=use_graph, tensor_parallel=group)
    if transport == "direct_unfused":   # the exchange as a kernel of its own instead of inside the projections
        from dfb_b200 import native
        dec.set_option(native.DFB_OPT_TP_FUSED, 0)
    dist.barrier()   # the ranks start their first step together (the exchange waits are bounded)
    rows = len(prompts)
    lens = [n + 1 for n in prompt_lens]
    logits_gpu = torch.zeros(rows, lg.vocab, dtype=torch.float32, device="cuda")
    worst, flips, bad_flips = 0.0, 0, 0
    for _ in range(steps):
        positions = [n - 1 for n in lens]
        want_logits, want_tok = O.decode_step(w, kv, cos_sin, cur, positions, tables)
        ids = torch.tensor(cur, dtype=torch.int64, device="cuda")
        pos = torch.tensor(positions, dtype=torch.int64, device="cuda")
        bt = H.padded_tables(tables, lens, g.block_size)
        dec.enqueue_rows(ids, pos, bt, out_logits=logits_gpu if not use_graph else None)
        torch.cuda.synchronize()
        got_tok = dec.tokens_device()[:rows].tolist()
        if not use_graph:
            mine = want_logits.float()[:, local.vocab_offset:local.vocab_offset + lg.vocab]
            worst = max(worst, float((logits_gpu.cpu() - mine).abs().max()))
        for r in range(rows):
            if got_tok[r] != int(want_tok[r]):
                flips += 1
                if not H.token_gap_ok(want_logits[r].float(), got_tok[r], int(want_tok[r]), 2 * H.TOKEN_GAP_ATOL):
                    bad_flips += 1
        cur = [int(t) for t in want_tok]
        lens = [n + 1 for n in lens]
    code, st = dec.status()
    kv_diff = float((kv_gpu.cpu().float() - kv[:, :, :, :, h0:h1, :].float()).abs().max())
    # every rank must have picked the same tokens
    toks = [None] * world
    dist.all_gather_object(toks, got_tok)
    report = dict(rank=rank, max_abs_logit_diff=worst, token_flips=flips, bad_flips=bad_flips,
                  device_status=int(st.device_status), kernels_per_step=int(st.kernels_per_step),
                  max_abs_kv_diff=kv_diff, ranks_agree=all(t == toks[0] for t in toks))
    Path(out_dir, f"rank{rank}.json").write_text(json.dumps(report))
    dec.close()
    torch.cuda.synchronize()
    dist.barrier()
    group.close()
    dist.destroy_process_group()


def tp_burst_worker(rank: int, world: int, port: int, out_dir: str, layers: int, vocab: int, steps: int):
    """Bursts and the fused sampler on a sharded decoder: every rank must publish the same tokens (the sampling
    noise is a function of the global vocabulary index, the shards' winners are merged by key), and a burst must
    equal the same steps issued one by one."""
    import numpy as np
    import torch
    import torch.distributed as dist

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from tests import harness as H
    from tests.harness import O
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.tensor_parallel import TensorParallelGroup, shard_weights

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    group = TensorParallelGroup.create(dist, rank, transport="direct")
    g = H.oracle_geometry(layers=layers, vocab=vocab)
    w = O.make_weights(g, seed=8, norm="random").to(torch.bfloat16)
    lens = [5, 70, 250]
    rows = len(lens)
    tables, nblocks = O.allocate_blocks([n + 2 * steps + 2 for n in lens], g.block_size)
    history = torch.from_numpy(np.random.Generator(np.random.Philox(key=81)).standard_normal(
        tuple(O.new_kv_cache(g, nblocks, torch.bfloat16).shape), dtype=np.float32) * 0.5).to(torch.bfloat16)
    local = shard_weights(H.to_decoder_weights(w), rank, world)
    lg = local.geom
    h0, h1 = rank * lg.kv_heads, (rank + 1) * lg.kv_heads
    temps = [0.0, 0.8, 1.3]
    first = [11, 22, 33]
    results = {}
    for mode in ("steps", "burst"):
        kv_gpu = history[:, :, :, :, h0:h1, :].contiguous().cuda()
        dec = StreamDecoder(local, kv_gpu[0], kv_gpu[1], block_size=g.block_size, num_cache_blocks=nblocks,
                            max_model_len=g.max_pos, tensor_parallel=group)
        dec.set_seed(4242)
        dist.barrier()
        if mode == "steps":
            out, ids = [], first
            for s in range(steps):
                ids = dec.decode_host(ids, [n + s for n in lens], tables, temperatures=temps)
                out.append(list(ids))
        else:
            out = dec.decode_burst(first, lens, tables, steps, temperatures=temps)
        code, st = dec.status()
        results[mode] = dict(tokens=out, status=int(st.device_status), kv=kv_gpu.cpu())
        dec.close()
        torch.cuda.synchronize()
        dist.barrier()
    toks = [None] * world
    dist.all_gather_object(toks, results["burst"]["tokens"])
    report = dict(rank=rank, ranks_agree=all(t == toks[0] for t in toks),
                  burst_equals_steps=results["burst"]["tokens"] == results["steps"]["tokens"],
                  kv_equal=bool(torch.equal(results["burst"]["kv"], results["steps"]["kv"])),
                  status=[results["steps"]["status"], results["burst"]["status"]],
                  sampled_rows_moved=any(a[1:] != b[1:] for a, b in zip(results["burst"]["tokens"][:-1],
                                                                        results["burst"]["tokens"][1:])),
                  tokens=results["burst"]["tokens"])
    Path(out_dir, f"rank{rank}.json").write_text(json.dumps(report))
    group.close()
    dist.destroy_process_group()
