#!/usr/bin/env python
"""Benchmark of the Qwen3-0.6B greedy decode step (one "step" = one decode step
of the whole batch).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--batch B] [--prompt P] [--sweep]

Default workload (N=1): batch 1, a one-token prompt (context 1), bf16
random-init weights of the Qwen3-0.6B geometry, W + K greedy decode steps, so
the step is pure weight streaming (1,192,099,840 B per step).

Prints ONE JSON line.  ``value`` is whole-job decode tokens/s with every input
resident on the device (CUDA events around K back-to-back steps, tokens fed
back on the device); ``e2e`` is the same metric through the user-facing
``MegakernelBackend.decode`` / ``decode_batch`` call with host inputs, i.e. one
host-to-device copy, the step, one device-to-host copy and one synchronisation
per step; ``roofline`` is the LM-head + argmax kernel (the largest single kernel)
timed alone, ``step_floor`` relates the whole step to its byte floor; ``cpu_baseline`` is the CPU oracle (a port of the reference torch path)
timed on the host cores for a bounded number of steps.

``--impl reference`` times that CPU path alone with all host threads.
With ``--gpus N`` (launched by torchrun) every rank runs an independent replica
of the workload (the step has no cross-sequence exchange): weak scaling, value
= tokens of all ranks / max-over-ranks time.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode_tokens_per_s"
UNIT = "tok/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one LM-head launch, from the
# Nsight Compute capture summarised under profiles/ (batch 1, full vocabulary).
LMHEAD_DRAM_TRAFFIC_BYTES = 316_430_080


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _loop(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [x.strip() for x in out.strip().split(",")]
                if len(parts) >= 6:
                    self.rows.append(parts)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._loop, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        mhz = sorted(float(r[0]) for r in self.rows)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


class BenchSeq:
    """The few Sequence attributes the backend reads (engine/sequence.py:22-28)."""

    def __init__(self, token, length, block_table):
        self.last_token, self._n, self.block_table, self.temperature = token, length, block_table, 0.0

    def __len__(self):
        return self._n


def cpu_reference_run(batch, prompt_len, steps, budget_s, threads=None, warmup=1):
    """The CPU oracle (fp32, the reference's torch-path arithmetic) on the same
    workload shape: returns (tokens/s, steps done, seconds, threads)."""
    import torch
    from oracle import qwen3_decode as O

    if threads:
        torch.set_num_threads(threads)
    g = O.QWEN3_06B
    w = O.make_weights(g, seed=0, norm="ones")
    cos_sin = O.rope_cos_sin_table(g)
    tables, nblocks = O.allocate_blocks([prompt_len + steps + warmup + 1] * batch, g.block_size)
    kv = O.new_kv_cache(g, nblocks, torch.float32)
    import numpy as np
    rng = np.random.Generator(np.random.Philox(key=1234))
    cur = rng.integers(0, g.vocab, batch).tolist()
    lens = [prompt_len] * batch
    if prompt_len > 1:  # fill the history with random K/V instead of timing a prefill
        kv.normal_(0, 1)
    done = 0
    for _ in range(max(warmup, 1)):   # untimed warm-up steps (page-in, thread pool), same feedback as the timed ones
        _, nxt = O.decode_step(w, kv, cos_sin, cur, [n - 1 for n in lens], tables)
        cur = [int(t) for t in nxt]
        lens = [n + 1 for n in lens]
    t0 = time.perf_counter()
    while done < steps and time.perf_counter() - t0 < budget_s:
        _, nxt = O.decode_step(w, kv, cos_sin, cur, [n - 1 for n in lens], tables)
        cur = [int(t) for t in nxt]
        lens = [n + 1 for n in lens]
        done += 1
    dt = time.perf_counter() - t0
    return batch * done / dt, done, dt, torch.get_num_threads()


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget = 60.0
    tps, done, dt, threads = cpu_reference_run(args.batch, args.prompt, args.steps, budget, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": done,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(done, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, n_gpus=args.gpus),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{done} decode steps of the same workload on the host CPU (fp32 oracle port "
                                   f"of the reference torch path; the Python reference itself cannot travel)"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, n_gpus):
    return {"workload": f"Qwen3-0.6B geometry, bf16 random init (seed 0, N(0,0.02)), batch {args.batch}, "
                        f"prompt {args.prompt} token(s), greedy decode, KV block 256",
            "batch": args.batch, "prompt_tokens": args.prompt, "kv_block_size": 256,
            "parallelism": f"replicas x{n_gpus}" if n_gpus > 1 else "single GPU",
            "l2_policy": "inputs larger than L2 (1.19 GB of weights streamed per step)"}


def time_step_loop(dec, torch, batch, prompt, warmup, steps, block_size, tables):
    """Device-resident loop: tokens fed back on the device, positions and block
    tables prepared before the timed region.  Returns ms for `steps` steps."""
    total = warmup + steps
    pos_all = torch.arange(prompt - 1, prompt - 1 + total, dtype=torch.int64, device="cuda").repeat(batch, 1).t().contiguous()
    first_ids = torch.randint(0, 151936, (batch,), dtype=torch.int64, device="cuda")
    pages = -(-(prompt + total) // block_size)
    bt = torch.tensor([t[:pages] for t in tables], dtype=torch.int32, device="cuda")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for s in range(total):
        if s == warmup:
            torch.cuda.synchronize()
            barrier()
            start.record()
        ctx = prompt + s
        dec.enqueue_rows(first_ids if s == 0 else None, pos_all[s], bt[:, : -(-ctx // block_size)], max_context=ctx)
    stop.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(stop)


_DIST = None


def barrier():
    from dfb_b200 import replicas
    replicas.barrier(_DIST)


def max_over_ranks(torch, value):
    from dfb_b200 import replicas
    return replicas.aggregate(_DIST, 0, value, device="cuda")[1]


def run_tensor_parallel_arm(args):
    """``--tp``: ONE model sharded over the ranks (strong scaling), batch 8 at context
    1024 by default.  Every rank holds 1/N of the projections, of the KV heads
    and of the LM head; the partial results are summed with NCCL after o_proj and
    down_proj.  Reports device us/step as the max over ranks next to the per-rank
    byte floor."""
    global _DIST
    import torch
    import torch.distributed as dist
    import __graft_entry__  # noqa: F401
    from dfb_b200 import native
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.geometry import QWEN3_06B
    from dfb_b200.synthetic import random_init_weights
    from dfb_b200.tensor_parallel import TensorParallelGroup, shard_weights

    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1")))
    if world not in (2, 4, 8):
        raise SystemExit("--tp needs 2, 4 or 8 ranks (launch with torch.distributed.run)")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _DIST = dist
    native.lib()
    group = TensorParallelGroup.create(dist, local, transport="nccl" if args.tp_transport == "nccl" else "direct")
    g = QWEN3_06B
    B, P, W, K = args.batch, args.prompt, args.warmup, args.steps
    if P + W + K > g.max_model_len:
        raise SystemExit(f"prompt {P} + {W + K} steps exceeds max_model_len {g.max_model_len}")
    full = random_init_weights(g, seed=0, norm="ones", device="cuda")
    weights = shard_weights(full, rank, world)
    del full.layers[:]          # the unsharded projections are not needed any more
    lg = weights.geom
    pages = g.max_pages
    kv = torch.empty(2, g.layers, B * pages, g.block_size, lg.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    kv.normal_(0, 1)            # a random KV history stands in for the prefill of the prompt
    tables = [list(range(r * pages, (r + 1) * pages)) for r in range(B)]
    dec = StreamDecoder(weights, kv[0], kv[1], g.block_size, B * pages, g.max_model_len, tensor_parallel=group)
    if args.tp_transport == "direct_unfused":
        dec.set_option(native.DFB_OPT_TP_FUSED, 0)
    barrier()
    sampler = ClockSampler(local)
    with sampler:
        time_step_loop(dec, torch, B, P, 3, 5, g.block_size, tables)
        ms = max_over_ranks(torch, time_step_loop(dec, torch, B, P, W, K, g.block_size, tables))
    code, st = dec.status()
    peak, peak_kind = measured_peaks()
    contexts = [sum(P + W + s for s in range(K)) / K] * B
    # bytes ONE rank streams per step: its shard of the layers and of the LM head, its KV heads
    rank_bytes = (lg.layers * lg.layer_weight_bytes() + 2 * lg.hidden + lg.lm_head_bytes()
                  + lg.kv_bytes_per_token() * int(sum(contexts)))
    us = 1e3 * ms / K
    line = {
        "metric": METRIC, "value": B * K / (ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"Qwen3-0.6B geometry, bf16 random init (seed 0, N(0,0.02)), batch {B}, prompt {P} "
                               f"token(s), greedy decode, KV block 256, one model over {world} GPUs",
                   "batch": B, "prompt_tokens": P, "kv_block_size": 256, "parallelism": f"tp{world}",
                   "collectives": ("exchange over peer-mapped memory fused into the kernels: o_proj / down_proj push "
                                   "tagged words into the peers' windows, the next fused norm pulls them (bounded wait)"
                                   if args.tp_transport == "direct" else
                                   "own exchange kernel over peer-mapped memory (push tagged words, bounded wait) after "
                                   "o_proj and down_proj" if args.tp_transport == "direct_unfused" else
                                   "ncclAllReduce (bf16 sum) after o_proj and down_proj, ncclAllGather of the "
                                   "per-rank greedy winners") + "; all captured in the step's CUDA graph",
                   "l2_policy": "inputs larger than L2 per rank" if rank_bytes > 126e6 else "per-rank bytes fit in L2"},
        "device_us_per_step": us,
        "step_floor": {"bytes_per_step_per_rank": rank_bytes, "floor_us": rank_bytes / (peak * 1e3),
                       "frac_of_floor": rank_bytes / (peak * 1e3) / us, "peak_gbs": peak, "peak": peak_kind},
        "gpu_launches": (int(st.kernels_per_step) + 1) * K, "collectives_per_step": 2 * g.layers + 1,
        "clocks": sampler.summary(), "device_status": int(st.device_status),
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    dec.close()
    torch.cuda.synchronize()
    dist.barrier()
    group.close()
    dist.destroy_process_group()


def run_own_arm(args):
    global _DIST
    import torch
    import __graft_entry__  # noqa: F401
    from dfb_b200 import MegakernelBackend, native
    from dfb_b200.geometry import QWEN3_06B
    from dfb_b200.synthetic import nano_model_view, random_init_weights

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        _DIST = dist
    native.lib()  # no fallback: fail here if the CUDA library is missing

    g = QWEN3_06B
    B, P, W, K = args.batch, args.prompt, args.warmup, args.steps
    total = W + K
    if P + total > g.max_model_len:
        raise SystemExit(f"prompt {P} + {total} steps exceeds max_model_len {g.max_model_len}")
    weights = random_init_weights(g, seed=0, norm="ones", device="cuda")
    model, hf = nano_model_view(weights)
    pages = g.max_pages
    kv_rows = 8 if args.sweep else B      # the sweep goes up to batch 8
    kv = torch.zeros(2, g.layers, kv_rows * pages, g.block_size, g.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    if P > 1:
        kv.normal_(0, 1)  # a random KV history stands in for the prefill of the prompt
    tables = [list(range(r * pages, (r + 1) * pages)) for r in range(B)]
    config = SimpleNamespace(hf_config=hf, max_model_len=g.max_model_len, max_num_seqs=B, tensor_parallel_size=1,
                             kvcache_block_size=g.block_size, decode_backend="megakernel")
    backend = MegakernelBackend(config, model)
    backend.set_kv_cache(kv)
    backend.ensure_ready()
    dec = backend.decoder

    sampler = ClockSampler(local)
    with sampler:
        # (1) device-resident throughput
        time_step_loop(dec, torch, B, P, 3, 5, g.block_size, tables)   # graph capture + warm caches
        ms = time_step_loop(dec, torch, B, P, W, K, g.block_size, tables)
        ms = max_over_ranks(torch, ms)

        # (2) end to end through the backend's public call, host inputs, one sync per step
        def e2e_loop(n_warm, n_timed):
            cur = [int(t) for t in torch.randint(0, g.vocab, (B,)).tolist()]
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = 0.0
            for s in range(n_warm + n_timed):
                if s == n_warm:
                    torch.cuda.synchronize(); barrier(); start.record(); t0 = time.perf_counter()
                n_tok = P + s + 1            # the sampled token was appended before the step
                nblk = -(-n_tok // g.block_size)
                if B == 1:
                    cur = backend.decode(BenchSeq(cur[0], n_tok, tables[0][:nblk]), tables[0][:nblk])
                else:
                    ids = torch.tensor(cur, dtype=torch.int64).pin_memory().cuda(non_blocking=True)
                    pos = torch.tensor([n_tok - 1] * B, dtype=torch.int64).pin_memory().cuda(non_blocking=True)
                    bt = torch.tensor([t[:nblk] for t in tables], dtype=torch.int32).pin_memory().cuda(non_blocking=True)
                    cur = backend.decode_batch(ids, pos, bt)
            stop.record(); torch.cuda.synchronize(); wall = time.perf_counter() - t0; barrier()
            return start.elapsed_time(stop), wall
        e2e_ms, e2e_wall = e2e_loop(W, K)
        e2e_ms = max_over_ranks(torch, max(e2e_ms, 1e3 * e2e_wall))

        # (3) the dominant kernel alone: LM head + argmax, 311 MB of weights per launch
        lm_iters = 20
        hid = torch.randn(B, g.hidden, device="cuda").to(torch.bfloat16)
        res = torch.randn(B, g.hidden, device="cuda").to(torch.bfloat16)
        stream = torch.cuda.current_stream().cuda_stream
        lm = lambda: native.check(native.lib().dfb_launch_lmhead_argmax(
            dec._handle, hid.data_ptr(), res.data_ptr(), None, None, B, stream), "lmhead")
        for _ in range(3):
            lm()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); s0.record()
        for _ in range(lm_iters):
            lm()
        s1.record(); torch.cuda.synchronize()
        lm_ms = s0.elapsed_time(s1) / lm_iters
    clocks = sampler.summary()
    code, st = dec.status()
    kernels_per_step = int(st.kernels_per_step) + 1   # + the input staging kernel
    step_kernel = ("decode_step_persistent_kernel (whole step: 28 layers + LM head + argmax)"
                   if int(st.kernels_per_step) == 1 else
                   f"chain of {int(st.kernels_per_step)} kernels in one CUDA graph with programmatic dependent launch")
    lm_kernel = ("row_gemv_kernel<1024,NB,NormArgmax> (LM head + greedy argmax, FP32 pipe)" if B <= 2 else
                 "pair_gemv_kernel<3,NormArgmax> (LM head + greedy argmax, mma.sync with 16 weight rows per MMA)")

    peak, peak_kind = measured_peaks()
    lm_bytes = g.lm_head_bytes() + 2 * g.hidden
    contexts = [sum(P + W + s for s in range(K)) / K] * B           # mean attended tokens per row
    step_bytes = g.step_bytes(contexts)
    us_per_step = 1e3 * ms / K
    tok_s = world * B * K / (ms / 1e3)
    line = {
        "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, world),
        "device_us_per_step": us_per_step,
        "step_floor": {"bytes_per_step": step_bytes, "floor_us": step_bytes / (peak * 1e3),
                       "frac_of_floor": step_bytes / (peak * 1e3) / us_per_step, "peak_gbs": peak, "peak": peak_kind},
        "e2e": {"value": world * B * K / (e2e_ms / 1e3), "unit": UNIT, "ms_per_step": e2e_ms / K,
                "h2d_bytes_per_step": 4 * (24 + 8 * g.max_pages) if B == 1 else 8 * B * 2 + 4 * B * g.max_pages,
                "d2h_bytes_per_step": 48, "api": "MegakernelBackend.decode" if B == 1 else "MegakernelBackend.decode_batch"},
        "gpu_launches": kernels_per_step * K,
        # the dominant kernel is the LM head + argmax kernel (26% of the step's bytes in one launch), timed alone
        "roofline": {"kernel": lm_kernel, "bound": "hbm", "achieved": lm_bytes / (lm_ms * 1e6), "peak": peak,
                     "unit": "GB/s", "frac": lm_bytes / (lm_ms * 1e6) / peak, "traffic": LMHEAD_DRAM_TRAFFIC_BYTES,
                     "bytes_per_launch": lm_bytes, "us_per_launch": 1e3 * lm_ms, "peak_source": peak_kind},
        "step_kernels": step_kernel,
        "clocks": clocks,
        "device_status": int(st.device_status),
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tps, done, dt, threads = cpu_reference_run(B, P, 400, budget_s=20.0)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"{done} decode steps of the same workload ({dt:.1f} s) by the fp32 CPU "
                                          "oracle, a port of the reference torch path"}
    if args.torch_arm and world == 1:
        try:
            line["torch_cudagraph"] = torch_cudagraph_arm(weights, g, B, P, W, K)
        except Exception as exc:   # the comparison arm must never break the bench line
            line["torch_cudagraph"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    if args.sweep and world == 1:
        line["sweep"] = sweep(dec, torch, g, peak, weights if args.torch_arm else None)
    if rank == 0:
        print(json.dumps(line), flush=True)
    dec.close()
    if world > 1:
        _DIST.destroy_process_group()


def torch_cudagraph_arm(weights, g, batch, prompt, warmup, steps, use_compile=True):
    """The reference's torch decode path restated on torch / cuBLAS ops, the way its
    CUDA-graph arm runs it (engine/model_runner.py:292-313,379-416: the graph covers
    the 28 layers, the LM head GEMM and the greedy sampler run outside it), on the
    same weights and workload.  A comparison arm only: it uses library kernels
    (cuBLAS, FlashAttention if it runs on this GPU, else SDPA) and is not part of
    the backend.  Returns a dict with the device us/step."""
    import torch
    import torch.nn.functional as F

    B, dev, bs = batch, "cuda", g.block_size
    eps, scale = g.eps, g.head_dim ** -0.5
    pages = g.max_pages
    kv = torch.zeros(2, g.layers, B * pages, bs, g.kv_heads, g.head_dim, dtype=torch.bfloat16, device=dev)
    if prompt > 1:
        kv.normal_(0, 1)
    cos_sin = weights.cos_sin

    def rms(x, w):
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return xf.to(x.dtype) * w

    def add_rms(x, res, w):
        xf = x.float() + res.float()
        res = xf.to(x.dtype)
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return xf.to(x.dtype) * w, res

    def rope(positions, q, k):
        cs = cos_sin[positions].unsqueeze(1)
        cos, sin = cs.chunk(2, dim=-1)

        def rot(x):
            x1, x2 = torch.chunk(x.float(), 2, dim=-1)
            return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)
        return rot(q), rot(k)

    def silu_mul(x):
        a, b = x.chunk(2, -1)
        return F.silu(a) * b

    compiled = False
    if use_compile:
        try:
            rms, add_rms, rope, silu_mul = (torch.compile(f) for f in (rms, add_rms, rope, silu_mul))
            compiled = True
        except Exception:
            compiled = False
    attention = "flash_attn_with_kvcache"
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception:
        flash_attn_with_kvcache, attention = None, "sdpa"

    st = dict(ids=torch.zeros(B, dtype=torch.int64, device=dev), pos=torch.zeros(B, dtype=torch.int64, device=dev),
              slots=torch.zeros(B, dtype=torch.int64, device=dev), lens=torch.zeros(B, dtype=torch.int32, device=dev),
              bt=torch.tensor([list(range(r * pages, (r + 1) * pages)) for r in range(B)], dtype=torch.int32, device=dev))

    def attn(q, k, v, layer):
        kc, vc = kv[0, layer], kv[1, layer]
        D = g.kv_heads * g.head_dim
        kc.view(-1, D).index_copy_(0, st["slots"], k.reshape(B, D))
        vc.view(-1, D).index_copy_(0, st["slots"], v.reshape(B, D))
        if attention == "flash_attn_with_kvcache":
            return flash_attn_with_kvcache(q.unsqueeze(1), kc, vc, cache_seqlens=st["lens"], block_table=st["bt"],
                                           softmax_scale=scale, causal=True).reshape(B, -1)
        kk = kc[st["bt"].long()].reshape(B, pages * bs, g.kv_heads, g.head_dim).transpose(1, 2)
        vv = vc[st["bt"].long()].reshape(B, pages * bs, g.kv_heads, g.head_dim).transpose(1, 2)
        mask = (torch.arange(pages * bs, device=dev)[None, :] < st["lens"][:, None])[:, None, None, :]
        o = F.scaled_dot_product_attention(q.unsqueeze(2), kk, vv, attn_mask=mask, scale=scale, enable_gqa=True)
        return o.reshape(B, -1)

    def model():
        h = F.embedding(st["ids"], weights.embed)
        res = None
        for li, lw in enumerate(weights.layers):
            if res is None:
                x, res = rms(h, lw.ln_in), h
            else:
                x, res = add_rms(h, res, lw.ln_in)
            qkv = F.linear(x, lw.wqkv)
            q, k, v = qkv.split([g.q_size, g.kv_size, g.kv_size], dim=-1)
            q = rms(q.reshape(B, g.q_heads, g.head_dim), lw.q_norm)
            k = rms(k.reshape(B, g.kv_heads, g.head_dim), lw.k_norm)
            q, k = rope(st["pos"], q, k)
            o = attn(q, k, v.reshape(B, g.kv_heads, g.head_dim), li)
            h = F.linear(o, lw.wo)
            x, res = add_rms(h, res, lw.ln_post)
            h = F.linear(silu_mul(F.linear(x, lw.wgu)), lw.wd)
        x, _ = add_rms(h, res, weights.final_norm)
        return x

    def set_step(ctx):           # staging copies of the step's inputs, as prepare_decode does
        st["pos"].fill_(ctx - 1)
        st["lens"].fill_(ctx)
        blk, off = (ctx - 1) // bs, (ctx - 1) % bs
        st["slots"].copy_(st["bt"][:, blk].long() * bs + off)

    with torch.inference_mode():
        set_step(prompt)
        try:
            for _ in range(3):
                model()
        except Exception as exc:
            if attention != "sdpa":
                attention, flash_attn_with_kvcache = "sdpa", None
                for _ in range(3):
                    model()
            else:
                return {"unavailable": f"torch arm failed: {type(exc).__name__}: {exc}"[:200]}
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            hidden = model()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for s in range(warmup + steps):
            if s == warmup:
                torch.cuda.synchronize()
                e0.record()
            set_step(prompt + s)
            graph.replay()
            logits = F.linear(hidden, weights.embed)
            st["ids"].copy_(logits.float().argmax(-1))
        e1.record()
        torch.cuda.synchronize()
    us = 1e3 * e0.elapsed_time(e1) / steps
    return {"device_us_per_step": us, "tok_s": B * 1e6 / us, "attention": attention, "compiled_elementwise": compiled,
            "what": "restatement of the reference torch decode path (CUDA graph over the layers; LM head GEMM, argmax and "
                    "input staging outside it) on torch / cuBLAS / FlashAttention library kernels, same weights and "
                    "workload; the reference package itself is not present on the GPU box"}


def sweep(dec, torch, g, peak, torch_arm_weights=None):
    """Extra device-time points: batch 1/2/4/8 at context 512..639 and batch 8 at
    mixed long contexts (not part of the headline line)."""
    out = []
    pages = g.max_pages
    for B, P in ((1, 1), (1, 512), (2, 512), (4, 512), (8, 512), (8, 1920)):
        if B * pages > dec._k_cache.shape[1]:
            continue
        tables = [list(range(r * pages, (r + 1) * pages)) for r in range(B)]
        time_step_loop(dec, torch, B, P, 2, 4, g.block_size, tables)
        ms = time_step_loop(dec, torch, B, P, 8, 120, g.block_size, tables)
        ctx = [P + 8 + 59.5] * B
        by = g.step_bytes(ctx)
        us = 1e3 * ms / 120
        entry = {"batch": B, "prompt": P, "device_us_per_step": us, "tok_s": B * 120 / (ms / 1e3),
                 "floor_us": by / (peak * 1e3), "frac_of_floor": by / (peak * 1e3) / us}
        if torch_arm_weights is not None:
            try:
                t = torch_cudagraph_arm(torch_arm_weights, g, B, P, 8, 120)
                entry["torch_cudagraph_us_per_step"] = t.get("device_us_per_step")
                entry["torch_attention"] = t.get("attention", t.get("unavailable"))
            except Exception as exc:
                entry["torch_cudagraph_us_per_step"] = None
                entry["torch_attention"] = f"{type(exc).__name__}: {exc}"[:120]
        out.append(entry)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=120)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=1)
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--torch-arm", action="store_true",
                    help="also time a torch / cuBLAS / CUDA-graph restatement of the reference decode path")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tp-transport", default="direct", choices=["direct", "direct_unfused", "nccl"])
    ap.add_argument("--tp", action="store_true",
                    help="tensor parallelism over the launched ranks (one model, strong scaling) instead of replicas")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.tp:
        run_tensor_parallel_arm(args)
    else:
        run_own_arm(args)


if __name__ == "__main__":
    main()
