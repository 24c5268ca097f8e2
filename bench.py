#!/usr/bin/env python
"""Benchmark of the Qwen3-0.6B greedy decode step (one "step" = one decode step
of the whole batch).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Default workload (N=1): batch 1, a one-token prompt (context 1), bf16
random-init weights of the Qwen3-0.6B geometry, W + K greedy decode steps, so
the step is pure weight streaming (1,192,099,840 B per step).

Prints ONE JSON line.  ``value`` is whole-job decode tokens/s with every input
resident on the device (CUDA events around K back-to-back steps, tokens fed
back on the device), the median of ``--repeats`` timed loops with their spread;
``e2e`` is the same metric through the user-facing ``MegakernelBackend.decode``
/ ``decode_batch`` call with host inputs (one host-to-device copy, the step,
one device-to-host copy and one synchronisation per step); ``step_floor``
relates the whole step to its byte floor; ``kernels`` lists the six kernels of
the step, each timed alone through its standalone C-ABI launcher over all 28
layers' weights (cold in L2, as inside a step) together with its share of the
live step's time taken from the library's own timeline; ``roofline`` is the
entry of that list with the largest share of the step's time; ``sweep`` holds
batch 1/2/4/8 at prompt 512 and the long-context point (batch 8, per-row
contexts uniform in [256, 2048), seeded block-table permutation) next to the
reference's torch-CUDA-graph arm; ``cpu_baseline`` is the CPU oracle (a port of
the reference torch path) timed on the host cores for a bounded number of
steps.

``--impl reference`` times that CPU path alone with all host threads.  With
``--gpus N`` (launched by torch.distributed.run) every rank runs an independent
replica of the workload (the step has no cross-sequence exchange: weak scaling,
value = tokens of all ranks / max-over-ranks time) and the line also carries a
``tensor_parallel`` block: ONE model sharded over the N ranks (batch 8, context
1024), device time as the max over ranks.

Profiling drivers (no JSON contract): ``--profile-step`` runs a few plain steps
or standalone LM-head launches for Nsight Compute; ``--cta-sweep`` prints the
per-op time of the persistent kernel against its CTA count.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
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
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of each kernel at batch 1, from the Nsight
# Compute captures summarised under profiles/ (None: not captured).
DRAM_TRAFFIC_BYTES = {
    "rmsnorm_qkv": 8_424_704,               # profiles/row_gemv_layer_kernels_rows1.md
    "o_proj": 4_217_856,
    "rmsnorm_gateup_swiglu": 12_620_288,
    "down_proj": 6_316_800,
    "lm_head_argmax": 316_430_080,          # profiles/lmhead_row_gemv_rows1_vocab151936.md
}


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


def spread(values):
    """min / max / coefficient of variation of repeated measurements (the
    reference reports mean, CoV, p50 and p95 of its runs: metrics.py:45-119)."""
    m = statistics.fmean(values)
    sd = statistics.pstdev(values) if len(values) > 1 else 0.0
    return {"min": min(values), "max": max(values), "mean": m, "cov": sd / m if m else 0.0, "n": len(values)}


# ----------------------------------------------------------------------------------------------------------
# CPU reference arm (the oracle port of the reference torch path)
# ----------------------------------------------------------------------------------------------------------
def cpu_reference_run(batch, prompt_len, steps, budget_s, threads=None, warmup=1):
    """The CPU oracle (fp32, the reference's torch-path arithmetic) on the same
    workload shape: returns (tokens/s, steps done, seconds, threads)."""
    import numpy as np
    import torch
    from oracle import qwen3_decode as O

    if threads:
        torch.set_num_threads(threads)
    g = O.QWEN3_06B
    w = O.make_weights(g, seed=0, norm="ones")
    cos_sin = O.rope_cos_sin_table(g)
    tables, nblocks = O.allocate_blocks([prompt_len + steps + warmup + 1] * batch, g.block_size)
    kv = O.new_kv_cache(g, nblocks, torch.float32)
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
    """``--impl reference``: rank 0 alone times the CPU path with every host core
    (torch.distributed.run exports OMP_NUM_THREADS=1, so the thread count is set
    explicitly); the other ranks exit without work."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    tps, done, dt, threads = cpu_reference_run(args.batch, args.prompt, args.steps, 60.0, threads=cores,
                                               warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": done,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(done, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, n_gpus=args.gpus),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{done} decode steps of the same workload on the host CPU, all {threads} host "
                                   "threads (fp32 oracle port of the reference torch path; one CPU job whatever "
                                   "the number of GPUs of the other arm)"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, n_gpus):
    return {"workload": f"Qwen3-0.6B geometry, bf16 random init (seed 0, N(0,0.02)), batch {args.batch}, "
                        f"prompt {args.prompt} token(s), greedy decode, KV block 256",
            "batch": args.batch, "prompt_tokens": args.prompt, "kv_block_size": 256,
            "parallelism": f"replicas x{n_gpus}" if n_gpus > 1 else "single GPU",
            "l2_policy": "inputs larger than L2 (1.19 GB of weights streamed per step)"}


# ----------------------------------------------------------------------------------------------------------
# timed loops
# ----------------------------------------------------------------------------------------------------------
_DIST = None


def barrier():
    from dfb_b200 import replicas
    replicas.barrier(_DIST)


def max_over_ranks(torch, value):
    from dfb_b200 import replicas
    return replicas.aggregate(_DIST, 0, value, device="cuda")[1]


def time_step_loop(dec, torch, prompts, warmup, steps, block_size, tables, sync=True):
    """Device-resident loop: tokens fed back on the device, positions and block
    tables prepared before the timed region.  ``prompts``: context length of every
    row before the first step.  Returns ms for ``steps`` steps."""
    batch, total = len(prompts), warmup + steps
    base = torch.tensor([p - 1 for p in prompts], dtype=torch.int64, device="cuda")
    pos_all = (base[None, :] + torch.arange(total, dtype=torch.int64, device="cuda")[:, None]).contiguous()
    first_ids = torch.randint(0, 151936, (batch,), dtype=torch.int64, device="cuda")
    top = max(prompts)
    pages = -(-(top + total) // block_size)
    bt = torch.tensor([t[:pages] for t in tables], dtype=torch.int32, device="cuda")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for s in range(total):
        if s == warmup:
            torch.cuda.synchronize()
            if sync:
                barrier()
            start.record()
        ctx = top + s
        dec.enqueue_rows(first_ids if s == 0 else None, pos_all[s], bt[:, : -(-ctx // block_size)], max_context=ctx)
    stop.record()
    torch.cuda.synchronize()
    if sync:
        barrier()
    return start.elapsed_time(stop)


def step_timeline(dec, torch, native, prompts, block_size, tables):
    """One traced step (the library's own globaltimer timeline): how much of the
    step's span each kernel kind accounts for, attributing to every kernel the time
    from its predecessor's end to its own end."""
    batch = len(prompts)
    top = max(prompts)
    pages = -(-(top + 4) // block_size)
    bt = torch.tensor([t[:pages] for t in tables], dtype=torch.int32, device="cuda")
    ids = torch.randint(0, 151936, (batch,), dtype=torch.int64, device="cuda")
    pos = torch.tensor([p - 1 for p in prompts], dtype=torch.int64, device="cuda")
    dec.set_option(native.DFB_OPT_TRACE, 1)
    names = ("rmsnorm_qkv", "attention", "o_proj", "rmsnorm_gateup_swiglu", "down_proj")
    shares = {n: 0.0 for n in names + ("lm_head_argmax",)}
    span = 0.0
    try:
        for _ in range(3):      # the last traced step counts (the first ones capture the graph and warm up)
            dec.read_trace()
            dec.enqueue_rows(ids, pos, bt, max_context=top)
            torch.cuda.synchronize()
        t = dec.read_trace()
        n = len(t)
        if n >= 6 and (n - 1) % 5 == 0:
            ends = [int(row[2]) for row in t]
            prev = int(t[0][0])
            for i in range(n):
                name = "lm_head_argmax" if i == n - 1 else names[i % 5]
                shares[name] += max(ends[i] - prev, 0) / 1e3
                prev = max(prev, ends[i])
            span = (max(ends) - int(t[0][0])) / 1e3
    finally:
        dec.set_option(native.DFB_OPT_TRACE, 0)
    return shares, span


def time_kernels_alone(dec, torch, native, weights, g, batch, context, peak):
    """Each kernel of the step alone through its standalone C-ABI launcher: one
    CUDA graph holds the launches of all 28 layers (so every launch finds its
    weights cold in L2, as inside a step), replayed and timed with CUDA events.
    These launches are serialised (no programmatic dependent launch), which is the
    view Nsight Compute has of them too."""
    lib = native.lib()
    B, L = batch, g.layers
    bf = torch.bfloat16
    h = torch.randn(B, g.hidden, device="cuda").to(bf)
    res = torch.randn(B, g.hidden, device="cuda").to(bf)
    res_out = torch.empty_like(res)
    qkv = torch.randn(B, g.qkv_rows, device="cuda").to(bf)
    attn = torch.randn(B, g.q_size, device="cuda").to(bf)
    act = torch.randn(B, g.intermediate, device="cuda").to(bf)
    hout = torch.empty(B, g.hidden, device="cuda", dtype=bf)
    pages = g.max_pages
    bt = torch.tensor([list(range(r * pages, (r + 1) * pages)) for r in range(B)], dtype=torch.int32, device="cuda")
    pos = torch.full((B,), context - 1, dtype=torch.int32, device="cuda")
    handle = dec._handle

    def launches(name, stream):
        for l, lw in enumerate(weights.layers):
            if name == "rmsnorm_qkv":
                rc = lib.dfb_launch_rmsnorm_qkv(h.data_ptr(), None, res.data_ptr(), res_out.data_ptr(), lw.ln_in.data_ptr(),
                                                lw.wqkv.data_ptr(), qkv.data_ptr(), B, g.hidden, g.qkv_rows, g.eps, stream)
            elif name == "attention":
                rc = lib.dfb_launch_attention(handle, l, qkv.data_ptr(), pos.data_ptr(), bt.data_ptr(), pages, None,
                                              attn.data_ptr(), B, context, stream)
            elif name == "o_proj":
                rc = lib.dfb_launch_linear(attn.data_ptr(), lw.wo.data_ptr(), hout.data_ptr(), B, g.hidden, g.q_size, stream)
            elif name == "rmsnorm_gateup_swiglu":
                rc = lib.dfb_launch_rmsnorm_gateup_swiglu(h.data_ptr(), res.data_ptr(), res_out.data_ptr(),
                                                          lw.ln_post.data_ptr(), lw.wgu.data_ptr(), act.data_ptr(), B,
                                                          g.hidden, g.intermediate, g.eps, stream)
            else:
                rc = lib.dfb_launch_linear(act.data_ptr(), lw.wd.data_ptr(), hout.data_ptr(), B, g.hidden,
                                           g.intermediate, stream)
            native.check(rc, name)

    kv_tok = 2 * g.kv_size * 2      # K and V bytes of one context token of one layer
    per_launch = {
        "rmsnorm_qkv": 2 * g.qkv_rows * g.hidden + 2 * g.hidden,
        "attention": kv_tok * context * B + 4 * g.head_dim,
        "o_proj": 2 * g.hidden * g.q_size,
        "rmsnorm_gateup_swiglu": 2 * 2 * g.intermediate * g.hidden + 2 * g.hidden,
        "down_proj": 2 * g.hidden * g.intermediate,
        "lm_head_argmax": g.lm_head_bytes() + 2 * g.hidden,
    }
    out = []
    reps = 10
    for name in ("rmsnorm_qkv", "attention", "o_proj", "rmsnorm_gateup_swiglu", "down_proj"):
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            launches(name, side.cuda_stream)       # warm-up outside the capture (function attributes, modules)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                launches(name, torch.cuda.current_stream().cuda_stream)
            for _ in range(2):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            side.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / (reps * L)
        out.append({"name": name, "launches_per_step": L, "bytes": per_launch[name], "us": us,
                    "achieved_gbs": per_launch[name] / (us * 1e3), "frac": per_launch[name] / (us * 1e3) / peak})
    # LM head + argmax: long enough to time with plain launches
    hid = torch.randn(B, g.hidden, device="cuda").to(bf)
    stream = torch.cuda.current_stream().cuda_stream
    lm = lambda: native.check(lib.dfb_launch_lmhead_argmax(handle, hid.data_ptr(), res.data_ptr(), None, None, B, stream),
                              "lmhead")
    for _ in range(3):
        lm()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(); s0.record()
    for _ in range(20):
        lm()
    s1.record(); torch.cuda.synchronize()
    us = 1e3 * s0.elapsed_time(s1) / 20
    out.append({"name": "lm_head_argmax", "launches_per_step": 1, "bytes": per_launch["lm_head_argmax"], "us": us,
                "achieved_gbs": per_launch["lm_head_argmax"] / (us * 1e3),
                "frac": per_launch["lm_head_argmax"] / (us * 1e3) / peak})
    return out


# ----------------------------------------------------------------------------------------------------------
# comparison arm: the reference's torch decode path with CUDA graphs
# ----------------------------------------------------------------------------------------------------------
def reference_cudagraph_points(points, steps):
    """The unmodified reference engine (baseline/_ref), torch-cudagraph arm, in a
    process of its own.  Returns {(batch, prompt): point} or {"unavailable": why}."""
    script = ROOT / "baseline" / "reference_engine.py"
    if not (ROOT / "baseline" / "_ref" / "nanovllm").exists():
        return {"unavailable": "baseline/_ref not installed (sh baseline/install_reference.sh)"}
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS"):
        env.pop(k, None)
    spec = ",".join(f"{b}:{p}" for b, p in points)
    try:
        proc = subprocess.run([sys.executable, str(script), "--points", spec, "--steps", str(steps)], env=env,
                              capture_output=True, text=True, timeout=900)
        last = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
        if not last:
            return {"unavailable": f"no output (rc {proc.returncode}): {proc.stderr[-300:]}"}
        data = json.loads(last[-1])
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    if "unavailable" in data:
        return {"unavailable": data["unavailable"]}
    return {(p["batch"], p["prompt"]): p for p in data["points"]}


def torch_cudagraph_standin(weights, g, batch, prompt, warmup, steps, use_compile=True):
    """Fallback comparison arm when baseline/_ref is absent: the reference's torch
    decode path restated on torch / cuBLAS / FlashAttention library kernels, the 28
    layers in one CUDA graph and the LM head GEMM + argmax outside it
    (engine/model_runner.py:292-313,379-416).  Labelled a stand-in wherever quoted."""
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

    if use_compile:
        try:
            rms, add_rms, rope, silu_mul = (torch.compile(f) for f in (rms, add_rms, rope, silu_mul))
        except Exception:
            pass
    from flash_attn import flash_attn_with_kvcache

    st = dict(ids=torch.zeros(B, dtype=torch.int64, device=dev), pos=torch.zeros(B, dtype=torch.int64, device=dev),
              slots=torch.zeros(B, dtype=torch.int64, device=dev), lens=torch.zeros(B, dtype=torch.int32, device=dev),
              bt=torch.tensor([list(range(r * pages, (r + 1) * pages)) for r in range(B)], dtype=torch.int32, device=dev))

    def attn(q, k, v, layer):
        kc, vc = kv[0, layer], kv[1, layer]
        D = g.kv_heads * g.head_dim
        kc.view(-1, D).index_copy_(0, st["slots"], k.reshape(B, D))
        vc.view(-1, D).index_copy_(0, st["slots"], v.reshape(B, D))
        return flash_attn_with_kvcache(q.unsqueeze(1), kc, vc, cache_seqlens=st["lens"], block_table=st["bt"],
                                       softmax_scale=scale, causal=True).reshape(B, -1)

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

    def set_step(ctx):
        st["pos"].fill_(ctx - 1)
        st["lens"].fill_(ctx)
        blk, off = (ctx - 1) // bs, (ctx - 1) % bs
        st["slots"].copy_(st["bt"][:, blk].long() * bs + off)

    with torch.inference_mode():
        set_step(prompt)
        for _ in range(3):
            model()
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
    return 1e3 * e0.elapsed_time(e1) / steps


def long_context_case(g, rows=8, seed=2024, steps=48):
    """BASELINE config 4: per-row contexts uniform in [256, 2048 - steps) and a
    seeded random permutation of the physical KV blocks."""
    import numpy as np

    rng = np.random.Generator(np.random.Philox(key=seed))
    ctx = [int(c) for c in rng.integers(256, 2048 - steps - 16, rows)]
    perm = rng.permutation(rows * g.max_pages).tolist()
    tables = [perm[r * g.max_pages:(r + 1) * g.max_pages] for r in range(rows)]
    return ctx, tables


def sweep(dec, torch, g, peak, repeats):
    """Device-time points beside the headline: BASELINE config 3 (batch 1/2/4/8,
    prompt 512) and config 4 (batch 8, mixed long contexts, scattered blocks)."""
    out = []
    pages = g.max_pages
    W, K = 4, 48
    cases = [(f"batch {B}, prompt 512", [512] * B, [list(range(r * pages, (r + 1) * pages)) for r in range(B)])
             for B in (1, 2, 4, 8)]
    ctx4, tables4 = long_context_case(g, steps=W + K)
    cases.append(("batch 8, contexts uniform in [256, 2048), permuted block tables", ctx4, tables4))
    for label, prompts, tables in cases:
        B = len(prompts)
        time_step_loop(dec, torch, prompts, 2, 3, g.block_size, tables, sync=False)
        runs = [1e3 * time_step_loop(dec, torch, prompts, W, K, g.block_size, tables, sync=False) / K
                for _ in range(max(repeats, 3))]
        us = statistics.median(runs)
        mean_ctx = [p + W + (K - 1) / 2 for p in prompts]
        by = g.step_bytes(mean_ctx)
        out.append({"case": label, "batch": B, "prompt": prompts if len(set(prompts)) > 1 else prompts[0],
                    "device_us_per_step": us, "spread_us": spread(runs), "tok_s": B * 1e6 / us,
                    "bytes_per_step": by, "floor_us": by / (peak * 1e3), "frac_of_floor": by / (peak * 1e3) / us})
    return out


# ----------------------------------------------------------------------------------------------------------
# tensor parallelism over the launched ranks
# ----------------------------------------------------------------------------------------------------------
def tensor_parallel_block(args, torch, dist, full_weights, local, transport="direct"):
    """BASELINE config 5: ONE model over all ranks (KV heads 8/N per rank, MLP split
    column/row, LM head by vocabulary), batch 8 at context 1024, device us/step as
    the max over ranks, next to one GPU running the same workload and to the
    per-rank byte floor.  Every rank must call this."""
    from dfb_b200 import native
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.geometry import QWEN3_06B as g
    from dfb_b200.tensor_parallel import TensorParallelGroup, shard_weights

    rank, world = dist.get_rank(), dist.get_world_size()
    B, P, W, K = 8, 1024, 4, max(16, min(args.steps, 64))
    peak, peak_kind = measured_peaks()
    pages = g.max_pages
    tables = [list(range(r * pages, (r + 1) * pages)) for r in range(B)]
    gen = torch.Generator(device="cuda").manual_seed(99)    # the same history on every rank
    kv_full = torch.empty(2, g.layers, B * pages, g.block_size, g.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    kv_full[0].normal_(0, 1.0, generator=gen)
    kv_full[1].normal_(0, 0.64, generator=gen)
    first_ids = torch.randint(0, g.vocab, (B,), dtype=torch.int64, device="cuda", generator=gen)

    def run(dec, record, forced=None):
        """W + K steps from the same first ids; returns (ms for K steps, tokens per step).  ``forced``: a
        [steps, B] token tensor fed in step by step instead of this decoder's own previous tokens (teacher
        forcing, so that two decoders can be compared beyond the first token that differs)."""
        total = W + K
        pos_all = torch.arange(P - 1, P - 1 + total, dtype=torch.int64, device="cuda").repeat(B, 1).t().contiguous()
        bt = torch.tensor([t[:-(-(P + total) // g.block_size)] for t in tables], dtype=torch.int32, device="cuda")
        toks = torch.zeros(total, B, dtype=torch.int32, device="cuda")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for s in range(total):
            if s == W:
                torch.cuda.synchronize(); barrier(); e0.record()
            ctx = P + s
            ids = first_ids if s == 0 else (forced[s - 1] if forced is not None else None)
            dec.enqueue_rows(ids, pos_all[s], bt[:, : -(-ctx // g.block_size)], max_context=ctx)
            if record:
                toks[s].copy_(dec.tokens_device()[:B])
        e1.record(); torch.cuda.synchronize(); barrier()
        return e0.elapsed_time(e1), toks.cpu()

    # one GPU, the same workload (every rank runs it, so that clocks and memory traffic are alike)
    single = StreamDecoder(full_weights, kv_full[0], kv_full[1], g.block_size, B * pages, g.max_model_len)
    run(single, False)
    ms_single, toks_single = run(single, True)
    ms_single_timed, _ = run(single, False)
    single.close()
    kv_local = kv_full[:, :, :, :, rank * (g.kv_heads // world):(rank + 1) * (g.kv_heads // world)].contiguous()
    del kv_full
    group = TensorParallelGroup.create(dist, local, transport="nccl" if transport == "nccl" else "direct")
    weights = shard_weights(full_weights, rank, world)
    lg = weights.geom
    dec = StreamDecoder(weights, kv_local[0], kv_local[1], g.block_size, B * pages, g.max_model_len, tensor_parallel=group)
    kv0 = kv_local.clone()
    run(dec, False)
    kv_local.copy_(kv0)
    ms_rec, toks_tp = run(dec, True, forced=toks_single.to("cuda").to(torch.int64))
    kv_local.copy_(kv0)
    ms_tp, _ = run(dec, False)
    ms_tp = max_over_ranks(torch, ms_tp)
    ms_one = max_over_ranks(torch, ms_single_timed)
    code, st = dec.status()
    same = int((toks_tp == toks_single).sum())      # (step, row) pairs, the sharded decoder fed the 1-GPU tokens
    mean_ctx = P + W + (K - 1) / 2
    rank_bytes = (lg.layers * lg.layer_weight_bytes() + 2 * lg.hidden + lg.lm_head_bytes()
                  + lg.kv_bytes_per_token() * int(B * mean_ctx))
    us = 1e3 * ms_tp / K
    block = {
        "workload": f"batch {B}, context {P}, {K} greedy steps, one model over {world} GPUs (KV heads "
                    f"{g.kv_heads // world} per rank, MLP split column/row, LM head by vocabulary)",
        "scaling": "strong", "ranks": world, "steps": K, "device_us_per_step": us, "tok_s": B * 1e6 / us,
        "one_gpu_same_workload_us_per_step": 1e3 * ms_one / K, "speedup_over_one_gpu": ms_one / ms_tp,
        "per_rank_bytes_per_step": rank_bytes, "per_rank_floor_us": rank_bytes / (peak * 1e3),
        "frac_of_floor": rank_bytes / (peak * 1e3) / us, "peak_gbs": peak, "peak": peak_kind,
        "exchanges_per_step": 2 * g.layers + 1,
        "exchange": "o_proj / down_proj push {2 x bf16, tag} words into the peers' windows (peer-mapped memory, "
                    "plain stores over NVLink), the next fused norm pulls them with a bounded wait; greedy winners "
                    "merged the same way" if transport == "direct" else "ncclAllReduce / ncclAllGather in the graph",
        "tokens_equal_to_one_gpu": same, "tokens_compared": int(toks_tp.numel()),
        "token_check": "every step of the sharded decoder is fed the one-GPU decoder's previous tokens (teacher forcing); "
                       "a pair differs where the bf16 rounding of the summed partial projections flips a near-tie of "
                       "this random-weight model",
        "device_status": int(st.device_status), "gpu_launches": (int(st.kernels_per_step) + 1) * K,
    }
    dec.close()
    torch.cuda.synchronize()
    dist.barrier()
    group.close()
    return block


# ----------------------------------------------------------------------------------------------------------
# this repository's arm
# ----------------------------------------------------------------------------------------------------------
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
    dist = None
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
    extras = world == 1 and not args.quick
    kv_rows = 8 if extras else B      # the sweep goes up to batch 8
    kv = torch.zeros(2, g.layers, kv_rows * pages, g.block_size, g.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    kv[0].normal_(0, 1.0)             # a random KV history stands in for the prefill of the prompts:
    kv[1].normal_(0, 0.64)            # K has unit RMS after its norm, V the scale of a N(0, 0.02) projection
    tables = [list(range(r * pages, (r + 1) * pages)) for r in range(B)]
    config = SimpleNamespace(hf_config=hf, max_model_len=g.max_model_len, max_num_seqs=kv_rows, tensor_parallel_size=1,
                             kvcache_block_size=g.block_size, decode_backend="megakernel")
    backend = MegakernelBackend(config, model)
    backend.set_kv_cache(kv)
    backend.ensure_ready()
    dec = backend.decoder
    for item in args.set_option:
        opt, val = item.split("=")
        dec.set_option(int(opt), int(val))
    peak, peak_kind = measured_peaks()

    sampler = ClockSampler(local)
    with sampler:
        # (1) device-resident throughput: `repeats` timed loops of exactly K steps each
        time_step_loop(dec, torch, [P] * B, 3, 5, g.block_size, tables)   # graph capture + warm caches
        runs_ms = [max_over_ranks(torch, time_step_loop(dec, torch, [P] * B, W, K, g.block_size, tables))
                   for _ in range(args.repeats)]
        ms = statistics.median(runs_ms)

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
            return max(start.elapsed_time(stop), 1e3 * wall)
        e2e_runs = [max_over_ranks(torch, e2e_loop(W, K)) for _ in range(max(3, args.repeats // 2))]
        e2e_ms = statistics.median(e2e_runs)

        # (2b) the same steps as ONE call: a burst of K steps from host inputs (one H2D, tokens fed back on the
        # device and published in pinned host memory by the device, one synchronisation per call)
        def burst_loop(n_warm, n_timed):
            cur = [int(t) for t in torch.randint(0, g.vocab, (B,)).tolist()]
            nblk = -(-(P + n_warm + n_timed + 1) // g.block_size)
            bt = [t[:nblk] for t in tables]
            if n_warm:
                cur = dec.decode_burst(cur, [P] * B, bt, n_warm)[-1]
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); barrier(); start.record(); t0 = time.perf_counter()
            dec.decode_burst(cur, [P + n_warm] * B, bt, n_timed)
            stop.record(); torch.cuda.synchronize(); wall = time.perf_counter() - t0; barrier()
            return max(start.elapsed_time(stop), 1e3 * wall)
        burst_ms = None
        if K <= native.DFB_MAX_BURST and P + W + K < g.max_model_len:
            burst_runs = [max_over_ranks(torch, burst_loop(W, K)) for _ in range(max(3, args.repeats // 2))]
            burst_ms = statistics.median(burst_runs)

        # (3) where the step's time goes: the library's own timeline of one live step, and every kernel alone
        shares, span_us = ({}, 0.0)
        kernels = []
        if rank == 0:
            shares, span_us = step_timeline(dec, torch, native, [P] * B, g.block_size, tables)
            kernels = time_kernels_alone(dec, torch, native, weights, g, B, max(P, 1), peak)
    clocks = sampler.summary()
    code, st = dec.status()
    kernels_per_step = int(st.kernels_per_step) + 1   # + the input staging kernel
    step_kernel = ("decode_step_persistent_kernel (whole step: 28 layers + LM head + argmax)"
                   if int(st.kernels_per_step) == 1 else
                   f"chain of {int(st.kernels_per_step)} kernels in one CUDA graph with programmatic dependent launch")
    total_share = sum(shares.values()) or 1.0
    for k in kernels:
        k["share_of_step"] = shares.get(k["name"], 0.0) / total_share
        k["live_us_per_step"] = shares.get(k["name"], 0.0)
        k["traffic"] = DRAM_TRAFFIC_BYTES.get(k["name"]) if B == 1 else None
    top = max(kernels, key=lambda k: k["share_of_step"]) if kernels else None

    contexts = [sum(P + W + s for s in range(K)) / K] * B           # mean attended tokens per row
    step_bytes = g.step_bytes(contexts)
    us_per_step = 1e3 * ms / K
    tok_s = world * B * K / (ms / 1e3)
    line = {
        "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, world),
        "repeats": args.repeats,
        "spread": {k: (world * B * K / (v / 1e3) if k in ("min", "max", "mean") else v)
                   for k, v in spread(runs_ms).items()},
        "device_us_per_step": us_per_step,
        "device_us_per_step_spread": spread([1e3 * r / K for r in runs_ms]),
        "step_floor": {"bytes_per_step": step_bytes, "floor_us": step_bytes / (peak * 1e3),
                       "frac_of_floor": step_bytes / (peak * 1e3) / us_per_step, "peak_gbs": peak, "peak": peak_kind},
        "e2e": {"value": world * B * K / (e2e_ms / 1e3), "unit": UNIT, "ms_per_step": e2e_ms / K,
                "h2d_bytes_per_step": 4 * (32 + 8 * g.max_pages) if B == 1 else 8 * B * 2 + 4 * B * g.max_pages,
                "d2h_bytes_per_step": 48, "api": "MegakernelBackend.decode" if B == 1 else "MegakernelBackend.decode_batch",
                "runs": len(e2e_runs)},
        "e2e_burst": None if burst_ms is None else {
            "value": world * B * K / (burst_ms / 1e3), "unit": UNIT, "ms_per_step": burst_ms / K, "steps_per_call": K,
            "h2d_bytes_per_call": 4 * (32 + 8 * g.max_pages), "api": "StreamDecoder.decode_burst "
            "(dfb_decode_burst_host: K steps per call, tokens fed back on the device, one synchronisation)"},
        "gpu_launches": kernels_per_step * K,
        "step_kernels": step_kernel,
        "clocks": clocks,
        "device_status": int(st.device_status),
    }
    if top is not None:
        # the kernel with the largest share of the step's TIME (not bytes), timed alone over all layers' weights
        line["roofline"] = {"kernel": top["name"], "bound": "hbm", "achieved": top["achieved_gbs"], "peak": peak,
                            "unit": "GB/s", "frac": top["frac"], "traffic": top["traffic"],
                            "bytes_per_launch": top["bytes"], "us_per_launch": top["us"],
                            "share_of_step": top["share_of_step"], "peak_source": peak_kind}
        line["kernels"] = kernels
        line["timeline_span_us"] = span_us
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tps, done, dt, threads = cpu_reference_run(B, P, 400, budget_s=15.0, threads=os.cpu_count())
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"{done} decode steps of the same workload ({dt:.1f} s) by the fp32 CPU "
                                          "oracle, a port of the reference torch path"}
    if extras:
        line["sweep"] = sweep(dec, torch, g, peak, args.repeats)
    dec.close()
    del backend, dec
    if extras and not args.no_torch_arm:
        # the comparison arm runs last, in a process of its own, after this arm's decoder is closed
        pts = [(1, 1), (1, 512), (2, 512), (4, 512), (8, 512), (8, 1150)]
        torch.cuda.empty_cache()
        ref = reference_cudagraph_points(pts, 64)
        if "unavailable" in ref:
            arm = {"arm": "stand-in: the reference torch decode path restated on torch / cuBLAS / FlashAttention "
                          "kernels with CUDA graphs (the reference package is not installed here)",
                   "why": ref["unavailable"], "points": []}
            for b, p in pts:
                try:
                    arm["points"].append({"batch": b, "prompt": p,
                                          "device_us_per_step": torch_cudagraph_standin(weights, g, b, p, 4, 48)})
                except Exception as exc:
                    arm["points"].append({"batch": b, "prompt": p, "unavailable": f"{type(exc).__name__}: {exc}"[:160]})
        else:
            arm = {"arm": "the unmodified reference engine (baseline/_ref): LLM(dir, decode_backend='torch', "
                          "enforce_eager=False), CUDA graphs, same seeded weights; per decode step: the reference's own "
                          "CUDA-event span, the host wall time and the summed GPU kernel time (torch.profiler)",
                   "points": list(ref.values())}
        line["torch_cudagraph"] = arm
    if world > 1:
        try:
            line["tensor_parallel"] = tensor_parallel_block(args, torch, dist, weights, local)
        except Exception as exc:
            line["tensor_parallel"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        _DIST.destroy_process_group()


# ----------------------------------------------------------------------------------------------------------
# profiling drivers
# ----------------------------------------------------------------------------------------------------------
def run_profile_step(args):
    """A few plain decode steps (or standalone LM-head launches) of a small or
    full model for Nsight Compute; nothing here checks results (the tests do)."""
    import torch
    import __graft_entry__  # noqa: F401
    from dfb_b200 import native
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.geometry import ModelGeometry
    from dfb_b200.synthetic import random_init_weights

    g = ModelGeometry(layers=args.layers, vocab=args.vocab)
    w = random_init_weights(g, seed=0, device="cuda")
    pages, B = g.max_pages, args.batch
    kv = torch.empty(2, g.layers, B * pages, g.block_size, g.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    kv.normal_(0, 1)
    dec = StreamDecoder(w, kv[0], kv[1], g.block_size, B * pages, g.max_model_len, use_graph=not args.no_graph,
                        persistent=args.mode == "persistent")
    if args.ctas:
        dec.set_option(native.DFB_OPT_PERSIST_CTAS, args.ctas)
    if args.row_gemv >= 0:
        dec.set_option(native.DFB_OPT_ROW_GEMV, args.row_gemv)
    tables = torch.tensor([list(range(r * pages, (r + 1) * pages)) for r in range(B)], dtype=torch.int32, device="cuda")
    ids = torch.randint(0, g.vocab, (B,), dtype=torch.int64, device="cuda")
    if args.lmhead_only:
        hid = torch.randn(B, g.hidden, device="cuda").to(torch.bfloat16)
        res = torch.randn(B, g.hidden, device="cuda").to(torch.bfloat16)
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(args.lmhead_only):
            native.check(native.lib().dfb_launch_lmhead_argmax(dec._handle, hid.data_ptr(), res.data_ptr(), None, None,
                                                               B, stream), "dfb_launch_lmhead_argmax")
        torch.cuda.synchronize()
        print(f"lm head launches={args.lmhead_only} rows={B} vocab={g.vocab}")
        dec.close()
        return
    for s in range(args.steps):
        ctx = args.prompt + s
        pos = torch.full((B,), ctx - 1, dtype=torch.int64, device="cuda")
        dec.enqueue_rows(ids if s == 0 else None, pos, tables[:, : -(-ctx // g.block_size)], max_context=ctx)
    torch.cuda.synchronize()
    code, st = dec.status()
    print(f"steps={args.steps} mode={args.mode} device_status={st.device_status} kernels_per_step={st.kernels_per_step}")
    dec.close()
    if code:
        raise SystemExit(1)


def run_store_kvcache(args):
    """``dfb_store_kvcache`` alone: N prompt tokens' K and V rows (2 KB each) scattered to random slots of one
    layer's cache, a fresh set of rows and slots per launch (inputs larger than L2 across the timed launches),
    CUDA events around each launch; bytes = N x 2 x 2 KB read + as many written."""
    import torch

    import __graft_entry__  # noqa: F401
    from dfb_b200.kv_store import store_kvcache

    n = int(args.store_kvcache)
    torch.cuda.set_device(0)
    peak, peak_kind = measured_peaks()
    heads, dim, bs = 8, 128, 256
    blocks = max(2 * -(-n // bs), 64)
    k_cache = torch.zeros(blocks, bs, heads, dim, dtype=torch.bfloat16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    sets = max(4, (256 << 20) // max(n * 8192, 1))          # enough distinct inputs to exceed L2
    sets = min(sets, 64)
    qkvs = [torch.randn(n, 4096, device="cuda").bfloat16() for _ in range(sets)]
    slots = [torch.randperm(blocks * bs, device="cuda")[:n].to(torch.int32) for _ in range(sets)]
    from dfb_b200 import native

    lib, stream = native.lib(), torch.cuda.current_stream().cuda_stream
    num_slots = blocks * bs

    def launch(i):   # the C entry point directly: the Python wrapper's checks would be what is timed at this size
        q = qkvs[i % sets]
        native.check(lib.dfb_store_kvcache(q.data_ptr() + 2 * 2048, q.data_ptr() + 2 * 3072, 4096, 4096,
                                           k_cache.data_ptr(), v_cache.data_ptr(), slots[i % sets].data_ptr(), n,
                                           heads * dim, num_slots, None, stream), "dfb_store_kvcache")

    burst = 8                                                # launches per timed sample, back to back
    store_kvcache(qkvs[0][:, 2048:3072].view(n, heads, dim), qkvs[0][:, 3072:4096].view(n, heads, dim), k_cache,
                  v_cache, slots[0])                         # once through the public wrapper
    times = []
    for it in range(args.warmup + max(args.steps, 8)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for j in range(burst):
            launch(it * burst + j)
        b.record()
        torch.cuda.synchronize()
        if it >= args.warmup:
            times.append(1e3 * a.elapsed_time(b) / burst)
    us = statistics.median(times)
    moved = 2 * n * 2 * heads * dim * 2                        # K and V rows, read and written
    print(json.dumps({"kernel": "store_kvcache_kernel", "tokens": n, "us": us, "bytes_read_plus_written": moved,
                      "achieved_gbs": moved / us / 1e3, "peak_gbs": peak, "frac": moved / us / 1e3 / peak,
                      "peak": peak_kind, "launches": len(times)}))


def run_prefill_attention(args):
    """``dfb_prefill_attention`` alone on BATCH sequences of LEN prompt tokens (q / k / v as slices of a fused
    projection output, 16 / 8 heads of 128): CUDA events around each launch, median; causal FLOPs =
    2 n^2 d Hq per sequence.  The library kernel the reference calls for this step (flash_attn_varlen_func) is
    timed on the same tensors when it can be imported, as the point of comparison."""
    import torch

    import __graft_entry__  # noqa: F401
    from dfb_b200.kv_store import prefill_attention

    batch, length = (int(x) for x in args.prefill_attention.lower().split("x"))
    torch.cuda.set_device(0)
    hq, hkv, d = 16, 8, 128
    n = batch * length
    qkv = torch.randn(n, 4096, device="cuda").bfloat16()
    q, k, v = qkv[:, :2048].view(n, hq, d), qkv[:, 2048:3072].view(n, hkv, d), qkv[:, 3072:].view(n, hkv, d)
    cu = torch.arange(0, n + 1, length, dtype=torch.int32, device="cuda")
    scale = d ** -0.5
    flops = batch * 2.0 * length * length * d * hq

    def timed(fn):
        ts = []
        for it in range(args.warmup + max(args.steps, 10)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); out = fn(); b.record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                ts.append(1e3 * a.elapsed_time(b))
        return statistics.median(ts), out

    us, mine = timed(lambda: prefill_attention(q, k, v, cu, length, scale))
    line = {"kernel": "prefill_attention_kernel", "batch": batch, "seq_len": length, "us": us,
            "causal_flops": flops, "achieved_tflops": flops / us / 1e6}
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak_tf = float(peaks.get("bf16_tflops", 0) or 0)
    if peak_tf:
        line.update(peak_tflops=peak_tf, frac=flops / us / 1e6 / peak_tf, peak="measured cuBLAS bf16 burst")
    try:
        from flash_attn import flash_attn_varlen_func

        fa_us, theirs = timed(lambda: flash_attn_varlen_func(q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu,
                                                             max_seqlen_q=length, max_seqlen_k=length,
                                                             softmax_scale=scale, causal=True))
        line.update(flash_attn_us=fa_us, flash_attn_tflops=flops / fa_us / 1e6,
                    max_abs_diff_to_flash_attn=float((mine.float() - theirs.float()).abs().max()))
    except Exception as exc:   # the comparison is optional
        line["flash_attn"] = f"not timed: {type(exc).__name__}"
    print(json.dumps(line))


def run_cta_sweep(args):
    """Per-op time against the CTA count (the reference's TG_NUM_SMS diagnostic,
    backends/megakernel/taskgraph.py:68-83): the persistent kernel at 1 ... 148
    CTAs from its own timeline, and the LM-head kernel of the chain against its
    grid size."""
    import torch
    import __graft_entry__  # noqa: F401
    from dfb_b200 import native
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.geometry import QWEN3_06B as g
    from dfb_b200.synthetic import random_init_weights

    w = random_init_weights(g, seed=0, device="cuda")
    pages = g.max_pages
    kv = torch.zeros(2, g.layers, pages, g.block_size, g.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    tables = [list(range(pages))]
    out = {"persistent_kernel": [], "chain_lm_head": [], "chain_step": None}
    ops = ("qkv", "attention", "o_proj", "gate_up", "down")
    for ctas in (1, 16, 64, 108, 148):
        dec = StreamDecoder(w, kv[0], kv[1], g.block_size, pages, g.max_model_len, persistent=True)
        dec.set_option(native.DFB_OPT_PERSIST_CTAS, ctas)
        steps = 2 if ctas == 1 else 16
        time_step_loop(dec, torch, [1], 1, 2, g.block_size, tables, sync=False)
        ms = time_step_loop(dec, torch, [1], 1, steps, g.block_size, tables, sync=False) / steps
        dec.set_option(native.DFB_OPT_TRACE, 1)
        ids = torch.randint(0, g.vocab, (1,), dtype=torch.int64, device="cuda")
        pos = torch.zeros(1, dtype=torch.int64, device="cuda")
        bt = torch.tensor([tables[0][:1]], dtype=torch.int32, device="cuda")
        for _ in range(2):
            dec.read_trace()
            dec.enqueue_rows(ids, pos, bt, max_context=1)
            torch.cuda.synchronize()
        t = dec.read_trace()
        per_op = {}
        if len(t) == 5 * g.layers + 1:
            for i, name in enumerate(ops):
                rows = t[i:5 * g.layers:5]
                per_op[name] = float(sum(int(r[2]) - int(r[0]) for r in rows)) / len(rows) / 1e3
            per_op["lm_head"] = (int(t[-1][2]) - int(t[-1][0])) / 1e3
        code, st = dec.status()
        out["persistent_kernel"].append({"ctas": ctas, "ms_per_step": ms, "us_per_op": per_op,
                                         "mean_us_per_op": 1e3 * ms / (5 * g.layers + 1),
                                         "device_status": int(st.device_status)})
        dec.close()
    dec = StreamDecoder(w, kv[0], kv[1], g.block_size, pages, g.max_model_len)
    time_step_loop(dec, torch, [1], 2, 3, g.block_size, tables, sync=False)
    out["chain_step"] = {"ms_per_step": time_step_loop(dec, torch, [1], 4, 64, g.block_size, tables, sync=False) / 64}
    hid = torch.randn(1, g.hidden, device="cuda").to(torch.bfloat16)
    res = torch.randn(1, g.hidden, device="cuda").to(torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    for ctas in (16, 64, 108, 148, 296, 444, 592):
        dec.set_option(native.DFB_OPT_LMHEAD_CTAS, ctas)
        lm = lambda: native.check(native.lib().dfb_launch_lmhead_argmax(dec._handle, hid.data_ptr(), res.data_ptr(), None,
                                                                        None, 1, stream), "lmhead")
        for _ in range(3):
            lm()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); e0.record()
        for _ in range(10):
            lm()
        e1.record(); torch.cuda.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / 10
        tiles = g.vocab // 16
        out["chain_lm_head"].append({"ctas": ctas, "us": us, "us_per_tile_per_cta": us / (-(-tiles // ctas))})
    dec.close()
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=120)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=1)
    ap.add_argument("--repeats", type=int, default=5, help="timed loops of --steps steps each; the median is reported")
    ap.add_argument("--quick", action="store_true", help="headline only: no sweep and no comparison arm")
    ap.add_argument("--no-torch-arm", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    # profiling drivers
    ap.add_argument("--profile-step", action="store_true", help="run plain steps for a profiler instead of the benchmark")
    ap.add_argument("--cta-sweep", action="store_true", help="per-op time against the CTA count")
    ap.add_argument("--prefill-attention", type=str, default="", metavar="BATCHxLEN",
                    help="time dfb_prefill_attention alone, e.g. 8x512, next to flash_attn_varlen_func on the same inputs")
    ap.add_argument("--store-kvcache", type=int, default=0, metavar="TOKENS",
                    help="time dfb_store_kvcache (prefill-side KV write) alone for this many prompt tokens")
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--mode", choices=["persistent", "chained"], default="chained")
    ap.add_argument("--lmhead-only", type=int, default=0, metavar="N")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--row-gemv", type=int, default=-1, help="profile driver: DFB_OPT_ROW_GEMV of the decoder")
    ap.add_argument("--set-option", action="append", default=[], metavar="ID=VALUE",
                    help="dfb_set_option on the benchmarked decoder (tuning experiments), e.g. 15=0")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    if args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # a rank that dies while its memory is bound to an in-switch reduction (NVLS) group faults its peers
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if args.profile_step:
        run_profile_step(args)
    elif args.cta_sweep:
        run_cta_sweep(args)
    elif args.store_kvcache:
        run_store_kvcache(args)
    elif args.prefill_attention:
        run_prefill_attention(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_own_arm(args)


if __name__ == "__main__":
    main()
