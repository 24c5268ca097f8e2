#!/usr/bin/env python
"""Run a few decode steps of a (small or full) model for a profiler.

Every kernel of the library is an ordinary launch, so Nsight Compute can
capture any of them from this driver, e.g. (one GPU, small case):

    python decode-fusion-boundary_b200/profile_step.py --layers 1 --lmhead-only 4
    ncu --set full --clock-control none -k regex:row_gemv_kernel -s 1 -c 2 \\
        -o prof python decode-fusion-boundary_b200/profile_step.py --layers 1 --lmhead-only 4

``--mode chained`` (default) runs the step as the chain of per-op kernels
(``row_gemv_kernel`` for one or two rows, ``pair_gemv_kernel`` / ``stream_gemv_kernel``
above that, ``paged_attention_kernel``), ``--mode persistent`` as the single persistent
kernel; ``--no-graph`` launches directly instead of replaying a CUDA graph.  Weights are seeded random
values; the KV history is random; nothing here checks results (the tests do).
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=1, help="context length before the first step")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--mode", choices=["persistent", "chained"], default="chained")
    ap.add_argument("--lmhead-only", type=int, default=0, metavar="N",
                    help="instead of whole steps, launch the standalone LM-head + argmax kernel N times")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--ctas", type=int, default=0, help="grid of the persistent kernel (0 = one per SM)")
    args = ap.parse_args()

    import torch
    import __graft_entry__  # noqa: F401
    from dfb_b200 import native
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.geometry import ModelGeometry
    from dfb_b200.synthetic import random_init_weights

    g = ModelGeometry(layers=args.layers, vocab=args.vocab)
    w = random_init_weights(g, seed=0, device="cuda")
    pages, B = g.max_pages, args.rows
    kv = torch.empty(2, g.layers, B * pages, g.block_size, g.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    kv.normal_(0, 1)
    dec = StreamDecoder(w, kv[0], kv[1], g.block_size, B * pages, g.max_model_len, use_graph=not args.no_graph,
                        persistent=args.mode == "persistent")
    if args.ctas:
        dec.set_option(native.DFB_OPT_PERSIST_CTAS, args.ctas)
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


if __name__ == "__main__":
    main()
