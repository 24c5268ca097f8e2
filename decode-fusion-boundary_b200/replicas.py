"""Multi-GPU execution of the decode step: independent replicas.

The decode step of one batch has no exchange between sequences, so with N GPUs
each rank (one process per GPU) runs its own batch on its own copy of the
weights and its own KV cache; there is no collective on the data path.  The only
communication is bookkeeping: a barrier around timed regions and a reduction of
the per-rank results (total tokens, slowest rank's time).
"""

from __future__ import annotations


def barrier(dist) -> None:
    if dist is not None and dist.is_initialized():
        dist.barrier()


def aggregate(dist, tokens: int, elapsed_ms: float, device="cpu") -> tuple[int, float]:
    """``(tokens of all ranks, slowest rank's elapsed ms)``.  Every rank calls
    this with its own numbers; works on any backend (``device`` must match it:
    "cuda" for NCCL, "cpu" for gloo)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return int(tokens), float(elapsed_ms)
    import torch

    total = torch.tensor([float(tokens)], dtype=torch.float64, device=device)
    slowest = torch.tensor([float(elapsed_ms)], dtype=torch.float64, device=device)
    dist.all_reduce(total, op=dist.ReduceOp.SUM)
    dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    return int(round(total.item())), float(slowest.item())


def shard_rows(num_rows: int, rank: int, world: int) -> range:
    """Rows of a global batch owned by ``rank`` (contiguous, as even as possible)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    base, extra = divmod(num_rows, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))
