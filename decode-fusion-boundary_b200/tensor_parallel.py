"""Tensor-parallel decode: weight sharding and the NCCL communicator the C
library calls through.

The reference's megakernel backend is single-GPU (tensor_parallel_size != 1 is
an explicit fallback reason, backends/megakernel/taskgraph.py:119-122); the
partitioning here is the one of its torch path: ``QKVParallelLinear`` /
``MergedColumnParallelLinear`` split output rows by head and by gate/up half,
``RowParallelLinear`` splits input columns and sums over the ranks
(layers/linear.py:54-153), ``ParallelLMHead`` splits the vocabulary
(layers/embed_head.py), and each rank's KV cache holds its KV heads only
(engine/model_runner.py:188).  Norm weights, the residual stream, token ids
and (here) the embedding table are replicated.

One process per GPU.  The communicator is created with NCCL's own C API
(``ncclGetUniqueId`` on rank 0, the id broadcast through ``torch.distributed``,
``ncclCommInitRank`` everywhere) because the C library needs the addresses of
``ncclAllReduce`` / ``ncclAllGather`` and a raw ``ncclComm_t`` to enqueue the
collectives on its own stream and to capture them in its CUDA graphs.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, replace
from pathlib import Path

from .geometry import ModelGeometry

NCCL_UNIQUE_ID_BYTES = 128
NCCL_INT8, NCCL_BFLOAT16, NCCL_SUM = 0, 9, 0   # ncclDataType_t / ncclRedOp_t codes (nccl.h)


def shard_geometry(geom: ModelGeometry, size: int) -> ModelGeometry:
    """Per-rank shapes.  Raises with the reason when the model does not split."""
    if size not in (1, 2, 4, 8):
        raise ValueError(f"tensor_parallel_size must be 1, 2, 4 or 8, got {size}")
    for name in ("q_heads", "kv_heads", "intermediate", "vocab"):
        if getattr(geom, name) % size:
            raise ValueError(f"{name}={getattr(geom, name)} is not divisible by tensor_parallel_size={size}")
    return replace(geom, q_heads=geom.q_heads // size, kv_heads=geom.kv_heads // size,
                   intermediate=geom.intermediate // size, vocab=geom.vocab // size)


def shard_layer_tensors(layer, geom: ModelGeometry, rank: int, size: int):
    """This rank's slices of one layer (contiguous copies)."""
    from .weights import LayerTensors

    d, q, kv, inter = geom.head_dim, geom.q_size, geom.kv_size, geom.intermediate
    ql, kvl, il = q // size, kv // size, inter // size
    wq = layer.wqkv[rank * ql:(rank + 1) * ql]
    wk = layer.wqkv[q + rank * kvl:q + (rank + 1) * kvl]
    wv = layer.wqkv[q + kv + rank * kvl:q + kv + (rank + 1) * kvl]
    gate = layer.wgu[rank * il:(rank + 1) * il]
    up = layer.wgu[inter + rank * il:inter + (rank + 1) * il]
    import torch

    cat = torch.cat
    assert d * (geom.q_heads // size) == ql
    return LayerTensors(
        ln_in=layer.ln_in, wqkv=cat([wq, wk, wv]).contiguous(), q_norm=layer.q_norm, k_norm=layer.k_norm,
        wo=layer.wo[:, rank * ql:(rank + 1) * ql].contiguous(), ln_post=layer.ln_post,
        wgu=cat([gate, up]).contiguous(), wd=layer.wd[:, rank * il:(rank + 1) * il].contiguous())


def shard_weights(weights, rank: int, size: int):
    """``DecoderWeights`` of rank ``rank``: sliced projections, the whole
    embedding table (rows ``[rank * vocab / size, ...)`` of it are the rank's
    LM head), replicated norms."""
    from .weights import DecoderWeights

    if size == 1:
        return weights
    local = shard_geometry(weights.geom, size)
    layers = [shard_layer_tensors(l, weights.geom, rank, size) for l in weights.layers]
    return DecoderWeights(local, weights.embed, layers, weights.final_norm, weights.cos_sin,
                          embed_rows=weights.geom.vocab, vocab_offset=rank * local.vocab)


def localize_nano_weights(weights, group):
    """``weights`` as read from ONE RANK of a tensor-parallel nano-vLLM model
    (``weights_from_nano_model``): the projections are already that rank's
    shards, and ``embed`` is the rank's slice ``[vocab / size, hidden]`` of the
    vocabulary-parallel embedding (layers/embed_head.py).  The decode step
    gathers embedding rows by token id on every rank, so the slices are
    collected once into the whole table; the rank's LM head is its slice of it."""
    import torch

    from .weights import DecoderWeights

    size, rank = group.size, group.rank
    g = weights.geom
    local_vocab = weights.embed.shape[0]
    parts = [torch.empty_like(weights.embed) for _ in range(size)]
    group.dist.all_gather(parts, weights.embed.contiguous())
    full = torch.cat(parts).contiguous()
    local = replace(g, q_heads=weights.layers[0].wo.shape[1] // g.head_dim,
                    kv_heads=(weights.layers[0].wqkv.shape[0] - weights.layers[0].wo.shape[1]) // (2 * g.head_dim),
                    intermediate=weights.layers[0].wd.shape[1], vocab=local_vocab)
    return DecoderWeights(local, full, weights.layers, weights.final_norm, weights.cos_sin,
                          embed_rows=full.shape[0], vocab_offset=rank * local_vocab)


def merge_shard_argmax(values, indices, shard_rows: int):
    """Host restatement of the device merge: ``values[r][b]`` / ``indices[r][b]``
    are rank r's best logit of row b and its shard-local index; the token is the
    largest value, the lowest global index among equals."""
    out = []
    for b in range(len(values[0])):
        best_v, best_i = float("-inf"), None
        for r in range(len(values)):
            gi = int(indices[r][b]) + r * shard_rows
            v = float(values[r][b])
            if best_i is None or v > best_v or (v == best_v and gi < best_i):
                best_v, best_i = v, gi
        out.append(best_i)
    return out


def _load_nccl():
    """The NCCL library of this Python environment (the one torch uses)."""
    import importlib.util

    spec = importlib.util.find_spec("nvidia.nccl")
    if spec is not None and spec.submodule_search_locations:
        for root in spec.submodule_search_locations:
            cand = Path(root) / "lib" / "libnccl.so.2"
            if cand.exists():
                return C.CDLL(str(cand), mode=C.RTLD_GLOBAL)
    return C.CDLL("libnccl.so.2", mode=C.RTLD_GLOBAL)


class _UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * NCCL_UNIQUE_ID_BYTES)]


@dataclass
class TensorParallelGroup:
    """An NCCL communicator owned by this process plus what the C library
    needs to call it."""

    rank: int
    size: int
    comm: C.c_void_p
    lib: object
    dist: object = None
    # "direct": the library's own exchange kernels over peer-mapped memory (NVLink, one node);
    # "nccl": ncclAllReduce / ncclAllGather on the library's stream
    transport: str = "direct"

    @classmethod
    def create(cls, dist, device_index: int, transport: str = "direct") -> "TensorParallelGroup":
        """``dist``: an initialised ``torch.distributed`` (any backend) used only
        to hand rank 0's NCCL id to the other ranks."""
        import torch

        rank, size = dist.get_rank(), dist.get_world_size()
        nccl = _load_nccl()
        uid = _UniqueId()
        if rank == 0:
            rc = nccl.ncclGetUniqueId(C.byref(uid))
            if rc:
                raise RuntimeError(f"ncclGetUniqueId failed with code {rc}")
        box = [bytes(C.string_at(C.byref(uid), NCCL_UNIQUE_ID_BYTES)) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        C.memmove(C.byref(uid), box[0], NCCL_UNIQUE_ID_BYTES)
        torch.cuda.set_device(device_index)
        comm = C.c_void_p()
        nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, _UniqueId, C.c_int]
        rc = nccl.ncclCommInitRank(C.byref(comm), size, uid, rank)
        if rc:
            raise RuntimeError(f"ncclCommInitRank failed with code {rc}")
        if transport not in ("direct", "nccl"):
            raise ValueError("transport must be 'direct' or 'nccl'")
        return cls(rank, size, comm, nccl, dist, transport)

    def gather_bytes(self, payload: bytes) -> list[bytes]:
        """Every rank's ``payload`` in rank order (host side, through torch.distributed)."""
        out = [None] * self.size
        self.dist.all_gather_object(out, payload)
        return out

    def descriptor(self, native, vocab_offset: int):
        return native.DfbTensorParallel(
            size=self.size, rank=self.rank, vocab_offset=vocab_offset, dtype_bf16=NCCL_BFLOAT16,
            dtype_int8=NCCL_INT8, op_sum=NCCL_SUM,
            all_reduce=C.cast(self.lib.ncclAllReduce, C.c_void_p).value,
            all_gather=C.cast(self.lib.ncclAllGather, C.c_void_p).value, comm=self.comm.value)

    def close(self) -> None:
        comm, self.comm = self.comm, None
        if comm:
            self.lib.ncclCommDestroy.argtypes = [C.c_void_p]
            self.lib.ncclCommDestroy(comm)
