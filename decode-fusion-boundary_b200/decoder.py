"""The decoder object behind ``decode_backend="megakernel"``.

Host-side replacement of the reference's ``TaskGraphDecoder``
(backends/megakernel/taskgraph.py:92-131 admission policy, :150-305 set-up,
:354-529 per-step protocol).  The reference builds a per-SM instruction stream
for one cooperative kernel; this decoder owns a native ``DfbHandle`` that runs
the step as a chain of ordinary sm_100a kernels inside a CUDA graph.  The
method set (``step`` / ``step_batch`` / ``decode_rows`` / ``decode_row``), the
argument meaning (pre-decode length as position, block tables right-padded
with block 0) and the error behaviour are the reference's.

``torch`` is imported lazily so the admission policy stays importable on a
machine without CUDA.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any

from .contracts import max_pages_per_seq, row_active_mask

# Compile-time row ceiling of the kernels (DFB_MAX_ROWS); the reference's
# TG_MAX_BATCH (taskgraph.py:33).
TG_MAX_BATCH = 8
# Tensor-parallel sizes the backend admits.  The reference admits only 1
# (taskgraph.py:119-122); this build also runs 2, 4 and 8 ranks, provided the
# engine attached a tensor-parallel group (``config.megakernel_tensor_parallel``,
# a ``tensor_parallel.TensorParallelGroup`` of that size) for the exchanges.
SUPPORTED_TP_SIZES = (1, 2, 4, 8)


@dataclass(frozen=True)
class TaskGraphCompatibility:
    supported: bool
    reason: str = ""


def taskgraph_compatibility(config: Any, seqs: list[Any], is_prefill: bool) -> TaskGraphCompatibility:
    """Torch-free admission policy; one explicit reason per rejection, in the
    reference's order (taskgraph.py:92-131)."""
    if is_prefill:
        return TaskGraphCompatibility(False, "Task-graph megakernel is decode-only; use the prefill backend")
    if not seqs:
        return TaskGraphCompatibility(False, "Task-graph megakernel needs at least one sequence")
    if len(seqs) > TG_MAX_BATCH:
        return TaskGraphCompatibility(
            False,
            f"Task-graph megakernel supports batch sizes 1..{TG_MAX_BATCH} "
            "(TG_MAX_BATCH, the compile-time scratch/bar ceiling)")
    max_num_seqs = getattr(config, "max_num_seqs", None)
    if isinstance(max_num_seqs, int) and max_num_seqs < len(seqs):
        return TaskGraphCompatibility(False, f"batch {len(seqs)} exceeds max_num_seqs={max_num_seqs}")
    tp_size = getattr(config, "tensor_parallel_size", 1)
    if tp_size not in SUPPORTED_TP_SIZES:
        return TaskGraphCompatibility(False, "Task-graph megakernel requires tensor_parallel_size in (1, 2, 4, 8)")
    if tp_size != 1:
        group = getattr(config, "megakernel_tensor_parallel", None)
        if group is None:
            return TaskGraphCompatibility(
                False, f"Task-graph megakernel at tensor_parallel_size={tp_size} needs a tensor-parallel group "
                       "(config.megakernel_tensor_parallel)")
        if getattr(group, "size", None) != tp_size:
            return TaskGraphCompatibility(
                False, f"tensor-parallel group has {getattr(group, 'size', None)} ranks but "
                       f"tensor_parallel_size={tp_size}")
    # Sampling.  The reference hands every non-greedy row back to torch (taskgraph.py:123-130); that stays the
    # default.  ``config.megakernel_sampling`` opts in to the sampler fused after the LM head
    # (layers/sampler.py:7-16 restated as a Gumbel-max draw): any true value admits a sampled single row, whose
    # temperature ``MegakernelBackend.decode`` reads from the sequence; the value "batch" also admits sampled
    # rows in batches, for engines that pass ``temperatures`` to ``MegakernelBackend.decode_batch`` (the stock
    # ``ModelRunner.run`` does not).
    sampling = getattr(config, "megakernel_sampling", False)
    for seq in seqs:
        if bool(getattr(seq, "is_greedy", False)):
            continue
        temperature = getattr(seq, "temperature", None)
        if temperature is None or temperature > 1e-10:
            if temperature is None or not sampling:
                return TaskGraphCompatibility(False, "Task-graph megakernel supports greedy sampling only")
            if len(seqs) > 1 and sampling != "batch":
                return TaskGraphCompatibility(
                    False, "Task-graph megakernel samples batches only when the engine passes temperatures to "
                           "decode_batch (config.megakernel_sampling = 'batch')")
    return TaskGraphCompatibility(True)


class StreamDecoder:
    """Owns the native decoder handle and runs one decode step per call."""

    def __init__(self, weights, k_cache, v_cache, block_size: int, num_cache_blocks: int,
                 max_model_len: int = 2048, attn_splits: int = 1, fusion_groups: int = 1,
                 verbose: bool = False, debug_bounds: bool = False, use_graph: bool = True,
                 use_pdl: bool = True, persistent: bool = False, tensor_parallel=None):
        import torch

        from . import native

        self._torch = torch
        self._native = native
        self._lib = native.lib()  # raises if the CUDA library has not been built
        if not torch.cuda.is_available():
            raise RuntimeError("Megakernel requires a CUDA device")
        g = weights.geom
        if max_model_len != g.max_model_len or block_size != g.block_size:
            raise ValueError("weights geometry disagrees with max_model_len / block_size")
        weights.validate()
        for name, cache in (("k_cache", k_cache), ("v_cache", v_cache)):
            want = (g.layers, num_cache_blocks, block_size, g.kv_heads, g.head_dim)
            if tuple(cache.shape) != want or cache.dtype != torch.bfloat16 or not cache.is_contiguous():
                raise RuntimeError(f"{name} must be a contiguous bf16 tensor of shape {want}")
        self._weights = weights  # keeps the tensors alive
        self._k_cache, self._v_cache = k_cache, v_cache
        self._max_rows = TG_MAX_BATCH
        self._max_pages = max_pages_per_seq(max_model_len, block_size)
        self._block_size = block_size
        self._max_model_len = max_model_len
        self._vocab = g.vocab
        # ``attn_splits`` / ``fusion_groups`` configure the reference's schedule
        # builder.  Here the split count follows the context length per step and
        # the step is always one graph, so both are accepted and not used.
        self._attn_splits, self._fusion_groups = int(attn_splits), int(fusion_groups)
        self._verbose, self._debug_bounds = bool(verbose), bool(debug_bounds)

        layer_arr = (native.DfbLayerWeights * g.layers)()
        for i, layer in enumerate(weights.layers):
            for name, _ in native.DfbLayerWeights._fields_:
                setattr(layer_arr[i], name, getattr(layer, name).data_ptr())
        desc = native.DfbModelDesc(
            abi_version=native.DFB_ABI_VERSION, hidden=g.hidden, layers=g.layers, q_heads=g.q_heads,
            kv_heads=g.kv_heads, head_dim=g.head_dim, intermediate=g.intermediate, vocab=g.vocab,
            max_model_len=max_model_len, block_size=block_size, num_blocks=num_cache_blocks, eps=g.eps,
            embed=weights.embed.data_ptr(), final_norm=weights.final_norm.data_ptr(),
            rope_cos_sin=weights.cos_sin.data_ptr(), layer_weights=layer_arr,
            k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr())
        handle = C.c_void_p()
        native.check(self._lib.dfb_create(C.byref(desc), C.byref(handle)), "dfb_create")
        self._handle = handle
        native.check(self._lib.dfb_set_option(handle, native.DFB_OPT_USE_GRAPH, int(use_graph)), "dfb_set_option")
        native.check(self._lib.dfb_set_option(handle, native.DFB_OPT_USE_PDL, int(use_pdl)), "dfb_set_option")
        native.check(self._lib.dfb_set_option(handle, native.DFB_OPT_STEP_MODE, int(persistent)), "dfb_set_option")
        # ``tensor_parallel``: a tensor_parallel.TensorParallelGroup; ``weights`` / the caches are then this
        # rank's shard (tensor_parallel.shard_weights) and every rank must issue the same steps
        self._tp = tensor_parallel
        if tensor_parallel is not None and tensor_parallel.size > 1:
            tp_desc = tensor_parallel.descriptor(native, weights.vocab_offset)
            native.check(self._lib.dfb_set_tensor_parallel(handle, C.byref(tp_desc)), "dfb_set_tensor_parallel")
            if tensor_parallel.transport == "loopback":
                # diagnostic: local stand-ins for the peers' windows, nobody fills them (timeout path on one GPU)
                native.check(self._lib.dfb_tp_open_loopback(handle), "dfb_tp_open_loopback")
            elif tensor_parallel.transport == "direct":
                mine = C.create_string_buffer(native.DFB_TP_HANDLE_BYTES)
                native.check(self._lib.dfb_tp_window_handle(handle, mine), "dfb_tp_window_handle")
                everyone = tensor_parallel.gather_bytes(mine.raw)
                native.check(self._lib.dfb_tp_open_peers(handle, b"".join(everyone)), "dfb_tp_open_peers")

        # persistent per-step buffers: no allocation on the step path
        self._result = torch.zeros(native.DFB_MAX_ROWS + 4, dtype=torch.int32, device="cuda")
        # explicit devices everywhere: the engine builds this object while torch's default device is "cuda"
        # (engine/model_runner.py:68-72), where a bare torch.zeros(...).pin_memory() fails
        self._result_host = torch.zeros(native.DFB_MAX_ROWS + 4, dtype=torch.int32, device="cpu").pin_memory()
        self._row_active = torch.ones(self._max_rows, dtype=torch.int32, device="cuda")
        self._h_ids = (C.c_int64 * self._max_rows)()
        self._h_pos = (C.c_int64 * self._max_rows)()
        self._h_bt = (C.c_int32 * (self._max_rows * self._max_pages))()
        self._h_out = (C.c_int32 * self._max_rows)()
        self._h_temp = (C.c_float * self._max_rows)()
        self._step_host = self._lib.dfb_decode_step_host_sampled
        self._current_stream = torch.cuda.current_stream
        self._step = native.DfbStepDesc()

    # -- lifecycle -----------------------------------------------------------
    def close(self) -> None:
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.dfb_destroy(handle)

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass

    def set_option(self, option: int, value: int) -> None:
        self._native.check(self._lib.dfb_set_option(self._handle, option, value), "dfb_set_option")

    def status(self):
        st = self._native.DfbStatus()
        code = self._lib.dfb_read_status(self._handle, C.byref(st))
        return code, st

    def read_trace(self):
        """Timeline of the last traced step: rows of ``(start, wait_done_last,
        end, wait_done_first, prologue_done, first_tile_mma_done, first_tile_done, 0)``
        in ns per kernel, in launch order; also re-arms the buffer (call once
        before the step to arm it)."""
        import numpy as np

        buf = np.zeros((1024, 8), dtype=np.uint64)
        n = self._lib.dfb_read_trace(self._handle, buf.ctypes.data, 1024)
        if n < 0:
            self._native.check(n, "dfb_read_trace")
        return buf[:n]

    def _stream(self) -> int:
        return self._torch.cuda.current_stream().cuda_stream

    def _raise_device_status(self) -> None:
        _, st = self.status()
        raise RuntimeError(
            f"megakernel decode step reported device status {st.device_status} "
            f"(kernel {st.detail[0]}, index {st.detail[1]}, value {st.detail[2]})")

    # -- decode --------------------------------------------------------------
    WARM_BURST, WARM_DEVICE, WARM_DEVICE_TOKENS, WARM_HOST, WARM_SAMPLING = 1, 2, 4, 8, 16

    def warm(self, max_rows: int | None = None, max_context: int | None = None,
             kinds: int = WARM_DEVICE_TOKENS | WARM_HOST) -> int:
        """Capture the graphs of every step geometry ahead of time (``dfb_warm``; the counterpart of
        ``ModelRunner.capture_cudagraph``).  The default prepares what ``MegakernelBackend`` calls: the
        host-buffer step of ``decode`` and the device-pointer step of ``decode_batch``.  Returns the number of
        graphs held."""
        n = C.c_int32(0)
        self._native.check(self._lib.dfb_warm(self._handle, int(max_rows or self._max_rows),
                                              int(max_context or self._max_model_len), int(kinds), C.byref(n)),
                           "dfb_warm")
        return n.value

    def set_seed(self, seed: int) -> None:
        """Seed of the sampling noise; restarts the noise stream (``dfb_set_seed``)."""
        self._native.check(self._lib.dfb_set_seed(self._handle, int(seed) & (2 ** 64 - 1)), "dfb_set_seed")

    def enqueue_rows(self, input_ids, positions, block_tables, active_rows=None, max_context: int = 0,
                     out_logits=None, temperatures=None) -> None:
        """Enqueue one step on the current stream without reading the result
        (device-resident loops; ``input_ids=None`` feeds the previous tokens
        back).  ``tokens_device()`` holds the token ids once the stream is done.
        ``temperatures``: ``None`` (greedy) or a float32 CUDA tensor ``[rows]``;
        rows above 1e-10 are sampled as ``layers/sampler.py:7-16`` does."""
        torch = self._torch
        rows = int(positions.numel())
        if rows > self._max_rows:
            raise RuntimeError(
                f"decode_rows got {rows} rows but this decoder is sized for {self._max_rows} (TG_MAX_BATCH); "
                "the backend's compatibility check should have rejected this batch upstream")
        cols = int(block_tables.size(1))
        if cols > self._max_pages:
            raise ValueError(
                f"block table has {cols} columns but the task-graph page_table stride is {self._max_pages} "
                "(max_model_len // block_size)")
        if positions.dtype != torch.int64 or (input_ids is not None and input_ids.dtype != torch.int64):
            raise TypeError("input_ids and positions must be int64 CUDA tensors")
        if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
            raise TypeError("block_tables must be an int32 CUDA tensor with unit column stride")
        s = self._step
        s.rows, s.block_table_cols, s.block_table_stride = rows, cols, int(block_tables.stride(0))
        s.max_context = int(max_context)
        s.input_ids = input_ids.data_ptr() if input_ids is not None else None
        s.positions = positions.data_ptr()
        s.block_tables = block_tables.data_ptr()
        if active_rows is not None:
            mask = row_active_mask(active_rows, rows)
            self._row_active[:rows].copy_(torch.tensor(mask, dtype=torch.int32, device="cpu"))
            s.row_active = self._row_active.data_ptr()
        else:
            s.row_active = None
        s.out_tokens = self._result.data_ptr()
        s.out_logits = out_logits.data_ptr() if out_logits is not None else None
        if temperatures is not None:
            if temperatures.dtype != torch.float32 or not temperatures.is_cuda or temperatures.numel() != rows:
                raise TypeError("temperatures must be a float32 CUDA tensor with one value per row")
            s.temperatures = temperatures.data_ptr()
        else:
            s.temperatures = None
        self._native.check(self._lib.dfb_decode_step(self._handle, C.byref(s), self._stream()), "dfb_decode_step")

    def tokens_device(self):
        return self._result

    def decode_rows(self, input_ids, positions, block_tables, active_rows=None, temperatures=None) -> list[int]:
        """One decode step for every row.  ``input_ids`` / ``positions`` are 1-D
        int64 CUDA tensors, ``block_tables`` the padded ``[rows, <= max_pages]``
        int32 CUDA tensor of ``ModelRunner.prepare_block_tables``; returns one
        token id per row after exactly one device-to-host read."""
        rows = int(input_ids.numel())
        if rows == 0:
            return []
        self.enqueue_rows(input_ids, positions, block_tables, active_rows, temperatures=temperatures)
        self._result_host.copy_(self._result, non_blocking=True)
        self._torch.cuda.current_stream().synchronize()
        out = self._result_host.tolist()
        if out[self._native.DFB_MAX_ROWS]:
            self._raise_device_status()
        return out[:rows]

    def decode_host(self, token_ids, positions, block_tables, active_rows=None, temperatures=None) -> list[int]:
        """One step from HOST data (lists of ints; one block-table list per
        row): one packed host-to-device copy, the step, one device-to-host
        copy, one synchronisation -- all inside the native call.
        ``temperatures``: ``None`` (greedy) or one float per row."""
        if len(token_ids) == 0:
            return []
        rows, cols, active, temps = self._pack_host(token_ids, positions, block_tables, active_rows, temperatures)
        code = self._lib.dfb_decode_step_host_sampled(self._handle, rows, self._h_ids, self._h_pos, self._h_bt, cols,
                                                      active, temps, self._h_out, self._stream())
        if code == -4:
            self._raise_device_status()
        self._native.check(code, "dfb_decode_step_host_sampled")
        return [int(self._h_out[r]) for r in range(rows)]

    def _pack_host(self, token_ids, positions, block_tables, active_rows, temperatures):
        rows = len(token_ids)
        if rows > self._max_rows:
            raise RuntimeError(f"got {rows} rows; the decoder is sized for {self._max_rows}")
        cols = max(len(t) for t in block_tables)
        if cols > self._max_pages:
            raise ValueError(
                f"block table has {cols} columns but the task-graph page_table stride is {self._max_pages} "
                "(max_model_len // block_size)")
        for r in range(rows):
            self._h_ids[r] = int(token_ids[r])
            self._h_pos[r] = int(positions[r])
            table = block_tables[r]
            base = r * cols
            for c in range(cols):
                self._h_bt[base + c] = int(table[c]) if c < len(table) else 0
        active = (C.c_int32 * rows)(*row_active_mask(active_rows, rows)) if active_rows is not None else None
        temps = None
        if temperatures is not None:
            if len(temperatures) != rows:
                raise ValueError("one temperature per row")
            temps = (C.c_float * rows)(*[float(t) for t in temperatures])
        return rows, cols, active, temps

    def burst_enqueue(self, token_ids, positions, block_tables, steps: int, active_rows=None,
                      temperatures=None) -> None:
        """Enqueue ``steps`` consecutive decode steps of the same rows (host lists as in
        ``decode_host``; row r's step s runs at ``positions[r] + s`` and the block tables must already hold
        the blocks up to ``positions[r] + steps - 1``).  Returns at once; the tokens feed back on the
        device and are published step by step in pinned host memory (``burst_collect``)."""
        rows, cols, active, temps = self._pack_host(token_ids, positions, block_tables, active_rows, temperatures)
        self._burst = (rows, int(steps), (C.c_int32 * (rows * int(steps)))())
        code = self._lib.dfb_decode_burst_enqueue(self._handle, rows, int(steps), self._h_ids, self._h_pos,
                                                  self._h_bt, cols, active, temps, self._stream())
        self._native.check(code, "dfb_decode_burst_enqueue")

    def burst_collect(self, wait: bool = True) -> list[list[int]]:
        """Tokens of the burst's finished steps, one list per step; ``wait=False`` returns what is there."""
        rows, steps, buf = self._burst
        done = C.c_int32(0)
        code = self._lib.dfb_decode_burst_collect(self._handle, int(wait), buf, C.byref(done))
        if code == -4:
            self._raise_device_status()
        self._native.check(code, "dfb_decode_burst_collect")
        return [[int(buf[s * rows + r]) for r in range(rows)] for s in range(done.value)]

    def decode_burst(self, token_ids, positions, block_tables, steps: int, active_rows=None,
                     temperatures=None) -> list[list[int]]:
        """``steps`` decode steps with one host-to-device copy and one synchronisation."""
        if not token_ids:
            return []
        self.burst_enqueue(token_ids, positions, block_tables, steps, active_rows, temperatures)
        return self.burst_collect(wait=True)

    def decode_row(self, token_id: int, position: int, block_table, temperature: float = 0.0) -> int:
        """Single-row path of ``ModelRunner`` (batch 1): takes the scheduler's
        host block table directly."""
        if self._torch.is_tensor(block_table):
            block_table = block_table.tolist()
        # the step every batch-1 token goes through: the persistent ctypes arrays are filled in place and the
        # native call made directly (no per-call lists or arrays)
        cols = min(len(block_table), self._max_pages)
        if cols < 1:
            raise ValueError("decode_row needs a block table")
        h_bt = self._h_bt
        for c in range(cols):
            h_bt[c] = block_table[c]
        self._h_ids[0] = token_id
        self._h_pos[0] = position
        temps = None
        if temperature and temperature > 1e-10:
            self._h_temp[0] = temperature
            temps = self._h_temp
        code = self._step_host(self._handle, 1, self._h_ids, self._h_pos, h_bt, cols, None, temps, self._h_out,
                               self._current_stream().cuda_stream)
        if code:
            if code == -4:
                self._raise_device_status()
            self._native.check(code, "dfb_decode_step_host_sampled")
        return self._h_out[0]

    # -- the one-step interface MegakernelBackend calls -----------------------
    def step(self, token_id: int, position: int | None = None, block_table=None, temperature: float = 0.0) -> int:
        if position is None or block_table is None:
            raise ValueError("task-graph decode requires position and block_table")
        return self.decode_row(token_id, position, block_table, temperature)

    def step_batch(self, input_token_ids, positions, block_tables, temperatures=None) -> list[int]:
        return self.decode_rows(input_token_ids, positions, block_tables, temperatures=temperatures)
