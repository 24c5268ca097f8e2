"""ctypes binding of ``libdfb_decode.so`` (the C ABI in ``include/dfb_decode.h``).

The library is built in-tree by :func:`build` (``nvcc`` for sm_100a).  Loading
fails loudly when it is missing: there is no Python or CPU fallback behind
these calls.
"""

from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libdfb_decode.so"
SOURCES = [PKG_DIR / "csrc" / "dfb_api.cu"]
HEADERS = [PKG_DIR / "csrc" / "dfb_kernels.cuh", PKG_DIR / "csrc" / "dfb_persistent.cuh", PKG_DIR / "csrc" / "dfb_rowgemv.cuh", PKG_DIR / "csrc" / "dfb_exchange.cuh", PKG_DIR / "csrc" / "dfb_pairgemv.cuh", PKG_DIR / "csrc" / "dfb_tcgemv.cuh", PKG_DIR / "csrc" / "dfb_attnring.cuh", PKG_DIR / "csrc" / "dfb_prefill.cuh", PKG_DIR.parent / "include" / "dfb_decode.h"]

DFB_ABI_VERSION = 2
DFB_MAX_ROWS = 8
DFB_MAX_BURST = 1024
DFB_MAX_SLOTS = 32
TOKEN_CALLBACK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_longlong), C.POINTER(C.c_int32), C.c_int32)
DFB_ATTN_CHUNK = 64
DFB_TP_HANDLE_BYTES = 64
DFB_OPT_USE_GRAPH, DFB_OPT_USE_PDL, DFB_OPT_LMHEAD_CTAS, DFB_OPT_TRACE = 1, 2, 3, 4
DFB_OPT_STEP_MODE, DFB_OPT_PERSIST_CTAS, DFB_OPT_ROW_GEMV, DFB_OPT_ATTN_WIDE = 5, 6, 7, 8
DFB_OPT_SMEM_CARVEOUT, DFB_OPT_SMEM_CARVEOUT_MMA, DFB_OPT_LATE_TRIGGER, DFB_OPT_PAIR_GEMV = 9, 10, 11, 12
DFB_OPT_BULK_X, DFB_OPT_TP_FUSED = 13, 14
DFB_OPT_LOOK_AHEAD, DFB_OPT_LMHEAD_AHEAD_MB, DFB_OPT_PEER_WAIT_US, DFB_OPT_TCGEN05 = 15, 16, 17, 18
DFB_OPT_ATTN_RING = 19
DFB_OPT_ATTN_CLUSTER = 20
DFB_OPT_ATTN_CHUNK128 = 21
DFB_OPT_ATTN_RING32 = 22
DFB_OPT_REG_WEIGHTS = 23
DFB_OPT_HOST_IO = 24
DFB_STATUS_BAD_POSITION, DFB_STATUS_BAD_BLOCK, DFB_STATUS_COPY_TIMEOUT = 1, 2, 3
DFB_STATUS_PEER_TIMEOUT, DFB_STATUS_BAD_TOKEN, DFB_STATUS_BAD_GRID, DFB_STATUS_BAD_SLOT = 4, 5, 6, 7

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]

EXPORTS = (
    "dfb_create", "dfb_destroy", "dfb_set_option", "dfb_decode_step", "dfb_decode_step_host",
    "dfb_read_status", "dfb_error_string", "dfb_read_trace", "dfb_launch_rmsnorm_qkv", "dfb_launch_attention",
    "dfb_launch_linear", "dfb_launch_rmsnorm_gateup_swiglu", "dfb_launch_lmhead_argmax",
    "dfb_lmhead_argmax_noalloc", "dfb_set_tensor_parallel", "dfb_tp_window_handle", "dfb_tp_open_peers",
    "dfb_tp_open_loopback", "dfb_decode_step_host_sampled", "dfb_set_seed", "dfb_launch_lmhead_sample",
    "dfb_decode_burst_enqueue", "dfb_decode_burst_collect", "dfb_decode_burst_host", "dfb_warm",
    "dfb_store_kvcache", "dfb_slot_set", "dfb_slot_get", "dfb_slots_step", "dfb_slots_run",
    "dfb_prefill_attention",
)


class DfbLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("ln_in", "wqkv", "q_norm", "k_norm", "wo", "ln_post", "wgu", "wd")]


class DfbModelDesc(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32), ("hidden", C.c_int32), ("layers", C.c_int32), ("q_heads", C.c_int32),
        ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("intermediate", C.c_int32), ("vocab", C.c_int32),
        ("max_model_len", C.c_int32), ("block_size", C.c_int32), ("num_blocks", C.c_int32), ("eps", C.c_float),
        ("embed", C.c_void_p), ("final_norm", C.c_void_p), ("rope_cos_sin", C.c_void_p),
        ("layer_weights", C.POINTER(DfbLayerWeights)), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
    ]


class DfbTensorParallel(C.Structure):
    """One rank of a tensor-parallel group; the two collectives are plain
    function addresses with ncclAllReduce's / ncclAllGather's signatures."""
    _fields_ = [
        ("size", C.c_int32), ("rank", C.c_int32), ("vocab_offset", C.c_int32), ("dtype_bf16", C.c_int32),
        ("dtype_int8", C.c_int32), ("op_sum", C.c_int32), ("all_reduce", C.c_void_p), ("all_gather", C.c_void_p),
        ("comm", C.c_void_p),
    ]


class DfbStepDesc(C.Structure):
    _fields_ = [
        ("rows", C.c_int32), ("block_table_cols", C.c_int32), ("block_table_stride", C.c_int32),
        ("max_context", C.c_int32), ("input_ids", C.c_void_p), ("positions", C.c_void_p),
        ("block_tables", C.c_void_p), ("row_active", C.c_void_p), ("out_tokens", C.c_void_p),
        ("out_logits", C.c_void_p), ("temperatures", C.c_void_p),
    ]


class DfbStatus(C.Structure):
    _fields_ = [("device_status", C.c_int32), ("detail", C.c_int32 * 3), ("steps", C.c_int64),
                ("kernels_per_step", C.c_int64)]


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS if p.exists())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA library for sm_100a next to this file."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libdfb_decode.so")
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(LIB_PATH), *map(str, SOURCES)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return LIB_PATH


_LIB = None


def lib() -> C.CDLL:
    """Load the library (once).  Raises if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`; "
            "the megakernel decode backend has no fallback implementation"
        )
    L = C.CDLL(str(LIB_PATH))
    vp, i32, f32 = C.c_void_p, C.c_int32, C.c_float
    L.dfb_create.argtypes = [C.POINTER(DfbModelDesc), C.POINTER(vp)]
    L.dfb_destroy.argtypes = [vp]
    L.dfb_destroy.restype = None
    L.dfb_set_option.argtypes = [vp, C.c_int, C.c_int]
    L.dfb_decode_step.argtypes = [vp, C.POINTER(DfbStepDesc), vp]
    L.dfb_decode_step_host.argtypes = [vp, i32, vp, vp, vp, i32, vp, vp, vp]
    L.dfb_decode_step_host_sampled.argtypes = [vp, i32, vp, vp, vp, i32, vp, vp, vp, vp]
    L.dfb_set_seed.argtypes = [vp, C.c_uint64]
    L.dfb_warm.argtypes = [vp, i32, i32, i32, vp]
    L.dfb_prefill_attention.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                        i32, i32, i32, f32, vp, i32, i32, i32, vp, vp]
    L.dfb_slot_set.argtypes = [vp, i32, i32, C.c_int64, C.c_int64, vp, i32, f32]
    L.dfb_slot_get.argtypes = [vp, i32, vp, vp, vp]
    L.dfb_slots_step.argtypes = [vp, vp, vp, vp]
    L.dfb_slots_run.argtypes = [vp, i32, TOKEN_CALLBACK, vp, vp]
    L.dfb_store_kvcache.argtypes = [vp, vp, C.c_int64, C.c_int64, vp, vp, vp, i32, i32, C.c_int64, vp, vp]
    L.dfb_decode_burst_enqueue.argtypes = [vp, i32, i32, vp, vp, vp, i32, vp, vp, vp]
    L.dfb_decode_burst_collect.argtypes = [vp, i32, vp, vp]
    L.dfb_decode_burst_host.argtypes = [vp, i32, i32, vp, vp, vp, i32, vp, vp, vp, vp]
    L.dfb_launch_lmhead_sample.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp]
    L.dfb_read_status.argtypes = [vp, C.POINTER(DfbStatus)]
    L.dfb_read_trace.argtypes = [vp, vp, i32]
    L.dfb_error_string.argtypes = [C.c_int]
    L.dfb_error_string.restype = C.c_char_p
    L.dfb_launch_rmsnorm_qkv.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, vp]
    L.dfb_launch_attention.argtypes = [vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, vp]
    L.dfb_launch_linear.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    L.dfb_launch_rmsnorm_gateup_swiglu.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, vp]
    L.dfb_launch_lmhead_argmax.argtypes = [vp, vp, vp, vp, vp, i32, vp]
    L.dfb_set_tensor_parallel.argtypes = [vp, C.POINTER(DfbTensorParallel)]
    L.dfb_tp_window_handle.argtypes = [vp, vp]
    L.dfb_tp_open_peers.argtypes = [vp, vp]
    L.dfb_tp_open_loopback.argtypes = [vp]
    L.dfb_lmhead_argmax_noalloc.argtypes = [vp, vp, vp, vp, i32, i32, i32, f32, vp, vp, vp]
    for name in EXPORTS:
        if name not in ("dfb_destroy", "dfb_error_string"):
            getattr(L, name).restype = C.c_int
    _LIB = L
    return L


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().dfb_error_string(code).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {code})")
