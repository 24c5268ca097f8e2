"""The C-ABI library loads and exports every function include/dfb_decode.h
declares; the ctypes structures have the header's layout.  No GPU work."""

import ctypes as C
import re
from pathlib import Path

from dfb_b200 import native

HEADER = Path(__file__).resolve().parents[1] / "include" / "dfb_decode.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return set(re.findall(r"\b(dfb_[a-z_0-9]+)\s*\(", text))


def test_library_exports_every_declared_symbol():
    native.build()
    lib = native.lib()
    names = declared_functions()
    assert names == set(native.EXPORTS)
    for n in names:
        assert hasattr(lib, n), n


def test_constants_match_header():
    text = HEADER.read_text()
    for name in ("DFB_ABI_VERSION", "DFB_MAX_ROWS", "DFB_ATTN_CHUNK", "DFB_OPT_USE_GRAPH", "DFB_OPT_USE_PDL",
                 "DFB_OPT_LMHEAD_CTAS", "DFB_OPT_TRACE", "DFB_OPT_STEP_MODE", "DFB_OPT_PERSIST_CTAS"):
        value = int(re.search(rf"#define {name}\s+(\d+)", text).group(1))
        assert getattr(native, name) == value


def test_struct_layouts():
    assert C.sizeof(native.DfbLayerWeights) == 64
    assert C.sizeof(native.DfbModelDesc) == 12 * 4 + 6 * 8
    assert native.DfbModelDesc.embed.offset == 48
    assert C.sizeof(native.DfbStepDesc) == 16 + 7 * 8
    assert native.DfbStepDesc.temperatures.offset == 16 + 6 * 8
    assert C.sizeof(native.DfbStatus) == 32


def test_argument_errors_need_no_device():
    lib = native.lib()
    handle = C.c_void_p()
    assert lib.dfb_create(None, C.byref(handle)) == -1
    bad = native.DfbModelDesc(abi_version=99)
    assert lib.dfb_create(C.byref(bad), C.byref(handle)) == -3
    bad = native.DfbModelDesc(abi_version=native.DFB_ABI_VERSION, hidden=512)
    assert lib.dfb_create(C.byref(bad), C.byref(handle)) == -2
    assert handle.value is None
    assert lib.dfb_decode_step(None, None, None) == -1
    assert lib.dfb_error_string(-2) == b"dfb: unsupported model geometry"
    assert lib.dfb_error_string(0) == b"success"


def test_store_kvcache_argument_checks_need_no_device():
    """dfb_store_kvcache validates before any launch."""
    lib = native.lib()
    one = 16
    assert lib.dfb_store_kvcache(None, one, 1024, 1024, one, one, one, 1, 1024, 10, None, None) == -1
    assert lib.dfb_store_kvcache(one, one, 1024, 1024, one, one, one, 1, 1020, 10, None, None) == -1   # row not in 16-byte pieces
    assert lib.dfb_store_kvcache(one, one, 512, 1024, one, one, one, 1, 1024, 10, None, None) == -1    # stride < row
    assert lib.dfb_store_kvcache(one, one + 2, 1024, 1024, one, one, one, 1, 1024, 10, None, None) == -1  # misaligned
    assert lib.dfb_store_kvcache(one, one, 1024, 1024, one, one, one, 0, 1024, 10, None, None) == 0    # nothing to do


def test_prefill_attention_argument_checks_need_no_device():
    lib = native.lib()
    one = 16
    ok = (one, one, one, one, one, None, 1, 8, 4096, 4096, 4096, 2048, 16, 8, 128, 0.088, None, 0, 0, 0, None, None)
    bad = list(ok); bad[0] = None
    assert lib.dfb_prefill_attention(*bad) == -1
    bad = list(ok); bad[14] = 64                 # head_dim the kernel is not built for
    assert lib.dfb_prefill_attention(*bad) == -2
    bad = list(ok); bad[12], bad[13] = 16, 5     # q heads not a multiple of kv heads
    assert lib.dfb_prefill_attention(*bad) == -2
    bad = list(ok); bad[8] = 1000                # q stride shorter than a row
    assert lib.dfb_prefill_attention(*bad) == -1
    bad = list(ok); bad[9] = 4100                # k stride not a multiple of 8
    assert lib.dfb_prefill_attention(*bad) == -1
    bad = list(ok); bad[16] = one                # a block table without its geometry
    assert lib.dfb_prefill_attention(*bad) == -1
