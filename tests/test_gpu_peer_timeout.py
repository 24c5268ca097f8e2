"""The bounded wait for a tensor-parallel peer, made to run out on ONE GPU.

A decoder is set up as rank 0 of two, but the "peer's" window is a plain local
allocation that nobody ever writes (``dfb_tp_open_loopback``).  With the wait
limit set to a few milliseconds every pull of the step gives up: the step
completes, the status word says which peer and tag were missing, the word can be
read and cleared, and the CUDA context stays usable.  No second rank exists, so
nothing is left waiting, and nothing faults, traps or hangs.
"""

import ctypes as C
import time

import pytest
import torch

from oracle import qwen3_decode as O
from tests import harness as H

pytestmark = pytest.mark.gpu


class LoopbackGroup:
    """The attributes ``StreamDecoder`` reads from a tensor-parallel group."""

    transport = "loopback"

    def __init__(self, size, rank):
        self.size, self.rank = size, rank

    def descriptor(self, native, vocab_offset):
        return native.DfbTensorParallel(size=self.size, rank=self.rank, vocab_offset=vocab_offset, dtype_bf16=9,
                                        dtype_int8=0, op_sum=0, all_reduce=None, all_gather=None, comm=None)


@pytest.mark.parametrize("fused", [1, 0])
@pytest.mark.parametrize("rows", [1, 4])
def test_missing_peer_times_out_with_status_4(cuda_device, rows, fused):
    from dfb_b200 import native
    from dfb_b200.decoder import StreamDecoder
    from dfb_b200.tensor_parallel import shard_weights

    size = 2
    g = H.oracle_geometry(layers=2, vocab=4096)
    w = O.make_weights(g, seed=61, norm="random").to(torch.bfloat16)
    local = shard_weights(H.to_decoder_weights(w), 0, size)
    lg = local.geom
    kv = torch.zeros(2, g.layers, 8, g.block_size, lg.kv_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    dec = StreamDecoder(local, kv[0], kv[1], g.block_size, 8, g.max_pos, tensor_parallel=LoopbackGroup(size, 0))
    dec.set_option(native.DFB_OPT_PEER_WAIT_US, 3000)       # 3 ms instead of the 2 s default
    dec.set_option(native.DFB_OPT_TP_FUSED, fused)
    ids = torch.tensor([5, g.vocab - 1, 7, 9][:rows], device="cuda")    # ids index the whole table, not the shard
    pos = torch.tensor([3, 40, 0, 100][:rows], device="cuda")
    bt = torch.arange(rows, dtype=torch.int32, device="cuda").reshape(rows, 1)
    for attempt in range(2):               # the second step finds a cleared status word and times out again
        t0 = time.perf_counter()
        dec.enqueue_rows(ids, pos, bt)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 5.0
        code, st = dec.status()
        assert code == -4 and st.device_status == native.DFB_STATUS_PEER_TIMEOUT, (code, st.device_status)
        assert st.detail[0] == 3 and st.detail[1] == 1, list(st.detail)      # exchange kernel id, the missing peer
        code, st = dec.status()
        assert code == 0 and st.device_status == 0                            # read once, cleared
    # the host-buffer step reports the same thing through its return code; an id of the upper vocabulary
    # shard is a valid id on a shard decoder
    with pytest.raises(RuntimeError, match="device status 4"):
        dec.decode_host([g.vocab - 1], [3], [[0]])
    dec.close()

    # the context is intact: an ordinary decoder runs and matches the oracle
    r = H.run_parity_case(layers=2, vocab=2048, prompt_lens=[9, 70], steps=2, seed=62)
    assert r["device_status"] == 0 and r["max_abs_logit_diff"] <= H.LOGIT_ATOL, r
