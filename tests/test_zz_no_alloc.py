"""The allocation-free LM-head entry point against the regular one.

``dfb_lmhead_argmax_noalloc`` is for callers that cannot allocate device memory
when they need the next token (the engine gave its free memory to the KV cache,
or the caller has no decoder handle).  It keeps its scratch in a fixed array
inside the library, shared by all calls, so this test calls it twice in a row and
compares both results with ``dfb_launch_lmhead_argmax``, which uses a decoder's
allocated scratch.  The file name sorts last so that it is collected last.
"""

import numpy as np
import pytest
import torch

from oracle import qwen3_decode as O
from tests import harness as H

pytestmark = pytest.mark.gpu


def _rand(shape, seed):
    rng = np.random.Generator(np.random.Philox(key=seed))
    return torch.from_numpy(rng.standard_normal(shape, dtype=np.float32)).to(torch.bfloat16)


@pytest.mark.parametrize("rows", [1, 2, 5])
def test_noalloc_matches_regular_entry_point_twice(cuda_device, rows):
    from dfb_b200 import native

    lib = native.lib()
    g = H.oracle_geometry(layers=1, vocab=4096)
    w = O.make_weights(g, seed=31, norm="random").to(torch.bfloat16)
    dec = H.make_decoder(w, O.new_kv_cache(g, 1, torch.bfloat16).cuda())
    embed, fnorm = dec._weights.embed, dec._weights.final_norm
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):          # the second call finds the first call's contents in the shared array
        h, res = _rand((rows, g.hidden), 40 + call).cuda(), _rand((rows, g.hidden), 50 + call).cuda()
        want_tok = torch.zeros(12, dtype=torch.int32, device="cuda")
        want_logits = torch.zeros(rows, g.vocab, dtype=torch.float32, device="cuda")
        native.check(lib.dfb_launch_lmhead_argmax(dec._handle, h.data_ptr(), res.data_ptr(), want_tok.data_ptr(),
                                                  want_logits.data_ptr(), rows, stream), "regular")
        got_tok = torch.full((8,), -1, dtype=torch.int32, device="cuda")
        got_logits = torch.zeros(rows, g.vocab, dtype=torch.float32, device="cuda")
        native.check(lib.dfb_lmhead_argmax_noalloc(embed.data_ptr(), fnorm.data_ptr(), h.data_ptr(), res.data_ptr(),
                                                   rows, g.hidden, g.vocab, g.eps, got_tok.data_ptr(),
                                                   got_logits.data_ptr(), stream), "noalloc")
        torch.cuda.synchronize()
        assert float((got_logits - want_logits).abs().max()) <= H.LOGIT_ATOL
        assert got_tok[:rows].tolist() == want_tok[:rows].tolist()
        # and against the oracle
        ref = O.op_final_norm_lmhead(h.cpu(), res.cpu(), w)
        assert float((got_logits.cpu() - ref.float()).abs().max()) <= 2.0 ** -5
    dec.close()


def test_noalloc_full_vocabulary_and_no_allocation(cuda_device):
    """The real vocabulary (151,936 rows: the 444-CTA grid of the one-row kernel) and a check that the call
    leaves the amount of free device memory exactly as it found it."""
    from dfb_b200 import native

    lib = native.lib()
    g = H.oracle_geometry(layers=1, vocab=151936)
    w = O.make_weights(g, seed=33, norm="random").to(torch.bfloat16)
    embed, fnorm = w.embed.cuda(), w.final_norm.cuda()
    stream = torch.cuda.current_stream().cuda_stream
    for rows in (1, 8):
        h, res = _rand((rows, g.hidden), 70 + rows).cuda(), _rand((rows, g.hidden), 80 + rows).cuda()
        tok = torch.full((8,), -1, dtype=torch.int32, device="cuda")
        logits = torch.zeros(rows, g.vocab, dtype=torch.float32, device="cuda")
        args = (embed.data_ptr(), fnorm.data_ptr(), h.data_ptr(), res.data_ptr(), rows, g.hidden, g.vocab, g.eps,
                tok.data_ptr(), logits.data_ptr(), stream)
        native.check(lib.dfb_lmhead_argmax_noalloc(*args), "noalloc warm-up")   # first call: symbol look-up, module load
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        for _ in range(2):
            native.check(lib.dfb_lmhead_argmax_noalloc(*args), "noalloc")
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before
        ref = O.op_final_norm_lmhead(h.cpu(), res.cpu(), w).float()
        assert float((logits.cpu() - ref).abs().max()) <= 2.0 ** -5
        got = tok[:rows].tolist()
        assert got == logits.argmax(-1).tolist()
        for r in range(rows):
            assert H.token_gap_ok(ref[r], got[r], int(ref[r].argmax()))


def test_noalloc_rejects_sizes_beyond_its_maximum(cuda_device):
    from dfb_b200 import native

    lib = native.lib()
    t = torch.zeros(8, 1024, dtype=torch.bfloat16, device="cuda")
    tok = torch.zeros(8, dtype=torch.int32, device="cuda")
    args = (t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr())
    assert lib.dfb_lmhead_argmax_noalloc(*args, 1, 1024, 262144 + 16, 1e-6, tok.data_ptr(), None, None) == -5
    assert lib.dfb_lmhead_argmax_noalloc(*args, 9, 1024, 4096, 1e-6, tok.data_ptr(), None, None) == -1
    assert lib.dfb_lmhead_argmax_noalloc(*args, 1, 512, 4096, 1e-6, tok.data_ptr(), None, None) == -2
    assert lib.dfb_lmhead_argmax_noalloc(*args, 1, 1024, 4100, 1e-6, tok.data_ptr(), None, None) == -2
    assert b"capacity" in lib.dfb_error_string(-5)
