"""Decode dispatch with the explicit-reason fallback contract.

This is the part of the reference's ``ModelRunner.run`` that chooses between the
megakernel backend and the torch path (engine/model_runner.py:315-376),
restated as a small object so the contract can be driven and tested without a
``ModelRunner``:

* an unsupported decode step falls back to the torch path and records why in
  ``last_fallback_reason``;
* a failure before a decoder exists disables the backend with a
  ``RuntimeWarning`` and falls back;
* a failure after a decoder exists raises and poisons the runner: the shared
  paged KV cache may already have been written, so silently producing tokens
  from the other path would be wrong.
"""

from __future__ import annotations

import warnings
from typing import Callable

from .backend import MegakernelBackend


class DecodeDispatch:
    def __init__(self, config, megakernel: MegakernelBackend | None,
                 prepare_decode: Callable | None = None):
        self.config = config
        self.megakernel = megakernel
        self.prepare_decode = prepare_decode
        self.last_backend_used = "torch"
        self.last_fallback_reason: str | None = None
        self._cuda_poisoned = False

    def run(self, seqs, is_prefill: bool, torch_path: Callable[[list, bool], list[int]]) -> list[int]:
        self.last_backend_used = "torch"
        self.last_fallback_reason = None
        mk = self.megakernel
        if mk is not None and not mk.disabled_reason:
            decision = MegakernelBackend.compatibility(self.config, seqs, is_prefill)
            if not decision.supported and not is_prefill:
                self.last_fallback_reason = decision.reason
            if decision.supported:
                try:
                    if len(seqs) == 1:
                        token_ids = mk.decode(seqs[0], seqs[0].block_table)
                    else:
                        input_ids, positions, block_tables = self.prepare_decode(seqs)
                        token_ids = mk.decode_batch(input_ids, positions, block_tables)
                except Exception as exc:
                    if mk.decoder is not None:
                        self._cuda_poisoned = True
                        raise RuntimeError(
                            "Megakernel decode failed after initialization: "
                            f"{exc}; restart with decode_backend=\"torch\"") from exc
                    mk.disable(str(exc))
                    self.last_fallback_reason = str(exc)
                    warnings.warn(
                        f"Megakernel unavailable; falling back to the standard backend: {exc}",
                        RuntimeWarning, stacklevel=2)
                else:
                    self.last_backend_used = self.config.decode_backend
                    return token_ids
        return torch_path(seqs, is_prefill)
