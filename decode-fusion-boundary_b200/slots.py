"""Fixed-slot decode runtime over the native library (``dfb_slot_*`` / ``dfb_slots_*``).

The reference designed this for its task-graph backend (fixed rows whose
sequences come and go, a token callback after every step:
``backends/megakernel/row_contract.py:1-24``, ``csrc/tg_abi.h:185-199``) and
left it unbuilt; its engine launches exactly the live rows instead.  Here the
slot state lives in the native decoder; this class is the thin host mirror an
engine's scheduler would drive: admit a sequence after its prefill, retire it
at end of sequence, append blocks as it grows.  Scheduling, preemption and
prefill stay with the engine.
"""

from __future__ import annotations

import ctypes as C


class SlotRuntime:
    def __init__(self, decoder):
        from . import native

        self._native = native
        self._lib = native.lib()
        self._dec = decoder                      # a StreamDecoder: owns the handle and the weights
        self.max_slots = native.DFB_MAX_SLOTS
        self._temperatures: dict[int, float] = {}
        self._tokens = (C.c_longlong * self.max_slots)()
        self._emitted = (C.c_int32 * self.max_slots)()

    def _stream(self) -> int:
        return self._dec._stream()

    def admit(self, slot: int, token: int, position: int, block_table, temperature: float = 0.0) -> None:
        """``token`` is the input of the slot's next step (the last prompt token's successor),
        ``position`` the sequence's length before that step, ``block_table`` its physical blocks."""
        table = (C.c_int32 * len(block_table))(*[int(b) for b in block_table])
        self._native.check(self._lib.dfb_slot_set(self._dec._handle, int(slot), 1, int(token), int(position), table,
                                                  len(block_table), float(temperature)), "dfb_slot_set")
        self._temperatures[int(slot)] = float(temperature)

    def extend(self, slot: int, block_table) -> None:
        """A longer block table for a live slot (the scheduler appended a block)."""
        active, token, position = self.state(slot)
        if not active:
            raise ValueError(f"slot {slot} is not live")
        self.admit(slot, token, position, block_table, self._temperatures.get(slot, 0.0))

    def retire(self, slot: int) -> None:
        self._native.check(self._lib.dfb_slot_set(self._dec._handle, int(slot), 0, 0, 0, None, 0, 0.0), "dfb_slot_set")
        self._temperatures.pop(int(slot), None)

    def state(self, slot: int):
        a, t, p = C.c_int32(0), C.c_int64(0), C.c_int64(0)
        self._native.check(self._lib.dfb_slot_get(self._dec._handle, int(slot), C.byref(a), C.byref(t), C.byref(p)),
                           "dfb_slot_get")
        return bool(a.value), int(t.value), int(p.value)

    def step(self) -> dict[int, int]:
        """One decode step of every live slot; ``{slot: token}`` of the slots that emitted."""
        code = self._lib.dfb_slots_step(self._dec._handle, self._tokens, self._emitted, self._stream())
        if code == -4:
            self._dec._raise_device_status()
        self._native.check(code, "dfb_slots_step")
        return {i: int(self._tokens[i]) for i in range(self.max_slots) if self._emitted[i]}

    def run(self, max_steps: int, on_tokens) -> None:
        """Step until ``max_steps``, until nothing emits, or until ``on_tokens({slot: token})`` returns true;
        the callback runs between steps and may admit, extend or retire slots."""
        failure = []

        def trampoline(_context, tokens, emitted, n):
            try:
                return 1 if on_tokens({i: int(tokens[i]) for i in range(n) if emitted[i]}) else 0
            except BaseException as exc:       # never unwind through the C frame
                failure.append(exc)
                return 1

        cb = self._native.TOKEN_CALLBACK(trampoline)
        code = self._lib.dfb_slots_run(self._dec._handle, int(max_steps), cb, None, self._stream())
        if failure:
            raise failure[0]
        if code == -4:
            self._dec._raise_device_status()
        self._native.check(code, "dfb_slots_run")
