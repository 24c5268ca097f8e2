"""CPU oracle for the Qwen3 greedy decode step.

TEST INFRASTRUCTURE ONLY. Nothing under this directory is part of the shipped
decode backend: it is imported by the test-suite, by the smoke check and by the
CPU-baseline / reference legs of the benchmark, where it plays the role of the
checker (or of the thing the GPU path is compared with), never of the product.
The CUDA backend never imports it and has no CPU fallback.

Parity status: PINNED. ``oracle.qwen3_decode`` is checked against outputs of the
reference project's own torch model (imported unmodified, with only its
FlashAttention/Triton ``Attention.forward`` swapped for a CPU restatement) that
are committed as fixtures under ``tests/golden/`` together with the script that
generated them (``tests/golden/make_golden.py``).
"""
