"""The package's seeded weight generator draws the same tensors as the oracle's
(so benchmark runs and oracle runs with one seed describe one model)."""

import torch

from dfb_b200.geometry import ModelGeometry
from dfb_b200.synthetic import random_init_weights
from dfb_b200.weights import LAYER_FIELDS, rope_cos_sin_table
from oracle import qwen3_decode as O


def test_same_stream_as_oracle():
    og = O.Geometry(layers=2, vocab=512)
    mg = ModelGeometry(layers=2, vocab=512)
    for norm in ("ones", "random"):
        a = O.make_weights(og, seed=5, norm=norm).to(torch.bfloat16)
        b = random_init_weights(mg, seed=5, norm=norm, device="cpu")
        assert torch.equal(a.embed, b.embed) and torch.equal(a.final_norm, b.final_norm)
        for la, lb in zip(a.layers, b.layers):
            for f in LAYER_FIELDS:
                assert torch.equal(getattr(la, f), getattr(lb, f)), f
    assert torch.equal(O.rope_cos_sin_table(og), rope_cos_sin_table(mg))
