"""The plain implementation against logits that the reference's own compiled CPU engine produced
(tests/golden/golden.json, made by tests/golden/make_golden.py from the reference's unmodified sources).
The reference quantizes activations to int8 and rounds to fp16, so agreement is to a few hundredths on
logits of spread one, with the same argmax everywhere; a misread formula is far outside that."""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402
import plain_model  # noqa: E402

TOLERANCE = 0.1          # measured when the file was made: 0.067


def _golden():
    with open(os.path.join(HERE, "golden", "golden.json")) as f:
        return json.load(f)


def test_plain_model_matches_the_reference_engine():
    g = _golden()
    assert g["config"] == make_golden.CFG and g["seed"] == make_golden.SEED and g["tokens"] == make_golden.TOKENS
    ref = np.array(g["reference_logits"])
    plain = plain_model.logits(plain_model.PlainModel(g["config"], make_golden.dequantized()), g["tokens"])
    assert float(np.abs(plain - ref).max()) < TOLERANCE
    assert (plain.argmax(-1) == ref.argmax(-1)).all()


def test_the_comparison_would_catch_a_misread_formula(monkeypatch):
    g = _golden()
    ref = np.array(g["reference_logits"])
    weights = make_golden.dequantized()

    def interleaved_pairs(x, positions, theta):           # the pairing of the other architecture family
        d = x.shape[-1]
        ang = plain_model.rope_angles(positions, d, theta).astype(np.float64)
        c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        out = x.copy()
        out[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s
        out[..., 1::2] = x[..., 0::2] * s + x[..., 1::2] * c
        return out

    monkeypatch.setattr(plain_model, "rope_neox", interleaved_pairs)
    wrong = plain_model.logits(plain_model.PlainModel(g["config"], weights), g["tokens"])
    assert float(np.abs(wrong - ref).max()) > 2 * TOLERANCE
    monkeypatch.undo()
    no_bias = dict(weights)
    for k in list(no_bias):
        if k.endswith("k_proj.bias") or k.endswith("q_proj.bias"):
            no_bias[k] = np.zeros_like(no_bias[k])
    wrong = plain_model.logits(plain_model.PlainModel(g["config"], no_bias), g["tokens"])
    assert float(np.abs(wrong - ref).max()) > 2 * TOLERANCE
