"""The plain implementation against logits that the reference's own compiled CPU engine produced
(tests/golden/golden.json, made by tests/golden/make_golden.py from the reference's unmodified sources).
The reference quantizes activations to int8 and rounds to fp16, so agreement is to a few hundredths on
logits of spread one, with the same argmax everywhere; a misread formula is far outside that."""
import json
import os
import sys

import numpy as np
import pytest

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


# ---------------------------------------------------------------------------------------
# Each operation alone against the reference's own host function (tests/golden/ops_golden.json,
# made by tests/golden/make_ops_golden.py from friday_cpu::rmsNorm, rope, decodeAttention, siluMul and
# addResidual: cpu_ops.h:12-28) at the tiny models' sizes.  The reference rounds outputs to fp16.
# ---------------------------------------------------------------------------------------

class Draws:
    """The input generator of tests/golden/ops_driver.cpp, repeated (float32 arithmetic as there)."""

    def __init__(self, seed):
        self.state = seed

    def take(self, n, scale):
        out = np.empty(n, dtype=np.float32)
        for i in range(n):
            self.state = (1103515245 * self.state + 12345) & 0x7FFFFFFF
            out[i] = (np.float32(self.state) / np.float32(2147483648.0) * np.float32(2.0) - np.float32(1.0)) * np.float32(scale)
        return out.astype(np.float64)


SHAPES = [("A", 64, 4, 2, 16, 176, 10000.0, 1e-6), ("B", 96, 3, 1, 32, 256, 1000000.0, 1e-5)]
OPS_RTOL = 2e-3          # fp16 outputs: 2^-11 relative, and the angle's fp32 rounding at position 200


def ops_cases(wrong=None):
    """(key, the plain implementation's result) for every entry of ops_golden.json; `wrong` names one
    operation to compute with a misread formula (the negative controls)."""
    for s, (name, width, heads, kv_heads, hd, inner, theta, eps) in enumerate(SHAPES):
        d = Draws(1000 + s)
        x, w = d.take(width, 3.0), d.take(width, 1.0)
        yield "%s.rms_norm" % name, plain_model.rms_norm(x[None], w, eps if wrong != "rms_norm" else 1.0)[0]
        for pos in (0, 1, 63, 200):
            q, k = d.take(heads * hd, 1.0).reshape(1, heads, hd), d.take(kv_heads * hd, 1.0).reshape(1, kv_heads, hd)
            p = [pos if wrong != "rope" else pos + 1]
            yield "%s.rope.%d" % (name, pos), np.concatenate([plain_model.rope_neox(q, p, theta).reshape(-1),
                                                              plain_model.rope_neox(k, p, theta).reshape(-1)])
        for seq in (1, 37, 200):
            q = d.take(heads * hd, 2.0).reshape(heads, hd)
            kc, vc = d.take(seq * kv_heads * hd, 1.0).reshape(seq, kv_heads, hd), d.take(seq * kv_heads * hd, 1.0).reshape(seq, kv_heads, hd)
            if wrong == "attention":
                q = q[::-1]                                   # heads on the wrong kv heads
            qs = np.zeros((seq, heads, hd))
            qs[-1] = q
            yield "%s.attention.%d" % (name, seq), plain_model.attention(qs, kc, vc)[-1].reshape(-1)
        gate, up = d.take(inner, 6.0), d.take(inner, 2.0)
        yield "%s.swiglu" % name, plain_model.swiglu(gate if wrong != "swiglu" else up, up if wrong != "swiglu" else gate)
        x, a = d.take(width, 2.0), d.take(width, 2.0)
        yield "%s.residual" % name, x + a


def _ops_golden():
    with open(os.path.join(HERE, "golden", "ops_golden.json")) as f:
        return {k: np.array(v) for k, v in json.load(f).items()}


def _off(got, ref):
    return float(np.abs(got - ref).max() / (np.abs(ref).max() + 1e-9))


def test_each_plain_function_matches_the_references_own():
    gold = _ops_golden()
    seen = 0
    for key, got in ops_cases():
        assert got.shape == gold[key].shape, key
        assert _off(got, gold[key]) <= OPS_RTOL, "%s: off by %.3g of the largest entry" % (key, _off(got, gold[key]))
        seen += 1
    assert seen == len(gold) == 20


@pytest.mark.parametrize("op", ["rms_norm", "rope", "attention", "swiglu"])
def test_a_misread_operation_would_be_caught(op):
    gold = _ops_golden()
    worst = max(_off(got, gold[key]) for key, got in ops_cases(wrong=op) if "." + op in key and ".rope.0" not in key)
    assert worst > 20 * OPS_RTOL
