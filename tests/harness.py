"""Shared by the tests that compare the engine with the plain implementation."""
import os

import numpy as np
import torch

import plain_model
import tiny_configs

# Largest allowed |engine - plain| on logits.  float32: everything is true 32-bit, the
# difference is summation order.  bfloat16: activations, weights and cache are rounded to
# 8 bits of mantissa after every operation; the bound is relative to the row's spread.
FP32_ABS = 2e-5


def bf16_ok(got, ref):
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    rms = np.sqrt((ref * ref).mean()) + 1e-12
    rel_l2 = np.sqrt(((got - ref) ** 2).mean()) / rms
    worst = np.abs(got - ref).max() / rms
    return rel_l2 < 0.03 and worst < 0.15, "rel-L2 %.4f (limit 0.03), worst/rms %.4f (limit 0.15)" % (rel_l2, worst)


def check_logits(got, ref, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == np.asarray(ref).shape, "%s: shape %s, plain %s" % (what, got.shape, np.asarray(ref).shape)
    assert np.isfinite(got).all(), "%s: logits are not finite" % what
    if dtype == "float32":
        err = float(np.abs(got - ref).max())
        assert err <= FP32_ABS, "%s: |engine - plain| = %.3g > %.3g" % (what, err, FP32_ABS)
    else:
        ok, text = bf16_ok(got, ref)
        assert ok, "%s: %s" % (what, text)


def sharpen(model_dir, factor=6.0):
    """Scales the query and key projections so that attention is peaked: with N(0, 0.02)
    weights every softmax is nearly flat and a wrong key would hardly show."""
    from friday_inference_engine_b200.weights import SafetensorsFile, write_safetensors
    path = os.path.join(model_dir, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {}
    for n in f.names():
        t = f.tensor(n).clone()
        if ".q_proj." in n or ".k_proj." in n:
            t = (t.float() * factor).to(t.dtype)
        if ".embed_tokens." in n:
            t = (t.float() * 10.0).to(t.dtype)
        tensors[n] = t
    f.close()
    write_safetensors(path, tensors)


_made = {}


def model_dir(tmp_root, name, sharp=True):
    key = (str(tmp_root), name, sharp)
    if key not in _made:
        cfg, seed = tiny_configs.CONFIGS[name]
        d = tiny_configs.make_model_dir(os.path.join(str(tmp_root), "model_%s_%d" % (name, sharp)), cfg, seed)
        if sharp:
            sharpen(d)
        _made[key] = (d, plain_model.PlainModel.from_dir(d))
    return _made[key]


def to_np(t):
    return t.detach().double().cpu().numpy()
