"""Shared by the tests that compare the engine with the plain implementation."""
import os

import numpy as np
import torch

import plain_model
import tiny_configs

# Largest allowed |engine - plain| on logits.  float32: everything is true 32-bit, the
# difference is summation order.  bfloat16: activations, weights and cache are rounded to
# 8 bits of mantissa after every operation; the bounds are relative to the row's spread
# (its root mean square): rel-L2 of the row and its worst entry.  They are twice the largest
# values measured over the whole suite on a B200 (tiny models: rel-L2 0.0072, worst 0.029;
# layers of the benchmark's width, tests/test_wide_gpu.py: 0.032 and 0.13).  FRIDAY_TEST_REPORT=<file>
# writes every measured pair there, so that the bounds can be checked against a new measurement.
FP32_ABS = 2e-5
BF16_TINY = (0.015, 0.06)
BF16_WIDE = (0.065, 0.27)


_report = os.environ.get("FRIDAY_TEST_REPORT")       # a file that receives every measured bfloat16 difference


def bf16_ok(got, ref, what="", limits=BF16_TINY):
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    rms = np.sqrt((ref * ref).mean()) + 1e-12
    rel_l2 = np.sqrt(((got - ref) ** 2).mean()) / rms
    worst = np.abs(got - ref).max() / rms
    if _report:
        with open(_report, "a") as f:
            f.write("%.5f %.5f %s\n" % (rel_l2, worst, what))
    return rel_l2 < limits[0] and worst < limits[1], "rel-L2 %.4f (limit %.3g), worst/rms %.4f (limit %.3g)" % (
        rel_l2, limits[0], worst, limits[1])


def check_logits(got, ref, dtype, what="", bf16_limits=BF16_TINY):
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == np.asarray(ref).shape, "%s: shape %s, plain %s" % (what, got.shape, np.asarray(ref).shape)
    assert np.isfinite(got).all(), "%s: logits are not finite" % what
    if dtype == "float32":
        err = float(np.abs(got - ref).max())
        assert err <= FP32_ABS, "%s: |engine - plain| = %.3g > %.3g" % (what, err, FP32_ABS)
    else:
        ok, text = bf16_ok(got, ref, what, bf16_limits)
        assert ok, "%s: %s" % (what, text)


def bf16_bytes_to_f32(raw):
    return (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bytes(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16                  # round to nearest, ties to even
    return u.astype("<u2").tobytes()


def rewrite(model_dir, change):
    """Rewrites model.safetensors: change(name, float32 array) -> float32 array (or None to keep).  BF16 and F32
    tensors only; other dtypes are copied as they are."""
    from friday_inference_engine_b200.weights import SafetensorsFile, write_safetensors
    path = os.path.join(model_dir, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = []
    for n in f.names():
        dtype, shape = f.dtype_shape(n)
        raw = f.raw(n)
        if dtype in ("BF16", "F32"):
            x = bf16_bytes_to_f32(raw) if dtype == "BF16" else np.frombuffer(raw, dtype="<f4")
            y = change(n, x.reshape(shape).copy())
            if y is not None:
                y = np.asarray(y, dtype=np.float32)
                raw = f32_to_bf16_bytes(y) if dtype == "BF16" else y.astype("<f4").tobytes()
        tensors.append((n, dtype, shape, raw))
    f.close()
    write_safetensors(path, tensors)


def sharpen(model_dir, factor=6.0):
    """Scales the query and key projections so that attention is peaked: with N(0, 0.02)
    weights every softmax is nearly flat and a wrong key would hardly show."""
    def change(n, x):
        if ".q_proj." in n or ".k_proj." in n:
            return x * np.float32(factor)
        if ".embed_tokens." in n:
            return x * np.float32(10.0)
        return None
    rewrite(model_dir, change)


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
