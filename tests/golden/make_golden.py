"""Compares the plain implementation (tests/plain_model.py) with the reference's own model code, once,
on a tiny random model, and writes the small outputs that tests/test_golden.py checks.

The reference (onurtamer/friday-inference-engine) is a C++ program that reads GGUF files with quantized
matrices.  Its CPU backend compiles here without CUDA:

    cmake -S <reference> -B baseline/_ref/build -G Ninja -DFRIDAY_ENABLE_CUDA=OFF -DFRIDAY_BUILD_TESTS=OFF \
          -DCMAKE_BUILD_TYPE=Release && cmake --build baseline/_ref/build

This script (python tests/golden/make_golden.py <reference dir> <build dir>)
  1. draws a tiny Qwen2 model that the reference accepts (it demands head_dim 128 and heads * head_dim ==
     hidden: model_config.cpp:59-60): 2 layers, hidden 256, 2 heads / 1 kv head, intermediate 512,
     vocabulary 64, q/k/v biases, an own head; matrices are quantized to Q8_0 (the reference's CPU path has
     no unquantized product: cpu_kquants.cpp:203-212), norms and biases are F32;
  2. writes it as GGUF with gguf-py, compiles reference_driver.cpp against libfriday_engine.a and runs the
     reference token by token on its CPU backend;
  3. runs the plain implementation on the DEQUANTIZED weights, whole sequence;
  4. writes golden.json: the seed, the tokens, the reference's logits, and the agreement found.

The reference quantizes activations to int8 per 32 values before every product and rounds every
intermediate to fp16 (cpu_backend.h:4-7), which the plain implementation does not; agreement is therefore
to a few hundredths on logits of spread 1 (and equal argmax), not to rounding.  What this pins is the
reading of the formulas: operation order, bias placement, NeoX pairing, grouped heads, SwiGLU, pre-norm
residuals, final norm and head.  Sliding windows, tied heads and head sizes other than 128 cannot run in
the reference; for those the plain implementation rests on the formulas alone.
"""
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_model  # noqa: E402

CFG = {"num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 2, "num_key_value_heads": 1,
       "head_dim": 128, "intermediate_size": 512, "vocab_size": 64, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
       "tie_word_embeddings": False, "max_position_embeddings": 64}
SEED = 1234
TOKENS = [3, 17, 42, 5, 63, 0, 21, 8, 33]


def q8_0(w):
    """Q8_0 of a [rows, k] matrix: per 32 values an fp16 scale d = max|x| / 127 and int8 round(x / d).
    Returns (bytes as uint8 [rows, k/32*34], dequantized float64 [rows, k])."""
    rows, k = w.shape
    blocks = w.reshape(rows, k // 32, 32).astype(np.float32)
    d = (np.abs(blocks).max(axis=-1, keepdims=True) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    q = np.where(df > 0, np.round(blocks / np.where(df > 0, df, 1)), 0).clip(-127, 127).astype(np.int8)
    raw = np.concatenate([d.view(np.uint8).reshape(rows, k // 32, 2), q.view(np.uint8)], axis=-1)
    return raw.reshape(rows, k // 32 * 34), (q.astype(np.float64) * df.astype(np.float64)).reshape(rows, k)


def draw():
    """HF-named float tensors of the tiny model, drawn from SEED (matrices ~ N(0, 0.3/sqrt(k)))."""
    rng = np.random.default_rng(SEED)
    c = CFG
    h, i, v = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    qd, kvd = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    t = {"model.embed_tokens.weight": rng.normal(size=(v, h)), "model.norm.weight": 1 + 0.1 * rng.normal(size=h),
         "lm_head.weight": rng.normal(size=(v, h)) / np.sqrt(h)}
    for l in range(c["num_hidden_layers"]):
        p = "model.layers.%d." % l
        t[p + "input_layernorm.weight"] = 1 + 0.1 * rng.normal(size=h)
        t[p + "post_attention_layernorm.weight"] = 1 + 0.1 * rng.normal(size=h)
        for n, rows in (("q", qd), ("k", kvd), ("v", kvd)):
            t[p + "self_attn.%s_proj.weight" % n] = rng.normal(size=(rows, h)) * 2.0 / np.sqrt(h)
            t[p + "self_attn.%s_proj.bias" % n] = 0.2 * rng.normal(size=rows)
        t[p + "self_attn.o_proj.weight"] = rng.normal(size=(h, qd)) / np.sqrt(qd)
        t[p + "mlp.gate_proj.weight"] = rng.normal(size=(i, h)) / np.sqrt(h)
        t[p + "mlp.up_proj.weight"] = rng.normal(size=(i, h)) / np.sqrt(h)
        t[p + "mlp.down_proj.weight"] = rng.normal(size=(h, i)) / np.sqrt(i)
    return t


GGUF_NAMES = {"input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
              "self_attn.q_proj.weight": "attn_q.weight", "self_attn.q_proj.bias": "attn_q.bias",
              "self_attn.k_proj.weight": "attn_k.weight", "self_attn.k_proj.bias": "attn_k.bias",
              "self_attn.v_proj.weight": "attn_v.weight", "self_attn.v_proj.bias": "attn_v.bias",
              "self_attn.o_proj.weight": "attn_output.weight", "mlp.gate_proj.weight": "ffn_gate.weight",
              "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight"}


def gguf_name(name):
    if name == "model.embed_tokens.weight":
        return "token_embd.weight"
    if name == "model.norm.weight":
        return "output_norm.weight"
    if name == "lm_head.weight":
        return "output.weight"
    _, _, layer, rest = name.split(".", 3)
    return "blk.%s.%s" % (layer, GGUF_NAMES[rest])


def dequantized():
    """What the reference's matrices hold after Q8_0; norms and biases as float32."""
    out = {}
    for name, w in draw().items():
        out[name] = q8_0(w)[1] if w.ndim == 2 else w.astype(np.float32).astype(np.float64)
    return out


def main(reference_dir, build_dir):
    from gguf import GGMLQuantizationType as T, GGUFWriter
    work = os.path.join(build_dir, "golden_work")
    os.makedirs(work, exist_ok=True)
    path = os.path.join(work, "tiny.gguf")
    w = GGUFWriter(path, "qwen2")
    c = CFG
    w.add_string("general.name", "tiny-golden")
    w.add_uint32("qwen2.block_count", c["num_hidden_layers"])
    w.add_uint32("qwen2.embedding_length", c["hidden_size"])
    w.add_uint32("qwen2.attention.head_count", c["num_attention_heads"])
    w.add_uint32("qwen2.attention.head_count_kv", c["num_key_value_heads"])
    w.add_uint32("qwen2.feed_forward_length", c["intermediate_size"])
    w.add_uint32("qwen2.context_length", c["max_position_embeddings"])
    w.add_float32("qwen2.attention.layer_norm_rms_epsilon", c["rms_norm_eps"])
    w.add_float32("qwen2.rope.freq_base", c["rope_theta"])
    for name, t in draw().items():
        if t.ndim == 2:
            w.add_tensor(gguf_name(name), q8_0(t)[0], raw_dtype=T.Q8_0)
        else:
            w.add_tensor(gguf_name(name), t.astype(np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    exe = os.path.join(work, "reference_driver")
    subprocess.run(["g++", "-O2", "-std=c++17", "-DFRIDAY_HAVE_CUDA=0", "-I", reference_dir,
                    "-I", os.path.join(reference_dir, "include"), os.path.join(HERE, "reference_driver.cpp"),
                    os.path.join(build_dir, "libfriday_engine.a"), "-lpthread", "-o", exe], check=True)
    res = subprocess.run([exe, path, "64"] + [str(t) for t in TOKENS], check=True, stdout=subprocess.PIPE, text=True)
    rows = [l for l in res.stdout.splitlines() if l and (l[0].isdigit() or l[0] == "-")]
    ref = np.array([[float(x) for x in l.split()] for l in rows[-len(TOKENS):]])
    assert ref.shape == (len(TOKENS), CFG["vocab_size"]), ref.shape
    plain = plain_model.logits(plain_model.PlainModel(CFG, dequantized()), TOKENS)
    diff = float(np.abs(plain - ref).max())
    rms = float(np.sqrt((ref ** 2).mean()))
    same = bool((plain.argmax(-1) == ref.argmax(-1)).all())
    out = {"config": CFG, "seed": SEED, "tokens": TOKENS, "reference_logits": [[round(float(v), 6) for v in r] for r in ref],
           "max_abs_diff": diff, "reference_rms": rms, "argmax_equal": same,
           "made_with": "reference CPU backend (friday::Engine, BackendKind::Cpu), Q8_0 matrices, one step() per token"}
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(out, f)
    print("max |plain - reference| = %.4f, reference logit rms = %.3f, argmax equal at every position: %s" % (diff, rms, same))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py REFERENCE_SOURCE_TREE [BUILD_DIR]")
    main(sys.argv[1],
         sys.argv[2] if len(sys.argv) > 2 else os.path.join(os.path.dirname(os.path.dirname(HERE)), "baseline", "_ref", "build"))
