"""Configuration, registry, safetensors, loader errors, sharded folders, random-weights mode (no GPU).
Everything asked here is answered by the library (config/*.cpp, weights/*.cpp) through its C interface."""
import json
import os

import numpy as np
import pytest
import torch

import harness
import plain_model
import tiny_configs
from friday_inference_engine_b200 import (ConfigError, WeightsError, check_weights, describe_model, read_config,
                                          registered_architectures, registered_parts)
from friday_inference_engine_b200.weights import SafetensorsFile, random_tensor, storage_plan, write_safetensors

BASE = {"architectures": ["Qwen2ForCausalLM"], "vocab_size": 100, "hidden_size": 64, "intermediate_size": 128,
        "num_hidden_layers": 2, "num_attention_heads": 4, "max_position_embeddings": 64, "rms_norm_eps": 1e-6}


def windows(cfg):
    d = describe_model(cfg)
    return [d["cache_requests"][str(c["cache"])]["window"] or None for c in d["program"]]


def test_defaults_follow_the_reference():
    c = read_config(BASE)
    assert c["num_key_value_heads"] == 4          # defaults to the head count
    assert c["head_dim"] == 16                    # hidden / heads
    assert c["rope_theta"] == 10000.0
    assert c["tie_word_embeddings"] is False and c["use_sliding_window"] is False
    assert c["max_window_layers"] == 2            # no window: no layer is below the limit
    assert windows(BASE) == [None, None]


def test_every_key_is_read_from_config():
    for cfg, _ in tiny_configs.CONFIGS.values():
        c = read_config(cfg)
        assert c["architectures"] == ["Qwen2ForCausalLM"]
        for k, v in cfg.items():
            if k in ("architectures", "model_type"):
                continue
            if k == "max_window_layers" and not cfg.get("use_sliding_window"):
                continue
            assert c[k] == v, k
        assert read_config(c) == c                 # the typed configuration reads back as itself


@pytest.mark.parametrize("change, word", [
    ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"rope_theta": 1.0}, "rope_theta"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"head_dim": 15}, "head_dim"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"use_sliding_window": True, "sliding_window": 16}, "max_window_layers"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}}, "rope_scaling"),
    ({"rope_scaling": {"rope_type": "linear", "factor": 2.0}}, "rope_scaling"),
])
def test_bad_config_names_the_key(change, word):
    d = dict(tiny_configs.TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k, None)
        else:
            d[k] = v
    with pytest.raises(ConfigError) as e:
        read_config(d)
    assert word in str(e.value)


def test_a_null_rope_scaling_is_no_scaling():
    assert read_config(dict(tiny_configs.TINY_A, rope_scaling=None))["rope_theta"] == 10000.0


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError) as e:
        read_config({"architectures": ["LlamaForCausalLM"]})
    assert "LlamaForCausalLM" in str(e.value) and registered_architectures()[0] in str(e.value)
    with pytest.raises(ConfigError):
        read_config({"model_type": "qwen2"})


def test_window_layers():
    assert windows(tiny_configs.TINY_C) == [None, None, 80, 80]
    assert windows(tiny_configs.TINY_B) == [24, 24, 24]
    assert windows(tiny_configs.TINY_A) == [None, None]


def test_shipped_parts_are_registered():
    assert registered_parts("norm") == ["rmsnorm"] and "gqa_attention" in registered_parts("mixer")
    assert set(registered_parts("position")) >= {"rotary_neox", "none"}
    assert registered_parts("feed_forward") == ["swiglu"] and registered_parts("block") == ["prenorm"]
    with pytest.raises(ConfigError):
        registered_parts("decoder")


NP = {"BF16": None, "F32": "<f4", "I64": "<i8", "F16": "<f2"}


def raw_of(t):
    return t.contiguous().view(torch.uint8).numpy().tobytes() if t.numel() else b""


NAMES = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int64: "I64", torch.float16: "F16"}


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2), "e": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, [(n, NAMES[v.dtype], tuple(v.shape), raw_of(v)) for n, v in t.items()], metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
    for n in t:
        assert f.dtype_shape(n) == (NAMES[t[n].dtype], tuple(t[n].shape))
        assert f.raw(n) == raw_of(t[n])
    # the installed safetensors package reads what we wrote, and we read what it writes
    from safetensors.torch import load_file, save_file
    theirs = load_file(p)
    assert all(torch.equal(theirs[n], t[n]) for n in t)
    q = str(tmp_path / "y.safetensors")
    save_file({k: v for k, v in t.items()}, q)
    g = SafetensorsFile(q)
    assert all(g.raw(n) == raw_of(t[n]) for n in t)


def folder(tmp_path, cfg=tiny_configs.TINY_A, seed=0, name="m"):
    return tiny_configs.make_model_dir(str(tmp_path / name), cfg, seed)


def edit(model_dir, drop=(), add=()):
    """Rewrites model.safetensors without the tensors `drop` and with the tensors `add` (name, dtype, shape, bytes)."""
    path = os.path.join(model_dir, "model.safetensors")
    f = SafetensorsFile(path)
    added = {a[0] for a in add}
    tensors = [(n,) + f.dtype_shape(n) + (f.raw(n),) for n in f.names() if n not in drop and n not in added]
    f.close()
    write_safetensors(path, tensors + list(add))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = folder(tmp_path)
    edit(d, drop=["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"],
         add=[("model.layers.0.mlp.up_proj.weight", "BF16", (5, 64), bytes(5 * 64 * 2)),
              ("model.layers.7.extra.weight", "F32", (1,), bytes(4))])
    with pytest.raises(WeightsError) as e:
        check_weights(d)
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.mlp.up_proj.weight", (5, 64), (176, 64))]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "k_proj.bias", "extra.weight", "[176, 64]"):
        assert word in text


def test_tied_head_ignores_a_stored_copy_and_untied_needs_one(tmp_path):
    d = folder(tmp_path)                                  # tied
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    assert "lm_head.weight" not in f.names()
    table = ("lm_head.weight",) + f.dtype_shape("model.embed_tokens.weight") + (f.raw("model.embed_tokens.weight"),)
    f.close()
    edit(d, add=[table])
    check_weights(d)                                      # a tied checkpoint may still carry a copy of the table
    assert "lm_head.weight" not in [s["name"] for s in storage_plan(d)]
    b = folder(tmp_path, tiny_configs.TINY_B, 1, "b")     # own head
    edit(b, drop=["lm_head.weight"])
    with pytest.raises(WeightsError) as e:
        check_weights(b)
    assert e.value.missing == ["lm_head.weight"]


def test_storage_rule(tmp_path):
    """bfloat16 unless the file stores 32 bits; a stacked tensor is promoted as a whole; float32 engines keep float32."""
    d = folder(tmp_path)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    wide = []
    for n in ("model.norm.weight", "model.layers.0.self_attn.q_proj.bias"):
        x = harness.bf16_bytes_to_f32(f.raw(n))
        wide.append((n, "F32", f.dtype_shape(n)[1], x.astype("<f4").tobytes()))
    n16 = "model.layers.1.mlp.down_proj.weight"
    x = harness.bf16_bytes_to_f32(f.raw(n16))
    wide.append((n16, "F16", f.dtype_shape(n16)[1], x.astype("<f2").tobytes()))
    f.close()
    edit(d, add=wide)
    plan = {s["name"]: s for s in storage_plan(d, "bfloat16")}
    assert plan["model.norm.weight"]["dtype"] == "float32"                      # stored in 32-bit: stays so
    assert plan["model.layers.0.self_attn.q_proj.bias"]["dtype"] == "float32"
    assert plan["model.layers.0.self_attn.k_proj.bias"] == {"name": "model.layers.0.self_attn.k_proj.bias",
                                                            "dtype": "float32", "into": "b_qkv"}   # promoted as a whole
    assert plan["model.layers.1.self_attn.k_proj.bias"]["dtype"] == "bfloat16"
    assert plan[n16]["dtype"] == "bfloat16" and plan["model.embed_tokens.weight"]["dtype"] == "bfloat16"
    assert plan["model.layers.0.mlp.gate_proj.weight"]["into"] == "w_gate_up"
    assert all(s["dtype"] == "float32" for s in storage_plan(d, "float32"))
    edit(d, add=[("model.norm.weight", "I64", (64,), bytes(64 * 8))])
    with pytest.raises(WeightsError) as e:
        storage_plan(d)
    assert "integer" in str(e.value)


def test_sharded_folder_reads_as_the_single_file(tmp_path):
    cfg, seed = tiny_configs.CONFIGS["B"]
    one = tiny_configs.make_model_dir(str(tmp_path / "one"), cfg, seed)
    three = tiny_configs.make_model_dir(str(tmp_path / "three"), cfg, seed, shards=3)
    files = sorted(os.listdir(three))
    assert files == ["config.json", "model-00001-of-00003.safetensors", "model-00002-of-00003.safetensors",
                     "model-00003-of-00003.safetensors", "model.safetensors.index.json"]
    check_weights(three)
    assert storage_plan(three) == storage_plan(one)
    whole = SafetensorsFile(os.path.join(one, "model.safetensors"))
    with open(os.path.join(three, "model.safetensors.index.json")) as f:
        index = json.load(f)["weight_map"]
    assert set(index) == set(whole.names()) and len(set(index.values())) == 3
    for n, shard in index.items():
        assert SafetensorsFile(os.path.join(three, shard)).raw(n) == whole.raw(n)
    # a tensor that the index lists but its shard lacks is reported with the rest, in the one error
    victim = "model.layers.1.mlp.up_proj.weight"
    path = os.path.join(three, index[victim])
    f = SafetensorsFile(path)
    keep = [(n,) + f.dtype_shape(n) + (f.raw(n),) for n in f.names() if n != victim]
    f.close()
    write_safetensors(path, keep)
    with pytest.raises(WeightsError) as e:
        check_weights(three)
    assert e.value.missing == [victim] and "absent from their shard" in str(e.value)
    os.remove(os.path.join(three, "model-00002-of-00003.safetensors"))
    with pytest.raises(WeightsError) as e:
        check_weights(three)
    assert "model-00002-of-00003.safetensors" in str(e.value)
    for name in os.listdir(three):
        if name != "config.json":
            os.remove(os.path.join(three, name))
    with pytest.raises(WeightsError) as e:
        check_weights(three)                              # no weights at all
    assert "model.safetensors" in str(e.value)


def test_random_mode_writes_a_folder_and_is_reproducible(tmp_path):
    cfg, seed = tiny_configs.CONFIGS["B"]
    a = tiny_configs.make_model_dir(str(tmp_path / "a"), cfg, seed)
    b = tiny_configs.make_model_dir(str(tmp_path / "b"), cfg, seed)
    c = tiny_configs.make_model_dir(str(tmp_path / "c"), cfg, seed + 1)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    with open(os.path.join(a, "config.json")) as f:
        assert json.load(f)["sliding_window"] == 24
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert set(fa.names()) == set(fb.names()) and "lm_head.weight" in fa.names()
    for n in fa.names():
        assert fa.raw(n) == fb.raw(n)
        assert fa.dtype_shape(n)[0] == "BF16"
    assert fa.raw("lm_head.weight") != fc.raw("lm_head.weight")
    w = harness.bf16_bytes_to_f32(fa.raw("model.layers.0.mlp.down_proj.weight"))
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    nw = harness.bf16_bytes_to_f32(fa.raw("model.norm.weight"))
    assert abs(float(nw.mean()) - 1.0) < 0.02
    # any tensor can be drawn alone and is the same
    name = "model.layers.2.self_attn.v_proj.bias"
    alone = random_tensor(seed, name, 32)
    assert harness.f32_to_bf16_bytes(alone) == fa.raw(name)
    # the plain implementation reads the folder
    pm = plain_model.PlainModel.from_dir(a)
    assert pm.vocab == 1000
    # and a float32 folder holds the numbers before the rounding
    d32 = tiny_configs.make_model_dir(str(tmp_path / "d"), cfg, seed, dtype="F32")
    f32 = SafetensorsFile(os.path.join(d32, "model.safetensors"))
    assert np.array_equal(np.frombuffer(f32.raw(name), dtype="<f4"), alone)
