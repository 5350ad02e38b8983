"""Configuration, registry, safetensors, loader errors, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

import tiny_configs
from friday_inference_engine_b200.config import ConfigError, Qwen2Config
from friday_inference_engine_b200.engine.model import DecoderModel
from friday_inference_engine_b200.registry import read_config, registered
from friday_inference_engine_b200.weights import (RandomSource, SafetensorsFile, WeightsError, expected_params,
                                                  load_weights, storage_dtype, write_safetensors)


def test_defaults_follow_the_reference():
    d = {"architectures": ["Qwen2ForCausalLM"], "vocab_size": 100, "hidden_size": 64, "intermediate_size": 128,
         "num_hidden_layers": 2, "num_attention_heads": 4, "max_position_embeddings": 64, "rms_norm_eps": 1e-6}
    c = Qwen2Config.from_dict(d)
    assert c.num_key_value_heads == 4          # defaults to the head count
    assert c.head_dim == 16                    # hidden / heads
    assert c.rope_theta == 10000.0
    assert c.tie_word_embeddings is False and c.use_sliding_window is False
    assert c.window_of(0) is None


def test_every_key_is_read_from_config():
    for cfg, _ in tiny_configs.CONFIGS.values():
        arch, c = read_config(cfg)
        assert arch.name == "Qwen2ForCausalLM"
        for k, v in cfg.items():
            if k in ("architectures", "model_type"):
                continue
            assert getattr(c, k) == v, k
        back = Qwen2Config.from_dict(c.to_dict())
        assert back == c


@pytest.mark.parametrize("change, word", [
    ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"rope_theta": 1.0}, "rope_theta"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"head_dim": 15}, "head_dim"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"hidden_act": "gelu"}, "hidden_act"),
])
def test_bad_config_names_the_key(change, word):
    d = dict(tiny_configs.TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k, None)
        else:
            d[k] = v
    with pytest.raises(ConfigError) as e:
        Qwen2Config.from_dict(d)
    assert word in str(e.value)


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError) as e:
        read_config({"architectures": ["LlamaForCausalLM"]})
    assert "LlamaForCausalLM" in str(e.value) and registered()[0] in str(e.value)
    with pytest.raises(ConfigError):
        read_config({"model_type": "qwen2"})


def test_window_layers():
    c = Qwen2Config.from_dict(tiny_configs.TINY_C)
    assert [c.window_of(l) for l in range(4)] == [None, None, 80, 80]


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2), "e": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
    for n in t:
        assert f.dtype_shape(n) == (t[n].dtype, tuple(t[n].shape))
        assert torch.equal(f.tensor(n), t[n])
    # the installed safetensors package reads what we wrote, and we read what it writes
    from safetensors.torch import load_file, save_file
    theirs = load_file(p)
    assert all(torch.equal(theirs[n], t[n]) for n in t)
    q = str(tmp_path / "y.safetensors")
    save_file({k: v for k, v in t.items()}, q)
    g = SafetensorsFile(q)
    assert all(torch.equal(g.tensor(n), t[n]) for n in t)


def _model(cfg=tiny_configs.TINY_A, dtype=torch.bfloat16):
    arch, c = read_config(cfg)
    return DecoderModel(arch.build_spec(c), dtype, torch.device("cpu"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    m = _model()
    src = RandomSource(expected_params(m), 0)
    tensors = {n: src.tensor(n) for n in src.names()}
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.up_proj.weight"] = torch.zeros(5, 64, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.zeros(1)
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, tensors)
    with pytest.raises(WeightsError) as e:
        load_weights(m, SafetensorsFile(p))
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.mlp.up_proj.weight", (5, 64), (176, 64))]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "k_proj.bias", "extra.weight", "[176, 64]"):
        assert word in text


def test_tied_head_ignores_a_stored_copy_and_untied_needs_one(tmp_path):
    m = _model(tiny_configs.TINY_A)                       # tied
    src = RandomSource(expected_params(m), 0)
    tensors = {n: src.tensor(n) for n in src.names()}
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, tensors)
    load_weights(m, SafetensorsFile(p))
    assert m.head is m.embedding
    mb = _model(tiny_configs.TINY_B)                      # own head
    srcb = RandomSource(expected_params(mb), 0)
    tb = {n: srcb.tensor(n) for n in srcb.names() if n != "lm_head.weight"}
    pb = str(tmp_path / "b.safetensors")
    write_safetensors(pb, tb)
    with pytest.raises(WeightsError) as e:
        load_weights(mb, SafetensorsFile(pb))
    assert e.value.missing == ["lm_head.weight"]


def test_storage_rule():
    bf, f32, f16 = torch.bfloat16, torch.float32, torch.float16
    assert storage_dtype(bf, "float", bf) == bf
    assert storage_dtype(f16, "float", bf) == bf
    assert storage_dtype(f32, "float", bf) == f32          # stored in 32-bit: stays so
    assert storage_dtype(bf, "float", f32) == f32
    assert storage_dtype(torch.int64, "int", bf) == torch.int32
    with pytest.raises(WeightsError):
        storage_dtype(torch.int64, "float", bf)


def test_fp32_stored_tensors_stay_fp32_in_bf16_mode(tmp_path):
    m = _model(tiny_configs.TINY_A, torch.bfloat16)
    src = RandomSource(expected_params(m), 0)
    tensors = {n: src.tensor(n) for n in src.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    tensors["model.layers.0.self_attn.q_proj.bias"] = tensors["model.layers.0.self_attn.q_proj.bias"].float()
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, tensors)
    load_weights(m, SafetensorsFile(p))
    assert m.final_norm.tensors["weight"].dtype == torch.float32
    assert m.layers[0].mixer.b_qkv.dtype == torch.float32      # the stacked bias is promoted as a whole
    assert m.layers[1].mixer.b_qkv.dtype == torch.bfloat16
    assert m.embedding.dtype == torch.bfloat16


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
        assert torch.equal(fa.tensor(n), fb.tensor(n))
        assert fa.dtype_shape(n)[0] == torch.bfloat16
    assert not torch.equal(fa.tensor("lm_head.weight"), fc.tensor("lm_head.weight"))
    w = fa.tensor("model.layers.0.mlp.down_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    nw = fa.tensor("model.norm.weight").float()
    assert abs(float(nw.mean()) - 1.0) < 0.02
    # any tensor can be drawn alone and is the same
    m = _model(cfg)
    alone = RandomSource(expected_params(m), seed).tensor("model.layers.2.self_attn.v_proj.bias")
    assert torch.equal(alone, fa.tensor("model.layers.2.self_attn.v_proj.bias"))
