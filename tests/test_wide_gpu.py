"""The engine at the layer sizes of the benchmark model (width 3584, 28 heads in 4 groups of head size
128, inner width 18944) with two layers and a smaller vocabulary, against the plain implementation:
the tiny test models never reach these tile counts, split-k ranges or head sizes."""
import numpy as np
import pytest
import torch

import harness
import plain_model

# In 32-bit the bound is the one the task states for the full-size models: |engine - plain| <= 1e-4 on the logits
# (sums over 18,944 terms in another order than the plain implementation's float64 move the last bits; the tiny
# models' tighter bound of 2e-5 is not meant for these sizes).
WIDE_FP32_ABS = 1e-4
import tiny_configs
from friday_inference_engine_b200 import Engine

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 2, "hidden_size": 3584,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944,
    "vocab_size": 5000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "use_sliding_window": False, "max_position_embeddings": 4096, "torch_dtype": "bfloat16",
}


# The layer sizes of the two larger models of the family (14B: 40 heads in 8 groups, width 5120, inner width 13824;
# 32B: the same heads and width, inner width 27648), one layer each, their norms' eps.
WIDER = dict(WIDE, num_hidden_layers=1, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
             intermediate_size=27648, rms_norm_eps=1e-5, vocab_size=3000)
WIDER_14B = dict(WIDER, intermediate_size=13824)


@pytest.mark.parametrize("config", [WIDER, WIDER_14B], ids=["32b_layer", "14b_layer"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_sizes_of_the_larger_models(config, dtype, tmp_path):
    """A prompt pass of unequal prompts and a one-token step at these sizes against the plain implementation."""
    d = str(tmp_path / "model")
    tiny_configs.make_model_dir(d, config, 11)
    harness.sharpen(d, 2.0)
    pm = plain_model.PlainModel.from_dir(d)
    eng = Engine(model_path=d, dtype=dtype, max_ctx=512, max_batch=2)
    lens = [150, 33]
    prompts = tiny_configs.random_prompts([n + 1 for n in lens], config["vocab_size"], 62)
    refs = [plain_model.logits(pm, p, at=[n - 1, n]) for p, n in zip(prompts, lens)]
    slots = [eng.alloc_slot() for _ in prompts]

    def check(got_rows, ref_rows, what):
        if dtype == "float32":
            err = float(np.abs(got_rows - ref_rows).max())
            assert err <= WIDE_FP32_ABS, "%s: |engine - plain| = %.3g > %.3g" % (what, err, WIDE_FP32_ABS)
        else:
            harness.check_logits(got_rows, ref_rows, dtype, what, harness.BF16_WIDE)

    got = eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[n - 1] for n in lens])
    for i in range(2):
        check(harness.to_np(got[i:i + 1]), refs[i][0:1], "prompt %d" % i)
    got = eng.step(slots, [[p[n]] for p, n in zip(prompts, lens)], [[0]] * 2)
    for i in range(2):
        check(harness.to_np(got[i:i + 1]), refs[i][1:2], "first token after prompt %d" % i)
    eng.check()


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("wide") / "model")
    tiny_configs.make_model_dir(d, WIDE, 9)
    harness.sharpen(d, 2.0)
    return d, plain_model.PlainModel.from_dir(d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_layers_prompt_then_tokens(wide, dtype):
    d, pm = wide
    eng = Engine(model_path=d, dtype=dtype, max_ctx=512, max_batch=3)
    lens, extra = [70, 9, 130], 3
    prompts = tiny_configs.random_prompts([n + extra for n in lens], WIDE["vocab_size"], 60)
    at = [[n - 1, n, n + extra - 1] for n in lens]
    refs = [plain_model.logits(pm, p, at=a) for p, a in zip(prompts, at)]
    slots = [eng.alloc_slot() for _ in prompts]
    got = eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[n - 1] for n in lens])
    def check(got_rows, ref_rows, what):
        if dtype == "float32":
            err = float(np.abs(got_rows - ref_rows).max())
            assert err <= WIDE_FP32_ABS, "%s: |engine - plain| = %.3g > %.3g" % (what, err, WIDE_FP32_ABS)
        else:
            harness.check_logits(got_rows, ref_rows, dtype, what, harness.BF16_WIDE)

    for i in range(3):
        check(harness.to_np(got[i:i + 1]), refs[i][0:1], "wide prompt %d" % i)
    for t in range(extra):
        got = eng.step(slots, [[p[n + t]] for p, n in zip(prompts, lens)], [[0]] * 3)
        if t in (0, extra - 1):
            for i in range(3):
                check(harness.to_np(got[i:i + 1]), refs[i][1 if t == 0 else 2][None], "wide decode %d of request %d" % (t, i))
    eng.check()


def test_wide_layers_device_decoder(wide):
    d, pm = wide
    eng = Engine(model_path=d, dtype="bfloat16", max_ctx=512, max_batch=2)
    lens, extra = [100, 61], 6
    prompts = tiny_configs.random_prompts([n + extra for n in lens], WIDE["vocab_size"], 61)
    refs = [plain_model.logits(pm, p, at=[len(p) - 1]) for p in prompts]
    slots = [eng.alloc_slot() for _ in prompts]
    eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[]] * 2)
    dec = eng.decoder(slots, [p[n] for p, n in zip(prompts, lens)])
    for t in range(extra):
        dec.step([p[n + t] for p, n in zip(prompts, lens)])
    got = harness.to_np(dec.logits)
    for i in range(2):
        harness.check_logits(got[i:i + 1], refs[i], "bfloat16", "wide decoder row %d" % i, harness.BF16_WIDE)
    dec.close()
    eng.check()


@pytest.mark.parametrize("rows", [17, 64, 100])
def test_wide_layers_decoder_of_many_rows(tmp_path, rows):
    """The benchmark's batch-64 step at its layer sizes (one layer): 32- and 64-row tiles with split k where all CTAs
    of a tile finish 16 rows each, the norm in the epilogues beside the rotary kernel, attention over 64 x 4 CTAs; and
    100 rows, whose 128-wide tiles go through the 16-row window."""
    cfg = dict(WIDE, num_hidden_layers=1, vocab_size=3000)
    d = tiny_configs.make_model_dir(str(tmp_path / "model"), cfg, 12)
    harness.sharpen(d, 2.0)
    pm = plain_model.PlainModel.from_dir(d)
    eng = Engine(model_path=d, dtype="bfloat16", max_ctx=128, max_batch=rows)
    steps = 4
    lens = [1 + (5 * i) % 23 for i in range(rows)]
    prompts = tiny_configs.random_prompts([n + steps for n in lens], cfg["vocab_size"], 63)
    refs = [plain_model.logits(pm, p, at=[n, n + steps - 1]) for p, n in zip(prompts, lens)]
    slots = [eng.alloc_slot() for _ in prompts]
    eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[]] * rows)
    dec = eng.decoder(slots, [p[n] for p, n in zip(prompts, lens)])
    live = [True] * rows
    for t in range(steps):
        dec.step([p[n + t] if live[i] else 0 for i, (p, n) in enumerate(zip(prompts, lens))])
        if t in (0, steps - 1):
            got = harness.to_np(dec.logits)
            for i in range(rows):
                if live[i]:
                    harness.check_logits(got[i:i + 1], refs[i][0 if t == 0 else 1][None], "bfloat16",
                                         "%d wide rows: row %d step %d" % (rows, i, t), harness.BF16_WIDE)
        if t == 1:
            for i in range(1, rows, 4):
                live[i] = False
                dec.retire(i)
                eng.free_slot(slots[i])
    dec.close()
    eng.check()


FULL_VOCABULARY = dict(WIDE, num_hidden_layers=1, vocab_size=152064, tie_word_embeddings=True, intermediate_size=2048)


@pytest.fixture(scope="module")
def full_vocabulary(tmp_path_factory):
    d = tiny_configs.make_model_dir(str(tmp_path_factory.mktemp("vocab") / "model"), FULL_VOCABULARY, 13)
    return d, plain_model.PlainModel.from_dir(d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_full_vocabulary(full_vocabulary, dtype):
    """One layer of the benchmark's width with its whole vocabulary of 152,064 (the head tied to the token table, so that
    the plain implementation holds the table once): the widest product of the model inside the engine."""
    cfg = FULL_VOCABULARY
    d, pm = full_vocabulary
    eng = Engine(model_path=d, dtype=dtype, max_ctx=64, max_batch=2)
    prompts = tiny_configs.random_prompts([12, 5], cfg["vocab_size"], 64)
    refs = [plain_model.logits(pm, p, at=[len(p) - 2, len(p) - 1]) for p in prompts]
    slots = [eng.alloc_slot() for _ in prompts]
    got = harness.to_np(eng.step(slots, [p[:-1] for p in prompts], [[len(p) - 2] for p in prompts]))
    more = harness.to_np(eng.step(slots, [[p[-1]] for p in prompts], [[0], [0]]))
    for i in range(2):
        for rows, ref, what in ((got[i:i + 1], refs[i][0:1], "prompt"), (more[i:i + 1], refs[i][1:2], "next token")):
            assert rows.shape == (1, 152064)
            if dtype == "float32":
                err = float(np.abs(rows - ref).max())
                assert err <= WIDE_FP32_ABS, "full vocabulary, %s %d: |engine - plain| = %.3g" % (what, i, err)
            else:
                harness.check_logits(rows, ref, dtype, "full vocabulary, %s %d" % (what, i), harness.BF16_WIDE)
    eng.check()
