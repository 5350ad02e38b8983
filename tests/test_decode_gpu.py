"""Decoding through the device decoder (static buffers, CUDA graph, and where it applies the fused
all-layers kernel) against the plain implementation, token by token with given tokens: across page
boundaries, with a window, with rows that end early, and once more with the fused kernel switched
off so that both ways stay covered."""
import numpy as np
import pytest
import torch

import harness
import plain_model
import tiny_configs
from friday_inference_engine_b200 import Engine

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("decode")


@pytest.mark.parametrize("fused", ["1", "0"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_device_decoder_follows_the_plain_model(root, monkeypatch, name, fused):
    monkeypatch.setenv("FRIDAY_FUSED_DECODE", fused)
    d, pm = harness.model_dir(root, name)
    eng = Engine(model_path=d, dtype="bfloat16", max_ctx=128 if name == "A" else 256, max_batch=4)
    limit = 120 if name == "A" else 200
    lens = [5, 60, 33]
    total = [limit, 150 if name != "A" else 110, 100]
    prompts = tiny_configs.random_prompts(total, eng.vocab_size, 50)
    refs = [plain_model.logits(pm, p) for p in prompts]
    slots = [eng.alloc_slot() for _ in prompts]
    eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[]] * 3)
    dec = eng.decoder(slots, [p[n] for p, n in zip(prompts, lens)])
    assert (dec.fused is not None) == (fused == "1")      # the fused kernel is an option, off unless asked for
    live = [True] * 3
    t = 0
    while any(live):
        feed = [prompts[i][lens[i] + t] if live[i] else 0 for i in range(3)]
        dec.step(feed)
        if t % 5 == 0 or t in (3, 4, 58, 59, 60, 62, 63, 64, 65):
            got = harness.to_np(dec.logits)
            for i in range(3):
                if live[i]:
                    at = lens[i] + t
                    harness.check_logits(got[i:i + 1], refs[i][at:at + 1], "bfloat16", "%s row %d token %d" % (name, i, at))
        t += 1
        for i in range(3):
            if live[i] and lens[i] + t >= total[i]:
                live[i] = False
                dec.retire(i)
                eng.free_slot(slots[i])
    dec.check()
    dec.close()
    eng.check()


def test_fused_and_general_decoding_choose_the_same_tokens(root, monkeypatch):
    d, pm = harness.model_dir(root, "D")
    outs = []
    for fused in ("1", "0"):
        monkeypatch.setenv("FRIDAY_FUSED_DECODE", fused)
        eng = Engine(model_path=d, dtype="bfloat16", max_ctx=256, max_batch=4)
        prompts = tiny_configs.random_prompts([7, 70, 20, 64], eng.vocab_size, 51)
        outs.append([g.tokens for g in eng.generate(prompts, max_new_tokens=40, temperature=0.7, seed=3)])
    same = sum(a == b for a, b in zip(*outs))
    assert same >= 3, outs          # bfloat16 sums in another order may flip a near-tie in one sequence
