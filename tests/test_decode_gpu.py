"""Decoding through the device decoder (long-lived buffers, CUDA graphs) against the plain implementation, token by
token with given tokens: across page boundaries, with a window, with rows that end early, at 17 to 64 rows (the
tiles and split-k schedules that a few rows never reach), and across the length bound at which the decoder changes
to another captured step."""
import numpy as np
import pytest

import harness
import plain_model
import tiny_configs
from friday_inference_engine_b200 import Engine

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("decode")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_device_decoder_follows_the_plain_model(root, name, dtype):
    d, pm = harness.model_dir(root, name)
    eng = Engine(model_path=d, dtype=dtype, max_ctx=128 if name == "A" else 256, max_batch=4)
    limit = 120 if name == "A" else 200
    lens = [5, 60, 33]
    total = [limit, 150 if name != "A" else 110, 100]
    prompts = tiny_configs.random_prompts(total, eng.vocab_size, 50)
    refs = [plain_model.logits(pm, p) for p in prompts]
    slots = [eng.alloc_slot() for _ in prompts]
    eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[]] * 3)
    dec = eng.decoder(slots, [p[n] for p, n in zip(prompts, lens)])
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
                    harness.check_logits(got[i:i + 1], refs[i][at:at + 1], dtype, "%s row %d token %d" % (name, i, at))
        t += 1
        for i in range(3):
            if live[i] and lens[i] + t >= total[i]:
                live[i] = False
                dec.retire(i)
                eng.free_slot(slots[i])
    assert dec.info()["graphs"] == 1                 # the first step ran eagerly, the rest from one captured step
    dec.close()
    eng.check()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("rows", [17, 32, 64, 100])
def test_decoder_of_many_rows(root, rows, dtype):
    """17 to 100 rows: the products put the weights on the tiles' M side with 32- and 64-wide row tiles, the norms
    ride in the epilogues but the rotation has its own kernel, and attention runs one CTA per (sequence, kv head).
    Unequal lengths, and every third row retires midway."""
    d, pm = harness.model_dir(root, "D")
    eng = Engine(model_path=d, dtype=dtype, max_ctx=192, max_batch=rows)
    steps = 12
    lens = [1 + (7 * i) % 90 for i in range(rows)]
    prompts = tiny_configs.random_prompts([n + steps for n in lens], eng.vocab_size, 52)
    refs = [plain_model.logits(pm, p, at=list(range(n, n + steps))) for p, n in zip(prompts, lens)]
    slots = [eng.alloc_slot() for _ in prompts]
    eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[]] * rows)
    dec = eng.decoder(slots, [p[n] for p, n in zip(prompts, lens)])
    live = [True] * rows
    for t in range(steps):
        dec.step([p[n + t] if live[i] else 0 for i, (p, n) in enumerate(zip(prompts, lens))])
        if t in (0, 1, 5, 6, 11):
            got = harness.to_np(dec.logits)
            for i in range(rows):
                if live[i]:
                    harness.check_logits(got[i:i + 1], refs[i][t:t + 1], dtype, "%d rows: row %d step %d" % (rows, i, t))
        if t == 5:
            for i in range(0, rows, 3):
                live[i] = False
                dec.retire(i)
                eng.free_slot(slots[i])
    dec.close()
    eng.check()


LONG = dict(tiny_configs.TINY_D, max_position_embeddings=2048, num_hidden_layers=2)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_decoder_crosses_its_length_bound(tmp_path_factory, dtype):
    """Captured steps serve lengths up to a bound (1,024, then doubling): a sequence that passes 1,024 tokens while it
    is decoded moves to the next bound's step, whose launch shapes differ (the keys are split more ways, the scratch
    for the splits grows).  A second batch then finds both steps captured."""
    root = tmp_path_factory.mktemp("long")
    d = tiny_configs.make_model_dir(str(root / "model"), LONG, 21)
    harness.sharpen(d)
    pm = plain_model.PlainModel.from_dir(d)
    eng = Engine(model_path=d, dtype=dtype, max_ctx=1280, max_batch=2)
    for batch in range(2):
        lens, steps = [1000, 40], 60
        prompts = tiny_configs.random_prompts([n + steps for n in lens], eng.vocab_size, 53 + batch)
        watch = [16, 17, 18, 19, 20, 21, 22, 23, 24, 25, 26, 27, 28, 29, 30, 59]
        refs = [plain_model.logits(pm, p, at=[n + t for t in watch]) for p, n in zip(prompts, lens)]
        slots = [eng.alloc_slot() for _ in prompts]
        eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[]] * 2)
        dec = eng.decoder(slots, [p[n] for p, n in zip(prompts, lens)])
        bounds = []
        for t in range(steps):
            dec.step([p[n + t] for p, n in zip(prompts, lens)])
            bounds.append(dec.info()["bound"])
            if t in watch:
                got = harness.to_np(dec.logits)
                for i in range(2):
                    harness.check_logits(got[i:i + 1], refs[i][watch.index(t)][None], dtype,
                                         "batch %d row %d at %d tokens" % (batch, i, lens[i] + t + 1))
        # the step that takes the sequence's 1,025th token is the first of the second bound
        assert bounds[23] == 1024 and bounds[24] == 1280 and len(set(bounds)) == 2
        assert dec.info()["graphs"] == 2
        dec.close()
        for s in slots:
            eng.free_slot(s)
    eng.check()


def test_generation_crosses_the_bound_in_float32(tmp_path_factory):
    """Engine.generate with two sequences of which one passes 1,024 tokens: in float32 the CUDA-core attention splits
    the keys by the bound, so the scratch grows exactly there."""
    root = tmp_path_factory.mktemp("long32")
    d = tiny_configs.make_model_dir(str(root / "model"), LONG, 22)
    pm = plain_model.PlainModel.from_dir(d)
    eng = Engine(model_path=d, dtype="float32", max_ctx=2048, max_batch=2)
    prompts = tiny_configs.random_prompts([1010, 30], eng.vocab_size, 55)
    out = eng.generate(prompts, max_new_tokens=30)
    for p, g in zip(prompts, out):
        assert g.finish_reason == "length" and len(g.tokens) == 30
        seq = list(p) + g.tokens
        ref = plain_model.logits(pm, seq, at=list(range(len(p) - 1, len(seq) - 1)))
        for k, tok in enumerate(g.tokens):
            assert tok == plain_model.greedy(ref[k]), "token %d of the sequence of %d" % (k, len(p))


def test_windowed_sequence_decoded_far_past_its_window(tmp_path_factory):
    """Every layer has a window of 24: a sequence of a thousand tokens gives its pages back as it goes and never
    holds more than three of them, and what a query sees stays exactly its last 24 keys."""
    root = tmp_path_factory.mktemp("window")
    cfg = dict(tiny_configs.TINY_B, max_position_embeddings=2048)
    d = tiny_configs.make_model_dir(str(root / "model"), cfg, 23)
    harness.sharpen(d)
    pm = plain_model.PlainModel.from_dir(d)
    eng = Engine(model_path=d, dtype="bfloat16", max_ctx=1100, max_batch=2, max_tokens=8 * 64)
    n = 1000
    prompts = tiny_configs.random_prompts([n, 300], eng.vocab_size, 56)
    watch = [40, 63, 64, 65, 500, 959, 960, 961, 999]
    refs = plain_model.logits(pm, prompts[0], at=watch)
    slots = [eng.alloc_slot(), eng.alloc_slot()]
    eng.step(slots, [prompts[0][:30], prompts[1][:10]], [[], []])
    dec = eng.decoder(slots, [prompts[0][30], prompts[1][10]])
    live = True
    for t in range(30, n):
        dec.step([prompts[0][t], prompts[1][t - 20] if live else 0])
        if t in watch:
            harness.check_logits(harness.to_np(dec.logits)[0:1], refs[watch.index(t)][None], "bfloat16", "token %d" % t)
        if t % 97 == 0:
            assert max(sum(p >= 0 for p in row) for row in eng.stats()["groups"][0]["table"]) <= 3
        if live and t - 20 == 299:
            live = False
            dec.retire(1)
            eng.free_slot(slots[1])
    dec.close()
    eng.free_slot(slots[0])
    assert eng.stats()["groups"][0]["pages_held"] == 0
    eng.check()
