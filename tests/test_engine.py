"""The engine against the plain implementation, however the work is cut: each request alone
and whole, the last 32 tokens one by one, batches of unequal lengths one after another in
reused slots, prompts cut into passes, mixed steps, long decoding, generation."""
import numpy as np
import pytest
import torch

import harness
import plain_model
import tiny_configs
from friday_inference_engine_b200 import Engine

pytestmark = pytest.mark.gpu
BACKENDS = [pytest.param(("cuda:0", "float32"), id="f32"), pytest.param(("cuda:0", "bfloat16"), id="bf16")]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("models")


@pytest.fixture(params=BACKENDS)
def where(request):
    return request.param


def nothing_held(eng):
    st = eng.stats()
    return st["slots_held"] == 0 and all(g["pages_held"] == 0 for g in st["groups"])


def engine(root, name, where, **kw):
    d, pm = harness.model_dir(root, name)
    device, dtype = where
    kw.setdefault("max_ctx", 512)
    kw.setdefault("max_batch", 6)
    return Engine(model_path=d, dtype=dtype, device=device, **kw), pm


LENGTHS = {"A": [5, 11, 17, 70], "B": [1, 19, 40, 64, 97], "C": [33, 130, 200]}


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_each_request_alone_and_whole(root, where, name):
    eng, pm = engine(root, name, where)
    for n, p in zip(LENGTHS[name], tiny_configs.random_prompts(LENGTHS[name], eng.vocab_size, 11)):
        s = eng.alloc_slot()
        got = eng.step([s], [p], [list(range(n))])
        eng.free_slot(s)
        harness.check_logits(harness.to_np(got), plain_model.logits(pm, p), where[1], "%s whole %d" % (name, n))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(root, where, name):
    eng, pm = engine(root, name, where)
    n = 100 if name != "C" else 180
    (p,) = tiny_configs.random_prompts([n], eng.vocab_size, 12)
    ref = plain_model.logits(pm, p)
    s = eng.alloc_slot()
    head = eng.step([s], [p[:n - 32]], [[n - 33]])
    harness.check_logits(harness.to_np(head), ref[n - 33:n - 32], where[1], "%s prompt's end" % name)
    for t in range(n - 32, n):
        got = eng.step([s], [[p[t]]], [[0]])
        harness.check_logits(harness.to_np(got), ref[t:t + 1], where[1], "%s decoded token at %d" % (name, t))
    eng.free_slot(s)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_one_after_another_reuse_slots(root, where, name):
    eng, pm = engine(root, name, where, max_batch=3, max_tokens=3 * 192 + 64, max_ctx=192)
    rounds = [[9, 70, 33], [64, 2, 65], [1, 110, 40]]
    for ri, lens in enumerate(rounds):
        extra = [3 + 2 * i + ri for i in range(len(lens))]          # tokens decoded after the prompt: unequal
        prompts = tiny_configs.random_prompts([a + b for a, b in zip(lens, extra)], eng.vocab_size, 20 + ri)
        refs = [plain_model.logits(pm, p) for p in prompts]
        slots = [eng.alloc_slot() for _ in prompts]
        got = eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [[n - 1] for n in lens])
        for i, n in enumerate(lens):
            harness.check_logits(harness.to_np(got[i:i + 1]), refs[i][n - 1:n], where[1],
                                 "%s round %d prompt %d" % (name, ri, i))
        live = list(range(len(prompts)))
        t = 0
        while live:
            got = eng.step([slots[i] for i in live], [[prompts[i][lens[i] + t]] for i in live], [[0]] * len(live))
            for k, i in enumerate(live):
                at = lens[i] + t
                harness.check_logits(harness.to_np(got[k:k + 1]), refs[i][at:at + 1], where[1],
                                     "%s round %d request %d token %d" % (name, ri, i, at))
            t += 1
            for i in [i for i in live if t >= extra[i]]:       # the shorter requests end earlier
                eng.free_slot(slots[i])
                live.remove(i)
        assert nothing_held(eng)


@pytest.mark.parametrize("name", ["B", "C"])
def test_cut_into_passes_and_continued(root, where, name):
    """A prompt longer than one pass, and a prompt given in two steps, equal the whole."""
    eng, pm = engine(root, name, where, prefill_chunk=48)
    (p,) = tiny_configs.random_prompts([150], eng.vocab_size, 13)
    ref = plain_model.logits(pm, p)
    s = eng.alloc_slot()
    got = eng.step([s], [p], [[149, 0, 47, 48, 100]])
    harness.check_logits(harness.to_np(got), ref[[149, 0, 47, 48, 100]], where[1], "in passes of 48")
    eng.free_slot(s)
    s = eng.alloc_slot()
    eng.step([s], [p[:82]], [[]])
    got = eng.step([s], [p[82:]], [[0, 67]])
    harness.check_logits(harness.to_np(got), ref[[82, 149]], where[1], "continued at 82")
    eng.free_slot(s)


def test_passes_of_equal_size(root, where):
    """Passes are cut as equal as whole pages allow, none longer than the limit: 200 tokens with a limit of 144 run as
    128 + 72 (two passes of 100, rounded up to pages of 64), 150 tokens with a limit of 80 as 80 + 70 (the rounded share
    would exceed the limit)."""
    for limit, n in ((80, 150), (144, 200)):
        eng, pm = engine(root, "B", where, prefill_chunk=limit)
        (p,) = tiny_configs.random_prompts([n], eng.vocab_size, 14)
        ref = plain_model.logits(pm, p)
        want = [n - 1, 0, 63, 64, 79, 80, 127, min(128, n - 1)]
        s = eng.alloc_slot()
        got = eng.step([s], [p], [want])
        harness.check_logits(harness.to_np(got), ref[want], where[1], "%d tokens in passes of at most %d" % (n, limit))
        eng.free_slot(s)


@pytest.mark.parametrize("name", ["B", "C"])
def test_several_sequences_over_several_passes(root, where, name):
    """Three sequences of unequal lengths cut into passes of 48 tokens: the later passes hold fewer sequences, and
    every pass finds the earlier tokens of its sequences in the cache."""
    eng, pm = engine(root, name, where, prefill_chunk=48)
    lens = [150, 40, 97]
    prompts = tiny_configs.random_prompts(lens, eng.vocab_size, 18)
    want = [[149, 0, 47, 48, 96], [39, 5], [96, 95, 48, 1]]
    slots = [eng.alloc_slot() for _ in prompts]
    got = harness.to_np(eng.step(slots, prompts, want))
    row = 0
    for i, (p, w) in enumerate(zip(prompts, want)):
        harness.check_logits(got[row:row + len(w)], plain_model.logits(pm, p)[w], where[1], "%s sequence %d in passes" % (name, i))
        row += len(w)
    for s in slots:
        eng.free_slot(s)
    assert nothing_held(eng)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_a_request_joins_a_running_batch(root, where, name):
    """One step carries one-token continuations of two running sequences and the whole prompt of a third; the next
    step continues all three by one token."""
    eng, pm = engine(root, name, where)
    prompts = tiny_configs.random_prompts([72, 30, 101], eng.vocab_size, 19)
    refs = [plain_model.logits(pm, p) for p in prompts]
    a, b, c = (eng.alloc_slot() for _ in range(3))
    eng.step([a, b], [prompts[0][:64], prompts[1][:20]], [[], []])
    got = harness.to_np(eng.step([a, c, b], [[prompts[0][64]], prompts[2][:95], [prompts[1][20]]], [[0], [94, 0], [0]]))
    harness.check_logits(got[0:1], refs[0][64:65], where[1], "%s running sequence a in a mixed step" % name)
    harness.check_logits(got[1:3], refs[2][[94, 0]], where[1], "%s joining prompt" % name)
    harness.check_logits(got[3:4], refs[1][20:21], where[1], "%s running sequence b in a mixed step" % name)
    got = harness.to_np(eng.step([a, b, c], [[prompts[0][65]], [prompts[1][21]], [prompts[2][95]]], [[0]] * 3))
    for k, (i, at) in enumerate([(0, 65), (1, 21), (2, 95)]):
        harness.check_logits(got[k:k + 1], refs[i][at:at + 1], where[1], "%s after the mixed step, request %d" % (name, i))
    for s in (a, b, c):
        eng.free_slot(s)


def test_first_tokens_of_a_sequence(root, where):
    eng, pm = engine(root, "B", where)
    (p,) = tiny_configs.random_prompts([6], eng.vocab_size, 14)
    ref = plain_model.logits(pm, p)
    s = eng.alloc_slot()
    for t in range(6):                                       # from the very first token, one by one
        got = eng.step([s], [[p[t]]], [[0]])
        harness.check_logits(harness.to_np(got), ref[t:t + 1], where[1], "token %d from empty" % t)
    eng.free_slot(s)


def test_long_decoding(root, where):
    eng, pm = engine(root, "C", where, max_ctx=512)
    n = 420
    (p,) = tiny_configs.random_prompts([n], eng.vocab_size, 15)
    ref = plain_model.logits(pm, p)
    s = eng.alloc_slot()
    eng.step([s], [p[:20]], [[]])
    for t in range(20, n):
        got = eng.step([s], [[p[t]]], [[0]])
        if t % 7 == 0 or t > n - 5 or t in (63, 64, 65, 127, 128, 129, 191, 192):
            harness.check_logits(harness.to_np(got), ref[t:t + 1], where[1], "decoded token %d" % t)
    eng.free_slot(s)


@pytest.mark.parametrize("name, temperature", [("A", 0.0), ("B", 0.8)])
def test_generation_through_the_entry_point(root, where, name, temperature):
    eng, pm = engine(root, name, where, max_batch=2, max_ctx=128)
    lens = [5, 11, 17] if name == "A" else [1, 19, 40, 64]
    prompts = tiny_configs.random_prompts(lens, eng.vocab_size, 16)
    steps = 8 if name == "A" else 16
    out = eng.generate(prompts, max_new_tokens=steps, temperature=temperature, seed=7)
    for i, (p, g) in enumerate(zip(prompts, out)):
        assert g.finish_reason == "length" and len(g.tokens) == steps
        # teacher forcing on the engine's own tokens: every choice must be the plain model's choice, or a
        # near-tie of it (bfloat16 only)
        seq = list(p)
        for k, tok in enumerate(g.tokens):
            row = plain_model.logits(pm, seq, at=[len(seq) - 1])[0]
            want = plain_model.sample(row, temperature, 7, i, k)
            if tok != want:
                assert where[1] == "bfloat16", "request %d token %d: %d, plain chose %d" % (i, k, tok, want)
                if temperature == 0:
                    assert row[want] - row[tok] < 0.05 * row.std(), "not a near-tie"
                else:
                    _, cdf = plain_model.temperature_cdf(row, temperature)
                    u = plain_model.uniform_for(7, i, k)
                    edge = min(abs(cdf[min(tok, want)] - u), abs(cdf[max(tok, want) - 1] - u))
                    assert abs(tok - want) == 1 and edge < 0.02, "not at the edge of the chosen interval"
            seq.append(tok)


@pytest.mark.parametrize("name", ["C", "B"])
def test_many_batches_of_random_shape(root, name):
    """Generation calls of random numbers of requests, lengths and budgets, one after another on one engine: batches of
    every size up to the engine's, kept decoders armed again and again, slots and pages used again, stop tokens.  In
    32-bit every chosen token must be the plain implementation's choice."""
    import random
    eng, pm = engine(root, name, ("cuda:0", "float32"), max_batch=3, max_ctx=200)
    rnd = random.Random(5)
    for call in range(10):
        lens = [rnd.choice([1, 2, 5, 31, 63, 64, 65, 100, 140]) for _ in range(rnd.randint(1, 7))]
        prompts = tiny_configs.random_prompts(lens, eng.vocab_size, 100 + call)
        budget = rnd.randint(1, 24)
        free = eng.generate(prompts, max_new_tokens=budget)
        stop = rnd.choice(free[0].tokens)
        out = eng.generate(prompts, max_new_tokens=budget, stop_token_ids=[stop]) if call % 2 else free
        for i, (p, g) in enumerate(zip(prompts, out)):
            seq = list(p)
            ref = plain_model.logits(pm, p + g.tokens + [0], at=list(range(len(p) - 1, len(p) + len(g.tokens))))
            for k, tok in enumerate(g.tokens):
                assert tok == plain_model.greedy(ref[k]), "call %d request %d token %d" % (call, i, k)
                seq.append(tok)
            if g.finish_reason == "stop":
                assert plain_model.greedy(ref[len(g.tokens)]) == stop and stop not in g.tokens
            elif g.finish_reason == "length":
                assert len(g.tokens) == budget
            else:
                assert g.finish_reason == "context" and len(p) + len(g.tokens) - 1 >= 200
        assert nothing_held(eng)
    eng.check()


def test_stop_tokens_end_sequences_early(root, where):
    eng, pm = engine(root, "A", where, max_batch=3, max_ctx=128)
    prompts = tiny_configs.random_prompts([5, 11, 17], eng.vocab_size, 17)
    free = eng.generate(prompts, max_new_tokens=12)
    stop = free[1].tokens[4]
    cut = eng.generate(prompts, max_new_tokens=12, stop_token_ids=[stop])
    for f, c in zip(free, cut):
        if stop in f.tokens:
            assert c.finish_reason == "stop" and c.tokens == f.tokens[:f.tokens.index(stop)]
        else:
            assert c.finish_reason == "length" and c.tokens == f.tokens
    assert nothing_held(eng)


def test_refusals(root, where):
    eng, _ = engine(root, "A", where, max_ctx=64, max_batch=2)
    from friday_inference_engine_b200.engine import StepError
    s = eng.alloc_slot()
    with pytest.raises(StepError):
        eng.step([s], [[512]], [[0]])                        # outside the vocabulary: an error, never remapped
    with pytest.raises(StepError):
        eng.step([s], [[1] * 65], [[0]])                     # longer than the context
    with pytest.raises(StepError):
        eng.step([s, s], [[1], [2]], [[0], [0]])
    eng.free_slot(s)


def test_a_kernel_that_gave_up_is_reported_and_the_word_is_cleared(root):
    """Every bounded wait of a kernel that runs out leaves a code in a status word on the device; Engine.check() raises
    on it and clears it.  The failure is made on the host: the code is written into the word with a copy, no kernel is
    made to wait."""
    try:
        from cuda.bindings import runtime as cudart
    except ImportError:
        from cuda import cudart
    from friday_inference_engine_b200 import KernelError
    eng, _ = engine(root, "A", ("cuda:0", "bfloat16"))
    eng.check()                                              # nothing has happened: no error
    word = eng.info()["status_word"]
    code = np.array([7], dtype=np.int32)
    (err,) = cudart.cudaMemcpy(word, code.ctypes.data, 4, cudart.cudaMemcpyKind.cudaMemcpyHostToDevice)
    assert int(err) == 0
    with pytest.raises(KernelError) as e:
        eng.check()
    assert "code 7" in str(e.value)
    eng.check()                                              # cleared: the engine goes on
    s = eng.alloc_slot()
    assert eng.step([s], [[1, 2, 3]], [[2]]).shape == (1, eng.vocab_size)
    eng.free_slot(s)
