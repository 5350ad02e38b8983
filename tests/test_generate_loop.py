"""The generation loop's decisions (engine/generate.cpp), with a scripted step function and sampler (no GPU)."""
import pytest

from friday_inference_engine_b200.engine import GenerationError, generate_loop as generate


class Script:
    """Sequences 'draw' from scripts; logits are stand-ins that name (request, step)."""

    def __init__(self, scripts, max_batch=2):
        self.scripts = scripts
        self.free = list(range(max_batch))[::-1]
        self.max_batch = max_batch
        self.held = {}
        self.steps = []           # (slots, tokens, want) of every step call
        self.by_slot = {}

    def alloc(self):
        s = self.free.pop()
        self.held[s] = 0
        return s

    def free_slot(self, s):
        assert s in self.held, "slot freed twice"
        del self.held[s]
        self.free.append(s)

    def step(self, slots, tokens, want):
        assert all(s in self.held for s in slots)
        self.steps.append((list(slots), [list(t) for t in tokens], [list(w) for w in want]))
        for s, t in zip(slots, tokens):
            self.held[s] += len(t)
        return list(slots)

    def sample(self, streams, steps):
        return [self.scripts[r][k] for r, k in zip(streams, steps)]

    def run(self, prompts, **kw):
        kw.setdefault("max_context", 100)
        return generate(prompts, step=self.step, sample=self.sample, alloc_slot=self.alloc, free_slot=self.free_slot,
                        max_batch=self.max_batch, vocab_size=1000, **kw)


def test_unequal_prompts_stops_and_shrinking_batches():
    sc = Script({0: [5, 6, 99, 0], 1: [7, 8, 9, 10, 11], 2: [99], 3: [1, 2, 3, 4, 5]}, max_batch=2)
    out = sc.run([[1, 2, 3], [4], [5, 5], [6, 6, 6, 6]], max_new_tokens=4, stop_token_ids=[99])
    assert [g.tokens for g in out] == [[5, 6], [7, 8, 9, 10], [], [1, 2, 3, 4]]
    assert [g.finish_reason for g in out] == ["stop", "length", "stop", "length"]
    # batch one: both prompts in one step, wanted at their last places
    assert sc.steps[0] == ([0, 1], [[1, 2, 3], [4]], [[2], [0]])
    assert sc.steps[1][1] == [[5], [7]] and sc.steps[2][1] == [[6], [8]]
    assert sc.steps[3] == ([1], [[9]], [[0]])              # request 0 ended: the batch shrank
    # batch two starts only after batch one ended, in slots that were given back
    assert sc.steps[4][1] == [[5, 5], [6, 6, 6, 6]]
    assert sorted(sc.steps[4][0]) == [0, 1]
    assert sc.steps[5][1] == [[1]]                          # request 2 stopped at once; only request 3 goes on
    # the last token of a finished sequence is never stepped
    assert len(sc.steps) == 4 + 1 + 3
    assert not sc.held and sorted(sc.free) == [0, 1]


def test_context_limit_and_ignore_eos():
    sc = Script({0: [9] * 20}, max_batch=1)
    out = sc.run([[1, 2, 3]], max_new_tokens=10, max_context=6)
    # positions 0..5: three prompt tokens, three generated ones can be stepped; the fourth cannot
    assert out[0].finish_reason == "context" and len(out[0].tokens) == 4
    assert sum(len(t[0]) for _, t, _ in sc.steps) == 6
    sc = Script({0: [99, 99, 99]}, max_batch=1)
    out = sc.run([[1]], max_new_tokens=3, stop_token_ids=[99], ignore_eos=True)
    assert out[0].tokens == [99, 99, 99] and out[0].finish_reason == "length"


def test_refusals_and_cleanup():
    sc = Script({0: [1]}, max_batch=1)
    with pytest.raises(GenerationError):
        sc.run([[]])
    with pytest.raises(GenerationError):
        sc.run([[1, 2, 3]], max_context=3)                 # the prompt would fill the context
    with pytest.raises(GenerationError):
        sc.run([[1, 5000]])
    assert sc.run([[1]], max_new_tokens=0)[0].finish_reason == "length" and not sc.steps

    def broken(slots, tokens, want):
        raise RuntimeError("boom")

    with pytest.raises(RuntimeError):
        generate([[1], [2]], step=broken, sample=sc.sample, alloc_slot=sc.alloc, free_slot=sc.free_slot,
                 max_batch=1, max_context=10, vocab_size=10)
    assert not sc.held                                     # the slot came back although the step failed


def test_streams_are_request_numbers():
    seen = []

    def sample(streams, steps):
        seen.append((list(streams), list(steps)))
        return [1] * len(streams)

    sc = Script({}, max_batch=2)
    generate([[1], [2], [3]], step=sc.step, sample=sample, alloc_slot=sc.alloc, free_slot=sc.free_slot, max_batch=2,
             max_context=10, vocab_size=10, max_new_tokens=2)
    assert seen == [([0, 1], [0, 0]), ([0, 1], [1, 1]), ([2], [0]), ([2], [1])]
