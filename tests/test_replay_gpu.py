"""bin/trace_run driven as a user drives it: a subprocess, one JSON step a line, the next
step only after `done <step>`.  The same requests are replayed whole, with the last 32
tokens one by one, and in batches of unequal lengths one after another; every file of
logits is compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import harness
import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Replay:
    def __init__(self, model_dir, dtype, out, max_tokens):
        self.out = out
        self.proc = subprocess.Popen(
            [os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out,
             "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)

    def step(self, number, entries, end=()):
        self.proc.stdin.write(json.dumps({"step": number, "entries": entries, "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == "done %d" % number, "trace_run answered %r (exit code %s)" % (line, self.proc.poll())

    def logits(self, number, vocab):
        return np.fromfile(os.path.join(self.out, "%d.f32" % number), dtype="<f4").reshape(-1, vocab)

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("replay")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_three_ways(root, name, dtype):
    d, pm = harness.model_dir(root, name)
    vocab = pm.vocab
    lens = [40, 75, 100, 33, 64, 90]
    reqs = tiny_configs.random_prompts(lens, vocab, 31)
    refs = [plain_model.logits(pm, p) for p in reqs]
    out = str(root / ("out_%s_%s" % (name, dtype)))
    # the most that is ever held: way three's first batch, 64 + 128 + 128 tokens in pages
    rp = Replay(d, dtype, out, max_tokens=320)
    n = 0
    # one: each request alone and whole
    for i, p in enumerate(reqs):
        rp.step(n, [{"id": "w%d" % i, "tokens": p, "want": list(range(len(p)))}], end=["w%d" % i])
        harness.check_logits(rp.logits(n, vocab), refs[i], dtype, "whole request %d" % i)
        n += 1
    # two: the last 32 tokens one by one
    for i, p in enumerate(reqs[:3]):
        cut = len(p) - 32
        rp.step(n, [{"id": "t%d" % i, "tokens": p[:cut], "want": [cut - 1]}])
        harness.check_logits(rp.logits(n, vocab), refs[i][cut - 1:cut], dtype, "prompt of request %d" % i)
        n += 1
        for t in range(cut, len(p)):
            last = t == len(p) - 1
            rp.step(n, [{"id": "t%d" % i, "tokens": [p[t]], "want": [0]}], end=["t%d" % i] if last else [])
            harness.check_logits(rp.logits(n, vocab), refs[i][t:t + 1], dtype, "request %d token %d" % (i, t))
            n += 1
    # three: batches of unequal lengths, shorter requests end earlier, one batch after another
    for batch in ([0, 1, 2], [3, 4, 5]):
        starts = {i: len(reqs[i]) - (6 + 5 * k) for k, i in enumerate(batch)}
        rp.step(n, [{"id": "b%d" % i, "tokens": reqs[i][:starts[i]], "want": [starts[i] - 1, 0]} for i in batch])
        got = rp.logits(n, vocab)
        for k, i in enumerate(batch):
            harness.check_logits(got[2 * k:2 * k + 2], refs[i][[starts[i] - 1, 0]], dtype, "batched prompt %d" % i)
        n += 1
        live, t = list(batch), 0
        while live:
            ending = [i for i in live if starts[i] + t == len(reqs[i]) - 1]
            rp.step(n, [{"id": "b%d" % i, "tokens": [reqs[i][starts[i] + t]], "want": [0]} for i in live],
                    end=["b%d" % i for i in ending])
            got = rp.logits(n, vocab)
            for k, i in enumerate(live):
                at = starts[i] + t
                harness.check_logits(got[k:k + 1], refs[i][at:at + 1], dtype, "batched request %d token %d" % (i, at))
            live = [i for i in live if i not in ending]
            t += 1
            n += 1
    rp.step(n, [{"id": "q", "tokens": reqs[0][:5], "want": []}], end=["q"])       # nothing wanted: no file
    assert not os.path.exists(os.path.join(out, "%d.f32" % n))
    rp.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_a_request_joins_a_running_batch(root, dtype):
    """Steps that mix one-token entries with a fresh prompt (the step function allows it), on the windowed model."""
    d, pm = harness.model_dir(root, "B")
    vocab = pm.vocab
    reqs = tiny_configs.random_prompts([90, 70, 40], vocab, 32)
    refs = [plain_model.logits(pm, p) for p in reqs]
    out = str(root / ("mixed_%s" % dtype))
    rp = Replay(d, dtype, out, max_tokens=320)
    rp.step(0, [{"id": "a", "tokens": reqs[0][:66], "want": [65]}])
    harness.check_logits(rp.logits(0, vocab), refs[0][65:66], dtype, "first prompt")
    rp.step(1, [{"id": "a", "tokens": [reqs[0][66]], "want": [0]}, {"id": "b", "tokens": reqs[1][:50], "want": [0, 49]}])
    got = rp.logits(1, vocab)
    harness.check_logits(got[0:1], refs[0][66:67], dtype, "running request in a mixed step")
    harness.check_logits(got[1:3], refs[1][[0, 49]], dtype, "joining prompt")
    rp.step(2, [{"id": "c", "tokens": reqs[2][:39], "want": [38]}, {"id": "b", "tokens": [reqs[1][50]], "want": [0]},
                {"id": "a", "tokens": [reqs[0][67]], "want": [0]}], end=["a"])
    got = rp.logits(2, vocab)
    harness.check_logits(got[0:1], refs[2][38:39], dtype, "second joining prompt")
    harness.check_logits(got[1:2], refs[1][50:51], dtype, "request b after joining")
    harness.check_logits(got[2:3], refs[0][67:68], dtype, "request a in its last step")
    rp.step(3, [{"id": "b", "tokens": [reqs[1][51]], "want": [0]}, {"id": "c", "tokens": [reqs[2][39]], "want": [0]}],
            end=["b", "c"])
    got = rp.logits(3, vocab)
    harness.check_logits(got[0:1], refs[1][51:52], dtype, "request b, one token more")
    harness.check_logits(got[1:2], refs[2][39:40], dtype, "request c, one token more")
    rp.close()
