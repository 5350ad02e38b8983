"""The library from C++: a program written against include/friday/engine.h alone is compiled here, linked with
libfriday_engine.so, run on a tiny model folder, and its tokens compared with the plain implementation."""
import os
import subprocess

import pytest

import harness
import plain_model
import tiny_configs
from friday_inference_engine_b200.ops import build

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_cpp_program_generates_the_plain_models_tokens(tmp_path, dtype):
    d, pm = harness.model_dir(tmp_path, "A")
    lib = build.ensure_engine_built()
    build.ensure_built(list(build.FAMILIES))                     # a C++ user builds the kernel libraries beforehand
    exe = str(tmp_path / "generate_main")
    subprocess.run([build._cxx(), "-std=c++17", "-O1", "-I", build.INCLUDE, os.path.join(HERE, "cpp", "generate_main.cpp"),
                    "-o", exe, lib, "-Wl,-rpath," + os.path.dirname(lib)], check=True)
    prompts = tiny_configs.random_prompts([5, 11, 17], pm.vocab, 40)       # three requests, two slots: two batches
    text = "\n".join(" ".join(str(t) for t in p) for p in prompts) + "\n"
    run = subprocess.run([exe, d, dtype, "8"], input=text, capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr
    lines = run.stdout.strip().split("\n")
    assert len(lines) == 5 and "Qwen2ForCausalLM" in run.stderr
    for p, line in zip(prompts, lines):
        tokens = [int(t) for t in line.split("[")[0].split()]
        assert len(tokens) == 8 and line.endswith("[length]")
        seq = list(p)
        for k, tok in enumerate(tokens):
            row = plain_model.logits(pm, seq, at=[len(seq) - 1])[0]
            want = plain_model.greedy(row)
            assert tok == want or (dtype == "bfloat16" and row[want] - row[tok] < 0.05 * row.std()), \
                "token %d: the program chose %d, the plain model %d" % (k, tok, want)
            seq.append(tok)
    ref = plain_model.logits(pm, prompts[0], at=[len(prompts[0]) - 2, len(prompts[0]) - 1])
    assert lines[3] == "prefill %d" % plain_model.greedy(ref[0]) or dtype == "bfloat16"
    assert lines[4] == "step %d" % plain_model.greedy(ref[1]) or dtype == "bfloat16"
