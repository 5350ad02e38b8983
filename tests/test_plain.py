"""The plain implementation checked against even plainer statements of the same
formulas (explicit loops), so that the oracle itself is not a misreading."""
import math

import numpy as np

import plain_model as pm


def test_philox_known_answers():
    # Known-answer vectors of Philox-4x32-10 from the Random123 distribution.
    assert pm.philox4x32((0, 0, 0, 0), (0, 0)) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert pm.philox4x32((0xffffffff,) * 4, (0xffffffff,) * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert pm.philox4x32((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0)) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_rms_norm_loop():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(3, 10)), rng.normal(size=10)
    y = pm.rms_norm(x, w, 1e-5)
    for r in range(3):
        ss = sum(v * v for v in x[r]) / 10
        for i in range(10):
            assert abs(y[r, i] - x[r, i] / math.sqrt(ss + 1e-5) * w[i]) < 1e-12


def test_rope_pairs_and_angle():
    rng = np.random.default_rng(1)
    x = rng.normal(size=(4, 2, 8))
    pos = [0, 1, 5, 77]
    y = pm.rope_neox(x, pos, 10000.0)
    assert np.allclose(y[0], x[0])                       # position 0 rotates nothing
    for t, p in enumerate(pos):
        for i in range(4):
            th = float(np.float32(p) / np.float32(np.power(np.float32(10000.0), np.float32(2 * i) / np.float32(8))))
            a, b = x[t, 1, i], x[t, 1, i + 4]
            assert abs(y[t, 1, i] - (a * math.cos(th) - b * math.sin(th))) < 1e-12
            assert abs(y[t, 1, i + 4] - (a * math.sin(th) + b * math.cos(th))) < 1e-12


def _attention_loops(q, k, v, window):
    T, nh, d = q.shape
    g = nh // k.shape[1]
    out = np.zeros_like(q)
    for t in range(T):
        lo = 0 if window is None else max(0, t - window + 1)
        for h in range(nh):
            s = [float(q[t, h] @ k[j, h // g]) / math.sqrt(d) for j in range(lo, t + 1)]
            m = max(s)
            e = [math.exp(v_ - m) for v_ in s]
            for n, j in enumerate(range(lo, t + 1)):
                out[t, h] += e[n] / sum(e) * v[j, h // g]
    return out


def test_attention_against_loops():
    rng = np.random.default_rng(2)
    q, k, v = rng.normal(size=(9, 6, 4)), rng.normal(size=(9, 2, 4)), rng.normal(size=(9, 2, 4))
    for window in (None, 1, 3, 9, 50):
        assert np.allclose(pm.attention(q, k, v, window), _attention_loops(q, k, v, window), atol=1e-12)


def test_swiglu_and_greedy():
    z = np.array([-30.0, -1.0, 0.0, 2.5, 30.0])
    assert np.allclose(pm.swiglu(z, np.ones(5)), [v / (1 + math.exp(-v)) for v in z])
    assert pm.greedy(np.array([1.0, 3.0, 3.0, 2.0])) == 1             # the first maximum wins
    assert pm.greedy(np.array([np.nan, np.inf, 1.0, -np.inf])) == 2     # NaN and Inf are skipped
    assert pm.greedy(np.array([np.nan, np.nan])) == -1


def test_sampling_is_a_function_of_seed_stream_step():
    row = np.random.default_rng(3).normal(size=50)
    a = [pm.sample(row, 0.8, 7, 2, s) for s in range(20)]
    assert a == [pm.sample(row, 0.8, 7, 2, s) for s in range(20)]
    assert a != [pm.sample(row, 0.8, 7, 3, s) for s in range(20)]
    assert len(set(a)) > 3
    # frequencies follow the distribution
    p, _ = pm.temperature_cdf(row, 0.8)
    draws = np.bincount([pm.sample(row, 0.8, 11, 0, s) for s in range(4000)], minlength=50) / 4000.0
    assert np.abs(draws - p).max() < 0.03


def _tiny(cfg_over=None, seed=0):
    cfg = {"num_hidden_layers": 2, "hidden_size": 16, "num_attention_heads": 4, "num_key_value_heads": 2,
           "head_dim": 4, "intermediate_size": 24, "vocab_size": 40, "rms_norm_eps": 1e-6, "rope_theta": 100.0,
           "tie_word_embeddings": True}
    cfg.update(cfg_over or {})
    rng = np.random.default_rng(seed)
    t = {"model.embed_tokens.weight": rng.normal(size=(40, 16)), "model.norm.weight": 1 + 0.1 * rng.normal(size=16)}
    for l in range(cfg["num_hidden_layers"]):
        p = "model.layers.%d." % l
        t[p + "input_layernorm.weight"] = 1 + 0.1 * rng.normal(size=16)
        t[p + "post_attention_layernorm.weight"] = 1 + 0.1 * rng.normal(size=16)
        for n, rows in (("q", 16), ("k", 8), ("v", 8)):
            t[p + "self_attn.%s_proj.weight" % n] = 0.3 * rng.normal(size=(rows, 16))
            t[p + "self_attn.%s_proj.bias" % n] = 0.3 * rng.normal(size=rows)
        t[p + "self_attn.o_proj.weight"] = 0.3 * rng.normal(size=(16, 16))
        t[p + "mlp.gate_proj.weight"] = 0.3 * rng.normal(size=(24, 16))
        t[p + "mlp.up_proj.weight"] = 0.3 * rng.normal(size=(24, 16))
        t[p + "mlp.down_proj.weight"] = 0.3 * rng.normal(size=(16, 24))
    return pm.PlainModel(cfg, t)


def test_causality_and_window():
    m = _tiny()
    toks = list(range(3, 15))
    full = pm.logits(m, toks)
    # a position's logits do not depend on later tokens
    assert np.allclose(pm.logits(m, toks[:7]), full[:7], atol=1e-12)
    # a window as long as the sequence changes nothing, a shorter one does
    mw = _tiny({"use_sliding_window": True, "sliding_window": 12, "max_window_layers": 0})
    assert np.allclose(pm.logits(mw, toks), full, atol=1e-12)
    mw = _tiny({"use_sliding_window": True, "sliding_window": 3, "max_window_layers": 1})
    assert mw.window_of(0) is None and mw.window_of(1) == 3
    cut = pm.logits(mw, toks)
    assert np.allclose(cut[:3], full[:3], atol=1e-12) and not np.allclose(cut[5:], full[5:], atol=1e-6)


def test_program_order_and_shared_keys():
    m = _tiny()
    toks = [1, 5, 9, 2, 7]
    base = pm.logits(m, toks)
    twice = _tiny()
    twice.program = [(0, None), (1, None), (1, None)]
    assert not np.allclose(pm.logits(twice, toks), base, atol=1e-6)
    shared = _tiny()
    shared.program = [(0, None), (1, 0)]          # layer 1 reads layer 0's keys and values
    assert not np.allclose(pm.logits(shared, toks), base, atol=1e-6)


def test_generate_stops():
    m = _tiny()
    out, why = pm.generate(m, [1, 2, 3], 6)
    assert why == "length" and len(out) == 6
    out2, why2 = pm.generate(m, [1, 2, 3], 6, stop_ids={out[2]})
    assert why2 == "stop" and out2 == out[:out.index(out[2])]
    out3, why3 = pm.generate(m, [1, 2, 3], 6, max_context=5)
    assert why3 == "context" and out3 == out[:3]      # positions 3 and 4 are stepped, the third token cannot be
