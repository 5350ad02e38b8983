"""Each shipped part alone against the plain function for it, and a toy architecture defined in the tests' own
plug-in (tests/cpp/toy_parts.cu): a mixer with state of its own, a feed-forward with routing, a second position
encoding, a layer order that names a layer twice and lets a layer read another's keys, an embedding multiplier
and a head with a bias, all registered from outside and run by the unchanged library."""
import ctypes
import json
import os
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_int64, c_void_p

import numpy as np
import pytest
import torch

import harness
import plain_model as pm
import tiny_configs
from friday_inference_engine_b200 import Engine, build_plugin, load_plugin, native, ops, registered_architectures
from friday_inference_engine_b200.cache import PAGE

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
HERE = os.path.dirname(os.path.abspath(__file__))
CODES = {torch.float32: 0, torch.bfloat16: 1}


@pytest.fixture(scope="module")
def plugin(tmp_path_factory):
    """Compiles and loads the plug-in once; returns its probe functions."""
    path = build_plugin(os.path.join(HERE, "cpp", "toy_parts.cu"), str(tmp_path_factory.mktemp("plugin") / "libtoy_parts.so"))
    load_plugin(path)
    lib = ctypes.CDLL(path)
    lib.probe_error.restype = c_char_p
    T, P = POINTER(native.Tensor), c_void_p
    lib.probe_new.argtypes = [c_char_p, c_char_p, c_int64, c_int, POINTER(c_void_p)]
    lib.probe_params.argtypes = [P, POINTER(c_char_p)]
    lib.probe_load.argtypes = [P, c_int, POINTER(c_char_p), POINTER(native.Tensor)]
    lib.probe_tensor.argtypes = [P, c_char_p, c_char_p, T]
    lib.probe_norm.argtypes = [P, T, T]
    lib.probe_rotary.argtypes = [P, c_void_p, POINTER(c_int)]
    lib.probe_mixer.argtypes = [P, T, T, c_float, T, POINTER(native.Geometry), POINTER(native.KV), P, T, T, T, POINTER(c_int)]
    lib.probe_feed_forward.argtypes = [P, T, T, c_float, T, P, T, T, T, POINTER(c_int)]
    lib.probe_free.argtypes = [P]
    lib.probe_free.restype = None
    return lib


def spec(kind, params=None, parts=None, prefix=""):
    return {"kind": kind, "params": params or {}, "prefix": prefix, "parts": parts or {}}


class Probe:
    """One part, built by the library's registry from a specification, with tensors of our making."""

    def __init__(self, lib, category, sp, width, dtype):
        self.lib, self.dtype = lib, dtype
        self.h = c_void_p()
        self.ok(lib.probe_new(category.encode(), json.dumps(sp).encode(), width, CODES[dtype], byref(self.h)))

    def ok(self, rc):
        assert rc == 0, self.lib.probe_error().decode()

    def fill(self, seed, scale=0.2):
        """Random parameters; returns them as float64 arrays by name."""
        out = c_char_p()
        self.ok(self.lib.probe_params(self.h, byref(out)))
        g = torch.Generator().manual_seed(seed)
        named, keep = {}, []
        for p in json.loads(out.value.decode()):
            t = (torch.randn(p["shape"], generator=g) * scale + (1.0 if p["one"] else 0.0)).to(self.dtype).to(DEV)
            keep.append((p["name"], t))
            named[p["name"]] = t.double().cpu().numpy()
        names = (c_char_p * len(keep))(*[n.encode() for n, _ in keep])
        tensors = (native.Tensor * len(keep))(*[ops._t(t) for _, t in keep])
        self.ok(self.lib.probe_load(self.h, len(keep), names, tensors))
        return named

    def tensor_info(self, path, name):
        t = native.Tensor()
        self.ok(self.lib.probe_tensor(self.h, path.encode(), name.encode(), byref(t)))
        return t.dtype, tuple(t.shape[i] for i in range(t.ndim))

    def __del__(self):
        if self.h:
            self.lib.probe_free(self.h)


def run_part(call, x, residual, then, rows, width, dtype):
    """Calls a probe's forward; returns (result, None | tensor | DeferredNorm)."""
    out = torch.empty((rows, width), dtype=dtype, device=DEV)
    normed = torch.empty_like(out)
    ssq = torch.empty((max(width // 16, 1), rows), dtype=torch.float32, device=DEV)
    ssq_d = ops._t(ssq)
    kind = c_int()
    xt, in_ssq, in_eps = (x.scaled, x.ssq, x.eps) if isinstance(x, ops.DeferredNorm) else (x, None, 0.0)
    call(ops._t(xt), ops._t(in_ssq), in_eps, ops._t(residual), then.h if then is not None else None, ops._t(out), ops._t(normed),
         ssq_d, byref(kind))
    torch.cuda.synchronize()
    if kind.value == 0:
        return out, None
    if kind.value == 1:
        return out, normed
    return out, ops.DeferredNorm(normed, ssq[:ssq_d.shape[0]], then.eps, out, then.weight)


def norm_probe(lib, dtype, width, seed, eps=1e-5):
    norm = Probe(lib, "norm", spec("rmsnorm", {"eps": eps}), width, dtype)
    norm.weight_np = norm.fill(seed)["weight"]
    norm.weight = torch.from_numpy(norm.weight_np).to(dtype).to(DEV)
    norm.eps = eps
    return norm


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(plugin, dtype):
    part = Probe(plugin, "norm", spec("rmsnorm", {"eps": 3e-6}), 120, dtype)
    w = part.fill(0)
    x = torch.randn(5, 120).to(dtype).to(DEV)
    out = torch.empty_like(x)
    part.ok(plugin.probe_norm(part.h, ops._t(x), ops._t(out)))
    ref = pm.rms_norm(x.double().cpu().numpy(), w["weight"], 3e-6)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(out.double().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()


def test_rotary_part_makes_the_reference_table(plugin):
    part = Probe(plugin, "position", spec("rotary_neox", {"theta": 1e6, "head_dim": 32}), 96, torch.float32)
    table = np.zeros(16, dtype=np.float32)
    dim = c_int()
    part.ok(plugin.probe_rotary(part.h, table.ctypes.data, byref(dim)))
    i = np.arange(16, dtype=np.float32)
    # the C library's powf (what the reference calls: cpu_ops.cpp:29) and numpy's may differ in the last bit
    want = np.power(np.float32(1e6), np.float32(2.0) * i / np.float32(32)).astype(np.float32)
    assert np.all(np.abs(table - want) <= np.spacing(want)) and table[0] == 1.0
    assert dim.value == 32
    none = Probe(plugin, "position", spec("none"), 96, torch.float32)
    none.ok(plugin.probe_rotary(none.h, table.ctypes.data, byref(dim)))
    assert dim.value == -1                      # "none" is honestly not rotary: the mixer rotates nothing


class OneSeq:
    """The geometry of one sequence given whole, with pools and a table made for one part; page 0 stays unused so
    that the part must follow the table."""

    def __init__(self, nkv, hd, n, dtype, window):
        pages = (n + PAGE - 1) // PAGE
        self.k = torch.full((pages + 2, PAGE, nkv, hd), float("nan"), dtype=dtype, device=DEV)
        self.v = self.k.clone()
        self.table = torch.tensor([[p + 1 for p in range(pages)][::-1]], dtype=torch.int32, device=DEV)
        i32 = dict(dtype=torch.int32, device=DEV)
        self.row_seq, self.row_pos = torch.zeros(n, **i32), torch.arange(n, **i32)
        self.start, self.qlen, self.pos0 = torch.zeros(1, **i32), torch.full((1,), n, **i32), torch.zeros(1, **i32)
        g = native.Geometry()
        g.rows, g.n_seqs, g.max_q_len, g.max_kv_len, g.decode = n, 1, n, n, 1 if n == 1 else 0
        g.row_seq, g.row_pos = self.row_seq.data_ptr(), self.row_pos.data_ptr()
        g.seq_start, g.seq_qlen, g.seq_pos0 = self.start.data_ptr(), self.qlen.data_ptr(), self.pos0.data_ptr()
        self.geometry = g
        self.kv = ops._kv(self.k, self.v, self.table, PAGE, window, write=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 10])
@pytest.mark.parametrize("nq,nkv,hd,width,n", [(6, 2, 48, 120, 90), (4, 2, 64, 256, 9)])
def test_attention_part(plugin, dtype, window, nq, nkv, hd, width, n):
    """The second shape is a step of few rows whose sizes let rotation, cache write and the following norm ride in
    the products' epilogues (bf16); the first goes through the kernels of their own."""
    sp = spec("gqa_attention", {"n_heads": nq, "n_kv_heads": nkv, "head_dim": hd, "window": window or 0},
              {"position": spec("rotary_neox", {"theta": 5e4, "head_dim": hd})})
    part = Probe(plugin, "mixer", sp, width, dtype)
    w = part.fill(1, scale=0.08)                     # scores of a few units: peaked, but not beyond what bf16 resolves
    code, shape = part.tensor_info("", "w_qkv")      # q, k and v were loaded into one stacked matrix
    assert shape == ((nq + 2 * nkv) * hd, width) and code == CODES[dtype]
    one = OneSeq(nkv, hd, n, dtype, window)
    h = torch.randn(n, width).to(dtype).to(DEV)
    res = torch.randn(n, width).to(dtype).to(DEV)

    def call(x, in_ssq, in_eps, residual, then, out, normed, ssq, kind):
        part.ok(plugin.probe_mixer(part.h, x, in_ssq, in_eps, residual, byref(one.geometry), byref(one.kv), then, out,
                                   normed, ssq, kind))

    out, nothing = run_part(call, h, res, None, n, width, dtype)
    assert nothing is None
    got = out.double().cpu().numpy()
    hn = h.double().cpu().numpy()
    q = pm.linear(hn, w["q_proj.weight"], w["q_proj.bias"]).reshape(n, nq, hd)
    k = pm.linear(hn, w["k_proj.weight"], w["k_proj.bias"]).reshape(n, nkv, hd)
    v = pm.linear(hn, w["v_proj.weight"], w["v_proj.bias"]).reshape(n, nkv, hd)
    pos = np.arange(n)
    o = pm.attention(pm.rope_neox(q, pos, 5e4), pm.rope_neox(k, pos, 5e4), v, window).reshape(n, nq * hd)
    ref = res.double().cpu().numpy() + pm.linear(o, w["o_proj.weight"])
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()
    # told which norm follows, it returns that norm of its result as well
    norm = norm_probe(plugin, dtype, width, 9)
    out2, normed = run_part(call, h, res, norm, n, width, dtype)
    assert torch.equal(out2, out) and normed is not None
    fused = ops.fusion_enabled() and dtype == torch.bfloat16 and n <= 64 and width % 128 == 0
    assert isinstance(normed, ops.DeferredNorm) == fused
    err = np.abs(ops.materialize(normed).double().cpu().numpy() - pm.rms_norm(out2.double().cpu().numpy(), norm.weight_np, 1e-5)).max()
    assert err <= tol * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,inner,n", [(120, 200, 7), (256, 384, 5)])
def test_feed_forward_part(plugin, dtype, width, inner, n):
    part = Probe(plugin, "feed_forward", spec("swiglu", {"inner": inner}), width, dtype)
    w = part.fill(2)
    assert part.tensor_info("", "w_gate_up")[1] == (2 * inner, width)       # gate and up, row by row in turn
    h = torch.randn(n, width).to(dtype).to(DEV)
    res = torch.randn(n, width).to(dtype).to(DEV)

    def call(x, in_ssq, in_eps, residual, then, out, normed, ssq, kind):
        part.ok(plugin.probe_feed_forward(part.h, x, in_ssq, in_eps, residual, then, out, normed, ssq, kind))

    def plain(hn, resn):
        return resn + pm.linear(pm.swiglu(pm.linear(hn, w["gate_proj.weight"]), pm.linear(hn, w["up_proj.weight"])),
                                w["down_proj.weight"])

    ref = plain(h.double().cpu().numpy(), res.double().cpu().numpy())
    out, nothing = run_part(call, h, res, None, n, width, dtype)
    assert nothing is None
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert np.abs(out.double().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    norm = norm_probe(plugin, dtype, width, 9)
    out2, normed = run_part(call, h, res, norm, n, width, dtype)
    assert torch.equal(out2, out)
    assert isinstance(normed, ops.DeferredNorm) == (ops.fusion_enabled() and dtype == torch.bfloat16 and width % 128 == 0)
    want = pm.rms_norm(out2.double().cpu().numpy(), norm.weight_np, 1e-5)
    assert np.abs(ops.materialize(normed).double().cpu().numpy() - want).max() <= tol * 4
    # and it takes such rows as its input: the norm is finished inside its first product
    if isinstance(normed, ops.DeferredNorm):
        ref2 = plain(want, out2.double().cpu().numpy())
        out3, _ = run_part(call, normed, out2, None, n, width, dtype)
        assert np.abs(out3.double().cpu().numpy() - ref2).max() <= tol * np.abs(ref2).max()


# ---------------------------------------------------------------------------------------
# The toy architecture of the plug-in, written out with the plain functions.
# ---------------------------------------------------------------------------------------

def toy_plain_logits(t, cfg, tokens):
    m = pm.PlainModel(cfg, t)
    T = len(tokens)
    pos = np.arange(T)
    x = pm.embed(t["model.embed_tokens.weight"], tokens) * 1.5                   # the embedding multiplier

    def attn(layer, x, rotate, kv=None):
        p = "model.layers.%d." % layer
        n = pm.rms_norm(x, t[p + "input_layernorm.weight"], m.eps)
        q = pm.linear(n, t[p + "self_attn.q_proj.weight"], t[p + "self_attn.q_proj.bias"]).reshape(T, m.n_heads, -1)
        k = pm.linear(n, t[p + "self_attn.k_proj.weight"], t[p + "self_attn.k_proj.bias"]).reshape(T, m.n_kv, -1)
        v = pm.linear(n, t[p + "self_attn.v_proj.weight"], t[p + "self_attn.v_proj.bias"]).reshape(T, m.n_kv, -1)
        if rotate:
            q, k = pm.rope_neox(q, pos, m.theta), pm.rope_neox(k, pos, m.theta)
        else:
            q, k = q.copy(), k.copy()
            q[:, :, 0] += pos[:, None] / 100.0
            k[:, :, 0] += pos[:, None] / 100.0
        if kv is not None:
            k, v = kv
        o = pm.attention(q, k, v, m.window_of(layer)).reshape(T, -1)
        return x + pm.linear(o, t[p + "self_attn.o_proj.weight"]), (k, v)

    x, _ = attn(0, x, True)
    x = pm.mlp_block(m, 0, x)
    n = pm.rms_norm(x, t["model.layers.1.input_layernorm.weight"], m.eps)
    mean = np.cumsum(n, axis=0) / np.arange(1, T + 1)[:, None]
    x = x + pm.linear(mean, t["model.layers.1.toy.mix.weight"])
    n = pm.rms_norm(x, t["model.layers.1.post_attention_layernorm.weight"], m.eps)
    logits = n @ t["model.layers.1.moe.router.weight"].T
    probs = np.exp(logits - logits.max(-1, keepdims=True))
    probs /= probs.sum(-1, keepdims=True)
    for row, e in enumerate(probs.argmax(-1)):
        y = np.maximum(n[row] @ t["model.layers.1.moe.experts.up"][e].T, 0.0) @ t["model.layers.1.moe.experts.down"][e].T
        x[row] = x[row] + y * probs[row, e]
    x, kv2 = attn(2, x, False)
    x = pm.mlp_block(m, 2, x)
    x, _ = attn(0, x, True)
    x = pm.mlp_block(m, 0, x)
    x, _ = attn(2, x, False, kv=kv2)
    x = pm.mlp_block(m, 2, x)
    head = pm.linear(pm.rms_norm(x, t["model.norm.weight"], m.eps), t["lm_head.weight"])
    return (head * 0.5) + t["lm_head.bias"]                                      # logit multiplier, then the bias


def test_toy_architecture_is_registered_built_and_stepped(plugin, tmp_path):
    assert "ToyForCausalLM" in registered_architectures()
    cfg = dict(tiny_configs.TINY_B)
    cfg["architectures"] = ["ToyForCausalLM"]
    cfg["use_sliding_window"] = False
    d = tiny_configs.make_model_dir(str(tmp_path / "toy"), cfg, 5)
    harness.sharpen(d, 4.0)
    harness.rewrite(d, lambda n, x: x * np.float32(40.0) if n == "lm_head.bias" else None)     # a bias that matters
    tensors = pm.read_safetensors(d + "/model.safetensors")
    assert "model.layers.1.toy.mix.weight" in tensors and "model.layers.1.self_attn.q_proj.weight" not in tensors
    assert tensors["model.layers.1.moe.experts.up"].shape == (3, 40, cfg["hidden_size"]) and \
        "model.layers.1.mlp.gate_proj.weight" not in tensors and "model.layers.0.mlp.gate_proj.weight" in tensors
    assert tensors["lm_head.bias"].shape == (cfg["vocab_size"],)
    eng = Engine(model_path=d, dtype="float32", max_ctx=256, max_batch=3, prefill_chunk=40)
    st = eng.stats()
    assert len(st["groups"]) == 1 and st["groups"][0]["entries"] == [0, 2, 3] and list(st["states"]) == ["1"]
    prompts = tiny_configs.random_prompts([70, 9, 33], cfg["vocab_size"], 6)
    refs = [toy_plain_logits(tensors, cfg, p) for p in prompts]
    for rnd in range(2):                                     # twice: the second time in used slots, states reset
        slots = [eng.alloc_slot() for _ in prompts]
        cut = [60, 5, 20]
        got = eng.step(slots, [p[:c] for p, c in zip(prompts, cut)], [[c - 1] for c in cut])
        for i, c in enumerate(cut):
            harness.check_logits(harness.to_np(got[i:i + 1]), refs[i][c - 1:c], "float32", "toy prompt %d" % i)
        for t in range(4):
            got = eng.step(slots, [[p[c + t]] for p, c in zip(prompts, cut)], [[0]] * 3)
            for i, c in enumerate(cut):
                harness.check_logits(harness.to_np(got[i:i + 1]), refs[i][c + t:c + t + 1], "float32",
                                     "toy decode %d of request %d" % (t, i))
        for s in slots:
            eng.free_slot(s)
    # the same model through the device decoder: the toy parts run inside the captured step like any other
    slots = [eng.alloc_slot() for _ in prompts]
    cut = [60, 5, 20]
    eng.step(slots, [p[:c] for p, c in zip(prompts, cut)], [[]] * 3)
    dec = eng.decoder(slots, [p[c] for p, c in zip(prompts, cut)])
    for t in range(4):
        dec.step([p[c + t] for p, c in zip(prompts, cut)])
        got = harness.to_np(dec.logits)
        for i, c in enumerate(cut):
            harness.check_logits(got[i:i + 1], refs[i][c + t:c + t + 1], "float32", "toy decoder step %d row %d" % (t, i))
    assert dec.info()["graphs"] == 1
    dec.close()
