"""Each part alone against the plain function for it, and a toy architecture defined
here: a mixer with state of its own, a second position encoding and a layer order that
names a layer twice and lets a layer read another's keys, all registered from outside
and run by the unchanged framework."""
import numpy as np
import pytest
import torch

import harness
import plain_model as pm
import tiny_configs
from friday_inference_engine_b200 import Engine, ops, register_architecture, register_part
from friday_inference_engine_b200.cache import PAGE, Cache
from friday_inference_engine_b200.config.qwen2 import Qwen2Config
from friday_inference_engine_b200.engine.step import StepContext
from friday_inference_engine_b200.parts import BuildEnv, LayerCall, PartSpec, StateRequest, build_part
from friday_inference_engine_b200.parts.base import Part
from friday_inference_engine_b200.architectures import qwen2_spec

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def env(width, dtype=torch.float32):
    return BuildEnv(width=width, dtype=dtype, device=DEV)


def fill(part, seed, scale=0.2):
    g = torch.Generator().manual_seed(seed)
    named = {}
    for name, owner, local, p in part.named_params():
        t = torch.randn(p.shape, generator=g) * scale + (1.0 if p.init == "one" else 0.0)
        owner.set_tensor(local, t.to(part.env.dtype).to(DEV))
        named[name] = t.to(part.env.dtype).double().numpy()
    part.finalize()
    return named


class OneSeq:
    """The geometry of one sequence given whole, with a cache made for one part."""

    def __init__(self, request, n, dtype):
        self.cache = Cache({0: request}, 4 * PAGE, 4 * PAGE, dtype, DEV, max_slots=2)
        self.cache.alloc_slot()                       # slot 0 stays unused: the part must follow the table
        self.slot = self.cache.alloc_slot()
        self.cache.reserve([self.slot], [n])
        ctx = StepContext(self, [self.slot], [n], [n])
        ctx.row_seq = torch.zeros(n, dtype=torch.int32, device=DEV)
        ctx.row_pos = torch.arange(n, dtype=torch.int32, device=DEV)
        ctx.tables = [torch.from_numpy(t).to(DEV) for t in self.cache.tables_for([self.slot])]
        ctx.seq_slots = torch.tensor([self.slot], dtype=torch.int64, device=DEV)
        ctx.seq_start = torch.zeros(1, dtype=torch.int32, device=DEV)
        ctx.seq_qlen = torch.full((1,), n, dtype=torch.int32, device=DEV)
        ctx.seq_pos0 = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.ctx = ctx
        self.view = self.cache.view(0, True, ctx.tables, ctx.seq_slots, [self.slot])

    def scratch(self, n, device):
        return torch.empty((max(n, 1),), dtype=torch.float32, device=device)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    part = build_part("norm", PartSpec("rmsnorm", {"eps": 3e-6}), env(120, dtype))
    w = fill(part, 0)
    x = torch.randn(5, 120).to(dtype).to(DEV)
    ref = pm.rms_norm(x.double().cpu().numpy(), w["weight"], 3e-6)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(part.forward(x).double().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()


def test_rotary_part_makes_the_reference_table():
    part = build_part("position", PartSpec("rotary_neox", {"theta": 1e6, "head_dim": 32}), env(96))
    d = part.denominators().cpu().numpy()
    i = np.arange(16, dtype=np.float32)
    assert np.array_equal(d, np.power(np.float32(1e6), np.float32(2.0) * i / np.float32(32)).astype(np.float32))
    assert part.rotary_dim == 32 and d.dtype == np.float32


def chained_norm(dtype, width, seed):
    """A norm part and a function that measures what a part returned beside its result when told that this norm
    follows: that norm of the result, as a tensor or as rows whose norm the next product finishes."""
    from friday_inference_engine_b200 import ops
    norm = build_part("norm", PartSpec("rmsnorm", {"eps": 1e-5}), env(width, dtype))
    g = fill(norm, seed)["weight"]
    return norm, lambda x, normed: np.abs(ops.materialize(normed).double().cpu().numpy()
                                          - pm.rms_norm(x.double().cpu().numpy(), g, 1e-5)).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 10])
@pytest.mark.parametrize("nq,nkv,hd,width,n", [(6, 2, 48, 120, 90), (4, 2, 64, 256, 9)])
def test_attention_part(dtype, window, nq, nkv, hd, width, n):
    """The second shape is a step of few rows whose sizes let rotation, cache write and the following norm ride in
    the products' epilogues (bf16); the first goes through the kernels of their own."""
    from friday_inference_engine_b200 import ops
    spec = PartSpec("gqa_attention", {"n_heads": nq, "n_kv_heads": nkv, "head_dim": hd, "window": window,
                                      "position": PartSpec("rotary_neox", {"theta": 5e4, "head_dim": hd})})
    part = build_part("mixer", spec, env(width, dtype))
    w = fill(part, 1, scale=0.08)                     # scores of a few units: peaked, but not beyond what bf16 resolves
    one = OneSeq(part.cache_request(), n, dtype)
    h = torch.randn(n, width).to(dtype).to(DEV)
    res = torch.randn(n, width).to(dtype).to(DEV)
    out, nothing = part.forward(h, res, one.ctx, one.view)
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
    norm, err = chained_norm(dtype, width, 9)
    out2, normed = part.forward(h, res, one.ctx, one.view, then=norm)
    assert torch.equal(out2, out) and normed is not None
    fused = ops.fusion_enabled() and dtype == torch.bfloat16 and n <= 64 and width % 128 == 0
    assert isinstance(normed, ops.DeferredNorm) == fused
    assert err(out2, normed) <= (2e-5 if dtype == torch.float32 else 3e-2) * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,inner,n", [(120, 200, 7), (256, 384, 5)])
def test_feed_forward_part(dtype, width, inner, n):
    from friday_inference_engine_b200 import ops
    part = build_part("feed_forward", PartSpec("swiglu", {"inner": inner}), env(width, dtype))
    w = fill(part, 2)
    h = torch.randn(n, width).to(dtype).to(DEV)
    res = torch.randn(n, width).to(dtype).to(DEV)
    hn = h.double().cpu().numpy()
    ref = res.double().cpu().numpy() + pm.linear(
        pm.swiglu(pm.linear(hn, w["gate_proj.weight"]), pm.linear(hn, w["up_proj.weight"])), w["down_proj.weight"])
    out, nothing = part.forward(h, res, None)
    assert nothing is None
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert np.abs(out.double().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    norm, err = chained_norm(dtype, width, 9)
    out2, normed = part.forward(h, res, None, then=norm)
    assert torch.equal(out2, out)
    assert isinstance(normed, ops.DeferredNorm) == (ops.fusion_enabled() and dtype == torch.bfloat16 and width % 128 == 0)
    assert err(out2, normed) <= tol * 4
    # and it takes such rows as its input: the norm is finished inside its first product
    if isinstance(normed, ops.DeferredNorm):
        hn2 = pm.rms_norm(out2.double().cpu().numpy(), norm.tensors["weight"].double().cpu().numpy(), 1e-5)
        ref2 = out2.double().cpu().numpy() + pm.linear(
            pm.swiglu(pm.linear(hn2, w["gate_proj.weight"]), pm.linear(hn2, w["up_proj.weight"])), w["down_proj.weight"])
        out3, _ = part.forward(normed, out2, None)
        assert np.abs(out3.double().cpu().numpy() - ref2).max() <= tol * np.abs(ref2).max()


# ---------------------------------------------------------------------------------------
# A toy architecture, defined wholly in this file.
# ---------------------------------------------------------------------------------------

@register_part("mixer", "toy_running_mean")
class RunningMean(Part):
    """out_t = W * mean(h_0 .. h_t): needs the sum so far and the count, kept per sequence."""
    category = "mixer"

    def __init__(self, env):
        super().__init__(env)
        self.declare("mix.weight", (env.width, env.width))

    def cache_request(self):
        return StateRequest((self.env.width + 1,), torch.float32)

    def forward(self, h, residual, ctx, cache):
        out = torch.empty_like(h)
        row = 0
        for b, q in enumerate(ctx.q_lens):                   # a scan over each sequence's rows, in order
            st = cache.state[ctx.slots[b]]
            sums = st[:-1] + torch.cumsum(h[row:row + q].float(), dim=0)
            counts = st[-1] + torch.arange(1, q + 1, device=h.device, dtype=torch.float32)
            out[row:row + q] = (sums / counts[:, None]).to(h.dtype)
            st[:-1] = sums[-1]
            st[-1] = counts[-1]
            row += q
        return ops.linear(out, self.tensors["mix.weight"], residual=residual)


@register_part("position", "toy_additive")
class AdditivePosition(Part):
    """Not rotary: adds pos/100 to the first dimension of every query and key head."""
    category = "position"
    rotary = False

    def __init__(self, env, head_dim):
        super().__init__(env)
        self.head_dim = head_dim

    def apply(self, qkv, ctx, n_heads, n_kv_heads, head_dim):
        v = qkv.view(qkv.shape[0], -1, head_dim)
        v[:, : n_heads + n_kv_heads, 0] += (ctx.row_pos.float() / 100.0).to(qkv.dtype)[:, None]


@register_part("feed_forward", "toy_top1")
class Top1Experts(Part):
    """A feed-forward with routing: a router picks one of a few small ReLU experts per row; the expert's output is
    weighted with the router's probability for it.  Rows are flat, so routing is a matter of row indices."""
    category = "feed_forward"

    def __init__(self, env, experts, inner):
        super().__init__(env)
        self.experts, self.inner = int(experts), int(inner)
        self.declare("router.weight", (self.experts, env.width))
        self.declare("experts.up", (self.experts, self.inner, env.width))
        self.declare("experts.down", (self.experts, env.width, self.inner))

    def forward(self, h, residual, ctx):
        t = self.tensors
        probs = torch.softmax(h.float() @ t["router.weight"].float().t(), dim=-1)      # router logits in 32-bit
        choice = probs.argmax(dim=-1)
        out = residual.clone()
        for e in range(self.experts):
            rows = (choice == e).nonzero(as_tuple=True)[0]
            if rows.numel():
                y = torch.relu(h[rows].float() @ t["experts.up"][e].float().t()) @ t["experts.down"][e].float().t()
                out[rows] += (y * probs[rows, e][:, None]).to(out.dtype)
        return out


def toy_spec(cfg):
    spec = qwen2_spec(cfg)
    layers = list(spec.layers)
    # layer 1: the toy mixer instead of attention; layer 2: attention with the toy position encoding
    p1 = dict(layers[1].params)
    p1["mixer"] = PartSpec("toy_running_mean", {}, prefix="toy.")
    p1["feed_forward"] = PartSpec("toy_top1", {"experts": 3, "inner": 40}, prefix="moe.")     # and routed experts
    layers[1] = PartSpec("prenorm", p1, prefix=layers[1].prefix)
    p2 = dict(layers[2].params)
    mp = dict(p2["mixer"].params)
    mp["position"] = PartSpec("toy_additive", {"head_dim": cfg.head_dim})
    p2["mixer"] = PartSpec("gqa_attention", mp, prefix="self_attn.")
    layers[2] = PartSpec("prenorm", p2, prefix=layers[2].prefix)
    spec.layers = layers
    spec.architecture = "ToyForCausalLM"
    # run order: 0, 1 (state), 2, then layer 0 AGAIN with a cache entry of its own, then layer 2 reading the
    # keys and values that the first call of layer 2 wrote
    spec.program = [LayerCall(0, cache=0), LayerCall(1, cache=1), LayerCall(2, cache=2), LayerCall(0, cache=3),
                    LayerCall(2, cache=2, write=False)]
    return spec


register_architecture("ToyForCausalLM", Qwen2Config, toy_spec)


def toy_plain_logits(t, cfg, tokens):
    """The toy model, whole sequence, written out with the plain functions."""
    m = pm.PlainModel(cfg, t)
    T = len(tokens)
    pos = np.arange(T)
    x = pm.embed(t["model.embed_tokens.weight"], tokens)

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
    return pm.linear(pm.rms_norm(x, t["model.norm.weight"], m.eps), t["lm_head.weight"])


def test_toy_architecture_is_registered_built_and_stepped(tmp_path):
    cfg = dict(tiny_configs.TINY_B)
    cfg["architectures"] = ["ToyForCausalLM"]
    cfg["use_sliding_window"] = False
    d = tiny_configs.make_model_dir(str(tmp_path / "toy"), cfg, 5)
    harness.sharpen(d, 4.0)
    tensors = pm.read_safetensors(d + "/model.safetensors")
    assert "model.layers.1.toy.mix.weight" in tensors and "model.layers.1.self_attn.q_proj.weight" not in tensors
    assert tensors["model.layers.1.moe.experts.up"].shape == (3, 40, cfg["hidden_size"]) and \
        "model.layers.1.mlp.gate_proj.weight" not in tensors and "model.layers.0.mlp.gate_proj.weight" in tensors
    eng = Engine(model_path=d, dtype="float32", max_ctx=256, max_batch=3, prefill_chunk=40)
    assert len(eng.cache.groups) == 1 and eng.cache.groups[0].entries == [0, 2, 3] and list(eng.cache.states) == [1]
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
