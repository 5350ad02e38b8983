"""Plain, slow statement of the Qwen2.5 dense decoder, written from the formulas of
onurtamer/friday-inference-engine (file:line given at each function).

It handles whole sequences only: no cache, no batching, no kernels, one function for
each part.  It shares no code with the package under test: it has its own reader of
config.json and of the safetensors file, and its own random numbers for sampling.

Arithmetic is float64 throughout, with two exceptions that follow the reference
literally because the result depends on them beyond rounding: the rotation angle of
the position encoding (fp32 `pos / pow(base, 2i/d)`) and the uniform number that the
sampler draws (a 24-bit fraction).

The reference rounds every intermediate to fp16, clamps to +-65504 and maps NaN to 0
(cpu_ops.cpp:23, cuda_math_kernels.cu:316-318).  Those are storage guards of an fp16
engine, not part of the model, and are left out here.

The reference cannot run these test configurations itself (model_config.cpp:59
demands head_dim 128 and has no sliding window), so this file rests on its formulas;
tests/golden/ holds a comparison with the reference's compiled CPU engine on a
configuration that it does accept.
"""
import json
import os
import struct

import numpy as np

F64 = np.float64


# ---------------------------------------------------------------------------
# reading a model folder (own reader; the product has another one)
# ---------------------------------------------------------------------------

_NP_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I32": np.int32, "I64": np.int64}


def read_safetensors(path):
    """name -> float64 (or integer) numpy array.  BF16 is widened by hand."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = blob[lo:hi]
        shape = tuple(info["shape"])
        if info["dtype"] == "BF16":
            u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(F64)
        else:
            arr = np.frombuffer(raw, dtype=_NP_DTYPES[info["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(F64)
        out[name] = arr.reshape(shape)
    return out


class PlainModel:
    """Weights by Hugging Face tensor name plus the numbers of config.json.

    `program` is the order in which layers run: a list of (layer, kv_source) where
    kv_source is None (the layer computes its own keys and values) or the index of an
    earlier program entry whose keys and values it reads instead.
    """

    def __init__(self, cfg, tensors, program=None):
        self.cfg = dict(cfg)
        self.t = tensors
        c = self.cfg
        self.n_layers = c["num_hidden_layers"]
        self.hidden = c["hidden_size"]
        self.n_heads = c["num_attention_heads"]
        self.n_kv = c.get("num_key_value_heads", self.n_heads)          # model_config.cpp:43
        self.head_dim = c.get("head_dim", self.hidden // self.n_heads)    # model_config.cpp:50
        self.eps = c["rms_norm_eps"]                                      # model_config.cpp:46 (required)
        self.theta = c.get("rope_theta", 10000.0)                         # model_config.cpp:47
        self.tied = bool(c.get("tie_word_embeddings", False))
        self.vocab = c["vocab_size"]
        self.program = program if program is not None else [(l, None) for l in range(self.n_layers)]

    @classmethod
    def from_dir(cls, model_dir, program=None):
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        return cls(cfg, read_safetensors(os.path.join(model_dir, "model.safetensors")), program)

    def window_of(self, layer):
        """Keys a query of this layer may see, or None for all earlier ones.

        The reference has no window.  The definition used here: a layer is windowed
        iff use_sliding_window and layer >= max_window_layers; a windowed query at
        position p sees keys max(0, p-W+1) .. p.
        """
        c = self.cfg
        if c.get("use_sliding_window", False) and layer >= c.get("max_window_layers", 0):
            return int(c["sliding_window"])
        return None


# ---------------------------------------------------------------------------
# the parts, one function each
# ---------------------------------------------------------------------------

def embed(table, tokens):
    """x = E[token]; an id outside [0, V) is an error (cpu_backend.cpp:160-166)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    if tokens.size and (tokens.min() < 0 or tokens.max() >= table.shape[0]):
        raise ValueError("token id out of range")
    return table[tokens].astype(F64)


def rms_norm(x, w, eps):
    """y = x / sqrt(mean(x^2) + eps) * w   (cpu_ops.cpp:10-24, cuda_math_kernels.cu:280-321)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x * (1.0 / np.sqrt(ms + eps)) * w


def linear(x, w, b=None):
    """y[n] = sum_k W[n][k] x[k] (+ b[n]); W is [out][in] (cuda_math_kernels.cu:35-45,
    bias in the epilogue: hpc_k_quants.cu:422-437)."""
    y = x @ w.T
    return y if b is None else y + b


def rope_angles(positions, head_dim, theta):
    """theta_i = pos / base^(2i/d) in fp32 (cpu_ops.cpp:26-30, cuda_math_kernels.cu:337-339)."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    denom = np.power(np.float32(theta), (np.float32(2.0) * i) / np.float32(head_dim)).astype(np.float32)
    pos = np.asarray(positions, dtype=np.float32)[:, None]
    return (pos / denom[None, :]).astype(np.float32)            # [T, d/2]


def rope_neox(x, positions, theta):
    """Pairs (i, i + d/2) of every head are rotated by theta_i (cpu_ops.cpp:31-40).
    x: [T, heads, d]."""
    d = x.shape[-1]
    ang = rope_angles(positions, d, theta).astype(F64)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., : d // 2], x[..., d // 2:]
    return np.concatenate([a * c - b * s, a * s + b * c], axis=-1)


def attention(q, k, v, window=None):
    """Causal grouped-query attention of one whole sequence.

    q: [T, n_heads, d]; k, v: [T, n_kv, d].  Head h reads kv head h // (n_heads/n_kv);
    s_j = q.k_j / sqrt(d) for j <= t; softmax; o = sum_j p_j v_j
    (cpu_ops.cpp:45-83, attention_kernels.cu:29-111).  The reference's "exp = 0 below
    -50" shortcut (cpu_ops.cpp:68) changes a weight by less than 2e-22 and is left out.
    """
    T, nh, d = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = np.zeros((T, nh, d), dtype=F64)
    scale = 1.0 / np.sqrt(F64(d))
    for h in range(nh):
        kh, vh = k[:, h // g, :], v[:, h // g, :]
        s = (q[:, h, :] @ kh.T) * scale                      # [T, T]
        t_idx = np.arange(T)[:, None]
        j_idx = np.arange(T)[None, :]
        ok = j_idx <= t_idx
        if window is not None:
            ok &= j_idx >= t_idx - window + 1
        s = np.where(ok, s, -np.inf)
        m = s.max(axis=-1, keepdims=True)
        e = np.exp(s - m)
        p = e / e.sum(axis=-1, keepdims=True)
        out[:, h, :] = p @ vh
    return out


def swiglu(gate, up):
    """a = silu(g) * u with silu(z) = z / (1 + e^-z) (cpu_ops.cpp:85-101; its shortcuts
    for |z| > 20 differ from the formula by less than 5e-8 and are left out)."""
    return gate / (1.0 + np.exp(-gate)) * up


def attention_block(m, layer, x, positions, kv_in=None):
    """n = norm(x); q,k,v = W n + b; rotate q,k; attend; x + Wo o
    (transformer.cpp:1013-1059, cpu_backend.cpp:65-110).  Returns (x, (k, v))."""
    p = "model.layers.%d." % layer
    t = m.t
    n = rms_norm(x, t[p + "input_layernorm.weight"], m.eps)
    T = x.shape[0]
    q = linear(n, t[p + "self_attn.q_proj.weight"], t[p + "self_attn.q_proj.bias"]).reshape(T, m.n_heads, m.head_dim)
    q = rope_neox(q, positions, m.theta)
    if kv_in is None:
        k = linear(n, t[p + "self_attn.k_proj.weight"], t[p + "self_attn.k_proj.bias"]).reshape(T, m.n_kv, m.head_dim)
        v = linear(n, t[p + "self_attn.v_proj.weight"], t[p + "self_attn.v_proj.bias"]).reshape(T, m.n_kv, m.head_dim)
        k = rope_neox(k, positions, m.theta)
    else:
        k, v = kv_in
    o = attention(q, k, v, m.window_of(layer)).reshape(T, m.n_heads * m.head_dim)
    return x + linear(o, t[p + "self_attn.o_proj.weight"]), (k, v)


def mlp_block(m, layer, x):
    """x + Wd (silu(Wg n) * (Wu n)), n = norm(x)  (transformer.cpp:1061-1072)."""
    p = "model.layers.%d." % layer
    t = m.t
    n = rms_norm(x, t[p + "post_attention_layernorm.weight"], m.eps)
    a = swiglu(linear(n, t[p + "mlp.gate_proj.weight"]), linear(n, t[p + "mlp.up_proj.weight"]))
    return x + linear(a, t[p + "mlp.down_proj.weight"])


def hidden_states(m, tokens):
    """The residual stream after the last layer, [T, hidden], for one whole sequence."""
    x = embed(m.t["model.embed_tokens.weight"], tokens)
    positions = np.arange(len(tokens))
    kvs = []
    for layer, kv_source in m.program:
        x, kv = attention_block(m, layer, x, positions, None if kv_source is None else kvs[kv_source])
        kvs.append(kv)
        x = mlp_block(m, layer, x)
    return x


def logits(m, tokens, at=None):
    """Final norm and head (transformer.cpp:1077-1113; tied head: cpu_backend.cpp:141-156).
    Returns float64 [len(at) or T, vocab]."""
    x = hidden_states(m, tokens)
    if at is not None:
        x = x[np.asarray(at, dtype=np.int64)]
    n = rms_norm(x, m.t["model.norm.weight"], m.eps)
    head = m.t["model.embed_tokens.weight"] if m.tied else m.t["lm_head.weight"]
    return linear(n, head)


# ---------------------------------------------------------------------------
# choosing a token
# ---------------------------------------------------------------------------

def greedy(row):
    """First maximum wins; NaN and Inf are skipped (main.cpp:90-101)."""
    best, best_v = -1, -1e30
    for i, v in enumerate(row):
        if np.isnan(v) or np.isinf(v):
            continue
        if v > best_v:
            best, best_v = i, v
    return best


def _mulhilo(a, b):
    p = (int(a) * int(b)) & 0xFFFFFFFFFFFFFFFF
    return (p >> 32) & 0xFFFFFFFF, p & 0xFFFFFFFF


def philox4x32(counter, key, rounds=10):
    """The public Philox-4x32-10 generator (Salmon et al., 2011)."""
    c = [int(v) & 0xFFFFFFFF for v in counter]
    k = [int(v) & 0xFFFFFFFF for v in key]
    for _ in range(rounds):
        hi0, lo0 = _mulhilo(0xD2511F53, c[0])
        hi1, lo1 = _mulhilo(0xCD9E8D57, c[2])
        c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
        k = [(k[0] + 0x9E3779B9) & 0xFFFFFFFF, (k[1] + 0xBB67AE85) & 0xFFFFFFFF]
    return c


def uniform_for(seed, stream, step):
    """The number in [0, 1) that decides draw `step` of sequence `stream`: the upper 24
    bits of the first Philox word, counter (step, stream, 0, 0), key (seed lo, seed hi).
    A sequence's draws depend on nothing else, so its batch-mates cannot change them."""
    w = philox4x32((step, stream, 0, 0), (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))[0]
    return (w >> 8) * (1.0 / 16777216.0)


def temperature_cdf(row, temperature):
    """p = softmax(logits / T) and its running sum, float64."""
    z = np.asarray(row, dtype=F64) / F64(temperature)
    e = np.exp(z - z.max())
    p = e / e.sum()
    return p, np.cumsum(p)


def sample(row, temperature, seed, stream, step):
    """temperature 0: greedy.  Otherwise the first token whose running probability
    exceeds u (the reference itself samples greedily only: main.cpp:90-101)."""
    if temperature == 0:
        return greedy(row)
    _, cdf = temperature_cdf(row, temperature)
    u = uniform_for(seed, stream, step)
    return int(min(np.searchsorted(cdf, u, side="right"), len(cdf) - 1))


def generate(m, prompt, max_new_tokens, stop_ids=(), temperature=0.0, seed=0, stream=0, max_context=None):
    """The reference's loop for one sequence (main.cpp:308-343): run the prompt, pick a
    token, stop on a stop token (which is not kept), on the limit, or on a full context.
    Every step runs the whole sequence again: slow on purpose."""
    toks = list(prompt)
    out = []
    for step in range(max_new_tokens):
        if max_context is not None and len(toks) > max_context:   # main.cpp:335
            return out, "context"
        row = logits(m, toks, at=[len(toks) - 1])[0]
        nxt = sample(row, temperature, seed, stream, step)
        if nxt in stop_ids:
            return out, "stop"
        out.append(nxt)
        toks.append(nxt)
    return out, "length"
