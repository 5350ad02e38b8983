"""The decode fast path for a stack of ordinary layers: all layers of a one-token step in ONE
persistent kernel (csrc/decode_layer.cu) instead of eight kernels per layer.

It applies when every layer is the arrangement the kernel implements (pre-norm block, RMSNorm,
grouped-query attention with rotary encoding or none, SwiGLU feed-forward), weights are bfloat16,
the run order is plain (each layer once, with a cache entry of its own) and the step has at most 16
rows.  It is an option (FRIDAY_FUSED_DECODE=1), not the default: see `applicable`.  The parts
themselves know nothing of this file: it reads their tensors and constants.
"""
import ctypes
import os

import numpy as np
import torch

from ..cache import PAGE
from ..ops import code_of, lib
from ..parts.attention import GQAttention
from ..parts.block import PreNormBlock
from ..parts.mlp import SwiGLU
from ..parts.norm import RMSNorm

MAX_ROWS = 16
_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _family():
    fam = lib.family("decode_layer")
    if not getattr(fam, "_declared", False):
        fam.declare("decode_layer_args_bytes", [])
        fam.declare("decode_layer_supports", [_I, _I, _I, _I])
        fam.declare("decode_layer_fill", [_P, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P, _P, _I, _F, _P, _I, _F,
                                          _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _I, _I])
        fam.declare("decode_layer_scratch", [_P, _I, _I, _I, _I, _I, _P])
        fam.declare("decode_layers_run", [_P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I,
                                          _I, _I, _F, _I, _P])
        fam._declared = True
    return fam


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def applicable(model, cache, rows):
    """True if the fused kernel can run this model's one-token steps."""
    # Off unless asked for: measured on B200 at the 7B shape and batch 8, a layer takes 165 us in this kernel
    # against 130 us as separate kernels chained by programmatic dependent launch (a grid barrier costs about
    # 3 us, a chained kernel boundary about 1.5 us), so the general path is the faster one today.
    if os.environ.get("FRIDAY_FUSED_DECODE", "0") != "1":
        return False
    env = model.env
    if env.dtype != torch.bfloat16 or env.device.type != "cuda" or not 1 <= rows <= MAX_ROWS:
        return False
    if [(c.layer, c.write) for c in model.program] != [(i, True) for i in range(len(model.layers))]:
        return False
    if len({c.cache for c in model.program}) != len(model.program) or any(c.cache is None for c in model.program):
        return False
    shape = None
    for block in model.layers:
        if type(block) is not PreNormBlock:
            return False
        mixer, ffn = block.mixer, block.feed_forward
        if type(mixer) is not GQAttention or type(ffn) is not SwiGLU:
            return False
        if type(block.norm1) is not RMSNorm or type(block.norm2) is not RMSNorm:
            return False
        if not getattr(mixer.position, "rotary", False) or mixer.out_bias:
            return False
        if mixer.scale != float(mixer.head_dim) ** -0.5 and mixer.scale <= 0:
            return False
        tensors = [mixer.w_qkv, mixer.w_o, ffn.w_gate_up, ffn.w_down]
        if any(t.dtype != torch.bfloat16 or t.shape[1] % 8 or not t.is_contiguous() for t in tensors):
            return False
        this = (mixer.n_heads, mixer.n_kv_heads, mixer.head_dim, ffn.inner, mixer.scale)
        if shape is not None and this != shape:
            return False
        shape = this
    if shape is None or shape[2] not in (16, 32, 64, 128):
        return False
    return all(call.cache in cache.group_of for call in model.program)


class FusedLayers:
    def __init__(self, decoder):
        self.decoder = decoder
        model, cache = decoder.model, decoder.cache
        self.fam = _family()
        dev = model.env.device
        rows, width = decoder.n, model.spec.width
        m0, f0 = model.layers[0].mixer, model.layers[0].feed_forward
        self.rows, self.width = rows, width
        self.nq, self.nkv, self.hd, self.inner, self.scale = m0.n_heads, m0.n_kv_heads, m0.head_dim, f0.inner, m0.scale
        self.ctas = torch.cuda.get_device_properties(dev).multi_processor_count
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.x = torch.zeros((rows, width), **bf)
        self.xn = torch.zeros((rows, width), **bf)
        self.qkv = torch.zeros((rows, (self.nq + 2 * self.nkv) * self.hd), **bf)
        self.attn = torch.zeros((rows, self.nq * self.hd), **bf)
        self.act = torch.zeros((rows, self.inner), **bf)
        size = self.fam.cdll.decode_layer_args_bytes()
        n = len(model.layers)
        raw = np.zeros((n * size + 64,), dtype=np.uint8)
        off = (-raw.ctypes.data) % 64
        host = raw[off:off + n * size]
        gemm_floats = gemm_counters = 0
        plan = (ctypes.c_longlong * 4)()
        for i, (block, call) in enumerate(zip(model.layers, model.program)):
            mixer, ffn = block.mixer, block.feed_forward
            group = cache.group_of[call.cache]
            gi = cache.groups.index(group)
            entry = group.index_of[call.cache]
            table = decoder.tables[gi]
            denom = mixer.position.denominators()
            n1, n2 = block.norm1.tensors["weight"], block.norm2.tensors["weight"]
            dst = host.ctypes.data + i * size
            self.fam.call("decode_layer_fill", dst, rows, width, self.nq, self.nkv, self.hd, self.inner,
                          _ptr(mixer.w_qkv), _ptr(mixer.b_qkv), code_of(mixer.b_qkv.dtype) if mixer.b_qkv is not None else 0,
                          _ptr(mixer.w_o), _ptr(ffn.w_gate_up), _ptr(ffn.w_down), _ptr(n1), code_of(n1.dtype),
                          float(block.norm1.eps), _ptr(n2), code_of(n2.dtype), float(block.norm2.eps), _ptr(self.x),
                          _ptr(self.xn), _ptr(self.qkv), _ptr(self.attn), _ptr(self.act), _ptr(group.k_pool[entry]),
                          _ptr(group.v_pool[entry]), _ptr(table), table.shape[1], mixer.window or 0, _ptr(denom),
                          mixer.position.rotary_dim if denom is not None else 0, self.ctas)
            self.fam.call("decode_layer_scratch", dst, rows, self.nq, self.nkv, self.hd, 1, ctypes.addressof(plan))
            gemm_floats, gemm_counters = max(gemm_floats, plan[0]), max(gemm_counters, plan[1])
        self._host_keepalive = raw
        self.layers = torch.from_numpy(host.copy()).to(dev)
        assert self.layers.data_ptr() % 64 == 0
        self.n_layers = n
        self.max_splits = 32
        row_tiles = (self.nq // self.nkv + 15) // 16
        self.items_base = rows * self.nkv * row_tiles
        self.gemm_scratch = torch.empty((max(int(gemm_floats), 4),), dtype=torch.float32, device=dev)
        self.gemm_counters = torch.zeros((max(int(gemm_counters), 4),), dtype=torch.int32, device=dev)
        self.attn_scratch = torch.empty((rows * self.nq * self.max_splits * (self.hd + 2),), dtype=torch.float32, device=dev)
        self.attn_counters = torch.zeros((self.items_base + 4,), dtype=torch.int32, device=dev)
        self.grid_bars = torch.zeros((32,), dtype=torch.int32, device=dev)
        self.status = torch.zeros((4,), dtype=torch.int32, device=dev)
        # FRIDAY_PROFILE=1, as in the reference (transformer.cpp:603-613): times of the phases of every layer
        self.trace = (torch.zeros((n * 8 + 1,), dtype=torch.int64, device=dev)
                      if os.environ.get("FRIDAY_PROFILE", "0") == "1" else None)

    def splits_for(self, bound):
        """CTAs that share one sequence's keys: enough to give every SM an item, a few blocks of keys each."""
        blocks = (bound + PAGE - 1) // PAGE
        return int(max(1, min(self.ctas // self.items_base, blocks // 2, self.max_splits)))

    def run(self, row_seq, row_pos, bound):
        """All layers on self.x, in place."""
        self.fam.call("decode_layers_run", _ptr(self.layers), self.n_layers, _ptr(self.x), _ptr(self.xn), _ptr(self.qkv),
                      _ptr(self.attn), _ptr(row_seq), _ptr(row_pos), _ptr(self.gemm_scratch), _ptr(self.gemm_counters),
                      _ptr(self.attn_scratch), _ptr(self.attn_counters), self.splits_for(bound), _ptr(self.grid_bars),
                      _ptr(self.status), _ptr(self.trace), self.rows, self.width, self.nq, self.nkv, self.hd, float(self.scale), self.ctas,
                      torch.cuda.current_stream().cuda_stream)
        return self.x

    PHASES = ("norm1", "qkv", "rotary+cache", "attention", "o_proj", "norm2", "gate_up", "down")

    def phase_times(self):
        """With FRIDAY_PROFILE=1: microseconds that CTA 0 spent in each phase (barrier included), mean over layers."""
        if self.trace is None:
            return None
        t = self.trace.cpu().numpy().astype(np.float64)
        d = np.diff(t).reshape(self.n_layers, 8) / 1e3
        return {name: float(d[:, i].mean()) for i, name in enumerate(self.PHASES)}

    def check(self):
        code = int(self.status[0].item())
        if code:
            self.status.zero_()
            self.grid_bars.zero_()
            self.gemm_counters.zero_()
            self.attn_counters.zero_()
            raise lib.KernelError("the fused decode kernel gave up waiting (code %d: 1-4 product pipeline, 5 producer, "
                                  "16+ grid barrier); its results are not valid" % code)
