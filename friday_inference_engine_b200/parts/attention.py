"""Grouped-query attention over the paged cache.

q = Wq h + bq, k = Wk h + bk, v = Wv h + bv (one product over the stacked matrices);
q and k are encoded with the position part; k and v go to the cache at each row's
(sequence, position); every query attends to the keys of its sequence up to its own
position, or to the last `window` of them; the result goes through Wo and the residual
is added in that product's epilogue.

Reference order of operations: transformer.cpp:1013-1059 (norm is the block's), q/k/v
bias in the product's epilogue (hpc_k_quants.cu:422-437), rotation and cache write in
one kernel (cuda_math_kernels.cu:363-404), grouped heads h -> h / (heads / kv heads)
and 1/sqrt(head_dim) scaling (attention_kernels.cu:45, cpu_ops.cpp:49-53), the output
product with the residual (transformer.cpp:1057-1059).
"""
import torch

from .. import ops
from .base import KVRequest, Part, build_part, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    category = "mixer"

    def __init__(self, env, n_heads, n_kv_heads, head_dim, position, qkv_bias=True, out_bias=False, window=None,
                 scale=None):
        super().__init__(env)
        if n_heads % n_kv_heads:
            raise ValueError("%d heads cannot share %d key/value heads" % (n_heads, n_kv_heads))
        self.n_heads, self.n_kv_heads, self.head_dim = int(n_heads), int(n_kv_heads), int(head_dim)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.qkv_bias, self.out_bias = bool(qkv_bias), bool(out_bias)
        self.position = self.adopt("", build_part("position", position, env))
        qd, kvd, w = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, env.width
        for name, rows in (("q_proj", qd), ("k_proj", kvd), ("v_proj", kvd)):
            self.declare(name + ".weight", (rows, w))
            if self.qkv_bias:
                self.declare(name + ".bias", (rows,))
        self.declare("o_proj.weight", (w, qd))
        if self.out_bias:
            self.declare("o_proj.bias", (w,))

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self.window)

    def finalize(self):
        super().finalize()
        t = self.tensors
        ws = [t.pop(n + ".weight") for n in ("q_proj", "k_proj", "v_proj")]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_qkv = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        self.b_qkv = None
        if self.qkv_bias:
            bs = [t.pop(n + ".bias") for n in ("q_proj", "k_proj", "v_proj")]
            bdt = torch.float32 if any(b.dtype == torch.float32 for b in bs) else bs[0].dtype
            self.b_qkv = torch.cat([b.to(bdt) for b in bs], dim=0).contiguous()
        self.w_o = t["o_proj.weight"]
        self.b_o = t.get("o_proj.bias")

    chains_norm = True

    def forward(self, h, residual, ctx, cache, then=None):
        nq, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        write = cache.write
        pools = (cache.k_pool, cache.v_pool, cache.block_table) if write else (None, None, None)
        if getattr(self.position, "rotary", False):
            qkv = ops.qkv_rope_write(h, self.w_qkv, self.b_qkv, ctx.row_seq, ctx.row_pos, self.position.denominators(),
                                     self.position.rotary_dim, nq, nkv, hd, *pools, cache.page_size)
        else:                                   # another encoding: it changes q and k itself
            qkv = ops.linear(h, self.w_qkv, bias=self.b_qkv)
            self.position.apply(qkv, ctx, nq, nkv, hd)
            if write:
                ops.rope_kv_write(qkv, ctx.row_seq, ctx.row_pos, None, 0, nq, nkv, hd, *pools, cache.page_size)
        mixed = torch.empty((qkv.shape[0], nq * hd), dtype=qkv.dtype, device=qkv.device)
        ops.attention(qkv, qkv.stride(0), mixed, cache.k_pool, cache.v_pool, cache.block_table, cache.page_size,
                      ctx.row_seq, ctx.row_pos, nq, nkv, hd, self.window, self.scale, ctx)
        norm = then.as_rmsnorm() if then is not None else None
        if norm is not None:
            return ops.linear_norm(mixed, self.w_o, norm[0], norm[1], bias=self.b_o, residual=residual)
        return ops.linear(mixed, self.w_o, bias=self.b_o, residual=residual), None
