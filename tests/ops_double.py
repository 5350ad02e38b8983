"""A stand-in for the kernel layer, for tests that run where there is no GPU.

It offers the same functions as the package's CudaOps, written with plain torch
operations on CPU tensors, in float64 inside.  It is not part of the product and the
product never loads it: tests install it with ops.set_backend to exercise the code
around the kernels (cache, pages, step function, generation loop, trace replay).
The kernels themselves are tested on the GPU against the plain implementation.
"""
import numpy as np
import torch

from plain_model import philox4x32  # noqa: F401  (kept here so that tests share one Philox)
import plain_model


class TorchOps:
    name = "torch-double"

    def embedding(self, tokens, table, out=None):
        if out is not None:
            out.copy_(table[tokens.long()])
            return out
        return table[tokens.long()]

    def gather_rows(self, rows, src):
        return src[rows.long()]

    def rmsnorm(self, x, weight, eps, out=None):
        xd = x.double()
        y = xd * (1.0 / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps)) * weight.double()
        return y.to(x.dtype)

    def swiglu(self, gate_up):
        g, u = gate_up[:, 0::2].double(), gate_up[:, 1::2].double()      # columns alternate gate, up
        return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)

    def linear_swiglu(self, x, weight_pairs):
        return self.swiglu(self.linear(x, weight_pairs))

    def rope_kv_write(self, qkv, row_seq, row_pos, denom, rotary_dim, n_heads, n_kv_heads, head_dim,
                      k_pool=None, v_pool=None, block_table=None, page_size=0):
        rows = qkv.shape[0]
        v3 = qkv.view(rows, n_heads + 2 * n_kv_heads, head_dim)
        live = row_seq >= 0
        if denom is not None:
            half = rotary_dim // 2
            ang = (row_pos.to(torch.float32)[:, None] / denom[None, :]).double()   # fp32 division, as the kernel
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            qk = v3[:, : n_heads + n_kv_heads, :].double()
            a, b = qk[..., :half].clone(), qk[..., half:rotary_dim].clone()
            qk[..., :half] = a * c - b * s
            qk[..., half:rotary_dim] = a * s + b * c
            v3[live, : n_heads + n_kv_heads, :] = qk[live].to(qkv.dtype)
        if k_pool is not None:
            for r in range(rows):
                if row_seq[r] < 0:
                    continue
                pos = int(row_pos[r])
                page = int(block_table[int(row_seq[r]), pos // page_size])
                assert page >= 0, "write to a page that is not held"
                k_pool[page, pos % page_size] = v3[r, n_heads:n_heads + n_kv_heads]
                v_pool[page, pos % page_size] = v3[r, n_heads + n_kv_heads:]

    def advance(self, tokens, sampled, row_pos, kv_len, row_seq, draws=None):
        if draws is not None:
            draws += 1
        live = row_seq >= 0
        tokens[live] = sampled[live]
        row_pos[live] += 1
        kv_len[live] += 1

    def linear(self, x, weight, bias=None, residual=None, out_dtype=None, out=None):
        y = x.double() @ weight.double().t()
        if bias is not None:
            y = y + bias.double()
        if residual is not None:
            y = y + residual.double()
        y = y.to(out_dtype or x.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def linear_norm(self, x, weight, norm_weight, eps, bias=None, residual=None):
        out = self.linear(x, weight, bias=bias, residual=residual)
        return out, self.rmsnorm(out, norm_weight, eps)

    def qkv_rope_write(self, x, weight, bias, row_seq, row_pos, denom, rotary_dim, n_heads, n_kv_heads, head_dim,
                       k_pool=None, v_pool=None, block_table=None, page_size=0):
        qkv = self.linear(x, weight, bias=bias)
        if denom is not None or k_pool is not None:
            self.rope_kv_write(qkv, row_seq, row_pos, denom, rotary_dim, n_heads, n_kv_heads, head_dim, k_pool, v_pool,
                               block_table, page_size)
        return qkv

    def attention(self, q, q_stride, out, k_pool, v_pool, block_table, page_size, row_seq, row_pos, n_heads,
                  n_kv_heads, head_dim, window, scale, geometry):
        rows = out.shape[0]
        g = n_heads // n_kv_heads
        for r in range(rows):
            if row_seq[r] < 0:
                out[r] = 0
                continue
            pos = int(row_pos[r])
            lo = max(0, pos - window + 1) if window else 0
            js = list(range(lo, pos + 1))
            pages = [int(block_table[int(row_seq[r]), j // page_size]) for j in js]
            assert all(p >= 0 for p in pages), "read of a page that is not held"
            k = torch.stack([k_pool[p, j % page_size] for p, j in zip(pages, js)]).double()   # [n, nkv, hd]
            v = torch.stack([v_pool[p, j % page_size] for p, j in zip(pages, js)]).double()
            qr = q[r, : n_heads * head_dim].view(n_heads, head_dim).double()
            for h in range(n_heads):
                s = (k[:, h // g, :] @ qr[h]) * scale
                p_ = torch.softmax(s, dim=0)
                out[r, h * head_dim:(h + 1) * head_dim] = (p_ @ v[:, h // g, :]).to(out.dtype)

    def sample(self, logits, temperature, streams, steps, seed, row_live=None, out=None):
        res = []
        for r in range(logits.shape[0]):
            if row_live is not None and row_live[r] < 0:
                res.append(0)
                continue
            res.append(plain_model.sample(logits[r].double().numpy(), float(temperature[r]), int(seed),
                                          int(streams[r]), int(steps[r])))
        t = torch.tensor(res, dtype=torch.int32)
        if out is not None:
            out.copy_(t)
            return out
        return t
