"""The library's operations, callable on torch tensors: what the tests of single kernels
and the measurements use.  Every function marshals its arguments to the C++ operation of
the same name (ops/ops.cpp, include/friday/ops.h), which chooses and launches this
library's own CUDA kernels; nothing is computed here, and there is no CPU path.

Kernels run on the legacy default stream, which is also torch's default, so they are
ordered with the torch operations around them.
"""
from ctypes import byref, c_int, c_void_p

from .. import native

_CODES = None


def _codes():
    global _CODES
    if _CODES is None:
        import torch
        _CODES = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2}
    return _CODES


def _t(t):
    """FridayTensor for a torch tensor (None -> a null pointer)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise native.KernelError("tensor on %s: this library runs on CUDA devices only, it has no CPU path" % t.device)
    try:
        code = _codes()[t.dtype]
    except KeyError:
        raise native.KernelError("no kernel for dtype %s (float32 and bfloat16 only)" % t.dtype) from None
    if t.dim() > 4 or t.dim() < 1 or t.stride(-1) != 1:
        raise native.KernelError("tensors must have 1 to 4 dimensions and unit inner stride, got shape %s strides %s"
                          % (tuple(t.shape), t.stride()))
    if t.dim() > 2 and not t.is_contiguous():
        raise native.KernelError("tensors of more than two dimensions must be contiguous")
    d = native.Tensor()
    d.data, d.dtype, d.ndim = t.data_ptr(), code, t.dim()
    for i, s in enumerate(t.shape):
        d.shape[i] = s
    d.ld = t.stride(0) if t.dim() == 2 else t.shape[-1]
    return d


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def _ref(struct):
    return None if struct is None else byref(struct)


class DeferredNorm:
    """Rows whose RMSNorm is half done by the product that made them (friday::Rows): `scaled` holds weight (*) x
    rounded to bf16, `ssq` [parts, rows] each part's share of the rows' sums of squares."""

    def __init__(self, scaled, ssq, eps, source, weight):
        self.scaled, self.ssq, self.eps, self.source, self.weight = scaled, ssq, float(eps), source, weight
        self.shape, self.dtype, self.device = scaled.shape, scaled.dtype, scaled.device

    def materialize(self):
        return rmsnorm(self.source, self.weight, self.eps)


def materialize(h):
    return h.materialize() if isinstance(h, DeferredNorm) else h


def _rows(x):
    """(tensor, ssq or None, eps, source, weight) of plain or deferred rows."""
    if isinstance(x, DeferredNorm):
        return x.scaled, x.ssq, x.eps, x.source, x.weight
    return x, None, 0.0, None, None


def _kv(k_pool, v_pool, block_table, page_size, window=None, write=True):
    if k_pool is None:
        return None
    kv = native.KV()
    kv.k_pool, kv.v_pool = k_pool.data_ptr(), v_pool.data_ptr()
    kv.pool_pages = k_pool.shape[0]
    kv.block_table = block_table.data_ptr()
    kv.table_width = block_table.shape[1]
    kv.page_size = int(page_size)
    kv.window = int(window or 0)
    kv.n_kv_heads, kv.head_dim = k_pool.shape[-2], k_pool.shape[-1]
    kv.dtype = _codes()[k_pool.dtype]
    kv.write = 1 if write else 0
    return kv


class CudaOps:
    """The handle of the library's operations on one device."""

    name = "cuda"

    def __init__(self, device=0):
        self._h = c_void_p()
        native.call("friday_ops_new", int(device), None, byref(self._h))

    def __del__(self):
        if getattr(self, "_h", None) and native is not None and native._lib is not None:      # None at interpreter exit
            native._lib.friday_ops_free(self._h)
            self._h = None

    def info(self):
        return native.call_json("friday_ops_info", self._h)

    def check_status(self):
        native.call("friday_ops_check_status", self._h)

    # -- row-wise ---------------------------------------------------------
    def embedding(self, tokens, table, out=None):
        import torch
        if out is None:
            out = torch.empty((tokens.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
        native.call("friday_ops_embedding", self._h, _p(tokens), tokens.numel(), _t(table), _t(out))
        return out

    def gather_rows(self, rows, src):
        import torch
        out = torch.empty((rows.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
        native.call("friday_ops_gather_rows", self._h, _p(rows), rows.numel(), _t(src), _t(out))
        return out

    def rmsnorm(self, x, weight, eps, out=None):
        import torch
        if out is None:
            out = torch.empty_like(x)
        native.call("friday_ops_rmsnorm", self._h, _t(x), _t(weight), float(eps), _t(out))
        return out

    def swiglu(self, gate_up):
        import torch
        out = torch.empty((gate_up.shape[0], gate_up.shape[1] // 2), dtype=gate_up.dtype, device=gate_up.device)
        native.call("friday_ops_swiglu", self._h, _t(gate_up), _t(out))
        return out

    def rope_kv_write(self, qkv, row_seq, row_pos, denom, rotary_dim, n_heads, n_kv_heads, head_dim, k_pool=None,
                      v_pool=None, block_table=None, page_size=0):
        kv = _kv(k_pool, v_pool, block_table, page_size)
        native.call("friday_ops_rope_kv_write", self._h, _t(qkv), _p(row_seq), _p(row_pos), _p(denom), int(rotary_dim),
                    n_heads, n_kv_heads, head_dim, _ref(kv))

    def advance(self, tokens, sampled, row_pos, kv_len, row_seq, draws=None):
        native.call("friday_ops_advance", self._h, _p(tokens), _p(sampled), _p(row_pos), _p(kv_len), _p(row_seq),
                    _p(draws), tokens.numel())

    def scale_rows(self, x, scale):
        native.call("friday_ops_scale_rows", self._h, _t(x), float(scale))
        return x

    def finish_logits(self, logits, bias=None, scale=1.0, softcap=0.0):
        native.call("friday_ops_finish_logits", self._h, _t(logits), _t(bias), float(scale), float(softcap))
        return logits

    # -- matrix products --------------------------------------------------
    def linear(self, x, weight, bias=None, residual=None, out_dtype=None, out=None):
        import torch
        xt, ssq, eps, source, nw = _rows(x)
        if out is None:
            out = torch.empty((xt.shape[0], weight.shape[0]), dtype=out_dtype or xt.dtype, device=xt.device)
        native.call("friday_ops_linear", self._h, _t(xt), _t(ssq), float(eps), _t(source), _t(nw), _t(weight), _t(bias),
                    _t(residual), _t(out))
        return out

    def _linear_tc(self, x, weight, bias, residual, out, swap=-1, bn=-1, splits=-1, act=0):
        native.call("friday_ops_linear_tc", self._h, _t(x), _t(weight), _t(bias), _t(residual), _t(out), swap, bn, splits, act)
        return out

    def _linear_simt(self, x, weight, bias, residual, out):
        native.call("friday_ops_linear_simt", self._h, _t(x), _t(weight), _t(bias), _t(residual), _t(out))
        return out

    def linear_norm(self, x, weight, norm_weight, eps, bias=None, residual=None):
        import torch
        xt, ssq, in_eps, _, _ = _rows(x)
        rows, n = xt.shape[0], weight.shape[0]
        out = torch.empty((rows, n), dtype=xt.dtype, device=xt.device)
        normed = torch.empty_like(out)
        parts = torch.empty((max(n // 16, 1), rows), dtype=torch.float32, device=xt.device)
        parts_d = _t(parts)
        deferred = c_int()
        native.call("friday_ops_linear_norm", self._h, _t(xt), _t(ssq), float(in_eps), _t(weight), _t(norm_weight),
                    float(eps), _t(bias), _t(residual), _t(out), _t(normed), parts_d, byref(deferred))
        if deferred.value:
            return out, DeferredNorm(normed, parts[:parts_d.shape[0]], eps, out, norm_weight)
        return out, normed

    def qkv_rope_write(self, x, weight, bias, row_seq, row_pos, denom, rotary_dim, n_heads, n_kv_heads, head_dim,
                       k_pool=None, v_pool=None, block_table=None, page_size=0):
        import torch
        xt, ssq, in_eps, _, _ = _rows(x)
        out = torch.empty((xt.shape[0], weight.shape[0]), dtype=xt.dtype, device=xt.device)
        kv = _kv(k_pool, v_pool, block_table, page_size)
        native.call("friday_ops_qkv_rope_write", self._h, _t(xt), _t(ssq), float(in_eps), _t(weight), _t(bias),
                    _p(row_seq), _p(row_pos), _p(denom), int(rotary_dim), n_heads, n_kv_heads, head_dim, _ref(kv), _t(out))
        return out

    def linear_swiglu(self, x, weight_pairs):
        import torch
        xt, ssq, in_eps, _, _ = _rows(x)
        out = torch.empty((xt.shape[0], weight_pairs.shape[0] // 2), dtype=xt.dtype, device=xt.device)
        native.call("friday_ops_linear_swiglu", self._h, _t(xt), _t(ssq), float(in_eps), _t(weight_pairs), _t(out))
        return out

    def tensor_core_ok(self, x, weight, out, residual=None):
        ok = c_int()
        native.call("friday_ops_tensor_core_ok", self._h, _t(x), _t(weight), _t(out), byref(ok))
        return bool(ok.value)

    def plan(self, rows, n, k):
        """(operands swapped, tile width, splits of k) that the tensor-core product chooses for a shape."""
        s, bn, sp = c_int(), c_int(), c_int()
        native.call("friday_ops_plan", self._h, rows, n, k, byref(s), byref(bn), byref(sp))
        return bool(s.value), bn.value, sp.value

    # -- attention --------------------------------------------------------
    def attention(self, q, q_stride, out, k_pool, v_pool, block_table, page_size, row_seq, row_pos, n_heads, n_kv_heads,
                  head_dim, window, scale, geometry):
        """geometry: an object with max_kv_len and, for the tensor-core kernels, n_seqs, max_q_len, decode and the
        per-sequence arrays seq_start, seq_qlen, seq_pos0 (int32, device)."""
        g = native.Geometry()
        g.rows = out.shape[0]
        g.n_seqs = int(getattr(geometry, "n_seqs", 0))
        g.max_q_len = int(getattr(geometry, "max_q_len", 0))
        g.max_kv_len = int(geometry.max_kv_len)
        g.decode = 1 if getattr(geometry, "decode", False) else 0
        g.row_seq, g.row_pos = row_seq.data_ptr(), row_pos.data_ptr()
        for name in ("seq_start", "seq_qlen", "seq_pos0"):
            t = getattr(geometry, name, None)
            setattr(g, name, None if t is None else t.data_ptr())
        kv = _kv(k_pool, v_pool, block_table, page_size, window, write=False)
        native.call("friday_ops_attention", self._h, _t(q), int(q_stride), _t(out), byref(kv), byref(g), n_heads,
                    n_kv_heads, head_dim, int(window or 0), float(scale))

    def decode_splits(self, n_seqs, n_heads, n_kv_heads, head_dim, max_kv_len):
        s = c_int()
        native.call("friday_ops_decode_splits", self._h, n_seqs, n_heads, n_kv_heads, head_dim, max_kv_len, byref(s))
        return s.value

    def attention_splits(self, rows, n_heads, max_kv_len):
        s = c_int()
        native.call("friday_ops_attention_splits", self._h, rows, n_heads, max_kv_len, byref(s))
        return s.value

    # -- one attention kernel's launcher, called directly with chosen arguments (tests of that kernel alone) -----
    def _test_buffers(self, device):
        import torch
        if getattr(self, "_tb", None) is None:
            self._tb = (torch.zeros((1 << 16,), dtype=torch.int32, device=device),
                        torch.zeros((4,), dtype=torch.int32, device=device))
        return self._tb

    def attention_tc(self, q, q_stride, out, k_pool, v_pool, block_table, seq_start, seq_qlen, seq_pos0, seq_live,
                     n_seqs, max_q_len, n_heads, n_kv_heads, head_dim, window, scale):
        from . import lib
        status = self._test_buffers(q.device)[1]
        lib.family("attention_tc").call(
            "attention_tc", q.data_ptr(), q_stride, q.shape[0], out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
            k_pool.shape[0], block_table.data_ptr(), block_table.shape[1], seq_start.data_ptr(), seq_qlen.data_ptr(),
            seq_pos0.data_ptr(), 0 if seq_live is None else seq_live.data_ptr(), n_seqs, max_q_len, n_heads, n_kv_heads,
            head_dim, window or 0, float(scale), status.data_ptr(), None)
        if int(status[0].item()):
            status.zero_()
            raise native.KernelError("the tcgen05 attention kernel gave up on one of its bounded waits")

    def attention_mma(self, q, q_stride, out, k_pool, v_pool, block_table, seq_start, seq_qlen, seq_pos0, seq_live,
                      n_seqs, max_q_len, n_heads, n_kv_heads, head_dim, window, scale, keys_mode, splits, geometry=None):
        import torch
        from . import lib
        rows = out.shape[0]
        counters, status = self._test_buffers(q.device)
        scratch = None
        if splits > 1:
            scratch = torch.empty((rows * n_heads * splits * (head_dim + 2),), dtype=torch.float32, device=q.device)
        lib.family("attention_mma").call(
            "attention_mma", q.data_ptr(), q_stride, out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0],
            block_table.data_ptr(), block_table.shape[1], 64, seq_start.data_ptr(), seq_qlen.data_ptr(),
            seq_pos0.data_ptr(), 0 if seq_live is None else seq_live.data_ptr(), n_seqs, rows, max_q_len, n_heads,
            n_kv_heads, head_dim, window or 0, float(scale), 1 if keys_mode else 0, splits,
            0 if scratch is None else scratch.data_ptr(), counters.data_ptr(), counters.numel(), status.data_ptr(), None)

    # -- sampling ---------------------------------------------------------
    def sample(self, logits, temperature, streams, steps, seed, row_live=None, out=None):
        import torch
        if out is None:
            out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        native.call("friday_ops_sample", self._h, _t(logits), _p(temperature), _p(streams), _p(steps),
                    int(seed) & 0xFFFFFFFFFFFFFFFF, _p(row_live), _p(out))
        return out


_backend = None


def backend():
    global _backend
    if _backend is None:
        _backend = CudaOps()
    return _backend


def fusion_enabled():
    """FRIDAY_FUSE=0 keeps norms, rotation and cache write in kernels of their own (for comparison)."""
    return backend().info()["fusion"]


def launch_count():
    return backend().info()["launches"]


def __getattr__(name):
    if name == "lib":          # direct access to the kernel libraries' C entry points, for tests of those
        import importlib
        return importlib.import_module(".lib", __name__)
    raise AttributeError(name)


def embedding(*a, **k):
    return backend().embedding(*a, **k)


def gather_rows(*a, **k):
    return backend().gather_rows(*a, **k)


def rmsnorm(*a, **k):
    return backend().rmsnorm(*a, **k)


def swiglu(*a, **k):
    return backend().swiglu(*a, **k)


def linear_swiglu(*a, **k):
    return backend().linear_swiglu(*a, **k)


def rope_kv_write(*a, **k):
    return backend().rope_kv_write(*a, **k)


def advance(*a, **k):
    return backend().advance(*a, **k)


def linear(*a, **k):
    return backend().linear(*a, **k)


def linear_norm(*a, **k):
    return backend().linear_norm(*a, **k)


def qkv_rope_write(*a, **k):
    return backend().qkv_rope_write(*a, **k)


def attention(*a, **k):
    return backend().attention(*a, **k)


def sample(*a, **k):
    return backend().sample(*a, **k)
