"""The operations that parts are made of, as functions on torch tensors.

Every function launches this library's own CUDA kernels on the current stream of the
tensors' device.  Tensors must live on a CUDA device: there is no CPU path, and a
kernel library that cannot be built or loaded is an error.

`set_backend` swaps the implementation object; the package itself never calls it.  It
exists so that tests of the code *around* the kernels (cache, step function, loop) can
run where there is no GPU, with a stand-in defined in the tests.
"""
import numpy as np
import torch

from . import lib
from .lib import KernelError

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def code_of(dtype):
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError("no kernel for dtype %s (float32 and bfloat16 only)" % dtype) from None


def _ptr(t):
    return 0 if t is None else t.data_ptr()


_raw_current_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle.  A prompt's pass launches some 170 kernels from Python: the direct query costs a
    fraction of a microsecond where building a torch.cuda.Stream object each time cost half of the pass's host time."""
    if _raw_current_stream is not None:
        return _raw_current_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("tensor on %s: this library runs on CUDA devices only, it has no CPU path" % t.device)


class DeferredNorm:
    """Rows whose RMSNorm is half done by the product that made them: `scaled` holds weight (*) x rounded to
    bf16, `ssq` [parts, rows] each part's share of the rows' sums of squares.  The product that takes the rows
    finishes the norm by scaling its own rows with 1 / sqrt(sum / width + eps); anything else asks for
    `materialize()`, which runs the norm's kernel on the rows themselves."""

    def __init__(self, scaled, ssq, eps, source, weight):
        self.scaled, self.ssq, self.eps, self.source, self.weight = scaled, ssq, float(eps), source, weight
        self.shape, self.dtype, self.device = scaled.shape, scaled.dtype, scaled.device

    def materialize(self):
        return rmsnorm(self.source, self.weight, self.eps)


def materialize(h):
    """The plain tensor behind what a product returned as normed rows."""
    return h.materialize() if isinstance(h, DeferredNorm) else h


def fusion_enabled():
    """FRIDAY_FUSE=0 keeps norms, rotation and cache write in kernels of their own (for comparison)."""
    import os
    return os.environ.get("FRIDAY_FUSE", "1") != "0"


def _rowmajor(t, what):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError("%s must be a 2-d tensor with unit inner stride, got shape %s strides %s"
                          % (what, tuple(t.shape), t.stride()))


class CudaOps:
    """The product's implementation: ctypes calls into the libraries built from csrc/."""

    name = "cuda"

    def __init__(self):
        self._tc = {}
        self._attn_counters = {}
        self._plans = {}
        self._cluster_fit = {}

    # -- row-wise ---------------------------------------------------------
    def embedding(self, tokens, table, out=None):
        _need_cuda(tokens, table)
        assert tokens.dtype == torch.int32 and tokens.is_contiguous() and table.is_contiguous()
        if out is None:
            out = torch.empty((tokens.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
        lib.family("rowwise").call("rowwise_embedding", _ptr(tokens), _ptr(table), _ptr(out), tokens.numel(),
                                   table.shape[1], code_of(table.dtype), _stream())
        return out

    def gather_rows(self, rows, src):
        _need_cuda(rows, src)
        assert rows.dtype == torch.int32 and src.is_contiguous()
        out = torch.empty((rows.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
        lib.family("rowwise").call("rowwise_gather_rows", _ptr(rows), _ptr(src), _ptr(out), rows.numel(),
                                   src.shape[1], code_of(src.dtype), _stream())
        return out

    def rmsnorm(self, x, weight, eps, out=None):
        _need_cuda(x, weight)
        assert x.is_contiguous() and weight.is_contiguous() and weight.numel() == x.shape[-1]
        if out is None:
            out = torch.empty_like(x)
        rows = x.numel() // x.shape[-1]
        lib.family("rowwise").call("rowwise_rmsnorm", _ptr(x), _ptr(weight), code_of(weight.dtype), _ptr(out), rows,
                                   x.shape[-1], float(eps), code_of(x.dtype), _stream())
        return out

    def swiglu(self, gate_up):
        _need_cuda(gate_up)
        assert gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
        inner = gate_up.shape[1] // 2
        out = torch.empty((gate_up.shape[0], inner), dtype=gate_up.dtype, device=gate_up.device)
        lib.family("rowwise").call("rowwise_swiglu", _ptr(gate_up), _ptr(out), gate_up.shape[0], inner,
                                   code_of(gate_up.dtype), _stream())
        return out

    def rope_kv_write(self, qkv, row_seq, row_pos, denom, rotary_dim, n_heads, n_kv_heads, head_dim,
                      k_pool=None, v_pool=None, block_table=None, page_size=0):
        """Rotates q and k inside `qkv` [rows, (nq + 2 nkv) * hd] (denom None: no rotation) and, if
        pools are given, writes k and v to the cache rows of (row_seq, row_pos)."""
        _need_cuda(qkv, row_seq, row_pos)
        assert qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
        write = k_pool is not None
        if write:
            assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
            assert k_pool.is_contiguous() and v_pool.is_contiguous() and block_table.dim() == 2
        if denom is not None:
            assert denom.dtype == torch.float32 and denom.numel() == rotary_dim // 2
        lib.family("rowwise").call(
            "rowwise_rope_kv_write", _ptr(qkv), _ptr(row_seq), _ptr(row_pos), _ptr(denom), rotary_dim, n_heads,
            n_kv_heads, head_dim, _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
            block_table.shape[1] if write else 0, page_size, 1 if write else 0, qkv.shape[0], code_of(qkv.dtype),
            _stream())

    def advance(self, tokens, sampled, row_pos, kv_len, row_seq, draws=None):
        lib.family("rowwise").call("rowwise_advance", _ptr(tokens), _ptr(sampled), _ptr(row_pos), _ptr(kv_len),
                                   _ptr(row_seq), _ptr(draws), tokens.numel(), _stream())

    # -- matrix products --------------------------------------------------
    def linear(self, x, weight, bias=None, residual=None, out_dtype=None, out=None):
        """x [rows, k] @ weight [n, k]^T (+ bias [n]) (+ residual [rows, n]).  x may be a DeferredNorm."""
        deferred = x if isinstance(x, DeferredNorm) else None
        if deferred is not None:
            x = deferred.scaled
        _need_cuda(x, weight, bias, residual)
        _rowmajor(x, "linear input")
        _rowmajor(weight, "linear weight")
        rows, k = x.shape
        n = weight.shape[0]
        if weight.shape[1] != k:
            raise KernelError("linear: input has %d columns, weight %s" % (k, tuple(weight.shape)))
        out_dtype = out_dtype or x.dtype
        if out is None:
            out = torch.empty((rows, n), dtype=out_dtype, device=x.device)
        if residual is not None:
            assert residual.shape == out.shape and residual.dtype == out.dtype and residual.stride() == out.stride()
        if self.tensor_core_ok(x, weight, out, residual):
            return self._linear_tc(x, weight, bias, residual, out, fusion=self._fusion_in(deferred))
        if deferred is not None:
            x = deferred.materialize()
        self._linear_simt(x, weight, bias, residual, out)
        return out

    @staticmethod
    def _fusion_in(deferred, fusion=None):
        """The fields of the fusion struct that finish a deferred norm of the input."""
        if deferred is None:
            return fusion
        fusion = fusion or lib.GemmFusion()
        fusion.in_ssq, fusion.in_parts = _ptr(deferred.ssq), deferred.ssq.shape[0]
        fusion.in_width, fusion.in_eps = float(deferred.scaled.shape[1]), deferred.eps
        return fusion

    def _plan(self, rows, n, k, device):
        """(operands swapped, tile width) that the tensor-core product will choose for a shape."""
        key = (rows, n, k, device)
        hit = self._plans.get(key)
        if hit is None:
            plan = np.zeros((8,), dtype=np.int64)
            lib.family("gemm_tc").call("gemm_tc_plan", rows, n, k, self._tc_buffers(device)[3], -1, -1, -1, plan.ctypes.data)
            if len(self._plans) > 4096:
                self._plans.clear()
            hit = self._plans[key] = (bool(plan[0]), int(plan[1]))
        return hit

    def _few_rows_tile_ok(self, x, weight, out, residual, max_rows, columns=128):
        """What the fused epilogues of the tensor-core product need: no more rows than max_rows, bf16, whole
        groups of `columns` output columns (128: the tiles of a one-token step's few rows)."""
        return (fusion_enabled() and out.dtype == torch.bfloat16 and x.shape[0] <= max_rows and weight.shape[0] % columns == 0
                and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
                and (residual is None or residual.data_ptr() % 16 == 0)
                and self.tensor_core_ok(x, weight, out, residual))

    def linear_norm(self, x, weight, norm_weight, eps, bias=None, residual=None):
        """linear(...) and the RMSNorm of its result: (out, normed).  For a few bf16 rows the norm is begun in
        the product's epilogue and `normed` is a DeferredNorm that the next product finishes; otherwise the
        norm's kernel runs and `normed` is a tensor."""
        deferred = x if isinstance(x, DeferredNorm) else None
        xt = deferred.scaled if deferred is not None else x
        _need_cuda(xt, weight, bias, residual, norm_weight)
        rows, n = xt.shape[0], weight.shape[0]
        if xt.dim() == 2 and weight.dim() == 2 and xt.shape[1] == weight.shape[1] and norm_weight.numel() == n:
            out = torch.empty((rows, n), dtype=xt.dtype, device=xt.device)
            if self._few_rows_tile_ok(xt, weight, out, residual, 64) and norm_weight.is_contiguous():
                if residual is not None:
                    assert residual.shape == out.shape and residual.dtype == out.dtype and residual.stride() == out.stride()
                scaled = torch.empty_like(out)
                ssq = torch.empty((n // 128, rows), dtype=torch.float32, device=out.device)
                fusion = self._fusion_in(deferred, lib.GemmFusion())
                fusion.norm_w, fusion.norm_w_dtype = _ptr(norm_weight), code_of(norm_weight.dtype)
                fusion.norm_out, fusion.out_ssq = _ptr(scaled), _ptr(ssq)
                self._linear_tc(xt, weight, bias, residual, out, fusion=fusion)
                return out, DeferredNorm(scaled, ssq, eps, out, norm_weight)
            if rows > 64 and n % 16 == 0 and self._few_rows_tile_ok(xt, weight, out, residual, rows, 16) \
                    and norm_weight.is_contiguous():
                # many rows: the rows lie on the tiles' M side and every column tile adds one partial sum per row
                if residual is not None:
                    assert residual.shape == out.shape and residual.dtype == out.dtype and residual.stride() == out.stride()
                swapped, bn = self._plan(rows, n, xt.shape[1], xt.device)
                if not swapped:
                    scaled = torch.empty_like(out)
                    ssq = torch.empty((-(-n // bn), rows), dtype=torch.float32, device=out.device)
                    fusion = self._fusion_in(deferred, lib.GemmFusion())
                    fusion.norm_w, fusion.norm_w_dtype = _ptr(norm_weight), code_of(norm_weight.dtype)
                    fusion.norm_out, fusion.out_ssq = _ptr(scaled), _ptr(ssq)
                    self._linear_tc(xt, weight, bias, residual, out, fusion=fusion)
                    return out, DeferredNorm(scaled, ssq, eps, out, norm_weight)
        out = self.linear(x, weight, bias=bias, residual=residual)
        return out, self.rmsnorm(out, norm_weight, eps)

    def qkv_rope_write(self, x, weight, bias, row_seq, row_pos, denom, rotary_dim, n_heads, n_kv_heads, head_dim,
                       k_pool=None, v_pool=None, block_table=None, page_size=0):
        """linear(x, weight, bias) followed by rope_kv_write on its result, which it returns.  For a few bf16
        rows and a head size that divides 128 both happen in the product's epilogue."""
        deferred = x if isinstance(x, DeferredNorm) else None
        xt = deferred.scaled if deferred is not None else x
        n = weight.shape[0]
        write = k_pool is not None
        if xt.dim() == 2 and weight.dim() == 2 and xt.shape[1] == weight.shape[1] and 128 % head_dim == 0 \
                and head_dim % 8 == 0 and n == (n_heads + 2 * n_kv_heads) * head_dim \
                and (denom is None or rotary_dim % 16 == 0):
            out = torch.empty((xt.shape[0], n), dtype=xt.dtype, device=xt.device)
            if self._few_rows_tile_ok(xt, weight, out, None, 16) and (not write or k_pool.dtype == torch.bfloat16):
                _need_cuda(xt, weight, bias, row_seq, row_pos, denom, k_pool, v_pool, block_table)
                fusion = self._fusion_in(deferred, lib.GemmFusion())
                fusion.row_seq, fusion.row_pos, fusion.denom = _ptr(row_seq), _ptr(row_pos), _ptr(denom)
                fusion.rot, fusion.nq, fusion.nkv, fusion.hd = int(rotary_dim), n_heads, n_kv_heads, head_dim
                if denom is not None:
                    assert denom.dtype == torch.float32 and denom.numel() == rotary_dim // 2
                if write:
                    assert k_pool.is_contiguous() and v_pool.is_contiguous() and block_table.dim() == 2
                    fusion.k_pool, fusion.v_pool, fusion.table = _ptr(k_pool), _ptr(v_pool), _ptr(block_table)
                    fusion.table_width, fusion.page = block_table.shape[1], int(page_size)
                return self._linear_tc(xt, weight, bias, None, out, fusion=fusion)
        qkv = self.linear(x, weight, bias=bias)
        if denom is not None or write:
            self.rope_kv_write(qkv, row_seq, row_pos, denom, rotary_dim, n_heads, n_kv_heads, head_dim, k_pool, v_pool,
                               block_table, page_size)
        return qkv

    # Scratch of the tensor-core product (partial tiles of split-k), its tile counters and the word in which
    # a kernel records a wait that gave up: one set per device, made once, so that captured graphs keep
    # their addresses.  At most two partial tiles of 128 x 256 floats per CTA, one CTA per SM.
    _TC_SCRATCH_FLOATS = 2 * 148 * 128 * 256
    _TC_COUNTERS = 4096

    def _tc_buffers(self, device):
        bufs = self._tc.get(device)
        if bufs is None:
            props = torch.cuda.get_device_properties(device)
            bufs = self._tc[device] = (
                torch.empty((self._TC_SCRATCH_FLOATS,), dtype=torch.float32, device=device),
                torch.zeros((self._TC_COUNTERS,), dtype=torch.int32, device=device),
                torch.zeros((4,), dtype=torch.int32, device=device),
                props.multi_processor_count)
        return bufs

    @staticmethod
    def tensor_core_ok(x, weight, out, residual):
        """The tensor-core kernel takes bf16 operands whose rows start on 16-byte boundaries."""
        return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and out.dtype in (torch.bfloat16, torch.float32)
                and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    # For measurements: a tensor [launches, 148, 16] of int64 that every tensor-core product from now on fills
    # with its CTAs' timestamps, one launch after the other (gemm_tc_fusion.h, part 4); None switches it off.
    trace = None
    trace_next = 0

    def _linear_tc(self, x, weight, bias, residual, out, swap=-1, bn=-1, splits=-1, act=0, fusion=None):
        import ctypes
        scratch, counters, status, sms = self._tc_buffers(x.device)
        rows, k = x.shape
        if self.trace is not None and self.trace_next < self.trace.shape[0]:
            fusion = fusion or lib.GemmFusion()
            fusion.trace = self.trace[self.trace_next].data_ptr()
            self.trace_next += 1
        lib.family("gemm_tc").call(
            "gemm_tc_fused", _ptr(x), _ptr(weight), _ptr(out), code_of(out.dtype), _ptr(bias),
            code_of(bias.dtype) if bias is not None else 0, _ptr(residual), rows, weight.shape[0], k, x.stride(0),
            weight.stride(0), out.stride(0), _ptr(scratch), scratch.numel(), _ptr(counters), counters.numel(),
            _ptr(status), sms, swap, bn, splits, act, ctypes.byref(fusion) if fusion is not None else None, _stream())
        return out

    def linear_swiglu(self, x, weight_pairs):
        """silu(x Wg^T) * (x Wu^T) for weight_pairs [2 * inner, k] whose rows alternate gate, up: one product
        with the activation in its epilogue on the tensor cores, else the product followed by the kernel."""
        deferred = x if isinstance(x, DeferredNorm) else None
        if deferred is not None:
            x = deferred.scaled
        _need_cuda(x, weight_pairs)
        _rowmajor(x, "linear input")
        _rowmajor(weight_pairs, "linear weight")
        rows, inner = x.shape[0], weight_pairs.shape[0] // 2
        out = torch.empty((rows, inner), dtype=x.dtype, device=x.device)
        if self.tensor_core_ok(x, weight_pairs, out, None) and out.dtype == torch.bfloat16:
            return self._linear_tc(x, weight_pairs, None, None, out, act=1, fusion=self._fusion_in(deferred))
        return self.swiglu(self.linear(deferred if deferred is not None else x, weight_pairs))

    def check_status(self):
        """Raises if a kernel recorded that one of its waits gave up (reads one word per device; call it
        where the host waits for the device anyway)."""
        for device, bufs in self._tc.items():
            code = int(bufs[2][0].item())
            if code:
                bufs[2].zero_()
                raise KernelError("a tensor-core kernel on %s gave up waiting (code %d: which of its bounded waits, "
                                  "see gemm_tc.cu and attention_tc.cu); its results are not valid" % (device, code))

    def _linear_simt(self, x, weight, bias, residual, out):
        """The CUDA-core product: true fp32, and the fallback of bf16 for sizes the tensor-core kernel refuses."""
        rows, k = x.shape
        n = weight.shape[0]
        lib.family("gemm_simt").call(
            "gemm_simt", _ptr(x), code_of(x.dtype), _ptr(weight), code_of(weight.dtype), _ptr(out),
            code_of(out.dtype), _ptr(bias), code_of(bias.dtype) if bias is not None else 0, _ptr(residual), rows, n,
            k, x.stride(0), weight.stride(0), out.stride(0), _stream())
        return out

    # -- attention --------------------------------------------------------
    def attention(self, q, q_stride, out, k_pool, v_pool, block_table, page_size, row_seq, row_pos, n_heads,
                  n_kv_heads, head_dim, window, scale, geometry):
        """Causal attention of the step's rows over the paged cache.

        q: the buffer that holds the queries, row stride q_stride (elements), head h at h * head_dim.
        geometry: the step's context: max_kv_len and scratch(); for the tensor-core kernel also n_seqs,
        max_q_len, decode and the per-sequence arrays seq_start, seq_qlen, seq_pos0 (int32, device).
        bf16 with a head size the tensor-core kernel is built for goes there; everything else (float32,
        other head sizes, a caller without per-sequence arrays) goes to the CUDA-core kernel.
        """
        _need_cuda(q, out, k_pool, v_pool, block_table, row_seq, row_pos)
        if (out.dtype == torch.bfloat16 and getattr(geometry, "seq_start", None) is not None
                and not geometry.decode and self.attention_tc_supports(head_dim, page_size, n_heads, n_kv_heads, q_stride)
                and k_pool.dim() == 4 and k_pool.is_contiguous() and v_pool.is_contiguous()):
            return self.attention_tc(q, q_stride, out, k_pool, v_pool, block_table, geometry.seq_start,
                                     geometry.seq_qlen, geometry.seq_pos0, row_seq, geometry.n_seqs,
                                     geometry.max_q_len, n_heads, n_kv_heads, head_dim, window, scale)
        if (out.dtype == torch.bfloat16 and getattr(geometry, "seq_start", None) is not None
                and self.attention_mma_supports(head_dim, page_size)):
            keys_mode = bool(geometry.decode)
            splits = 1
            if keys_mode:
                splits = self.decode_splits(geometry.n_seqs, n_heads, n_kv_heads, head_dim, geometry.max_kv_len, q.device)
            return self.attention_mma(q, q_stride, out, k_pool, v_pool, block_table, geometry.seq_start,
                                      geometry.seq_qlen, geometry.seq_pos0, row_seq, geometry.n_seqs,
                                      geometry.max_q_len, n_heads, n_kv_heads, head_dim, window, scale, keys_mode,
                                      splits, geometry)
        rows = out.shape[0]
        splits = self.attention_splits(rows, n_heads, geometry.max_kv_len)
        scratch = None
        if splits > 1:
            scratch = geometry.scratch(rows * n_heads * splits * (head_dim + 2), q.device)
        lib.family("attention_simt").call(
            "attention_simt", _ptr(q), q_stride, _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
            block_table.shape[1], page_size, _ptr(row_seq), _ptr(row_pos), rows, n_heads, n_kv_heads, head_dim,
            window or 0, float(scale), splits, _ptr(scratch), code_of(out.dtype), _stream())

    def attention_tc_supports(self, head_dim, page_size, n_heads, n_kv_heads, q_stride):
        """Prompts: both products of attention on tcgen05 (csrc/attention_tc.cu).  FRIDAY_ATTN_TC=0 keeps the
        mma.sync kernel for them."""
        import os
        return (os.environ.get("FRIDAY_ATTN_TC", "1") != "0" and head_dim % 16 == 0 and 16 <= head_dim <= 128
                and page_size == 64 and n_kv_heads > 0 and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 128
                and q_stride % 8 == 0)

    def attention_tc(self, q, q_stride, out, k_pool, v_pool, block_table, seq_start, seq_qlen, seq_pos0, seq_live,
                     n_seqs, max_q_len, n_heads, n_kv_heads, head_dim, window, scale):
        """Causal attention of whole prompts (or their continuation) over the paged cache: up to 128 rows of
        (token, group head) pairs per CTA, blocks of 128 keys."""
        status = self._tc_buffers(q.device)[2]
        lib.family("attention_tc").call(
            "attention_tc", _ptr(q), q_stride, q.shape[0], _ptr(out), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0],
            _ptr(block_table), block_table.shape[1], _ptr(seq_start), _ptr(seq_qlen), _ptr(seq_pos0), _ptr(seq_live),
            n_seqs, max_q_len, n_heads, n_kv_heads, head_dim, window or 0, float(scale), _ptr(status), _stream())

    def attention_mma_supports(self, head_dim, page_size):
        return head_dim % 16 == 0 and 16 <= head_dim <= 128 and page_size == 64

    def attention_mma(self, q, q_stride, out, k_pool, v_pool, block_table, seq_start, seq_qlen, seq_pos0, seq_live,
                      n_seqs, max_q_len, n_heads, n_kv_heads, head_dim, window, scale, keys_mode, splits, geometry):
        """The tensor-core kernel; keys_mode: one-token steps (rows of a CTA share a token, warps and `splits`
        CTAs share the keys); otherwise CTAs own 64 rows of (token, group head) pairs."""
        rows = out.shape[0]
        scratch = None
        if splits > 1:
            scratch = geometry.scratch(rows * n_heads * splits * (head_dim + 2), q.device)
        counters = self._attention_counters(q.device)
        lib.family("attention_mma").call(
            "attention_mma", _ptr(q), q_stride, _ptr(out), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table),
            block_table.shape[1], 64, _ptr(seq_start), _ptr(seq_qlen), _ptr(seq_pos0), _ptr(seq_live), n_seqs, rows,
            max_q_len, n_heads, n_kv_heads, head_dim, window or 0, float(scale), 1 if keys_mode else 0, splits,
            _ptr(scratch), _ptr(counters), counters.numel(), _ptr(self._tc_buffers(q.device)[2]), _stream())

    def _attention_counters(self, device):
        """Zeroed ints, one per (sequence, kv head, row tile) of a one-token step; the kernel leaves them zero."""
        c = self._attn_counters.get(device)
        if c is None:
            c = self._attn_counters[device] = torch.zeros((1 << 16,), dtype=torch.int32, device=device)
        return c

    def decode_splits(self, n_seqs, n_heads, n_kv_heads, head_dim, max_kv_len, device):
        """CTAs that share one sequence's keys in a one-token step: as many as leave every CTA at least two blocks
        of keys, up to the 8 of a thread-block cluster, as long as all clusters run at once (a second wave would
        cost a whole CTA's set-up and merge again).  The device says how many clusters of a size it holds when it
        is empty; SMs that the kernel before frees one by one are packed less well (measured on a B200: 32 clusters
        of 8 ran in two waves although 33 fit), hence the margin of one half."""
        group = n_heads // n_kv_heads
        base = n_seqs * n_kv_heads * ((group + 15) // 16)              # clusters of the launch
        blocks = (max_kv_len + 63) // 64
        fits = lib.family("attention_mma").cdll.attention_mma_clusters_at_once
        for size in range(min(8, max(1, blocks // 2)), 1, -1):
            key = (device, head_dim, size)
            if key not in self._cluster_fit:
                self._cluster_fit[key] = int(fits(head_dim, size))
            if 2 * self._cluster_fit[key] >= 3 * base:
                return size
        return 1

    @staticmethod
    def attention_splits(rows, n_heads, max_kv_len):
        """CUDA-core kernel: few rows facing long contexts are cut along the keys so that the device fills."""
        warps = rows * n_heads
        want = 148 * 16
        if warps >= want or max_kv_len <= 128:
            return 1
        return int(max(1, min(want // max(warps, 1), (max_kv_len + 63) // 64, 64)))

    # -- sampling ---------------------------------------------------------
    def sample(self, logits, temperature, streams, steps, seed, row_live=None, out=None):
        _need_cuda(logits, temperature, streams, steps)
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        assert temperature.dtype == torch.float32 and streams.dtype == torch.int32 and steps.dtype == torch.int32
        if out is None:
            out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        lib.family("sampling").call("sampling_sample", _ptr(logits), logits.shape[0], logits.shape[1],
                                    logits.stride(0), _ptr(temperature), _ptr(streams), _ptr(steps),
                                    int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(row_live), _ptr(out), _stream())
        return out


_backend = CudaOps()


def set_backend(obj):
    """Replaces the implementation object and returns the previous one."""
    global _backend
    prev, _backend = _backend, obj
    return prev


def backend():
    return _backend


def embedding(*a, **k):
    return _backend.embedding(*a, **k)


def gather_rows(*a, **k):
    return _backend.gather_rows(*a, **k)


def rmsnorm(*a, **k):
    return _backend.rmsnorm(*a, **k)


def swiglu(*a, **k):
    return _backend.swiglu(*a, **k)


def linear_swiglu(*a, **k):
    return _backend.linear_swiglu(*a, **k)


def rope_kv_write(*a, **k):
    return _backend.rope_kv_write(*a, **k)


def advance(*a, **k):
    return _backend.advance(*a, **k)


def linear(*a, **k):
    return _backend.linear(*a, **k)


def linear_norm(*a, **k):
    return _backend.linear_norm(*a, **k)


def qkv_rope_write(*a, **k):
    return _backend.qkv_rope_write(*a, **k)


def attention(*a, **k):
    return _backend.attention(*a, **k)


def sample(*a, **k):
    return _backend.sample(*a, **k)
