"""Each kernel alone against the plain implementation's function for the same step, at
sizes other than the test models': widths and vocabularies that are no power of two,
head sizes in steps of 16 up to 256, odd head counts and groups, long contexts."""
import os

import numpy as np
import pytest
import torch

import plain_model as pm
from friday_inference_engine_b200 import ops
from friday_inference_engine_b200.cache import PAGE

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def f64(t):
    return t.detach().double().cpu().numpy()


def close(got, ref, dtype, what, fp32_tol=2e-5, bf16_rel=0.02):
    got, ref = f64(got) if torch.is_tensor(got) else got, np.asarray(ref)
    scale = np.abs(ref).max() + 1e-12
    err = np.abs(got - ref).max() / scale
    tol = fp32_tol if dtype == torch.float32 else bf16_rel
    assert err <= tol, "%s: relative error %.3g > %.3g" % (what, err, tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_gather(dtype):
    table = rnd((777, 100), dtype, 0)
    toks = torch.tensor([0, 776, 5, 5, 300], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embedding(toks, table), table[toks.long()])
    assert torch.equal(ops.gather_rows(toks, table), table[toks.long()])
    # an id outside the table (what a sampler leaves for a row without a finite logit) reads nothing: zeros
    bad = torch.tensor([3, -1, 777, 2], dtype=torch.int32, device=DEV)
    got = ops.embedding(bad, table)
    assert torch.equal(got[[0, 3]], table[[3, 2]]) and float(got[[1, 2]].float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [100, 3584, 5000])
def test_rmsnorm(dtype, width):
    x, w = rnd((7, width), dtype, 1, 3.0), rnd((width,), dtype, 2)
    close(ops.rmsnorm(x, w, 1e-5), pm.rms_norm(f64(x), f64(w), 1e-5), dtype, "rmsnorm %d" % width)
    w32 = w.float()                     # a weight stored in 32-bit stays so beside bf16 activations
    close(ops.rmsnorm(x, w32, 1e-6), pm.rms_norm(f64(x), f64(w32), 1e-6), dtype, "rmsnorm fp32 weight")


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    gu = rnd((9, 2 * 177), dtype, 3, 4.0)
    ref = pm.swiglu(f64(gu)[:, 0::2], f64(gu)[:, 1::2])      # columns alternate gate, up
    close(ops.swiglu(gu), ref, dtype, "swiglu")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (37, 200, 1024), (130, 96, 768), (5, 1001, 333), (64, 177, 3584)])
def test_gemm_simt(dtype, m, n, k):
    a, w = rnd((m, k), dtype, 4), rnd((n, k), dtype, 5, 0.05)
    bias, res = rnd((n,), dtype, 6), rnd((m, n), dtype, 7)
    close(ops.backend()._linear_simt(a, w, None, None, torch.empty((m, n), dtype=dtype, device=DEV)),
          pm.linear(f64(a), f64(w)), dtype, "product")
    ref = pm.linear(f64(a), f64(w), f64(bias)) + f64(res)
    out = res.clone()                                     # the residual in place, as the blocks use it
    close(ops.backend()._linear_simt(a, w, bias, out, out), ref, dtype, "product + bias + residual in place")
    lg = ops.backend()._linear_simt(a, w, None, None, torch.empty((m, n), dtype=torch.float32, device=DEV))
    assert lg.dtype == torch.float32
    close(lg, pm.linear(f64(a), f64(w)), torch.float32 if dtype == torch.float32 else dtype, "fp32 output",
          bf16_rel=1e-4)                                  # bf16 inputs are exact; only the sum is rounded (fp32)


def test_gemm_simt_mixed_storage():
    a, w = rnd((9, 96), torch.bfloat16, 8), rnd((50, 96), torch.float32, 9)
    bias = rnd((50,), torch.float32, 10)
    out = torch.empty((9, 50), dtype=torch.bfloat16, device=DEV)
    ops.backend()._linear_simt(a, w, bias, None, out)
    close(out, pm.linear(f64(a), f64(w), f64(bias)), torch.bfloat16, "bf16 rows, fp32 matrix")


def paged(k, v, dtype, extra_pages=3, seed=0):
    """Scatters [n, nkv, hd] keys and values over shuffled pages; returns pools and table."""
    n = k.shape[0]
    n_pages = (n + PAGE - 1) // PAGE
    perm = torch.randperm(n_pages + extra_pages, generator=torch.Generator().manual_seed(seed))[:n_pages]
    kp = torch.full((n_pages + extra_pages, PAGE) + tuple(k.shape[1:]), float("nan"), dtype=dtype, device=DEV)
    vp = kp.clone()
    for lp in range(n_pages):
        rows = slice(lp * PAGE, min((lp + 1) * PAGE, n))
        kp[perm[lp], : rows.stop - rows.start] = k[rows]
        vp[perm[lp], : rows.stop - rows.start] = v[rows]
    return kp, vp, perm.to(torch.int32).to(DEV).view(1, -1)


class Geo:
    def __init__(self, max_kv_len):
        self.max_kv_len = max_kv_len
        self._s = None

    def scratch(self, n, device):
        self._s = torch.empty((max(n, 1),), dtype=torch.float32, device=device)
        return self._s


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,n,window", [
    (4, 2, 16, 37, None), (3, 1, 32, 130, 24), (28, 4, 128, 300, None), (6, 2, 48, 257, 80), (5, 5, 256, 70, None),
    (8, 1, 112, 64, 64), (14, 2, 64, 1000, None)])
def test_attention_rows_of_a_whole_sequence(dtype, nq, nkv, hd, n, window):
    q, k, v = rnd((n, nq, hd), dtype, 11), rnd((n, nkv, hd), dtype, 12), rnd((n, nkv, hd), dtype, 13)
    q = q * 2                                            # sharper softmax, as the reference's test does
    ref = pm.attention(f64(q), f64(k), f64(v), window).reshape(n, nq * hd)
    kp, vp, table = paged(k, v, dtype)
    row_seq = torch.zeros(n, dtype=torch.int32, device=DEV)
    row_pos = torch.arange(n, dtype=torch.int32, device=DEV)
    out = torch.empty((n, nq * hd), dtype=dtype, device=DEV)
    qf = q.reshape(n, nq * hd).contiguous()
    ops.attention(qf, nq * hd, out, kp, vp, table, PAGE, row_seq, row_pos, nq, nkv, hd, window, hd ** -0.5, Geo(n))
    close(out, ref, dtype, "whole sequence")
    # the last row alone, as decoding sees it (few rows, long context: the keys are split)
    out1 = torch.empty((1, nq * hd), dtype=dtype, device=DEV)
    ops.attention(qf[n - 1:], nq * hd, out1, kp, vp, table, PAGE, row_seq[:1], row_pos[n - 1:], nq, nkv, hd, window,
                  hd ** -0.5, Geo(n))
    close(out1, ref[n - 1:], dtype, "last row alone")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(dtype):
    """One key among a thousand matches the query; its value must come out."""
    nq, nkv, hd, n = 4, 2, 64, 1000
    k = rnd((n, nkv, hd), dtype, 14, 0.1)
    v = rnd((n, nkv, hd), dtype, 15)
    q = rnd((1, nq, hd), dtype, 16, 0.1)
    far = 3
    k[far, :, :] = 0
    k[far, :, 0] = 8.0
    q[0, :, 0] = 8.0 * (hd ** 0.5)                        # score 64 for the far key, about 0 elsewhere
    kp, vp, table = paged(k, v, dtype)
    out = torch.empty((1, nq * hd), dtype=dtype, device=DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    ops.attention(q.reshape(1, -1).contiguous(), nq * hd, out, kp, vp, table, PAGE, torch.zeros(1, dtype=torch.int32, device=DEV),
                  pos, nq, nkv, hd, None, hd ** -0.5, Geo(n))
    want = f64(v)[far].repeat(nq // nkv, axis=0).reshape(-1)
    close(out[0], want, dtype, "the far key's value", fp32_tol=1e-4)
    # with a window that ends one short of it, it must NOT be seen
    ops.attention(q.reshape(1, -1).contiguous(), nq * hd, out, kp, vp, table, PAGE, torch.zeros(1, dtype=torch.int32, device=DEV),
                  pos, nq, nkv, hd, n - 1 - far, hd ** -0.5, Geo(n))
    assert np.abs(f64(out[0]) - want).max() > 0.5
    ops.attention(q.reshape(1, -1).contiguous(), nq * hd, out, kp, vp, table, PAGE, torch.zeros(1, dtype=torch.int32, device=DEV),
                  pos, nq, nkv, hd, n - far, hd ** -0.5, Geo(n))
    close(out[0], want, dtype, "the window's first key", fp32_tol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope_and_cache_write(dtype):
    nq, nkv, hd = 5, 2, 48
    rows = 10
    qkv = rnd((rows, (nq + 2 * nkv) * hd), dtype, 17)
    before = f64(qkv).reshape(rows, nq + 2 * nkv, hd)
    row_seq = torch.tensor([0, 0, 0, 1, 1, -1, 1, 0, 0, 0], dtype=torch.int32, device=DEV)
    row_pos = torch.tensor([62, 63, 64, 0, 1, 0, 2, 65, 66, 200], dtype=torch.int32, device=DEV)
    table = torch.tensor([[3, 1, 7, 5], [2, 0, -1, -1]], dtype=torch.int32, device=DEV)
    kp = torch.zeros((8, PAGE, nkv, hd), dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    denom = torch.from_numpy(np.power(np.float32(50000.0), np.float32(2.0) * np.arange(hd // 2, dtype=np.float32)
                                      / np.float32(hd)).astype(np.float32)).to(DEV)
    ops.rope_kv_write(qkv, row_seq, row_pos, denom, hd, nq, nkv, hd, kp, vp, table, PAGE)
    after = f64(qkv).reshape(rows, nq + 2 * nkv, hd)
    tbl = table.cpu().numpy()
    for r in range(rows):
        if int(row_seq[r]) < 0:
            assert np.array_equal(after[r], before[r])      # a padding row is left alone
            continue
        p = int(row_pos[r])
        ref = pm.rope_neox(before[r:r + 1, : nq + nkv], [p], 50000.0)[0]
        close(after[r, : nq + nkv], ref, dtype, "rotated q and k, row %d" % r)
        assert np.array_equal(after[r, nq + nkv:], before[r, nq + nkv:])          # v is untouched
        page = tbl[int(row_seq[r]), p // PAGE]
        assert np.array_equal(f64(kp[page, p % PAGE]), after[r, nq:nq + nkv])
        assert np.array_equal(f64(vp[page, p % PAGE]), after[r, nq + nkv:])
    assert int((kp != 0).any(dim=-1).any(dim=-1).sum()) == rows - 1                # nothing else was written


def test_sampling_greedy_rule():
    x = torch.tensor([[1.0, 3.0, 3.0, 2.0], [float("nan"), float("inf"), 1.0, -float("inf")],
                      [-5.0, -5.0, -5.0, -5.0]], device=DEV)
    t = torch.zeros(3, device=DEV)
    z = torch.zeros(3, dtype=torch.int32, device=DEV)
    assert ops.sample(x, t, z, z, 0).tolist() == [1, 2, 0]


@pytest.mark.parametrize("vocab", [50, 1000, 152064])
def test_sampling_matches_plain_draws(vocab):
    rows = 24
    logits = rnd((rows, vocab), torch.float32, 18, 3.0)
    temp = torch.full((rows,), 0.8, device=DEV)
    streams = torch.arange(rows, dtype=torch.int32, device=DEV) % 5
    steps = torch.arange(rows, dtype=torch.int32, device=DEV) * 3
    got = ops.sample(logits, temp, streams, steps, 7).tolist()
    host = logits.cpu().numpy()
    exact = 0
    for r in range(rows):
        want = pm.sample(host[r], 0.8, 7, int(streams[r]), int(steps[r]))
        if got[r] == want:
            exact += 1
            continue
        # fp32 running sums may move an interval's edge by a rounding: then u must sit on that edge
        _, cdf = pm.temperature_cdf(host[r], 0.8)
        u = pm.uniform_for(7, int(streams[r]), int(steps[r]))
        lo, hi = min(got[r], want), max(got[r], want)
        assert abs(cdf[lo] - u) < 1e-5 and cdf[hi - 1] - cdf[lo] < 1e-5, "row %d: %d, plain %d" % (r, got[r], want)
    assert exact >= rows - 2
    # greedy on the same rows
    g = ops.sample(logits, torch.zeros(rows, device=DEV), streams, steps, 7).tolist()
    assert g == [pm.greedy(host[r]) for r in range(rows)]


def test_sampling_draws_do_not_depend_on_the_batch():
    logits = rnd((6, 300), torch.float32, 19, 2.0)
    temp = torch.full((6,), 1.3, device=DEV)
    streams = torch.tensor([4, 9, 1, 0, 7, 2], dtype=torch.int32, device=DEV)
    steps = torch.tensor([0, 5, 2, 2, 9, 1], dtype=torch.int32, device=DEV)
    whole = ops.sample(logits, temp, streams, steps, 3).tolist()
    for r in (0, 3, 5):
        alone = ops.sample(logits[r:r + 1].contiguous(), temp[:1], streams[r:r + 1].contiguous(),
                           steps[r:r + 1].contiguous(), 3).tolist()
        assert alone == [whole[r]]


# ------------------------------------------------------------------ tensor-core product
TC_SHAPES = [
    # m, n, k: rows of activations, out features, in features
    (1, 128, 64), (1, 4608, 3584), (8, 3584, 3584), (7, 1001, 328), (16, 777, 96), (17, 256, 512), (33, 200, 1024),
    (64, 3584, 18944), (64, 130, 72), (65, 96, 768), (130, 96, 768), (200, 1001, 328), (257, 300, 64),
    (512, 4608, 3584), (2048, 512, 1024),
    # few rows, more tiles of weights than SMs with a half-empty last wave: k is cut although every SM has a tile
    (8, 27648, 5120), (3, 128 * 160, 1024),
    # more than 128 rows and at least 256 columns: 256-row tiles on pairs of SMs; a last row tile whose second half is
    # empty, widths that are no multiple of the tile width, of 16 or of 8, more tiles than pairs
    (129, 256, 64), (256, 1000, 136), (300, 1001, 328), (513, 4104, 72), (1300, 2400, 4096), (2500, 9000, 128),
]


@pytest.mark.parametrize("m,n,k", TC_SHAPES)
def test_gemm_tensor_core(m, n, k):
    dt = torch.bfloat16
    a, w = rnd((m, k), dt, 20), rnd((n, k), dt, 21, 0.05)
    bias, res = rnd((n,), dt, 22), rnd((m, n), dt, 23)
    ref0 = pm.linear(f64(a), f64(w))
    be = ops.backend()
    assert be.tensor_core_ok(a, w, res, res)
    # fp32 output shows the sums themselves: inputs are exact in bf16, only the order of the fp32 sum differs
    lg = be._linear_tc(a, w, None, None, torch.empty((m, n), dtype=torch.float32, device=DEV))
    close(lg, ref0, torch.float32, "tensor-core product, fp32 out", fp32_tol=3e-5)
    out = be._linear_tc(a, w, None, None, torch.empty((m, n), dtype=dt, device=DEV))
    close(out, ref0, dt, "tensor-core product", bf16_rel=0.01)
    ref = pm.linear(f64(a), f64(w), f64(bias)) + f64(res)
    io = res.clone()
    close(be._linear_tc(a, w, bias, io, io), ref, dt, "bias + residual in place", bf16_rel=0.01)
    io = res.clone()
    close(be._linear_tc(a, w, bias.float(), io, io), ref, dt, "fp32 bias", bf16_rel=0.01)
    be.check_status()


@pytest.mark.parametrize("m,n,k,swap,bn,splits", [
    (8, 512, 1024, 1, 16, 1), (8, 512, 1024, 1, 16, 4), (8, 512, 1024, 1, 64, 16), (40, 300, 2048, 1, 64, 3),
    (40, 300, 2048, 0, 64, 1), (300, 300, 2048, 0, 128, 2), (300, 700, 2048, 0, 256, 5), (128, 256, 4096, 0, 256, 64),
    (100, 100, 64, 0, 128, 1), (5, 130, 72, 0, 256, 1), (300, 40, 2048, 1, 32, 1),
    (300, 1000, 256, 0, 208, 1), (2048, 3584, 512, 0, 208, 1), (256, 700, 128, 0, 144, 3), (130, 1001, 328, 0, 240, 1),
    # tiles narrower than 128 on pairs of SMs (more than 128 rows, k not split)
    (256, 1000, 512, 0, 64, 1), (300, 700, 328, 0, 112, 1), (513, 333, 256, 0, 80, 1), (200, 4608, 192, 0, 96, 1),
    # weights on the M side with the rows as a 128-wide tile that is finished through a window of 16 rows
    (128, 512, 1024, 1, 128, 1), (100, 384, 2048, 1, 128, 3), (65, 300, 512, 1, 128, 2), (128, 1024, 4096, 1, 128, 16)])
def test_gemm_tensor_core_every_tiling(m, n, k, swap, bn, splits):
    """Orientation, tile width and split-k are choices of the launcher; each must give the same product."""
    dt = torch.bfloat16
    a, w = rnd((m, k), dt, 24), rnd((n, k), dt, 25, 0.05)
    bias, res = rnd((n,), dt, 26), rnd((m, n), torch.float32, 27)
    ref = pm.linear(f64(a), f64(w), f64(bias)) + f64(res)
    be = ops.backend()
    for _ in range(2):                                       # twice: the tile counters must be back at zero
        io = res.clone()
        got = be._linear_tc(a, w, bias, io, io, swap=swap, bn=bn, splits=splits)
        close(got, ref, torch.float32, "swap %d bn %d splits %d" % (swap, bn, splits), fp32_tol=3e-5)
    be.check_status()


def test_linear_chooses_a_kernel_that_can_do_the_shape():
    dt = torch.bfloat16
    a, w = rnd((9, 100), dt, 28), rnd((50, 100), dt, 29)     # k = 100: rows are not 16-byte multiples
    assert not ops.backend().tensor_core_ok(a, w, a, None)
    close(ops.linear(a, w), pm.linear(f64(a), f64(w)), dt, "falls back to CUDA cores")
    a, w = rnd((9, 104), dt, 28), rnd((50, 104), dt, 29)
    assert ops.backend().tensor_core_ok(a, w, a, None)
    close(ops.linear(a, w), pm.linear(f64(a), f64(w)), dt, "tensor cores")


# ------------------------------------------------------------------ tensor-core attention
class SeqGeo(Geo):
    pass


def mma_case(seqs, nq, nkv, hd, window, keys_mode, splits, seed=30, tcgen05=False):
    """seqs: list of (tokens held before the step, tokens in the step).  Builds a paged cache that holds
    every sequence's keys and values (shuffled pages, NaN elsewhere), runs the tensor-core kernel on the
    step's rows (the mma.sync one, or with tcgen05 the one for prompts) and compares with the plain attention
    of each whole sequence."""
    dt = torch.bfloat16
    n_pages_each = [(a + q + PAGE - 1) // PAGE for a, q in seqs]
    total_pages = sum(n_pages_each) + 3
    perm = torch.randperm(total_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    kp = torch.full((total_pages, PAGE, nkv, hd), float("nan"), dtype=dt, device=DEV)
    vp = kp.clone()
    width = max(n_pages_each) + 1
    table = torch.full((len(seqs), width), -1, dtype=torch.int32)
    rows = sum(q for _, q in seqs)
    qbuf = torch.empty((rows, (nq + 2 * nkv) * hd), dtype=dt, device=DEV)     # q sits inside a wider row, as in qkv
    refs, starts, row = [], [], 0
    for s, (a, q) in enumerate(seqs):
        n = a + q
        qs, ks, vs = rnd((n, nq, hd), dt, seed + 3 * s + 1) * 2, rnd((n, nkv, hd), dt, seed + 3 * s + 2), \
            rnd((n, nkv, hd), dt, seed + 3 * s + 3)
        refs.append(pm.attention(f64(qs), f64(ks), f64(vs), window).reshape(n, nq * hd)[a:])
        for lp in range(n_pages_each[s]):
            page = perm.pop()
            table[s, lp] = page
            lo, hi = lp * PAGE, min((lp + 1) * PAGE, n)
            kp[page, : hi - lo] = ks[lo:hi]
            vp[page, : hi - lo] = vs[lo:hi]
        qbuf[row:row + q, : nq * hd] = qs[a:].reshape(q, nq * hd)
        starts.append(row)
        row += q
    i32 = dict(dtype=torch.int32, device=DEV)
    geo = Geo(max(a + q for a, q in seqs))
    out = torch.full((rows, nq * hd), float("nan"), dtype=dt, device=DEV)
    if tcgen05:
        ops.backend().attention_tc(
            qbuf, qbuf.stride(0), out, kp, vp, table.to(DEV), torch.tensor(starts, **i32),
            torch.tensor([q for _, q in seqs], **i32), torch.tensor([a for a, _ in seqs], **i32), None, len(seqs),
            max(q for _, q in seqs), nq, nkv, hd, window, hd ** -0.5)
        ops.backend().check_status()
    else:
        ops.backend().attention_mma(
            qbuf, qbuf.stride(0), out, kp, vp, table.to(DEV), torch.tensor(starts, **i32),
            torch.tensor([q for _, q in seqs], **i32), torch.tensor([a for a, _ in seqs], **i32), None, len(seqs),
            max(q for _, q in seqs), nq, nkv, hd, window, hd ** -0.5, keys_mode, splits, geo)
    close(out, np.concatenate(refs, axis=0), dt, "tensor-core attention", bf16_rel=0.02)


@pytest.mark.parametrize("nq,nkv,hd,window", [
    (4, 2, 16, None), (3, 1, 32, 24), (28, 4, 128, None), (6, 2, 48, 80), (8, 1, 112, 64), (14, 2, 64, None),
    (5, 5, 80, None), (9, 3, 96, 100), (32, 1, 64, None)])
def test_attention_mma_prompts_of_unequal_lengths(nq, nkv, hd, window):
    # whole prompts, a continued one, one token, lengths around the 64-key blocks
    mma_case([(0, 37), (0, 130), (70, 65), (0, 1), (63, 2), (0, 64)], nq, nkv, hd, window, False, 1)


@pytest.mark.parametrize("nq,nkv,hd,window", [
    (4, 2, 16, None), (3, 1, 32, 24), (28, 4, 128, None), (6, 2, 48, 80), (8, 1, 112, 64), (14, 2, 64, None),
    (5, 5, 80, None), (9, 3, 96, 100), (32, 1, 64, None), (40, 8, 128, 300), (128, 1, 16, None), (3, 3, 128, 128)])
def test_attention_tcgen05_prompts_of_unequal_lengths(nq, nkv, hd, window):
    """The kernel for prompts with both products on tcgen05: the same cases as the mma.sync kernel (stale pages
    hold NaN), lengths around its 64-key blocks and twice that, 128 heads on one kv head (one token per tile), and a window
    that is exactly one block."""
    mma_case([(0, 37), (0, 130), (70, 65), (0, 1), (63, 2), (0, 64)], nq, nkv, hd, window, False, 1, tcgen05=True)
    mma_case([(0, 128), (0, 129), (127, 2), (255, 258), (0, 700)], nq, nkv, hd, window, False, 1, seed=77, tcgen05=True)


@pytest.mark.parametrize("nq,nkv,hd,window,splits", [
    (4, 2, 16, None, 1), (3, 1, 32, 24, 2), (28, 4, 128, None, 5), (28, 4, 128, None, 1), (6, 2, 48, 80, 3),
    (8, 1, 112, 64, 4), (40, 8, 128, None, 7), (32, 1, 64, None, 2), (5, 5, 80, 130, 16),
    # more than 8: partial rows through memory, merged by the last CTA (12 and 16 rows per tile, head sizes whose rows do
    # not fill a warp's lanes evenly, more splits than a short sequence has blocks)
    (24, 2, 96, None, 37), (28, 4, 128, None, 64), (16, 1, 48, 200, 23), (6, 3, 16, None, 9)])
def test_attention_mma_one_token_steps(nq, nkv, hd, window, splits):
    mma_case([(0, 1), (63, 1), (64, 1), (65, 1), (299, 1), (1000, 1), (127, 1)], nq, nkv, hd, window, True, splits)


def test_attention_mma_long_prompt_sizes_of_the_7b_shape():
    mma_case([(0, 700), (300, 500)], 28, 4, 128, None, False, 1)
    mma_case([(0, 2048), (1000, 1100)], 28, 4, 128, None, False, 1, tcgen05=True)


def sampled_columns(n, count, seed):
    g = torch.Generator().manual_seed(seed)
    cols = torch.randperm(n, generator=g)[:count].sort().values
    return torch.cat([torch.tensor([0, 127, 128, n - 129, n - 128, n - 1]), cols]).unique()


@pytest.mark.parametrize("m", [65, 100, 128, 129, 256, 300, 512, 640])
@pytest.mark.parametrize("n,k", [(4608, 3584), (3584, 3584), (7168, 5120)])
def test_products_of_prompts_of_a_few_hundred_rows(m, n, k):
    """The tilings the planner picks between one and a few row tiles (narrow tiles on pairs of SMs among them), with
    bias and residual, against float64."""
    dt = torch.bfloat16
    a, w = rnd((m, k), dt, 210 + m), rnd((n, k), dt, 211, 0.02)
    bias, res = rnd((n,), dt, 212), rnd((m, n), dt, 213)
    ref = pm.linear(f64(a), f64(w), f64(bias)) + f64(res)
    close(ops.linear(a, w, bias, res), ref, dt, "%d x %d x %d as planned" % (m, n, k), bf16_rel=0.01)
    ops.backend().check_status()


@pytest.mark.parametrize("m", [1, 8, 64, 130])
def test_products_at_the_full_width_of_the_head(m):
    """n = 152,064 columns with k = 3,584: the head's 1,188 weight tiles (eight waves and four tiles of a ninth) on the
    tensor cores, and the same product in true 32-bit on the CUDA cores, against float64 on 4,096 sampled columns."""
    n, k = 152064, 3584
    x, w = rnd((m, k), torch.bfloat16, 200 + m), rnd((n, k), torch.bfloat16, 201, 0.02)
    cols = sampled_columns(n, 4096, 202).to(DEV)
    ref = f64(x) @ f64(w[cols]).T
    out = ops.linear(x, w, out_dtype=torch.float32)
    assert out.shape == (m, n) and bool(torch.isfinite(out).all())
    close(out[:, cols], ref, torch.float32, "tensor cores, fp32 logits", fp32_tol=2e-5)      # bf16 inputs are exact
    out16 = ops.linear(x, w)
    close(out16[:, cols], ref, torch.bfloat16, "tensor cores, bf16 out")
    if m <= 8:
        x32, w32 = x.float(), w.float()
        out32 = ops.linear(x32, w32)
        close(out32[:, cols], ref, torch.float32, "CUDA cores, true 32-bit", fp32_tol=2e-5)
    ops.backend().check_status()


class StepGeo:
    """The geometry of a step as the engine hands it to attention: per-sequence arrays on the device."""

    def __init__(self, seqs):
        i32 = dict(dtype=torch.int32, device=DEV)
        self.n_seqs = len(seqs)
        self.max_q_len = max(q for _, q in seqs)
        self.max_kv_len = max(a + q for a, q in seqs)
        self.decode = self.max_q_len == 1
        starts = np.concatenate([[0], np.cumsum([q for _, q in seqs])[:-1]])
        self.seq_start = torch.tensor(starts.tolist(), **i32)
        self.seq_qlen = torch.tensor([q for _, q in seqs], **i32)
        self.seq_pos0 = torch.tensor([a for a, _ in seqs], **i32)
        self.row_seq = torch.tensor(np.repeat(np.arange(len(seqs)), [q for _, q in seqs]).tolist(), **i32)
        self.row_pos = torch.tensor(np.concatenate([np.arange(a, a + q) for a, q in seqs]).tolist(), **i32)


def rows_reference(q, pos, k, v, window):
    """Attention of a few query rows at positions `pos` over keys 0 .. pos (the last `window` of them), float64; the
    formula of cpu_ops.cpp:45-83.  q [rows, nq, hd], k and v [n, nkv, hd]."""
    rows, nq, hd = q.shape
    group = nq // k.shape[1]
    out = np.zeros((rows, nq, hd))
    for r in range(rows):
        lo = 0 if not window else max(0, pos[r] - window + 1)
        for h in range(nq):
            kk, vv = k[lo:pos[r] + 1, h // group], v[lo:pos[r] + 1, h // group]
            s = kk @ q[r, h] * hd ** -0.5
            e = np.exp(s - s.max())
            out[r, h] = (e / e.sum()) @ vv
    return out.reshape(rows, nq * hd)


def long_case(seqs, nq, nkv, hd, window, dtype=torch.bfloat16, width=None, seed=60):
    """seqs: (tokens held, tokens of the step).  Through ops.attention with the step's full geometry, so the kernel and
    the number of splits are the ones the engine picks for these lengths."""
    n_pages_each = [(a + q + PAGE - 1) // PAGE for a, q in seqs]
    total_pages = sum(n_pages_each) + 2
    perm = torch.randperm(total_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    kp = torch.full((total_pages, PAGE, nkv, hd), float("nan"), dtype=dtype, device=DEV)
    vp = kp.clone()
    table = torch.full((len(seqs), width or max(n_pages_each)), -1, dtype=torch.int32)
    rows = sum(q for _, q in seqs)
    qbuf = torch.zeros((rows, (nq + 2 * nkv) * hd), dtype=dtype, device=DEV)
    refs, row = [], 0
    for s, (a, q) in enumerate(seqs):
        n = a + q
        qs = rnd((q, nq, hd), dtype, seed + 3 * s + 1) * 2
        ks, vs = rnd((n, nkv, hd), dtype, seed + 3 * s + 2), rnd((n, nkv, hd), dtype, seed + 3 * s + 3)
        far = 7 + s                                       # one key far back matches the first query's first head
        ks[far, :, :] = 0
        ks[far, :, 1] = 6.0
        qs[0, 0, :] = 0
        qs[0, 0, 1] = 6.0 * hd ** 0.5
        refs.append(rows_reference(f64(qs), list(range(a, n)), f64(ks), f64(vs), window))
        pages = [perm.pop() for _ in range(n_pages_each[s])]
        table[s, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        pad = len(pages) * PAGE - n
        kp[pages] = torch.cat([ks, torch.full((pad, nkv, hd), float("nan"), dtype=dtype, device=DEV)]).view(len(pages), PAGE, nkv, hd)
        vp[pages] = torch.cat([vs, torch.full((pad, nkv, hd), float("nan"), dtype=dtype, device=DEV)]).view(len(pages), PAGE, nkv, hd)
        qbuf[row:row + q, : nq * hd] = qs.reshape(q, nq * hd)
        row += q
    geo = StepGeo(seqs)
    out = torch.full((rows, nq * hd), float("nan"), dtype=dtype, device=DEV)
    ops.attention(qbuf, qbuf.stride(0), out, kp, vp, table.to(DEV), PAGE, geo.row_seq, geo.row_pos, nq, nkv, hd, window,
                  hd ** -0.5, geo)
    ops.backend().check_status()
    close(out, np.concatenate(refs, axis=0), dtype, "attention over long contexts", bf16_rel=0.02)
    return geo


@pytest.mark.parametrize("nq,nkv", [(28, 4), (40, 8)])
@pytest.mark.parametrize("longest", [4096, 8192])
def test_one_token_steps_over_long_contexts(nq, nkv, longest):
    """Page tables of 64 and 128 entries and as many splits as the engine picks for the longest sequence."""
    geo = long_case([(longest - 1, 1), (longest // 2 + 5, 1), (99, 1)], nq, nkv, 128, None)
    assert ops.backend().decode_splits(3, nq, nkv, 128, geo.max_kv_len) >= 4       # really split, as the engine would


@pytest.mark.parametrize("seqs", [[(16383, 1)], [(20000, 1), (700, 1)]])
def test_one_token_steps_of_few_sequences_over_very_long_contexts(seqs):
    """Few sequences with many keys: more CTAs share a sequence than a cluster holds, and the last one merges their
    partial rows through memory."""
    geo = long_case(seqs, 28, 4, 128, None)
    assert ops.backend().decode_splits(len(seqs), 28, 4, 128, geo.max_kv_len) > 8


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_token_steps_with_a_page_table_wider_than_a_cta(dtype):
    """More pages than the kernel's CTA has threads (one sequence really holds 130 of them, the table has room for
    170): the first pages come from shared memory, the rest from the table itself."""
    long_case([(8300, 1), (69, 1)], 2, 1, 16, None, dtype=dtype, width=170)
    long_case([(8300, 1), (69, 1)], 2, 1, 16, 4000, dtype=dtype, width=170)


@pytest.mark.parametrize("nq,nkv", [(28, 4), (40, 8)])
def test_continued_prompt_over_a_long_context(nq, nkv):
    long_case([(6000, 300), (0, 130)], nq, nkv, 128, None)


def test_attention_mma_dead_rows_give_zero():
    dt = torch.bfloat16
    nq, nkv, hd = 4, 2, 32
    kp = torch.full((2, PAGE, nkv, hd), float("nan"), dtype=dt, device=DEV)
    q = rnd((2, (nq + 2 * nkv) * hd), dt, 40)
    out = torch.full((2, nq * hd), float("nan"), dtype=dt, device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    live = torch.tensor([-1, -1], **i32)
    ops.backend().attention_mma(q, q.stride(0), out, kp, kp, torch.zeros((2, 1), **i32), torch.tensor([0, 1], **i32),
                                torch.ones(2, **i32), torch.tensor([5, 9], **i32), live, 2, 1, nq, nkv, hd, None, 1.0,
                                True, 2, Geo(10))
    assert float(out.float().abs().max()) == 0.0


@pytest.mark.parametrize("m,inner,k", [(1, 64, 64), (8, 18944, 3584), (8, 13824, 5120), (40, 177, 512), (64, 200, 96), (100, 177, 512),
                                       (100, 18944, 3584), (128, 1024, 512),
                                       (300, 1000, 1024), (2048, 2368, 512)])
def test_gemm_tensor_core_gated_epilogue(m, inner, k):
    dt = torch.bfloat16
    x = rnd((m, k), dt, 41)
    wg, wu = rnd((inner, k), dt, 42, 0.05), rnd((inner, k), dt, 43, 0.05)
    pairs = torch.stack([wg, wu], dim=1).reshape(2 * inner, k).contiguous()
    ref = pm.swiglu(pm.linear(f64(x), f64(wg)), pm.linear(f64(x), f64(wu)))
    close(ops.linear_swiglu(x, pairs), ref, dt, "product with silu(gate) * up in the epilogue", bf16_rel=0.01)
    be = ops.backend()
    for swap, bn, splits in ((1, 64, 3), (0, 128, 2), (0, 256, 1), (0, 176, 1)):
        if (swap and m > 64) or 2 * inner * max(m, 128) > 2000000:     # forced tilings only where their scratch fits
            continue
        out = torch.empty((m, inner), dtype=dt, device=DEV)
        close(be._linear_tc(x, pairs, None, None, out, swap=swap, bn=bn, splits=splits, act=1), ref, dt,
              "gated, swap %d bn %d splits %d" % (swap, bn, splits), bf16_rel=0.01)
    be.check_status()


@pytest.mark.parametrize("m,n,k", [(2048, 3584, 512), (1100, 3584 + 256, 1024), (2048 + 77, 2400, 320), (2048, 3584, 18944),
                                   (4096, 3584, 1024), (19 * 128, 2048, 4096)])
def test_gemm_tensor_core_partial_last_wave(m, n, k, monkeypatch):
    """More 128 x 256 tiles than SMs with a remainder: with FRIDAY_STREAM_K=1 the last wave is cut along k over
    all SMs.  The switch is read once per process, so this test runs the product in a child process."""
    import subprocess
    import sys
    code = ("import os, sys; os.environ['FRIDAY_STREAM_K']='1'; sys.path.insert(0, %r); sys.path.insert(0, %r);"
            "import test_kernels_gpu as t; t.partial_last_wave(%d, %d, %d)"
            % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), os.path.dirname(os.path.abspath(__file__)), m, n, k))
    subprocess.run([sys.executable, "-c", code], check=True)
    partial_last_wave(m, n, k)


def partial_last_wave(m, n, k):
    dt = torch.bfloat16
    a, w = rnd((m, k), dt, 44), rnd((n, k), dt, 45, 0.05)
    res = rnd((m, n), dt, 46)
    io = res.clone()
    ops.linear(a, w, residual=io, out=io)
    ref = (a.float() @ w.float().t()).double() + res.double()          # fp32 matmul of exact bf16 inputs as the yardstick
    err = float((io.double() - ref).abs().max() / ref.abs().max())
    assert err <= 0.01, err
    # the same product with a bias, beginning a norm: the tile's last CTA has whole rows of the tile
    b, g = rnd((n,), dt, 47), rnd((n,), dt, 48) + 1.0
    out, h = ops.linear_norm(a, w, g, 1e-6, bias=b, residual=res)
    assert isinstance(h, ops.DeferredNorm)
    close(out, f64(a) @ f64(w).T + f64(b) + f64(res), dt, "product")
    close(h.ssq.sum(0), (f64(out) ** 2).sum(-1), torch.float32, "sums of squares", fp32_tol=1e-5)
    close(h.scaled, f64(out) * f64(g), dt, "rows times the norm's weights")
    ops.backend().check_status()


# ---------------------------------------------------------------- work fused into the tensor-core product's ends
def denominators(theta, rot):
    return torch.from_numpy(np.power(np.float32(theta), np.float32(2.0) * np.arange(rot // 2, dtype=np.float32)
                                     / np.float32(rot)).astype(np.float32)).to(DEV)


@pytest.mark.parametrize("m,nq,nkv,hd,rot,k", [(1, 4, 2, 32, 32, 64), (8, 28, 4, 128, 128, 3584), (16, 2, 1, 64, 32, 512),
                                                 (5, 6, 1, 16, 16, 1024), (9, 2, 3, 128, 64, 200),
                                                 (17, 28, 4, 128, 128, 3584), (33, 2, 1, 32, 32, 200), (40, 6, 2, 64, 64, 512),
                                                 (64, 28, 4, 128, 128, 3584), (64, 4, 2, 16, 16, 96)])
def test_gemm_with_rotation_and_cache_write_in_its_epilogue(m, nq, nkv, hd, rot, k, monkeypatch):
    """The fused epilogue against the product followed by the rotation kernel: same bits in q, k, v and in the
    cache; against the plain rotation for the values."""
    n = (nq + 2 * nkv) * hd
    x, w, b = rnd((m, k), torch.bfloat16, 70, 0.5), rnd((n, k), torch.bfloat16, 71, 0.1), rnd((n,), torch.bfloat16, 72)
    row_seq = torch.tensor([i % 2 for i in range(m)], dtype=torch.int32, device=DEV)
    if m > 2:
        row_seq[2] = -1                                                   # a padding row
    row_pos = torch.tensor([60 + 3 * i for i in range(m)], dtype=torch.int32, device=DEV)
    table = torch.tensor([[3, 1, 7, 5], [2, 0, 6, 4]], dtype=torch.int32, device=DEV)
    denom = denominators(1e6, rot)
    results = []
    for fuse in ("1", "0"):
        monkeypatch.setenv("FRIDAY_FUSE", fuse)
        kp = torch.zeros((8, PAGE, nkv, hd), dtype=torch.bfloat16, device=DEV)
        vp = torch.zeros_like(kp)
        before = ops.launch_count()
        qkv = ops.qkv_rope_write(x, w, b, row_seq, row_pos, denom, rot, nq, nkv, hd, kp, vp, table, PAGE)
        assert ops.launch_count() - before == (1 if fuse == "1" else 2), "fused: one launch; else two"
        results.append((qkv, kp, vp))
    ops.backend().check_status()
    live = (row_seq >= 0).cpu().numpy()
    for got, want, what in zip(results[0], results[1], ("q, k, v", "key cache", "value cache")):
        if what == "q, k, v":
            got, want = got[torch.from_numpy(live).to(DEV)], want[torch.from_numpy(live).to(DEV)]
        assert torch.equal(got, want), what
    plain = f64(x) @ f64(w).T + f64(b)
    plain = np.asarray(f64(torch.from_numpy(plain).to(torch.bfloat16))).reshape(m, nq + 2 * nkv, hd)
    for r in range(m):
        if not live[r]:
            continue
        ref = plain[r].copy()
        ref[: nq + nkv, :rot] = pm.rope_neox(plain[r:r + 1, : nq + nkv, :rot], [int(row_pos[r])], 1e6)[0]
        close(results[0][0][r].reshape(nq + 2 * nkv, hd), ref, torch.bfloat16, "row %d" % r)
    # no rotation and no cache: the product alone
    qkv = ops.qkv_rope_write(x, w, b, row_seq, row_pos, None, 0, nq, nkv, hd)
    assert torch.equal(qkv, ops.linear(x, w, bias=b))


@pytest.mark.parametrize("m,n,k,k2", [(1, 128, 64, 64), (8, 3584, 3584, 1024), (16, 256, 18944, 512), (7, 640, 200, 136),
                                      (33, 384, 1024, 192), (64, 3584, 512, 64)])
def test_gemm_begins_a_norm_that_the_next_gemm_finishes(m, n, k, k2, monkeypatch):
    x, w = rnd((m, k), torch.bfloat16, 80, 0.5), rnd((n, k), torch.bfloat16, 81, 0.05)
    res = rnd((m, n), torch.bfloat16, 82, 2.0)
    g = rnd((n,), torch.bfloat16, 83) + 1.0
    eps = 1e-5
    out, h = ops.linear_norm(x, w, g, eps, residual=res)
    assert isinstance(h, ops.DeferredNorm), "few bf16 rows and whole tiles: the norm is begun in the epilogue"
    assert torch.equal(out, ops.linear(x, w, residual=res)), "the product itself is unchanged"
    normed = pm.rms_norm(f64(out), f64(g), eps)
    close(h.materialize(), normed, torch.bfloat16, "materialised")
    # the sums of squares: shares of 128 columns each
    ssq = (f64(out) ** 2).reshape(m, n // 128, 128).sum(-1).T
    close(h.ssq, ssq, torch.float32, "partial sums of squares", fp32_tol=1e-5)
    # consumers: a plain product with bias (bf16 and fp32 output), the gated one, and one that begins the next norm
    w2, b2 = rnd((k2 * 2, n), torch.bfloat16, 84, 0.05), rnd((k2 * 2,), torch.bfloat16, 85)
    ref = normed @ f64(w2).T
    close(ops.linear(h, w2, bias=b2), ref + f64(b2), torch.bfloat16, "consumer with bias")
    close(ops.linear(h, w2, out_dtype=torch.float32), ref, torch.bfloat16, "consumer with fp32 output", bf16_rel=0.01)
    close(ops.linear_swiglu(h, w2), pm.swiglu(ref[:, 0::2], ref[:, 1::2]), torch.bfloat16, "gated consumer")
    if (2 * k2) % 128 == 0:
        g2 = rnd((2 * k2,), torch.bfloat16, 86) + 1.0
        out2, h2 = ops.linear_norm(h, w2, g2, eps)
        assert isinstance(h2, ops.DeferredNorm)
        close(out2, ref, torch.bfloat16, "consumer that begins a norm")
        close(h2.materialize(), pm.rms_norm(f64(out2), f64(g2), eps), torch.bfloat16, "second norm")
    # a consumer that cannot finish the norm itself (a k that is no multiple of 8 is not for the tensor cores;
    # here: fp32 weights) gets the rows from the norm's own kernel
    close(ops.linear(h, w2.float()), ref, torch.bfloat16, "consumer on the CUDA cores")
    monkeypatch.setenv("FRIDAY_FUSE", "0")
    out3, h3 = ops.linear_norm(x, w, g, eps, residual=res)
    assert torch.is_tensor(h3), "switched off: the norm's own kernel runs and a tensor comes back"
    close(h3, pm.rms_norm(f64(out3), f64(g), eps), torch.bfloat16, "unfused norm")
    ops.backend().check_status()


@pytest.mark.parametrize("m,n,k,k2", [(80, 3584, 512, 96), (128, 640, 4096, 64), (65, 48, 64, 24), (300, 3584, 1024, 128),
                                      (2048, 3584, 256, 104), (257, 208, 72, 512), (130, 272, 18944, 40)])
def test_gemm_of_many_rows_begins_a_norm(m, n, k, k2):
    """More than 128 rows (and fewer whose width is no multiple of 128) lie on the tiles' M side: every column tile,
    whatever its width, adds one share of each row's sum of squares; up to 128 rows with the weights on the M side add
    one share per 128 columns.  The next product, either way round, finishes the norm."""
    x, w = rnd((m, k), torch.bfloat16, 180, 0.5), rnd((n, k), torch.bfloat16, 181, 0.05)
    res, b = rnd((m, n), torch.bfloat16, 182, 2.0), rnd((n,), torch.bfloat16, 183)
    g = rnd((n,), torch.bfloat16, 184) + 1.0
    eps = 1e-6
    out, h = ops.linear_norm(x, w, g, eps, bias=b, residual=res)
    assert isinstance(h, ops.DeferredNorm)
    assert torch.equal(out, ops.linear(x, w, bias=b, residual=res)), "the product itself is unchanged"
    plan = np.zeros(5, dtype=np.int64)
    ops.lib.family("gemm_tc").call("gemm_tc_plan", m, n, k, ops.backend().info()["sm_count"], -1, -1, -1, plan.ctypes.data)
    assert plan[0] == (1 if m <= 128 else 0)
    if plan[0] == 1 and n % 128 == 0:
        bn = 128
    else:
        ops.lib.family("gemm_tc").call("gemm_tc_plan", m, n, k, ops.backend().info()["sm_count"], 0, -1, -1, plan.ctypes.data)
        bn = int(plan[1])
    assert h.ssq.shape == (-(-n // bn), m)
    sq = f64(out) ** 2
    ssq = np.stack([sq[:, c:c + bn].sum(-1) for c in range(0, n, bn)])
    close(h.ssq, ssq, torch.float32, "partial sums of squares", fp32_tol=1e-5)
    close(h.scaled, f64(out) * f64(g), torch.bfloat16, "rows times the norm's weights")
    normed = pm.rms_norm(f64(out), f64(g), eps)
    close(h.materialize(), normed, torch.bfloat16, "materialised")
    w2 = rnd((k2 * 2, n), torch.bfloat16, 185, 0.05)
    ref = normed @ f64(w2).T
    close(ops.linear(h, w2), ref, torch.bfloat16, "consumer")
    close(ops.linear_swiglu(h, w2), pm.swiglu(ref[:, 0::2], ref[:, 1::2]), torch.bfloat16, "gated consumer")
    if (2 * k2) % 16 == 0:
        g2 = rnd((2 * k2,), torch.bfloat16, 186) + 1.0
        out2, h2 = ops.linear_norm(h, w2, g2, eps)
        assert isinstance(h2, ops.DeferredNorm)
        close(out2, ref, torch.bfloat16, "consumer that begins a norm")
        close(h2.materialize(), pm.rms_norm(f64(out2), f64(g2), eps), torch.bfloat16, "second norm")
    # a width that is no multiple of 16: the norm's own kernel
    out3, h3 = ops.linear_norm(x, w[:n - 8], g[:n - 8], eps)
    assert torch.is_tensor(h3)
    close(h3, pm.rms_norm(f64(out3), f64(g[:n - 8]), eps), torch.bfloat16, "unfused norm")
    ops.backend().check_status()


def test_norm_and_rotation_fused_into_split_k_products():
    """Shapes whose k is split over several CTAs: the last one to arrive runs the fused epilogue."""
    m, nq, nkv, hd, k = 4, 2, 1, 128, 4096
    n = (nq + 2 * nkv) * hd
    x, w = rnd((m, k), torch.bfloat16, 90, 0.5), rnd((n, k), torch.bfloat16, 91, 0.05)
    plan = np.zeros(5, dtype=np.int64)
    ops.lib.family("gemm_tc").call("gemm_tc_plan", m, n, k, ops.backend().info()["sm_count"], -1, -1, -1, plan.ctypes.data)
    assert plan[0] == 1 and plan[2] > 1, "this shape is meant to be split along k"
    g = rnd((n,), torch.bfloat16, 92) + 1.0
    out, h = ops.linear_norm(x, w, g, 1e-6)
    assert isinstance(h, ops.DeferredNorm) and torch.equal(out, ops.linear(x, w))
    w2 = rnd((256, n), torch.bfloat16, 93, 0.05)
    close(ops.linear(h, w2), pm.rms_norm(f64(out), f64(g), 1e-6) @ f64(w2).T, torch.bfloat16, "split-k consumer")
