"""gemm_tc_noalloc, the entry point for callers that cannot allocate device memory (a
server that gave all of it away at start-up, a loop that cannot afford an allocation's
synchronisation, a host program without an allocator): called through its exported C
symbol, twice in a row, and compared with the ordinary entry point, which takes its
scratch from the caller.  The file sorts last so that a run that stops at the first
failure has already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_entry_point_matches_the_ordinary_one_twice():
    from friday_inference_engine_b200 import ops
    from friday_inference_engine_b200.ops import lib

    dev = torch.device("cuda:0")
    fam = lib.family("gemm_tc")                      # builds the library if needed; gives its path
    cdll = ctypes.CDLL(fam.path)
    fn = cdll.gemm_tc_noalloc
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, I, P, I, P, I, I, I, I, I, I, P, P]
    fn.restype = I
    err = cdll.gemm_tc_last_error
    err.restype = ctypes.c_char_p

    g = torch.Generator().manual_seed(5)
    be = ops.backend()
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    # a decoding shape that splits k (36 tiles on 148 SMs) with the last CTA finishing the tile, one of 17 to 64 rows
    # whose CTAs all finish 16 rows each of a split tile, and one that does not split
    for m, n, k in ((8, 4608, 3584), (40, 4608, 3584), (40, 18944, 512)):
        x = torch.randn((m, k), generator=g).to(torch.bfloat16).to(dev)
        w = (torch.randn((n, k), generator=g) * 0.05).to(torch.bfloat16).to(dev)
        bias = torch.randn((n,), generator=g).to(torch.bfloat16).to(dev)
        res = torch.randn((m, n), generator=g).to(dev)
        want = be._linear_tc(x, w, bias, res, torch.empty((m, n), dtype=torch.float32, device=dev))
        ref = x.double() @ w.double().t() + bias.double() + res.double()
        scale = float(ref.abs().max())
        assert float((want.double() - ref).abs().max()) <= 3e-5 * scale          # the ordinary entry point is right
        for call in range(2):                                                   # two calls in a row share the area
            out = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
            rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, bias.data_ptr(), 1, res.data_ptr(), m, n, k,
                    x.stride(0), w.stride(0), out.stride(0), status.data_ptr(), stream)
            assert rc == 0, err().decode()
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            diff = float((out.double() - want.double()).abs().max())
            assert diff <= 3e-5 * scale, "call %d of %dx%dx%d differs from gemm_tc by %.3g" % (call, m, n, k, diff)
    # beyond the built-in area: refused with a message, nothing launched.  How k is split depends on the number of
    # SMs, so the shape is chosen by asking the planner with this device's count.
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    plan = (ctypes.c_longlong * 8)()
    too_big = None
    for m, n, k in ((128, 9216, 8192), (300, 700, 8192), (128, 5120, 16384), (128, 4608, 32768), (256, 2304, 65536)):
        cdll.gemm_tc_plan(m, n, k, sms, -1, -1, -1, plan)
        if plan[3] > 2 * 1024 * 1024:
            too_big = (m, n, k)
            break
    assert too_big is not None, "the test's premise: one of these shapes needs more partial tiles than the area holds"
    m, n, k = too_big
    x = torch.zeros((m, k), dtype=torch.bfloat16, device=dev)
    w = torch.zeros((n, k), dtype=torch.bfloat16, device=dev)
    out = torch.zeros((m, n), dtype=torch.float32, device=dev)
    rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, None, 0, None, m, n, k, k, k, n, status.data_ptr(), stream)
    assert rc != 0 and b"built-in area" in err()
    torch.cuda.synchronize()
