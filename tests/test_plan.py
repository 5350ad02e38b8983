"""The launcher's choices for the tensor-core product (which operand feeds the M side, tile width, how k is cut), asked
of the built library on the host: no GPU is needed to plan a product."""
import ctypes

import pytest

from friday_inference_engine_b200.ops import lib

SMS = 148


@pytest.fixture(scope="module", autouse=True)
def library():
    """Built on first use (nvcc cross-compiles without a GPU); where it cannot be built or loaded there is nothing to ask."""
    try:
        return lib.family("gemm_tc")
    except Exception as e:           # no compiler, or no CUDA runtime library to load against
        pytest.skip("the gemm_tc library is not available here: %s" % e)


def plan(m, n, k, swap=-1, bn=-1, splits=-1):
    out = (ctypes.c_longlong * 8)()
    lib.family("gemm_tc").cdll.gemm_tc_plan(m, n, k, SMS, swap, bn, splits, out)
    return {"swap": int(out[0]), "bn": int(out[1]), "splits": int(out[2]), "scratch": int(out[3]), "counters": int(out[4])}


def tiles_of(p, m, n):
    rows, cols = (n, m) if p["swap"] else (m, n)
    return -(-rows // 128) * -(-cols // p["bn"])


@pytest.mark.parametrize("m", [1, 8, 16])
def test_few_rows_put_the_weights_on_the_m_side(m):
    # 7B shapes: q/k/v (36 tiles of 128 weight rows), gate and up (296: two whole waves of 148 SMs), down (28)
    p = plan(m, 4608, 3584)
    assert (p["swap"], p["bn"], p["splits"]) == (1, 16, 4)
    assert plan(m, 37888, 3584)["splits"] == 1
    p = plan(m, 3584, 18944)
    assert p["splits"] == 5 and p["counters"] == 28 and p["scratch"] == 28 * 5 * 128 * 16
    # 14B gate and up: 216 tiles would leave the second wave half empty; k is cut in two
    assert plan(m, 27648, 5120)["splits"] == 2
    # 32B gate and up (432 tiles, 2.9 waves) and the head (1,188 tiles) are left whole
    assert plan(m, 55296, 5120)["splits"] == 1 and plan(m, 152064, 3584)["splits"] == 1


def test_tile_width_follows_the_rows():
    assert [plan(m, 3584, 3584)["bn"] for m in (16, 17, 32, 33, 64, 65, 128)] == [16, 32, 32, 64, 64, 128, 128]
    assert all(plan(m, 3584, 3584)["swap"] == 1 for m in (1, 64, 65, 128)) and plan(129, 3584, 3584)["swap"] == 0
    # wide partial tiles are costly to merge: rows on the M side are cut at most four ways, and only where a split keeps
    # 64 k blocks
    assert plan(130, 3584, 18944)["splits"] <= 4 and plan(256, 4608, 3584)["splits"] == 1
    # pairs of SMs take narrower tiles where k is short and wider ones leave pairs idle
    assert plan(256, 4608, 3584)["bn"] == 64 and plan(512, 3584, 3584)["bn"] == 112 and plan(512, 3584, 18944)["bn"] == 128


def test_many_rows_fill_whole_waves_of_pairs():
    # 2,048 rows are 8 tiles of 256 rows on 74 pairs of SMs; the width is the multiple of 16 that wastes the least
    assert plan(2048, 37888, 3584)["bn"] == 256                 # 8 x 148 tiles: 16 whole waves
    p = plan(2048, 3584, 18944)
    assert p["swap"] == 0 and p["splits"] == 1 and 128 <= p["bn"] <= 256 and p["bn"] % 16 == 0
    waves = -(-8 * -(-3584 // p["bn"]) // 74)
    assert waves * (p["bn"] + 16) <= 2 * (256 + 16), "no worse than two waves of the widest tile"


@pytest.mark.parametrize("m,n,k", [(8, 3584, 18944), (3, 128 * 160, 1024), (130, 272, 18944), (40, 4608, 3584)])
def test_scratch_and_counters_match_the_split(m, n, k):
    p = plan(m, n, k)
    if p["splits"] > 1:
        assert p["counters"] == tiles_of(p, m, n) and p["scratch"] == p["counters"] * p["splits"] * 128 * p["bn"]
    else:
        assert p["counters"] == 0 and p["scratch"] == 0
    forced = plan(m, n, k, splits=3)
    assert forced["splits"] <= 3 and forced["bn"] == p["bn"]
