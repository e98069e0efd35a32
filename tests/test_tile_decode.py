"""The tile decode of the persistent GEMM kernels divides by run-time divisors with a float reciprocal and one
correction step (``fast_div`` in ``ops/csrc/gemm_sm100.cuh``).  This mirrors that arithmetic in fp32 on the CPU and
checks it against integer division over the whole range the kernels use (work items and tiles stay far below 2^22).
"""
import numpy as np
import pytest


def fast_div(x, d):
    xf = x.astype(np.float32)
    inv = np.float32(1.0) / np.float32(d)                      # a correctly rounded reciprocal, as __frcp_rn
    q = np.trunc(xf * inv).astype(np.int64)                    # __float2int_rz
    r = x - q * d
    return q + (r >= d).astype(np.int64) - (r < 0).astype(np.int64)


@pytest.mark.parametrize("d", [1, 2, 3, 5, 7, 13, 16, 25, 74, 100, 147, 148, 255, 296, 448, 1792, 7168, 65536, 99991])
def test_fast_div_matches_integer_division(d):
    x = np.arange(0, 1 << 22, dtype=np.int64)
    assert np.array_equal(fast_div(x, d), x // d)


def test_decode_work_covers_every_tile_once():
    """The grouped tile order (16 row blocks per group) enumerates every (tile_m, tile_n) exactly once."""
    for tiles_m, tiles_n in [(1, 1), (7, 3), (16, 5), (17, 7), (256, 7), (50, 25)]:
        seen = set()
        num = tiles_m * tiles_n
        for t in range(num):
            per_group = 16 * tiles_n
            group = t // per_group
            first_m = group * 16
            gsz = min(tiles_m - first_m, 16)
            in_group = t - group * per_group
            tn = in_group // gsz
            tm = first_m + in_group - tn * gsz
            assert 0 <= tm < tiles_m and 0 <= tn < tiles_n
            seen.add((tm, tn))
        assert len(seen) == num
