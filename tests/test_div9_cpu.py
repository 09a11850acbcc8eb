"""The 3x3 average-pool fast path divides by 9 with a rounded reciprocal and one exact FMA
residual.  That sequence must equal the correctly rounded x / 9 for every float it is used on.
Division by a constant is invariant under scaling by powers of two, so one full binade
(all 2^23 significands, both signs) covers every normal input; the float64 emulation of the
two FMAs below is exact (products of two 24-bit significands and the following sums fit in 53 bits)."""
import numpy as np


def test_fma_division_by_nine_is_correctly_rounded_over_a_full_binade():
    m = np.arange(1 << 23, dtype=np.uint32)
    for sign in (0, 0x80000000):
        x = (m | np.uint32(0x3F800000) | np.uint32(sign)).view(np.float32)       # [1, 2) and (-2, -1]
        r = np.float32(1.0) / np.float32(9.0)
        q0 = x * r
        e = (x.astype(np.float64) - q0.astype(np.float64) * 9.0).astype(np.float32)
        assert np.array_equal(e.astype(np.float64), x.astype(np.float64) - q0.astype(np.float64) * 9.0)  # exact
        q = (q0.astype(np.float64) + e.astype(np.float64) * np.float64(r)).astype(np.float32)
        assert np.array_equal(q, x / np.float32(9.0))
