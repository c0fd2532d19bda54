"""The kernels form scale = amax / 127 as q = RN(amax*y), r = amax - 127*q, RN(q + r*y) with
y = RN(1/127) instead of calling the division subroutine.  That must be the IEEE quotient for
every fp32 amax in [1e-30, 1e30] (outside it the kernels divide).  The full range (1.67e9 values)
was checked once with the same arithmetic; this test walks every 97th value plus both ends."""
import numpy as np


def quotient_by_correction(a):
    y = np.float32(1.0) / np.float32(127.0)
    a64 = a.astype(np.float64)
    q0 = (a64 * np.float64(y)).astype(np.float32)                     # the product is exact in fp64
    rem = (a64 - q0.astype(np.float64) * 127.0).astype(np.float32)      # exact (as in the FMA)
    return (q0.astype(np.float64) + rem.astype(np.float64) * np.float64(y)).astype(np.float32)


def test_three_instruction_quotient_equals_ieee_division():
    lo = int(np.float32(1e-30).view(np.uint32))
    hi = int(np.float32(1e30).view(np.uint32))
    bits = np.concatenate([np.arange(lo, hi + 1, 97, dtype=np.uint32),
                           np.arange(lo, lo + 4096, dtype=np.uint32), np.arange(hi - 4095, hi + 1, dtype=np.uint32)])
    a = bits.view(np.float32)
    want = (a / np.float32(127.0)).astype(np.float32)
    got = quotient_by_correction(a)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
