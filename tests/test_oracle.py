"""CPU tests of the oracle: it must reproduce the vectors generated from the reference's own
PyTorch helpers, and the reference's four policy tests
(tools/tests/test_w8a8_quantization.py:23-74) must hold when re-expressed on the oracle."""
import math

import numpy as np
import pytest
import torch


@pytest.mark.parametrize("case", ["a", "b", "d", "e"])
def test_oracle_matches_reference_golden_linear(ref, golden, case):
    x = torch.from_numpy(golden[f"{case}_x"].astype(np.float32))
    w = torch.from_numpy(golden[f"{case}_w"].astype(np.float32))
    out, qx, qw, sx, sw, acc = ref.w8a8_linear_reference(x, w)
    assert np.array_equal(qx.numpy(), golden[f"{case}_qx"])
    assert np.array_equal(qw.numpy(), golden[f"{case}_qw"])
    assert np.array_equal(sx.numpy().view(np.uint32), golden[f"{case}_sx"].view(np.uint32))
    assert np.array_equal(sw.numpy().view(np.uint32), golden[f"{case}_sw"].view(np.uint32))
    assert np.array_equal(acc.numpy(), golden[f"{case}_acc"])
    assert np.array_equal(out.numpy().view(np.uint32), golden[f"{case}_out"].view(np.uint32))
    # the exact-in-fp64 GEMM the large tests use gives the same integers
    assert np.array_equal(ref.gemm_i8_i32(qx, qw, exact_fast=True).numpy(), golden[f"{case}_acc"])


def test_oracle_matches_reference_golden_zero_rows(ref, golden):
    q, s = ref.quantize_rows(torch.from_numpy(golden["c_x"]))
    assert np.array_equal(q.numpy(), golden["c_q"])
    assert np.array_equal(s.numpy(), golden["c_s"])


def test_zero_rows_have_unit_scale_and_zero_codes(ref):
    x = torch.zeros(3, 128)
    x[1] = torch.linspace(-2.0, 2.0, 128)
    q, s = ref.quantize_rows(x)
    assert s[0].item() == 1.0 and s[2].item() == 1.0
    assert torch.count_nonzero(q[0]).item() == 0 and torch.count_nonzero(q[2]).item() == 0
    assert q.min().item() >= -127 and q.max().item() <= 127


def test_outer_scale_dequantization_matches_elementwise_formula(ref):
    torch.manual_seed(0x57A8)
    x = torch.randn(17, 128)
    w = torch.randn(33, 128)
    out, qx, qw, sx, sw, acc = ref.w8a8_linear_reference(x, w)
    for row, col in ((0, 0), (3, 7), (16, 32)):
        exact = sum(int(qx[row, i]) * int(qw[col, i]) for i in range(128))
        assert exact == int(acc[row, col])
        expected = float(exact) * float(sx[row]) * float(sw[col])
        assert math.isclose(float(out[row, col]), expected, rel_tol=1e-6, abs_tol=1e-6)


def test_quality_with_row_scale_variation_and_outliers(ref):
    torch.manual_seed(1234)
    m, k, n = 32, 256, 64
    x = torch.randn(m, k)
    w = torch.randn(n, k)
    x *= torch.exp2(torch.linspace(-1.5, 1.5, m))[:, None]
    w *= torch.exp2(torch.linspace(-1.0, 1.0, n))[:, None]
    x[1, k // 3] *= 10.0
    w[1, k // 5] *= -10.0
    out, *_ = ref.w8a8_linear_reference(x, w)
    assert torch.isfinite(out).all()
    assert ref.sqnr_db(x @ w.T, out) >= 30.0


def test_maximum_k_has_int32_headroom(ref):
    assert 127 * 127 * 8192 == 132_128_768 < torch.iinfo(torch.int32).max
    qx = torch.full((1, 8192), 127, dtype=torch.int8)
    qw = torch.full((2, 8192), -127, dtype=torch.int8)
    qw[1] = 127
    acc = ref.gemm_i8_i32(qx, qw)
    assert acc.tolist() == [[-132_128_768, 132_128_768]]


def test_fused_norm_matches_unfused_composition(ref):
    torch.manual_seed(3)
    x = torch.randn(9, 96)
    mod = torch.randn(96) * 0.1
    bias = torch.randn(96) * 0.1
    q, s = ref.rms_norm_quantize_rows(x, mod, bias, 1e-6, scale_is_mod=True)
    v = x * torch.rsqrt((x.double() ** 2).mean(dim=1) + 1e-6).float()[:, None] * (1 + mod) + bias
    q2, s2 = ref.quantize_rows(v)
    assert (q.int() - q2.int()).abs().max() <= 1  # rsqrt vs 1/sqrt may move a tie
    assert torch.allclose(s, s2, rtol=1e-6)


def test_epilogue_forms(ref):
    torch.manual_seed(4)
    acc = torch.randint(-50000, 50000, (5, 16), dtype=torch.int32)
    sa, sw = torch.rand(5) + 0.1, torch.rand(16) * 1e-3
    res, gate = torch.randn(5, 16), torch.randn(16)
    a = ref.dequant_gated_residual(acc, sa, sw, res, gate)
    assert torch.equal(a, res + acc.float() * sa[:, None] * sw[None, :] * gate[None, :])
    b = ref.dequant_add_residual(acc, sa, sw, res)
    assert torch.equal(b, res + acc.float() * sa[:, None] * sw[None, :])
    q, s = ref.dequant_silu_quantize_rows(acc, sa, sw, None)
    v = acc.float() * sa[:, None] * sw[None, :]
    q2, s2 = ref.quantize_rows(v / (1 + torch.exp(-v)))
    assert torch.equal(q, q2) and torch.equal(s, s2)


def test_layer_stack_runs_small(ref):
    d, nq, hid = 128, 384, 512
    lw = ref.make_layer(0, d, nq, hid)
    x = ref.make_tokens(16, 0, torch.float16, d)
    tr = {}
    y = ref.layer_forward(x, lw, trace=tr)
    assert y.shape == x.shape and y.dtype == torch.float16 and torch.isfinite(y.float()).all()
    assert tr["q5"].shape == (16, hid) and tr["qkv"].shape == (16, nq)
    y2 = ref.stack_forward(x, [lw, ref.make_layer(1, d, nq, hid)], steps=2)
    assert torch.isfinite(y2.float()).all()
    assert ref.stack_ops_per_row() == 109_051_904


def test_fma_f32_is_correctly_rounded(ref):
    """The oracle's fp32 fused multiply-add against exact rational arithmetic, including the case where rounding
    to fp64 first and to fp32 second would give the other neighbour."""
    from fractions import Fraction
    import numpy as np

    def exact_fma(a, b, c):
        x = Fraction(float(a)) * Fraction(float(b)) + Fraction(float(c))
        lo = np.float32(float(x))                       # some nearby fp32; walk to the bracketing pair
        cands = [lo, np.nextafter(lo, np.float32(np.inf)), np.nextafter(lo, np.float32(-np.inf))]
        best = min(cands, key=lambda v: (abs(Fraction(float(v)) - x), int(np.float32(v).view(np.uint32)) & 1))
        return np.float32(best)

    g = torch.Generator().manual_seed(3)
    a = torch.randint(-(1 << 21), (1 << 21) + 1, (4000,), generator=g).to(torch.float32)
    b = torch.randn(4000, generator=g) * 1e-4
    c = torch.randn(4000, generator=g) * torch.tensor([1e-3, 1.0, 1e3, 1e6]).repeat(1000)
    # crafted: the exact sum lies 2^-60 below the midpoint between two fp32 values; fp64 rounds onto the midpoint,
    # and round-to-even from there would go UP to the wrong neighbour
    a = torch.cat([a, torch.tensor([float(2 ** 18 + 1), float(2 ** 18 + 1)])])
    b = torch.cat([b, torch.tensor([2.0 ** -42 * (1 - 2.0 ** -18), -(2.0 ** -42) * (1 - 2.0 ** -18)])])
    c = torch.cat([c, torch.tensor([1.0 + 2.0 ** -23, -(1.0 + 2.0 ** -23)])])
    got = ref.fma_f32(a, b, c)
    want = torch.tensor([exact_fma(x, y, z) for x, y, z in zip(a.tolist(), b.tolist(), c.tolist())])
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    assert float(got[-2]) == 1.0 + 2.0 ** -23 and float(got[-1]) == -(1.0 + 2.0 ** -23)
    naive = (a.double() * b.double() + c.double()).float()
    assert float(naive[-2]) != float(got[-2])           # the case really needs the correction
