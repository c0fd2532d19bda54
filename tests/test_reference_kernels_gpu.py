"""Same-GPU parity against the reference's OWN CUDA operators (its src/world_cuda_ops.cu
compiled in place into oracle/_ref/, see oracle/build_reference_ops.py).

Integer work must agree bit for bit.  The reference is built with --use_fast_math
(reciprocal multiplies, contracted multiply-adds, __sinf/__cosf) while this library follows
the IEEE rule of the reference's PyTorch parity test, so floating-point results are compared
with the tolerances written below: scales within 1e-6 relative, codes never more than one
step apart and different in fewer than 1e-4 of the positions."""
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "oracle"))
import ref_cuda_ops as rk  # noqa: E402

if not rk.available():
    pytest.skip("the reference operator library is not built", allow_module_level=True)


def gen(seed):
    return torch.Generator().manual_seed(seed)


def codes_close(q, q_ref):
    d = (q.int() - q_ref.int()).abs()
    assert int(d.max()) <= 1
    assert float((d > 0).float().mean()) < 1e-4


def scales_close(s, s_ref):
    assert float(((s - s_ref).abs() / s_ref.abs().clamp_min(1e-30)).max()) <= 1e-6


@pytest.mark.parametrize("m,k,n", [(512, 2048, 6144), (512, 2048, 4096), (128, 2048, 2048), (512, 8192, 2048),
                                   (77, 256, 320), (16, 2048, 8192), (2048, 2048, 8192), (1000, 96, 1028)])
def test_int8_gemm_equals_the_reference_cutlass_kernel(pkg, m, k, n):
    g = gen(m + n)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).to(DEV)
    w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).to(DEV)
    acc_ref = torch.empty(m, n, dtype=torch.int32, device=DEV)
    rk.call("gemm_i8_i32", a, w, acc_ref, m, k, n)
    torch.cuda.synchronize()
    assert torch.equal(pkg.gemm_i8_i32(a, w), acc_ref)
    assert pkg.poll_status() == 0


def test_quantizers_against_the_reference_kernels(pkg):
    g = gen(3)
    rows, cols = 512, 2048
    x = torch.randn(rows, cols, generator=g) * 1.7
    x[:, 5] *= 30.0
    x = x.to(DEV)
    q_ref = torch.empty(rows, cols, dtype=torch.int8, device=DEV)
    s_ref = torch.empty(rows, device=DEV)
    rk.call("quantize_rows_f32_i8", x, q_ref, s_ref, rows, cols)
    torch.cuda.synchronize()
    q, s = pkg.quantize_rows(x)
    scales_close(s, s_ref)
    codes_close(q, q_ref)

    mod = (torch.randn(cols, generator=g) * 0.1).to(DEV)
    bias = (torch.randn(cols, generator=g) * 0.1).to(DEV)
    for vec, b in ((mod, bias), (mod, None), (None, None)):
        rk.call("rms_norm_quantize_rows_i8", x, vec, b, q_ref, s_ref, rows, cols, 1e-6)
        torch.cuda.synchronize()
        q, s = pkg.rms_norm_quantize_rows(x, vec, b, 1e-6, scale_is_mod=True)
        scales_close(s, s_ref)
        codes_close(q, q_ref)

    acc = torch.randint(-300000, 300000, (rows, cols), generator=g, dtype=torch.int32).to(DEV)
    sa = (torch.rand(rows, generator=g) * 0.05 + 0.01).to(DEV)
    sw = (torch.rand(cols, generator=g) * 2e-4 + 1e-5).to(DEV)
    for b in (bias, None):
        rk.call("dequant_silu_quantize_rows_i8", acc, sa, sw, b, q_ref, s_ref, rows, cols)
        torch.cuda.synchronize()
        q, s = pkg.dequant_act_quantize_rows(acc, sa, sw, bias=b, act=pkg.ACT_SILU)
        scales_close(s, s_ref)
        codes_close(q, q_ref)


def test_dequantizers_against_the_reference_kernels(pkg):
    g = gen(4)
    rows, cols = 333, 2048
    acc = torch.randint(-300000, 300000, (rows, cols), generator=g, dtype=torch.int32).to(DEV)
    sa = (torch.rand(rows, generator=g) * 0.05 + 0.01).to(DEV)
    sw = (torch.rand(cols, generator=g) * 2e-4 + 1e-5).to(DEV)
    res = torch.randn(rows, cols, generator=g).to(DEV)
    gate = torch.randn(cols, generator=g).to(DEV)
    out_ref = torch.empty(rows, cols, device=DEV)
    rk.call("dequant_gated_residual_f32", acc, sa, sw, res, gate, out_ref, rows, cols)
    torch.cuda.synchronize()
    # the reference contracts residual + v * gate into one fused multiply-add: one rounding fewer
    assert torch.allclose(pkg.dequant_residual(acc, sa, sw, residual=res, gate=gate), out_ref, rtol=1e-6, atol=2e-6)
    rk.call("dequant_add_residual_f32", acc, sa, sw, res, out_ref, rows, cols)
    torch.cuda.synchronize()
    assert torch.allclose(pkg.dequant_residual(acc, sa, sw, residual=res), out_ref, rtol=1e-6, atol=2e-6)


def test_qkv_consumer_and_its_fused_form_against_the_reference_kernel(pkg, ref):
    T, Hq, Hkv, d, W, H, eps = 512, 32, 16, 64, 32, 16, 1e-6
    g = gen(5)
    n = (Hq + 2 * Hkv) * d
    x = torch.randn(T, 2048, generator=g)
    qx, sx = ref.quantize_rows(x)
    qw, sw = ref.quantize_weight(torch.randn(n, 2048, generator=g) * 0.03)
    qx, sx, qw, sw = qx.to(DEV), sx.to(DEV), qw.to(DEV), sw.to(DEV)
    xp = torch.randint(0, W, (T,), generator=g).to(DEV)
    yp = torch.randint(0, H, (T,), generator=g).to(DEV)
    tp = torch.randint(0, 64, (T,), generator=g).to(DEV)
    xy = (torch.rand(d // 8, generator=g) * 6).to(DEV)
    inv_t = torch.rand(d // 2 - 2 * (d // 8), generator=g).to(DEV)
    acc = torch.empty(T, n, dtype=torch.int32, device=DEV)
    q_ref = torch.empty(Hq, T, d, device=DEV)
    k_ref = torch.empty(Hkv, T, d, device=DEV)
    v_ref = torch.empty(Hkv, T, d, device=DEV)
    rk.call("gemm_i8_i32", qx, qw, acc, T, 2048, n)
    rk.call("qkv_fused_rms_rope_i32_dequant", acc, sx, sw, q_ref, k_ref, v_ref, xp, yp, tp, xy, inv_t, T, Hq, Hkv, d,
            W, H, eps)
    torch.cuda.synchronize()
    cos, sin = pkg.rope_tables(xp, yp, tp, xy, inv_t, d, W, H)
    q, k, v = pkg.linear_qkv_heads(qx, sx, qw, sw, cos, sin, Hq, Hkv, d, eps)
    assert torch.equal(v, v_ref)  # plain dequantization: two multiplies either way
    # normalised heads are O(1); fast-math sine/cosine of phases up to ~60 rad are good to ~1e-5
    assert torch.allclose(q, q_ref, rtol=1e-5, atol=2e-4)
    assert torch.allclose(k, k_ref, rtol=1e-5, atol=2e-4)


def test_seeded_random_shapes_against_the_reference_kernels(pkg):
    """Forty seeded shapes (ragged M, N any multiple of 4, K any multiple of 32): raw accumulators equal the
    reference's CUTLASS kernel bit for bit; the fused fp32 linear with residual equals the reference's
    GEMM + dequant_add_residual pair within one rounding (the reference contracts the last multiply-add);
    for M <= 128 the grouped launch equals the single one bit for bit."""
    import random
    rnd = random.Random(7)
    for it in range(40):
        m = rnd.choice([1, 7, 16, 33, 64, 100, 128, 129, 200, 256, 300, 511, 512, 777, 1024])
        k = 128 * rnd.randint(1, 64) if rnd.random() < 0.5 else 32 * rnd.randint(1, 96)
        n = 64 * rnd.randint(1, 96) if rnd.random() < 0.4 else 4 * rnd.randint(1, 700)
        g = gen(1000 + it)
        a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).to(DEV)
        w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).to(DEV)
        acc_ref = torch.empty(m, n, dtype=torch.int32, device=DEV)
        rk.call("gemm_i8_i32", a, w, acc_ref, m, k, n)
        torch.cuda.synchronize()
        assert torch.equal(pkg.gemm_i8_i32(a, w), acc_ref), (m, k, n)
        sa = (torch.rand(m, generator=g) * 0.05 + 0.01).to(DEV)
        sw = (torch.rand(n, generator=g) * 2e-4 + 1e-5).to(DEV)
        res = torch.randn(m, n, generator=g).to(DEV)
        out_ref = torch.empty(m, n, device=DEV)
        rk.call("dequant_add_residual_f32", acc_ref, sa, sw, res, out_ref, m, n)
        torch.cuda.synchronize()
        y = pkg.linear(a, sa, w, sw, residual=res, out_dtype=torch.float32)
        assert torch.allclose(y, out_ref, rtol=1e-6, atol=2e-6), (m, k, n)
        if m <= 128:
            yg = pkg.linear_grouped([dict(x_i8=a, x_scales=sa, w_i8=w, w_scales=sw, n=n, residual=res)],
                                    out_dtype=torch.float32)[0]
            assert torch.equal(yg, y), (m, k, n)
    assert pkg.poll_status() == 0
