"""GPU parity of the activation quantizers and accumulator consumers against the CPU oracle.
Codes and scales must be bit-exact wherever no transcendental function is involved."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int32)


def tokens(rows, cols, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    x *= torch.exp2(torch.linspace(-3, 3, rows))[:, None]
    if cols >= 8:
        x[:, :: max(cols // 8, 1)] *= 20.0
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(3, 128), (17, 128), (512, 2048), (33, 100), (7, 8200), (5000, 2048),
                                       (64, 8192), (2, 20000), (130, 24), (1, 8)])
def test_quantize_rows_bit_exact(pkg, ref, dtype, rows, cols):
    x = tokens(rows, cols, rows * 131 + cols, dtype)
    if rows >= 3:
        x[2] = 0
    q_ref, s_ref = ref.quantize_rows(x)
    q, s = pkg.quantize_rows(x.to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(bits(s), bits(s_ref))
    assert torch.equal(q.cpu(), q_ref)


def test_quantize_rows_reference_golden(pkg, golden):
    for case in ("a", "b", "d", "e"):
        x = torch.from_numpy(golden[f"{case}_x"].astype(np.float32))
        q, s = pkg.quantize_rows(x.to(DEV))
        assert np.array_equal(q.cpu().numpy(), golden[f"{case}_qx"])
        assert np.array_equal(s.cpu().numpy().view(np.uint32), golden[f"{case}_sx"].view(np.uint32))
    q, s = pkg.quantize_rows(torch.from_numpy(golden["c_x"]).to(DEV))
    assert np.array_equal(q.cpu().numpy(), golden["c_q"]) and np.array_equal(s.cpu().numpy(), golden["c_s"])


def test_quantize_rows_strided_view_and_empty(pkg, ref):
    x = tokens(96, 6144, 5, torch.float16).to(DEV)
    q, s = pkg.quantize_rows(x, cols=2048)  # first 2048 columns of rows 6144 apart
    q_ref, s_ref = ref.quantize_rows(x.cpu()[:, :2048])
    assert torch.equal(q.cpu(), q_ref) and torch.equal(bits(s), bits(s_ref))
    q, s = pkg.quantize_rows(torch.empty(0, 128, device=DEV))
    assert q.shape == (0, 128)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(512, 2048), (9, 96), (4100, 2048), (33, 100), (16, 8192)])
@pytest.mark.parametrize("variant", ["plain", "mod", "mod_bias", "gamma"])
def test_rms_norm_quantize_rows_bit_exact(pkg, ref, dtype, rows, cols, variant):
    x = tokens(rows, cols, rows + cols, dtype)
    g = torch.Generator().manual_seed(11)
    vec = torch.randn(cols, generator=g) * 0.05
    bias = torch.randn(cols, generator=g) * 0.1
    scale_is_mod = variant != "gamma"
    if variant == "plain":
        vec_in, bias_in = None, None
    elif variant == "mod":
        vec_in, bias_in = vec, None
    elif variant == "mod_bias":
        vec_in, bias_in = vec, bias
    else:
        vec_in, bias_in = 1.0 + vec, None
    eps = 1e-6
    q_ref, s_ref = ref.rms_norm_quantize_rows(x, vec_in, bias_in, eps, scale_is_mod)
    q, s = pkg.rms_norm_quantize_rows(x.to(DEV), None if vec_in is None else vec_in.to(DEV),
                                      None if bias_in is None else bias_in.to(DEV), eps, scale_is_mod)
    mism = int((q.cpu() != q_ref).sum())
    smism = int((bits(s) != bits(s_ref)).sum())
    # the fp64 sum of squares may differ in its last bit between summation orders, which can
    # move the fp32 inv_rms of a row by one ulp about once per 1e9 rows; anything else is a bug
    assert smism == 0 and mism == 0, f"{mism} code and {smism} scale mismatches"


@pytest.mark.parametrize("act", [1, 2])
@pytest.mark.parametrize("rows,cols,with_bias", [(128, 2048, True), (512, 8192, False), (19, 72, True)])
def test_dequant_act_quantize_rows(pkg, ref, parity_log, act, rows, cols, with_bias):
    g = torch.Generator().manual_seed(rows + act)
    acc = torch.randint(-120000, 120000, (rows, cols), generator=g, dtype=torch.int32)
    sa = torch.rand(rows, generator=g) * 0.05 + 0.01
    sw = torch.rand(cols, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(cols, generator=g) * 0.2 if with_bias else None
    q_ref, s_ref = ref.dequant_silu_quantize_rows(acc, sa, sw, bias, act=act)
    sa_dev = sa.to(DEV)
    # in and out scale vectors alias, as at the reference's call sites (src/world_cuda.cu:2131,2135)
    q, s = pkg.dequant_act_quantize_rows(acc.to(DEV), sa_dev, sw.to(DEV), None if bias is None else bias.to(DEV),
                                         act=act, out_row_scales=sa_dev)
    assert s.data_ptr() == sa_dev.data_ptr()
    assert torch.allclose(s.cpu(), s_ref, rtol=2e-6, atol=0)
    diff = (q.cpu().int() - q_ref.int()).abs()
    row = parity_log(f"dequant_act_quantize_rows act={act} {rows}x{cols}", int((diff != 0).sum()), diff.numel(),
                     max_step=int(diff.max()))
    assert int(diff.max()) <= 1
    # exp/tanh differ in the last ulps between libraries: a code may move across a rounding tie.
    # Measured on B200: 8 and 6 of 4 194 304 positions (1.9e-6, 1.4e-6) at 512 x 8192, none at the small
    # sizes; the bound is twice the largest measured rate (one position at 128 x 2048).
    assert row["rate"] < 4e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(512, 2048), (33, 100), (70000, 8), (16384, 2048)])
@pytest.mark.parametrize("gated", [False, True])
def test_dequant_residual_bit_exact(pkg, ref, dtype, rows, cols, gated):
    g = torch.Generator().manual_seed(rows)
    acc = torch.randint(-2 ** 27, 2 ** 27, (rows, cols), generator=g, dtype=torch.int32)
    sa = torch.rand(rows, generator=g) * 0.05 + 0.01
    sw = torch.rand(cols, generator=g) * 2e-4 + 1e-5
    res = torch.randn(rows, cols, generator=g).to(dtype)
    gate = torch.randn(cols, generator=g) if gated else None
    want = (ref.dequant_gated_residual(acc, sa, sw, res, gate) if gated
            else ref.dequant_add_residual(acc, sa, sw, res)).to(dtype)
    got = pkg.dequant_residual(acc.to(DEV), sa.to(DEV), sw.to(DEV), res.to(DEV), None if gate is None else gate.to(DEV))
    assert got.dtype == dtype
    assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8))


def test_qkv_rms_rope_dequant(pkg, ref):
    T, Hq, Hkv, d, W, H = 96, 8, 4, 64, 16, 8
    g = torch.Generator().manual_seed(2)
    n = (Hq + 2 * Hkv) * d
    acc = torch.randint(-200000, 200000, (T, n), generator=g, dtype=torch.int32)
    sa = torch.rand(T, generator=g) * 0.05 + 0.01
    sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
    xp = torch.randint(0, W, (T,), generator=g)
    yp = torch.randint(0, H, (T,), generator=g)
    tp = torch.randint(0, 32, (T,), generator=g)
    xy = torch.rand(d // 8, generator=g) * 6.0
    inv_t = torch.rand(d // 2 - 2 * (d // 8), generator=g)
    eps = 1e-6
    q_ref, k_ref, v_ref = ref.qkv_fused_rms_rope_i32_dequant(acc, sa, sw, xp, yp, tp, xy, inv_t, Hq, Hkv, d, W, H, eps)
    q, k, v = pkg.qkv_rms_rope_dequant(acc.to(DEV), sa.to(DEV), sw.to(DEV), xp.to(DEV), yp.to(DEV), tp.to(DEV),
                                       xy.to(DEV), inv_t.to(DEV), Hq, Hkv, d, W, H, eps)
    assert torch.equal(v.cpu(), v_ref)  # plain dequant: exact
    assert torch.allclose(q.cpu(), q_ref, rtol=1e-5, atol=2e-6)  # cos/sin differ in the last ulps
    assert torch.allclose(k.cpu(), k_ref, rtol=1e-5, atol=2e-6)


def test_quantize_rows_many_scales_bit_exact(pkg, ref):
    """The kernel divides by the row scale with a refined reciprocal multiply instead of a division
    instruction; that must still be the correctly rounded quotient for every scale.  65536 rows with
    scales over 60 binades, values placed at and next to rounding ties, plus tiny and huge rows."""
    g = torch.Generator().manual_seed(99)
    rows, cols = 65536, 64
    amax = torch.exp2(torch.rand(rows, generator=g) * 60 - 30) * (1 + torch.rand(rows, generator=g))
    codes = torch.randint(-127, 128, (rows, cols), generator=g).float()
    frac = torch.tensor([0.0, 0.5, -0.5, 0.49999997, 0.50000006, 0.25, -0.49999997, 0.5])[
        torch.randint(0, 8, (rows, cols), generator=g)]
    x = (codes + frac) * (amax / 127.0)[:, None]
    x[:, 0] = amax
    x[:16] *= 1e-35   # near the subnormal range: the plain-division path
    x[16:32] *= 1e30
    q_ref, s_ref = ref.quantize_rows(x)
    q, s = pkg.quantize_rows(x.to(DEV))
    assert torch.equal(bits(s), bits(s_ref))
    assert torch.equal(q.cpu(), q_ref)


def test_qkv_consumer_refuses_a_misaligned_accumulator(pkg):
    """The stand-alone QKV consumer reads accumulators and weight scales two at a time: a view that starts on an odd
    element must come back as an error (return 1 + message), not as a misaligned access on the device."""
    T, Hq, Hkv, d = 8, 2, 1, 64
    n = (Hq + 2 * Hkv) * d
    acc = torch.zeros(T * n + 1, dtype=torch.int32, device=DEV)[1:].view(T, n)   # 4-byte offset
    sa, sw = torch.ones(T, device=DEV), torch.ones(n, device=DEV)
    pos = torch.zeros(T, dtype=torch.int64, device=DEV)
    xy, inv_t = torch.ones(d // 8, device=DEV), torch.ones(d // 2 - 2 * (d // 8), device=DEV)
    with pytest.raises(pkg.W8A8Error, match="8-byte aligned"):
        pkg.qkv_rms_rope_dequant(acc, sa, sw, pos, pos, pos, xy, inv_t, Hq, Hkv, d, 16, 8, 1e-6)


def test_mma_rate_self_test_reports_a_plausible_ceiling(pkg):
    rate = pkg.mma_rate(4096)
    assert 1000.0 < rate < 9000.0, rate   # TOP/s: above any GEMM of this library, below twice the nominal dense figure
    assert pkg.poll_status() == 0
