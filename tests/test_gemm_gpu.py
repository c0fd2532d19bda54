"""GPU parity of the tcgen05 int8 GEMM and the fused linear against the CPU oracle.
int32 accumulators must be bit-exact; fused outputs without a transcendental activation
are expected bit-exact too (and are required to be within 2 ulp of the 16-bit output)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def codes(rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-127, 128, (rows, cols), generator=g, dtype=torch.int8)


def slab(w):
    n, k = w.shape
    return w.view(n, k // 128, 128).permute(1, 0, 2).contiguous()


def test_single_mma_known_answer(pkg, ref):
    """128 x 16 x 32: one instruction.  Operands are small distinct integers so that a wrong
    descriptor field shows up as a structured error rather than as noise."""
    m, n, k = 128, 16, 32
    a = ((torch.arange(m)[:, None] * 3 + torch.arange(k)[None, :]) % 11 - 5).to(torch.int8)
    b = ((torch.arange(n)[:, None] * 5 + torch.arange(k)[None, :] * 2) % 7 - 3).to(torch.int8)
    acc = pkg.gemm_i8_i32(a.to(DEV), b.to(DEV))
    assert pkg.poll_status() == 0
    assert torch.equal(acc.cpu(), ref.gemm_i8_i32(a, b))


SHAPES = [(32, 128, 64), (128, 128, 256), (128, 2048, 2048), (512, 2048, 6144), (512, 8192, 2048),
          (512, 2048, 8192), (100, 96, 72), (130, 160, 264), (1, 32, 1), (16, 2048, 2048), (300, 4096, 520),
          (2048, 2048, 2048), (4224, 256, 384)]


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_gemm_i8_i32_bit_exact(pkg, ref, m, k, n):
    a, b = codes(m, k, m + k), codes(n, k, n + k + 1)
    acc = pkg.gemm_i8_i32(a.to(DEV), b.to(DEV))
    assert pkg.poll_status() == 0
    assert torch.equal(acc.cpu(), ref.gemm_i8_i32(a, b))


def test_gemm_extreme_codes_use_full_int32_range(pkg):
    m, k, n = 128, 8192, 128
    a = torch.full((m, k), 127, dtype=torch.int8)
    b = torch.full((n, k), -127, dtype=torch.int8)
    b[1::2] = 127
    acc = pkg.gemm_i8_i32(a.to(DEV), b.to(DEV)).cpu()
    assert int(acc[0, 0]) == -132_128_768 and int(acc[5, 1]) == 132_128_768
    assert torch.equal(acc[:, 0::2], torch.full((m, n // 2), -132_128_768, dtype=torch.int32))


@pytest.mark.parametrize("m,k,n", [(512, 2048, 6144), (64, 8192, 2048), (130, 256, 264)])
def test_gemm_slab_layout_equals_row_major(pkg, ref, m, k, n):
    a, b = codes(m, k, 1), codes(n, k, 2)
    acc_rm = pkg.gemm_i8_i32(a.to(DEV), b.to(DEV))
    acc_sl = pkg.gemm_i8_i32(a.to(DEV), slab(b).to(DEV), n=n, w_layout=pkg.W_SLAB128)
    assert torch.equal(acc_rm, acc_sl)
    assert torch.equal(acc_rm.cpu(), ref.gemm_i8_i32(a, b))


def test_gemm_reference_golden(pkg, golden):
    for case in ("a", "b", "d", "e"):
        qx = torch.from_numpy(golden[f"{case}_qx"])
        qw = torch.from_numpy(golden[f"{case}_qw"])
        if qx.shape[1] % 32:
            continue
        acc = pkg.gemm_i8_i32(qx.to(DEV), qw.to(DEV))
        assert np.array_equal(acc.cpu().numpy(), golden[f"{case}_acc"])


def test_gemm_rejects_bad_arguments(pkg):
    a, b = codes(128, 100, 0).to(DEV), codes(128, 100, 1).to(DEV)
    with pytest.raises(pkg.W8A8Error, match="divisible by 32"):
        pkg.gemm_i8_i32(a, b)


def test_cfg0_single_qkv_linear(pkg, ref):
    """Config 0: X fp16 [512,2048] with x20 outlier channels, W fp16 [6144,2048] ~ N(0,0.02),
    bias ~ N(0,0.01), fp16 output: codes and accumulators bit-exact, output <= 2 fp16 ulp."""
    x, w, bias = ref.make_cfg0()
    qx_ref, sx_ref = ref.quantize_rows(x)
    qw_ref, sw_ref = ref.quantize_weight(w.float())
    acc_ref = ref.gemm_i8_i32(qx_ref, qw_ref)
    y_ref = ref.linear_w8a8(qx_ref, sx_ref, qw_ref, sw_ref, bias=bias, out_dtype=torch.float16)

    packed, sw = pkg.pack_weight(w.float(), layout=pkg.W_SLAB128)
    assert torch.equal(sw.view(torch.int32), sw_ref.view(torch.int32))
    qx, sx = pkg.quantize_rows(x.to(DEV))
    assert torch.equal(qx.cpu(), qx_ref) and torch.equal(sx.cpu().view(torch.int32), sx_ref.view(torch.int32))
    acc = pkg.gemm_i8_i32(qx, packed.to(DEV), n=6144, w_layout=pkg.W_SLAB128)
    assert torch.equal(acc.cpu(), acc_ref)
    y = pkg.linear(qx, sx, packed.to(DEV), sw.to(DEV), w_layout=pkg.W_SLAB128, bias=bias.to(DEV),
                   out_dtype=torch.float16)
    assert pkg.poll_status() == 0
    ulp = ref.ulp_distance_f16(y.cpu(), y_ref)
    assert int(ulp.max()) <= 2
    rel = ((y.cpu().float() - y_ref.float()).abs() / y_ref.float().abs().clamp_min(1e-3)).max()
    assert float(rel) <= 1e-3
    assert int((ulp != 0).sum()) == 0  # same fp32 operation order on both sides: expected identical
    # quality versus the unquantized linear: the x20 outlier channels of this config cost
    # per-token int8 about 5 dB against the reference's 30 dB gate on outlier-free inputs
    assert ref.sqnr_db(x.float() @ w.float().T + bias, y.cpu().float()) >= 20.0


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,k,n", [(512, 2048, 2048), (130, 256, 264), (77, 128, 100)])
@pytest.mark.parametrize("parts", ["plain", "bias", "res", "gate_res", "all"])
def test_fused_linear_bit_exact(pkg, ref, out_dtype, m, k, n, parts):
    g = torch.Generator().manual_seed(m + n)
    a, b = codes(m, k, 3), codes(n, k, 4)
    sx = torch.rand(m, generator=g) * 0.05 + 0.01
    sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(n, generator=g) * 0.1 if parts in ("bias", "all") else None
    gate = torch.randn(n, generator=g) if parts in ("gate_res", "all") else None
    res = torch.randn(m, n, generator=g).to(out_dtype) if parts in ("res", "gate_res", "all") else None
    want = ref.linear_w8a8(a, sx, b, sw, bias=bias, gate=gate, residual=res, out_dtype=out_dtype)
    dv = lambda t: None if t is None else t.to(DEV)
    got = pkg.linear(a.to(DEV), sx.to(DEV), b.to(DEV), sw.to(DEV), bias=dv(bias), gate=dv(gate), residual=dv(res),
                     out_dtype=out_dtype)
    assert pkg.poll_status() == 0
    assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8))


@pytest.mark.parametrize("act", [1, 2])
def test_fused_linear_activation(pkg, ref, act):
    m, k, n = 256, 2048, 1024
    g = torch.Generator().manual_seed(9)
    a, b = codes(m, k, 5), codes(n, k, 6)
    sx = torch.rand(m, generator=g) * 0.02 + 0.005
    sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
    want = ref.epilogue_f32(ref.gemm_i8_i32(a, b), sx, sw, None, act)
    got = pkg.linear(a.to(DEV), sx.to(DEV), b.to(DEV), sw.to(DEV), act=act, out_dtype=torch.float32)
    assert torch.allclose(got.cpu(), want, rtol=4e-6, atol=1e-6)  # SFU exp/rcp: a few ulp
    got16 = pkg.linear(a.to(DEV), sx.to(DEV), b.to(DEV), sw.to(DEV), act=act, out_dtype=torch.float16)
    assert int(ref.ulp_distance_f16(got16.cpu(), want.to(torch.float16)).max()) <= 2


@pytest.mark.parametrize("act", [1, 2])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("pair", [0, 1])
def test_vector_activation_epilogue_equals_the_guarded_one(pkg, act, out_dtype, pair):
    """A linear that dequantizes and activates (the MLP's up linear) through the lean kernel's vector epilogue, and
    the same call with a column-scale vector that is not 16-byte aligned, which takes the general kernel's guarded
    per-element epilogue.  Same operations in the same order: the two must agree bit for bit."""
    m, k, n = 512, 1024, 1024
    g = torch.Generator().manual_seed(12)
    a, b = codes(m, k, 13).to(DEV), codes(n, k, 14).to(DEV)
    sx = (torch.rand(m, generator=g) * 0.02 + 0.005).to(DEV)
    sw_buf = torch.zeros(n + 4, device=DEV)
    sw_buf[1:n + 1] = (torch.rand(n, generator=g) * 2e-4 + 1e-5).to(DEV)
    sw_aligned = sw_buf[1:n + 1].clone()
    pkg.lib().b200_w8a8_set_pair_mma(pair)   # 1: the CTA-pair kernel where it is legal (aligned vectors only)
    try:
        fast = pkg.linear(a, sx, b, sw_aligned, act=act, out_dtype=out_dtype)
        slow = pkg.linear(a, sx, b, sw_buf[1:n + 1], act=act, out_dtype=out_dtype)
    finally:
        pkg.lib().b200_w8a8_set_pair_mma(0)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    assert torch.equal(fast.view(torch.uint8), slow.view(torch.uint8))


def test_fused_linear_strided_output(pkg, ref):
    """Output written into a column block of a wider buffer (row stride > N)."""
    m, k, n = 256, 256, 512
    a, b = codes(m, k, 7), codes(n, k, 8)
    sx, sw = torch.rand(m) * 0.05 + 0.01, torch.rand(n) * 2e-4 + 1e-5
    buf = torch.zeros(m, 3 * n, dtype=torch.float16, device=DEV)
    pkg.linear(a.to(DEV), sx.to(DEV), b.to(DEV), sw.to(DEV), out=buf[:, n:2 * n])
    want = ref.linear_w8a8(a, sx, b, sw, out_dtype=torch.float16)
    assert torch.equal(buf[:, n:2 * n].cpu(), want)
    assert int(buf[:, :n].abs().max()) == 0 and int(buf[:, 2 * n:].abs().max()) == 0


@pytest.mark.parametrize("m,k,n", [(16, 2048, 2048), (64, 8192, 2048), (128, 2048, 8192), (32, 2048, 2048),
                                   (100, 1024, 520), (512, 8192, 2048), (48, 9 * 128, 256)])
@pytest.mark.parametrize("forced", [(0, 0), (64, 4), (128, 2), (256, 8)])
def test_split_k_linear_bit_exact(pkg, ref, m, k, n, forced):
    """Skinny / few-tile shapes with the K range split over several CTAs: integer partial sums are
    added in the workspace, so the result is identical to the unsplit kernel and to the oracle.
    `forced` pins (tile width, K ranges); (0, 0) lets the planner choose.  (9 K slabs in 4 ranges would
    leave the last range empty: the launcher must lower the count rather than reduce a stale accumulator.)"""
    g = torch.Generator().manual_seed(m + k)
    a, b = codes(m, k, 11), codes(n, k, 12)
    sx = torch.rand(m, generator=g) * 0.05 + 0.01
    sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
    res = torch.randn(m, n, generator=g).half()
    want = ref.linear_w8a8(a, sx, b, sw, residual=res, out_dtype=torch.float16)
    splits = forced[1] if forced[1] else 8
    ws = torch.zeros(4096 + splits * m * n * 4, dtype=torch.uint8, device=DEV)
    pkg.lib().b200_w8a8_debug_force_plan(forced[0], forced[1], 1 if forced[1] else 0)
    try:
        for _ in range(2):  # twice through the same workspace: it must come back zero-filled where it matters
            got = pkg.linear(a.to(DEV), sx.to(DEV), b.to(DEV), sw.to(DEV), residual=res.to(DEV),
                             out_dtype=torch.float16, workspace=ws)
            assert pkg.poll_status() == 0
            assert torch.equal(got.cpu(), want)
            assert int(ws[:4096].view(torch.int32).abs().max()) == 0  # ticket counters are back at zero
    finally:
        pkg.lib().b200_w8a8_debug_force_plan(0, 0, 0)


def test_split_k_planner_reports_workspace(pkg):
    lib = pkg.lib()
    # one tile, very long K that no cluster size divides (515 slabs): the split goes through the workspace
    assert lib.b200_w8a8_linear_workspace_size(16, 515 * 128, 64) > 0
    assert lib.b200_w8a8_linear_workspace_size(16, 65536, 64) == 0      # a cluster split needs no workspace
    assert lib.b200_w8a8_linear_workspace_size(16384, 2048, 6144) == 0  # plenty of tiles: no split


@pytest.mark.parametrize("m,k,n", [(512, 8192, 2048), (512, 2048, 2048), (100, 1024, 520), (16, 2048, 2048),
                                   (300, 512, 6144)])
@pytest.mark.parametrize("bn,splits", [(256, 4), (256, 2), (128, 4), (128, 2), (64, 2)])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_cluster_split_k_linear_bit_exact(pkg, ref, m, k, n, bn, splits, out_dtype):
    """K split over the CTAs of a thread-block cluster; partial sums meet in shared memory.
    Needs no workspace and must give the same bits as the unsplit kernel and the oracle."""
    g = torch.Generator().manual_seed(m + k + bn)
    a, b = codes(m, k, 31), codes(n, k, 32)
    sx = torch.rand(m, generator=g) * 0.05 + 0.01
    sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(n, generator=g) * 0.1
    res = torch.randn(m, n, generator=g).to(out_dtype)
    want = ref.linear_w8a8(a, sx, b, sw, bias=bias, residual=res, out_dtype=out_dtype)
    pkg.lib().b200_w8a8_debug_force_plan(bn, splits, 2)
    try:
        got = pkg.linear(a.to(DEV), sx.to(DEV), b.to(DEV), sw.to(DEV), bias=bias.to(DEV), residual=res.to(DEV),
                         out_dtype=out_dtype)
        assert pkg.poll_status() == 0
        assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8))
        acc = pkg.gemm_i8_i32(a.to(DEV), b.to(DEV))
        assert torch.equal(acc.cpu(), ref.gemm_i8_i32(a, b))
    finally:
        pkg.lib().b200_w8a8_debug_force_plan(0, 0, 0)


@pytest.fixture
def pair_mma(pkg):
    pkg.lib().b200_w8a8_set_pair_mma(1)  # two CTAs per 256 x 256 tile wherever the launch allows it
    yield
    pkg.lib().b200_w8a8_set_pair_mma(0)


@pytest.mark.parametrize("m,k,n", [(256, 128, 256), (512, 2048, 6144), (130, 256, 512), (300, 4096, 544),
                                   (2048, 2048, 2048), (4224, 256, 384), (1024, 8192, 2048)])
def test_pair_mma_gemm_bit_exact(pkg, ref, pair_mma, m, k, n):
    """cta_group::2: a cluster of two CTAs shares one tile (each loads half of the W rows)."""
    a, b = codes(m, k, m + 3), codes(n, k, n + 5)
    acc = pkg.gemm_i8_i32(a.to(DEV), b.to(DEV))
    assert pkg.poll_status() == 0
    assert torch.equal(acc.cpu(), ref.gemm_i8_i32(a, b))
    g = torch.Generator().manual_seed(m)
    sx = torch.rand(m, generator=g) * 0.05 + 0.01
    sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(n, generator=g) * 0.1
    res = torch.randn(m, n, generator=g).half()
    want = ref.linear_w8a8(a, sx, b, sw, bias=bias, residual=res, out_dtype=torch.float16)
    got = pkg.linear(a.to(DEV), sx.to(DEV), slab(b).to(DEV), sw.to(DEV), n=n, w_layout=pkg.W_SLAB128,
                     bias=bias.to(DEV), residual=res.to(DEV), out_dtype=torch.float16)
    assert pkg.poll_status() == 0
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("m,k,n", [(512, 2048, 2048), (100, 512, 520), (16, 2048, 2048), (300, 256, 64), (640, 8192, 2048)])
@pytest.mark.parametrize("use_slab", [False, True])
def test_two_slab_stages_of_narrow_tiles_bit_exact(pkg, ref, m, k, n, use_slab):
    """64-wide tiles of an unsplit launch bring two K slabs per copy and pipeline stage.  Forced to that tile width,
    with and without the two-slab stages, the accumulators and a fused fp16 linear must equal the oracle."""
    a, b = codes(m, k, m + 1), codes(n, k, n + 2)
    g = torch.Generator().manual_seed(m + n)
    sx = torch.rand(m, generator=g) * 0.05 + 0.01
    sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
    res = torch.randn(m, n, generator=g).half()
    want_acc = ref.gemm_i8_i32(a, b)
    want = ref.linear_w8a8(a, sx, b, sw, residual=res, out_dtype=torch.float16)
    wd = (slab(b) if use_slab else b).to(DEV)
    layout = pkg.W_SLAB128 if use_slab else pkg.W_ROW_MAJOR
    lib = pkg.lib()
    lib.b200_w8a8_debug_force_plan(64, 1, 0)
    try:
        for one_slab in (0, 1):
            lib.b200_w8a8_debug_one_slab_stages(one_slab)
            acc = pkg.gemm_i8_i32(a.to(DEV), wd, n=n, w_layout=layout)
            y = pkg.linear(a.to(DEV), sx.to(DEV), wd, sw.to(DEV), n=n, w_layout=layout, residual=res.to(DEV),
                           out_dtype=torch.float16)
            assert pkg.poll_status() == 0
            assert torch.equal(acc.cpu(), want_acc), f"accumulators differ (one_slab={one_slab})"
            assert torch.equal(y.cpu(), want), f"fused linear differs (one_slab={one_slab})"
    finally:
        lib.b200_w8a8_debug_one_slab_stages(0)
        lib.b200_w8a8_debug_force_plan(0, 0, 0)
