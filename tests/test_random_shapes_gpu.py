"""Seeded random shapes through the operators against the oracle: the fixed lists of the other files name the
shapes the model uses; this one walks the space between them (odd row counts, N that is no multiple of the tile
width, K of one to many slabs, every output type, every optional epilogue input, both weight layouts)."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def codes(rows, cols, gen, lo=-127):
    return torch.randint(lo, 128, (rows, cols), generator=gen, dtype=torch.int8)


def slab(w):
    n, k = w.shape
    return w.view(n, k // 128, 128).permute(1, 0, 2).contiguous().view(-1)


@pytest.mark.parametrize("seed", range(24))
def test_random_fused_linear_bit_exact(pkg, ref, seed):
    rnd = random.Random(seed)
    m = rnd.choice([1, 7, 16, 33, 100, 128, 129, 255, 300, 511, 640])
    k = 32 * rnd.randint(1, 48) if seed % 3 else 128 * rnd.randint(1, 20)
    n = rnd.choice([4, 8, 24, 64, 100, 128, 136, 200, 256, 264, 520, 1000, 1280])
    dtype = rnd.choice([torch.float16, torch.bfloat16, torch.float32])
    layout = pkg.W_SLAB128 if k % 128 == 0 and rnd.random() < 0.6 else pkg.W_ROW_MAJOR
    g = torch.Generator().manual_seed(1000 + seed)
    a, b = codes(m, k, g), codes(n, k, g)
    sx = torch.rand(m, generator=g) * 0.05 + 0.01
    sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
    bias = torch.randn(n, generator=g) * 0.1 if rnd.random() < 0.5 else None
    gate = torch.randn(n, generator=g) if rnd.random() < 0.4 else None
    res = torch.randn(m, n, generator=g).to(dtype) if (gate is not None or rnd.random() < 0.5) else None
    want = ref.linear_w8a8(a, sx, b, sw, bias=bias, gate=gate, residual=res, out_dtype=dtype)
    dv = lambda t: None if t is None else t.to(DEV)
    w_dev = (slab(b) if layout == pkg.W_SLAB128 else b.reshape(-1)).to(DEV)
    got = pkg.linear(a.to(DEV), sx.to(DEV), w_dev, sw.to(DEV), n=n, w_layout=layout, bias=dv(bias), gate=dv(gate),
                     residual=dv(res), out_dtype=dtype)
    assert pkg.poll_status() == 0
    assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8)), (m, k, n, dtype, layout)
    acc = pkg.gemm_i8_i32(a.to(DEV), w_dev, n=n, w_layout=layout)
    assert torch.equal(acc.cpu(), ref.gemm_i8_i32(a, b)), (m, k, n, layout)


@pytest.mark.parametrize("seed", range(12))
def test_random_quantizers_bit_exact(pkg, ref, seed):
    rnd = random.Random(100 + seed)
    rows = rnd.choice([1, 3, 31, 64, 127, 500, 1025])
    cols = rnd.choice([8, 32, 40, 96, 256, 520, 1000, 2048, 4096, 8192])
    dtype = rnd.choice([torch.float16, torch.bfloat16, torch.float32])
    g = torch.Generator().manual_seed(2000 + seed)
    x = (torch.randn(rows, cols, generator=g) * (10.0 ** rnd.uniform(-3, 2))).to(dtype)
    if rows > 2:
        x[rows // 2] = 0.0
    q, s = pkg.quantize_rows(x.to(DEV))
    q_ref, s_ref = ref.quantize_rows(x)
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32)) and torch.equal(q.cpu(), q_ref), (rows, cols, dtype)
    gamma = torch.randn(cols, generator=g) * 0.2
    beta = torch.randn(cols, generator=g) * 0.1 if rnd.random() < 0.5 else None
    is_mod = rnd.random() < 0.5
    q, s = pkg.rms_norm_quantize_rows(x.to(DEV), gamma.to(DEV), None if beta is None else beta.to(DEV), eps=1e-6,
                                      scale_is_mod=is_mod)
    q_ref, s_ref = ref.rms_norm_quantize_rows(x, gamma, beta, 1e-6, is_mod)
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32)) and torch.equal(q.cpu(), q_ref), (rows, cols, dtype)


@pytest.mark.parametrize("seed", range(10))
def test_random_blockwise_linear_bit_exact(pkg, ref, seed):
    rnd = random.Random(200 + seed)
    m = rnd.choice([1, 16, 100, 128, 129, 300, 640])
    k = 128 * rnd.randint(1, 24)
    n = rnd.choice([8, 64, 128, 136, 200, 520, 1000, 1280])
    dtype = rnd.choice([torch.float16, torch.bfloat16, torch.float32])
    layout = rnd.choice([pkg.W_SLAB128, pkg.W_ROW_MAJOR])
    g = torch.Generator().manual_seed(3000 + seed)
    x = torch.randn(m, k, generator=g) * (10.0 ** rnd.uniform(-2, 1))
    w = torch.randn(n, k, generator=g) * 0.03
    bias = torch.randn(n, generator=g) * 0.1 if rnd.random() < 0.5 else None
    qx, sx = pkg.quantize_blocks128(x.to(DEV))
    packed, sw = pkg.pack_weight_blocks128(w, layout=layout)
    y = pkg.linear_blocks128(qx, sx, packed.to(DEV), sw.to(DEV), n=n, w_layout=layout,
                             bias=None if bias is None else bias.to(DEV), out_dtype=dtype)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    qx_ref, sx_ref = ref.quantize_blocks128(x)
    qw_ref, sw_ref = ref.quantize_blocks128(w)
    assert torch.equal(qx.cpu(), qx_ref) and torch.equal(sx.cpu(), sx_ref)
    want = ref.linear_blocks128(qx_ref, sx_ref, qw_ref, sw_ref, bias=bias, out_dtype=dtype)
    assert torch.equal(y.cpu().view(torch.uint8), want.view(torch.uint8)), (m, k, n, dtype, layout)
