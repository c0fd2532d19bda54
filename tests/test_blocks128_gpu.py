"""The 128 x 128 blockwise numerics (b200_w8a8_quantize_blocks128 / _pack_weight_blocks128_host /
_linear_blocks128) against the CPU restatement of the rule.  The reference describes this rule in its notes
(docs/cuda_w8a8_optimization.md:319-321) but ships no implementation of it, so there are no reference vectors."""
import pytest
import torch

DEV = "cuda:0"


def acts(rows, cols, seed, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    x[:, : min(cols, 128)] *= 6.0        # one K block with a wider range than the others
    if rows > 3:
        x[3] = 0.0
    return x.to(dtype)


def unslab(packed, n, k):
    return packed.view(k // 128, n, 128).permute(1, 0, 2).reshape(n, k)


@pytest.mark.parametrize("layout", [0, 1])
def test_blockwise_weight_packer_matches_the_oracle(pkg, ref, layout):
    g = torch.Generator().manual_seed(11)
    n, k = 200, 384
    w = torch.randn(n, k, generator=g) * 0.02
    w[:128, 128:256] = 0.0               # an all-zero block takes the floor scale 1e-8 / 128
    w[130, 5] = -1.0                     # a block whose extreme is negative reaches code -128
    packed, scales = pkg.pack_weight_blocks128(w, layout=layout, threads=3)
    q_ref, s_ref = ref.quantize_blocks128(w)
    codes = packed.view(n, k) if layout == pkg.W_ROW_MAJOR else unslab(packed, n, k)
    assert torch.equal(scales.view(torch.int32), s_ref.view(torch.int32))
    assert torch.equal(codes, q_ref)
    assert scales[0, 1].item() == torch.tensor(1e-8, dtype=torch.float32).item() / 128 and int(codes[:128, 128:256].abs().max()) == 0
    assert int(codes.min()) == -128 and int(codes.max()) == 127
    bad = w.clone()
    bad[7, 300] = float("inf")
    with pytest.raises(pkg.W8A8Error, match="not finite"):
        pkg.pack_weight_blocks128(bad, layout=layout)
    with pytest.raises(pkg.W8A8Error, match="128"):
        pkg.pack_weight_blocks128(torch.randn(8, 96), layout=layout)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 128), (128, 128), (300, 256), (2048, 2048), (1000, 8192)])
def test_block_quantizer_bit_exact(pkg, ref, rows, cols, dtype):
    x = acts(rows, cols, rows + cols, dtype)
    q, s = pkg.quantize_blocks128(x.to(DEV))
    q_ref, s_ref = ref.quantize_blocks128(x)
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))
    assert torch.equal(q.cpu(), q_ref)


@pytest.mark.gpu
def test_block_quantizer_rounding_ties_and_extremes(pkg, ref):
    # every block is scaled so that scale = 2^e exactly: quotients k + 0.5 are then exact ties
    rows, cols = 256, 256
    x = torch.zeros(rows, cols)
    base = torch.arange(-128, 128, dtype=torch.float32)
    for r in range(rows):
        x[r] = (base + 0.5).roll(r)[:cols] if cols <= 256 else 0
    x[0, 0] = 128.0   # amax 128 -> scale 1 in the first block column
    x[0, 128] = -128.0
    x[128, 0] = 128.0
    x[128, 128] = 128.0
    q, s = pkg.quantize_blocks128(x.to(DEV))
    q_ref, s_ref = ref.quantize_blocks128(x)
    assert torch.equal(s.cpu(), s_ref) and float(s_ref[0, 0]) == 1.0
    assert torch.equal(q.cpu(), q_ref)
    assert int(q_ref.max()) == 127 and int(q_ref.min()) == -128   # +128 saturates, -128 is kept


@pytest.mark.gpu
def test_block_quantizer_rejects_bad_shapes(pkg):
    with pytest.raises(pkg.W8A8Error, match="divisible by 128"):
        pkg.quantize_blocks128(torch.zeros(16, 96, device=DEV))
    with pytest.raises(pkg.W8A8Error, match="aligned"):
        pkg.quantize_blocks128(torch.zeros(16, 130, device=DEV, dtype=torch.float16)[:, 1:129])
    with pytest.raises(pkg.W8A8Error, match="128 or 1"):
        pkg.quantize_blocks128(torch.zeros(16, 128, device=DEV), block_rows=64)


@pytest.mark.gpu
def test_the_library_picks_the_wide_tile_when_it_fills_the_machine(pkg, ref):
    """Unforced: 2048 x 6144 is 384 wide tiles (>= one per SM) -> 256-wide kernel; the same problem forced to 128-wide
    tiles gives the same bits."""
    m, k, n = 2048, 256, 6144
    g = torch.Generator().manual_seed(31)
    x = acts(m, k, 9)
    w = torch.randn(n, k, generator=g) * 0.03
    qx, sx = pkg.quantize_blocks128(x.to(DEV))
    packed, sw = pkg.pack_weight_blocks128(w)
    packed, sw = packed.to(DEV), sw.to(DEV)
    y_auto = pkg.linear_blocks128(qx, sx, packed, sw, n=n)
    pkg.lib().b200_w8a8_debug_force_plan(128, 0, 0)
    try:
        y_128 = pkg.linear_blocks128(qx, sx, packed, sw, n=n)
    finally:
        pkg.lib().b200_w8a8_debug_force_plan(0, 0, 0)
    torch.cuda.synchronize()
    qx_ref, sx_ref = ref.quantize_blocks128(x)
    qw_ref, sw_ref = ref.quantize_blocks128(w)
    want = ref.linear_blocks128(qx_ref, sx_ref, qw_ref, sw_ref, out_dtype=torch.float16)
    assert torch.equal(y_auto.cpu(), want) and torch.equal(y_128.cpu(), want)


CASES = [  # m, k, n, out dtype, layout, bias
    (128, 128, 128, torch.float32, 0, False),
    (100, 256, 200, torch.float16, 1, True),      # ragged rows and columns
    (16, 2048, 2048, torch.float16, 1, False),    # skinny
    (512, 2048, 6144, torch.float16, 1, True),    # QKV at 512 rows
    (2048, 2048, 2048, torch.bfloat16, 1, False),
    (300, 8192, 2048, torch.float32, 0, True),    # 64 K blocks: every accumulator slot is reused 16 times
    (1500, 1024, 520, torch.bfloat16, 0, False),  # several tiles per CTA, N not a multiple of 128
]


@pytest.fixture
def tile_width(pkg, request):
    """Forces the kernel's tile width (the library picks 256 only when that still gives every SM a tile)."""
    pkg.lib().b200_w8a8_debug_force_plan(request.param, 0, 0)
    yield request.param
    pkg.lib().b200_w8a8_debug_force_plan(0, 0, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("tile_width", [128, 256], indirect=True)
@pytest.mark.parametrize("m,k,n,dtype,layout,with_bias", CASES)
def test_blockwise_linear_bit_exact(pkg, ref, tile_width, m, k, n, dtype, layout, with_bias):
    g = torch.Generator().manual_seed(m + k + n)
    x = acts(m, k, m + n)
    w = torch.randn(n, k, generator=g) * 0.03
    w[:, -128:] *= 4.0
    bias = torch.randn(n, generator=g) * 0.1 if with_bias else None
    qx, sx = pkg.quantize_blocks128(x.to(DEV))
    packed, sw = pkg.pack_weight_blocks128(w, layout=layout)
    y = pkg.linear_blocks128(qx, sx, packed.to(DEV), sw.to(DEV), n=n, w_layout=layout,
                             bias=None if bias is None else bias.to(DEV), out_dtype=dtype)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    qx_ref, sx_ref = ref.quantize_blocks128(x)
    qw_ref, sw_ref = ref.quantize_blocks128(w)
    want = ref.linear_blocks128(qx_ref, sx_ref, qw_ref, sw_ref, bias=bias, out_dtype=dtype)
    assert torch.equal(y.cpu().view(torch.uint8), want.view(torch.uint8))
    # and it is a sane linear: close to the fp32 product
    exact = x.double() @ w.double().T + (0 if bias is None else bias.double())
    assert ref.sqnr_db(exact.float(), y.cpu().float()) > 30.0


@pytest.mark.gpu
@pytest.mark.parametrize("tile_width", [128, 256], indirect=True)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("parts", ["res", "gate_res", "all"])
def test_blockwise_linear_gate_and_residual_bit_exact(pkg, ref, tile_width, dtype, parts):
    """The row/channel linear's epilogue on top of the blockwise accumulation: no transcendental, so exact."""
    m, k, n = 300, 512, 264
    g = torch.Generator().manual_seed(17)
    x = acts(m, k, 3)
    w = torch.randn(n, k, generator=g) * 0.03
    bias = torch.randn(n, generator=g) * 0.1 if parts == "all" else None
    gate = torch.randn(n, generator=g) if parts in ("gate_res", "all") else None
    res = torch.randn(m, n, generator=g).to(dtype)
    qx, sx = pkg.quantize_blocks128(x.to(DEV))
    packed, sw = pkg.pack_weight_blocks128(w)
    dv = lambda t: None if t is None else t.to(DEV)
    y = pkg.linear_blocks128(qx, sx, packed.to(DEV), sw.to(DEV), n=n, bias=dv(bias), gate=dv(gate), residual=dv(res),
                             out_dtype=dtype)
    torch.cuda.synchronize()
    qx_ref, sx_ref = ref.quantize_blocks128(x)
    qw_ref, sw_ref = ref.quantize_blocks128(w)
    want = ref.linear_blocks128(qx_ref, sx_ref, qw_ref, sw_ref, bias=bias, gate=gate, residual=res, out_dtype=dtype)
    assert torch.equal(y.cpu().view(torch.uint8), want.view(torch.uint8))


@pytest.mark.gpu
@pytest.mark.parametrize("act", [1, 2])
def test_blockwise_linear_activation_then_block_requantization(pkg, ref, act):
    """MLP shape of the layer: fc1 + SiLU / GELU in fp32, block quantizer on the hidden, fc2 + residual.  The
    activation uses the hardware exp2 / reciprocal like the row/channel epilogue: a few fp32 ulp."""
    m, k, n = 256, 512, 1024
    g = torch.Generator().manual_seed(23)
    x = acts(m, k, 4)
    w1 = torch.randn(n, k, generator=g) * 0.03
    b1 = torch.randn(n, generator=g) * 0.1
    w2 = torch.randn(k, n, generator=g) * 0.03
    res = torch.randn(m, k, generator=g)
    qx, sx = pkg.quantize_blocks128(x.to(DEV))
    p1, s1 = pkg.pack_weight_blocks128(w1)
    p2, s2 = pkg.pack_weight_blocks128(w2)
    h = pkg.linear_blocks128(qx, sx, p1.to(DEV), s1.to(DEV), n=n, bias=b1.to(DEV), act=act, out_dtype=torch.float32)
    qh, sh = pkg.quantize_blocks128(h)
    y = pkg.linear_blocks128(qh, sh, p2.to(DEV), s2.to(DEV), n=k, residual=res.to(DEV), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    qx_ref, sx_ref = ref.quantize_blocks128(x)
    q1, t1 = ref.quantize_blocks128(w1)
    q2, t2 = ref.quantize_blocks128(w2)
    h_ref = ref.linear_blocks128(qx_ref, sx_ref, q1, t1, bias=b1, act=act, out_dtype=torch.float32)
    assert torch.allclose(h.cpu(), h_ref, rtol=4e-6, atol=1e-6)
    # downstream of the GPU's own hidden everything is exact again
    qh_ref, sh_ref = ref.quantize_blocks128(h.cpu())
    assert torch.equal(qh.cpu(), qh_ref) and torch.equal(sh.cpu(), sh_ref)
    want = ref.linear_blocks128(qh_ref, sh_ref, q2, t2, residual=res, out_dtype=torch.float32)
    assert torch.equal(y.cpu().view(torch.uint8), want.view(torch.uint8))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 128), (130, 256), (1000, 2048)])
def test_row_group_quantizer_bit_exact(pkg, ref, rows, cols, dtype):
    """block_rows = 1: every token row keeps its own scale per K block."""
    x = acts(rows, cols, rows + cols + 1, dtype)
    q, s = pkg.quantize_blocks128(x.to(DEV), block_rows=1)
    q_ref, s_ref = ref.quantize_row_blocks128(x)
    assert s.shape == (rows, cols // 128)
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))
    assert torch.equal(q.cpu(), q_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("tile_width", [128, 256], indirect=True)
@pytest.mark.parametrize("m,k,n,dtype", [(100, 256, 200, torch.float16), (300, 1024, 520, torch.float32),
                                         (1100, 512, 1280, torch.bfloat16)])
def test_blockwise_linear_with_row_groups_bit_exact(pkg, ref, tile_width, m, k, n, dtype):
    g = torch.Generator().manual_seed(m + n)
    x = acts(m, k, m)
    x[::7] *= 25.0                       # token rows of very different range
    w = torch.randn(n, k, generator=g) * 0.03
    bias = torch.randn(n, generator=g) * 0.1
    res = torch.randn(m, n, generator=g).to(dtype)
    qx, sx = pkg.quantize_blocks128(x.to(DEV), block_rows=1)
    packed, sw = pkg.pack_weight_blocks128(w)
    y = pkg.linear_blocks128(qx, sx, packed.to(DEV), sw.to(DEV), n=n, bias=bias.to(DEV), residual=res.to(DEV),
                             out_dtype=dtype, x_block_rows=1)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    qx_ref, sx_ref = ref.quantize_row_blocks128(x)
    qw_ref, sw_ref = ref.quantize_blocks128(w)
    want = ref.linear_blocks128(qx_ref, sx_ref, qw_ref, sw_ref, bias=bias, residual=res, out_dtype=dtype,
                                x_scale_per_row=True)
    assert torch.equal(y.cpu().view(torch.uint8), want.view(torch.uint8))


@pytest.mark.gpu
def test_row_groups_keep_ordinary_rows_next_to_outlier_rows(pkg, ref):
    """Every 64th token 20x larger: with 128 x 128 activation blocks the ordinary rows share a scale with an outlier
    row and lose ~20 dB; with 1 x 128 groups they keep the row/channel rule's quality (and the K-block scales on top)."""
    g = torch.Generator().manual_seed(8)
    m, k, n = 512, 2048, 1024
    x = torch.randn(m, k, generator=g)
    x[::64] *= 20.0
    w = torch.randn(n, k, generator=g) * 0.02
    exact = (x.double() @ w.double().T).float()
    packed, sw = pkg.pack_weight_blocks128(w)
    packed, sw = packed.to(DEV), sw.to(DEV)
    q2, s2 = pkg.quantize_blocks128(x.to(DEV))
    y_blocks = pkg.linear_blocks128(q2, s2, packed, sw, n=n, out_dtype=torch.float32)
    q1, s1 = pkg.quantize_blocks128(x.to(DEV), block_rows=1)
    y_groups = pkg.linear_blocks128(q1, s1, packed, sw, n=n, out_dtype=torch.float32, x_block_rows=1)
    qr, sr = pkg.quantize_rows(x.to(DEV))
    pw, swr = pkg.pack_weight(w)
    y_rows = pkg.linear(qr, sr, pw.to(DEV), swr.to(DEV), n=n, w_layout=pkg.W_SLAB128, out_dtype=torch.float32)
    torch.cuda.synchronize()
    ordinary = torch.ones(m, dtype=torch.bool)
    ordinary[::64] = False
    db = lambda y: ref.sqnr_db(exact[ordinary], y.cpu()[ordinary])
    blocks, groups, rows = db(y_blocks), db(y_groups), db(y_rows)
    assert groups > blocks + 10.0, (blocks, groups, rows)
    assert groups > rows - 1.0, (blocks, groups, rows)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols,form", [(1, 128, "gamma"), (77, 384, "mod_bias"), (300, 2048, "gamma"),
                                            (64, 4096, "none"), (33, 8192, "mod_bias")])
def test_fused_rms_norm_row_group_quantizer_bit_exact(pkg, ref, rows, cols, form, dtype):
    g = torch.Generator().manual_seed(rows + cols)
    x = acts(rows, cols, rows * 3 + cols, dtype)
    vec = None if form == "none" else torch.randn(cols, generator=g) * 0.2 + (0.0 if form == "mod_bias" else 1.0)
    bias = torch.randn(cols, generator=g) * 0.1 if form == "mod_bias" else None
    is_mod = form == "mod_bias"
    dv = lambda t: None if t is None else t.to(DEV)
    q, s = pkg.rms_norm_quantize_row_blocks128(x.to(DEV), dv(vec), dv(bias), eps=1e-6, scale_is_mod=is_mod)
    q_ref, s_ref = ref.rms_norm_quantize_row_blocks128(x, vec, bias, 1e-6, is_mod)
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))
    assert torch.equal(q.cpu(), q_ref)


@pytest.mark.gpu
def test_norm_then_blockwise_linear_chain_matches_the_oracle(pkg, ref):
    """RMSNorm -> group codes -> blockwise linear + residual, the three operators of an attention-out style step."""
    g = torch.Generator().manual_seed(41)
    m, d, n = 200, 1024, 1024
    x = (torch.randn(m, d, generator=g) * 1.5).to(torch.float16)
    gamma = torch.randn(d, generator=g) * 0.05 + 1.0
    w = torch.randn(n, d, generator=g) * 0.03
    q, s = pkg.rms_norm_quantize_row_blocks128(x.to(DEV), gamma.to(DEV), None, eps=1e-6, scale_is_mod=False)
    packed, sw = pkg.pack_weight_blocks128(w)
    y = pkg.linear_blocks128(q, s, packed.to(DEV), sw.to(DEV), n=n, residual=x.to(DEV), out_dtype=torch.float16,
                             x_block_rows=1)
    torch.cuda.synchronize()
    q_ref, s_ref = ref.rms_norm_quantize_row_blocks128(x, gamma, None, 1e-6, False)
    qw_ref, sw_ref = ref.quantize_blocks128(w)
    want = ref.linear_blocks128(q_ref, s_ref, qw_ref, sw_ref, residual=x, out_dtype=torch.float16, x_scale_per_row=True)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(y.cpu(), want)


@pytest.mark.gpu
def test_accuracy_on_config0_outlier_channels(pkg, ref, parity_log):
    """Config 0 (fp16 tokens with eight x20 outlier channels, N(0, 0.02) weights): SQNR against the fp64 product of the
    row/channel rule, of 128 x 128 blocks on both operands, and of 1 x 128 activation groups with 128 x 128 weight
    blocks.  Measured 25.3 / 24.6 / 32.9 dB; the bounds keep the ordering and most of the margin."""
    x, w, bias = ref.make_cfg0()
    exact = (x.double() @ w.double().T + bias.double()).float()
    n = w.shape[0]
    qr, sr = pkg.quantize_rows(x.to(DEV))
    pw, swr = pkg.pack_weight(w.float())
    y_rows = pkg.linear(qr, sr, pw.to(DEV), swr.to(DEV), n=n, w_layout=pkg.W_SLAB128, bias=bias.to(DEV),
                        out_dtype=torch.float32)
    pb, swb = pkg.pack_weight_blocks128(w.float())
    pb, swb = pb.to(DEV), swb.to(DEV)
    q2, s2 = pkg.quantize_blocks128(x.to(DEV))
    y_blocks = pkg.linear_blocks128(q2, s2, pb, swb, n=n, bias=bias.to(DEV), out_dtype=torch.float32)
    q1, s1 = pkg.quantize_blocks128(x.to(DEV), block_rows=1)
    y_groups = pkg.linear_blocks128(q1, s1, pb, swb, n=n, bias=bias.to(DEV), out_dtype=torch.float32, x_block_rows=1)
    torch.cuda.synchronize()
    rows, blocks, groups = (ref.sqnr_db(exact, y.cpu()) for y in (y_rows, y_blocks, y_groups))
    parity_log("config0_sqnr_db", 0, exact.numel(), row_channel=rows, blocks_128x128=blocks, groups_1x128=groups)
    assert groups > rows + 5.0 and groups > blocks + 5.0, (rows, blocks, groups)
    assert abs(blocks - rows) < 2.0, (rows, blocks)


@pytest.mark.gpu
def test_blockwise_beats_rowwise_when_k_ranges_differ(pkg, ref):
    """What the option is for: a few K segments with a much wider range cost the row/channel rule resolution
    everywhere else in the row; per-block scales keep it."""
    g = torch.Generator().manual_seed(5)
    m, k, n = 256, 2048, 1024
    x = torch.randn(m, k, generator=g)
    x[:, 256:384] *= 40.0
    w = torch.randn(n, k, generator=g) * 0.02
    w[:, 256:384] *= 0.05       # the wide activations meet small weights: their product is ordinary
    exact = (x.double() @ w.double().T).float()
    qx, sx = pkg.quantize_blocks128(x.to(DEV))
    packed, sw = pkg.pack_weight_blocks128(w)
    y_blk = pkg.linear_blocks128(qx, sx, packed.to(DEV), sw.to(DEV), n=n, out_dtype=torch.float32)
    qr, sr = pkg.quantize_rows(x.to(DEV))
    pw, swr = pkg.pack_weight(w)
    y_row = pkg.linear(qr, sr, pw.to(DEV), swr.to(DEV), n=n, w_layout=pkg.W_SLAB128, out_dtype=torch.float32)
    torch.cuda.synchronize()
    blk, row = ref.sqnr_db(exact, y_blk.cpu()), ref.sqnr_db(exact, y_row.cpu())
    assert blk > row + 6.0, (blk, row)


@pytest.mark.gpu
def test_blockwise_linear_rejects_bad_arguments(pkg):
    qx = torch.zeros(16, 192, dtype=torch.int8, device=DEV)
    s = torch.ones(1, 2, device=DEV)
    w = torch.zeros(128 * 192, dtype=torch.int8, device=DEV)
    with pytest.raises(pkg.W8A8Error, match="K divisible by 128"):
        pkg.linear_blocks128(qx, s, w, s, n=128, w_layout=pkg.W_ROW_MAJOR)
    qx = torch.zeros(16, 256, dtype=torch.int8, device=DEV)
    w = torch.zeros(100 * 256, dtype=torch.int8, device=DEV)
    out = torch.empty(16, 104, dtype=torch.float16, device=DEV)[:, 1:101]
    with pytest.raises(pkg.W8A8Error, match="aligned"):
        pkg.linear_blocks128(qx, s, w, s, n=100, w_layout=pkg.W_ROW_MAJOR, out=out)


@pytest.mark.gpu
def test_four_layers_row_group_numerics_against_the_row_channel_stack(pkg, ref, parity_log):
    """The ten-operator layer of the linear stack (norm -> A8 -> QKV -> A8 -> out + residual -> norm -> A8 -> controller +
    residual -> norm -> A8 -> up + GELU -> A8 -> down + residual) composed from the blockwise operators with a scale per
    token row and K block, next to the row/channel stack driver, both against the same layers in fp64 without any
    quantization: synthetic tokens with eight x20 outlier channels, four layers."""
    d, nqkv, hid, rows, n_layers = 512, 1536, 2048, 256, 4
    layers = [ref.make_layer_fp32(l, d, nqkv, hid) for l in range(n_layers)]
    x = ref.make_tokens(rows, 3, torch.float16, d)

    def rms(v, g):
        return v / torch.sqrt((v * v).mean(dim=1, keepdim=True) + 1e-6) * g.double()

    ideal = x.double()
    for ws, gs in layers:
        w = [t.double() for t in ws]
        ideal = ideal + (rms(ideal, gs[0]) @ w[0].T)[:, :d] @ w[1].T
        ideal = ideal + rms(ideal, gs[1]) @ w[2].T
        ideal = ideal + torch.nn.functional.gelu(rms(ideal, gs[2]) @ w[3].T, approximate="tanh") @ w[4].T

    stack = pkg.LinearStack(d, nqkv, hid, n_layers, max_rows=rows)
    for l, (ws, gs) in enumerate(layers):
        stack.set_layer(l, ws, gs)
    y_rows = stack.forward(x.to(DEV)).cpu()
    stack.close()

    cur = x.to(DEV)
    for ws, gs in layers:
        packed = [tuple(t.to(DEV) for t in pkg.pack_weight_blocks128(w)) for w in ws]
        g = [t.to(DEV) for t in gs]
        lin = lambda q, s, i, n, **kw: pkg.linear_blocks128(q, s, packed[i][0], packed[i][1], n=n, x_block_rows=1, **kw)
        q, s = pkg.rms_norm_quantize_row_blocks128(cur, g[0], None, scale_is_mod=False)
        qkv = lin(q, s, 0, nqkv, out_dtype=torch.float16)
        q, s = pkg.quantize_blocks128(qkv[:, :d], block_rows=1)
        x1 = lin(q, s, 1, d, residual=cur, out_dtype=torch.float16)
        q, s = pkg.rms_norm_quantize_row_blocks128(x1, g[1], None, scale_is_mod=False)
        x2 = lin(q, s, 2, d, residual=x1, out_dtype=torch.float16)
        q, s = pkg.rms_norm_quantize_row_blocks128(x2, g[2], None, scale_is_mod=False)
        h = lin(q, s, 3, hid, act=pkg.ACT_GELU_TANH, out_dtype=torch.float32)
        q, s = pkg.quantize_blocks128(h, block_rows=1)
        cur = lin(q, s, 4, d, residual=x2, out_dtype=torch.float16)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    y_groups = cur.cpu()
    db_rows = ref.sqnr_db(ideal.float(), y_rows.float())
    db_groups = ref.sqnr_db(ideal.float(), y_groups.float())
    # the same for what the four layers added to the stream (the stream itself is carried exactly in both)
    delta = (ideal - x.double()).float()
    dd_rows = ref.sqnr_db(delta, y_rows.float() - x.float())
    dd_groups = ref.sqnr_db(delta, y_groups.float() - x.float())
    parity_log("four_layer_stack_sqnr_db", 0, ideal.numel(), row_channel=db_rows, groups_1x128=db_groups,
               update_row_channel=dd_rows, update_groups_1x128=dd_groups)
    assert db_groups > db_rows + 1.0, (db_rows, db_groups)
    assert dd_groups > dd_rows + 1.0, (dd_rows, dd_groups)
