"""Parity at the sizes bench.py times: the planner's own choices at those sizes are what is tested.

  config 2  M=2048, bf16, chained passes through the C++ driver with graph replay;
  config 3  bands of rows on two lanes at full width, worlds independent of one another,
            and a launch large enough for the planner to pick the CTA-pair kernel by itself;
  config 4  all twelve skinny (M, K, N) shapes, as single launches and as one grouped launch.

Every operator is checked against the CPU oracle on the GPU's own inputs (codes, scales and
accumulator-derived outputs bit for bit; the fp32 hidden after GELU within the stated tolerance,
with the measured number of differing re-quantized codes recorded)."""
import pytest
import torch

from test_stack_gpu import dev_layer, gpu_layer, same

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
D, NQKV, HID = 2048, 6144, 8192


def check_layer_against_oracle(ref, lw, c, dtype, parity_log, tag):
    """c: the GPU's tensors of one layer (on the CPU).  Each operator is re-run by the oracle on the
    GPU's inputs of that operator."""
    q, s = ref.rms_norm_quantize_rows(c["x"], lw.g_attn, None, 1e-6, scale_is_mod=False)
    assert same(c["q1"], q) and same(c["s1"], s)
    assert same(c["qkv"], ref.linear_w8a8(c["q1"], c["s1"], *lw.qkv, out_dtype=dtype))
    q, s = ref.quantize_rows(c["qkv"][:, :D])
    assert same(c["q2"], q) and same(c["s2"], s)
    assert same(c["x1"], ref.linear_w8a8(c["q2"], c["s2"], *lw.out, residual=c["x"], out_dtype=dtype))
    q, s = ref.rms_norm_quantize_rows(c["x1"], lw.g_ctrl, None, 1e-6, scale_is_mod=False)
    assert same(c["q3"], q) and same(c["s3"], s)
    assert same(c["x2"], ref.linear_w8a8(c["q3"], c["s3"], *lw.ctrl, residual=c["x1"], out_dtype=dtype))
    q, s = ref.rms_norm_quantize_rows(c["x2"], lw.g_mlp, None, 1e-6, scale_is_mod=False)
    assert same(c["q4"], q) and same(c["s4"], s)
    q5_ref, s5_ref, h_ref = ref.linear_w8a8_requant(c["q4"], c["s4"], *lw.up, act=ref.ACT_GELU_TANH)
    assert torch.allclose(c["h"], h_ref, rtol=4e-6, atol=1e-6)
    q, s = ref.quantize_rows(c["h"])  # the oracle's quantizer on the GPU's own fp32 hidden: exact
    assert same(c["q5"], q) and same(c["s5"], s)
    # against the oracle's own hidden a code may sit on the other side of a rounding tie: count them
    diff = (c["q5"].int() - q5_ref.int()).abs()
    row = parity_log(f"{tag}: codes of the hidden vs the oracle's own hidden", int((diff != 0).sum()), diff.numel(),
                     max_step=int(diff.max()), scale_mismatches=int((c["s5"] != s5_ref).sum()))
    # measured on B200: 9 to 15 of 16 777 216 codes (5.4e-7 to 8.9e-7), never more than one step; the row
    # scale differs in its last bits in about 37 % of the rows (the maxima differ by a few fp32 ulp)
    assert int(diff.max()) <= 1 and row["rate"] < 2e-6
    assert same(c["x3"], ref.linear_w8a8(c["q5"], c["s5"], *lw.down, residual=c["x2"], out_dtype=dtype))


def build_stack(pkg, ref, n_layers, rows, band, dtype):
    stack = pkg.LinearStack(D, NQKV, HID, n_layers, max_rows=rows, band_rows=band, dtype=dtype)
    lws = []
    for l in range(n_layers):
        ws, gs = ref.make_layer_fp32(l)
        stack.set_layer(l, ws, gs)
        lws.append(ref.make_layer(l))
    return stack, lws


def test_config2_m2048_bf16_chained_graph_replay(pkg, ref, parity_log):
    n_layers, steps, rows, dtype = 2, 2, 2048, torch.bfloat16
    stack, lws = build_stack(pkg, ref, n_layers, rows, 0, dtype)
    Ls = [dev_layer(pkg, lw) for lw in lws]
    x = ref.make_tokens(rows, 0, dtype).to(DEV)
    cur, traces = x, []
    for st in range(steps):
        for l in range(n_layers):
            t = {}
            cur = gpu_layer(pkg, cur, Ls[l], t)
            traces.append((st, l, {k: v.cpu() for k, v in t.items()}))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        y = stack.forward(x, steps=steps, use_graph=True)
        y2 = stack.forward(x, steps=steps, use_graph=True)
    stream.synchronize()
    assert pkg.poll_status() == 0
    assert same(y, cur) and same(y2, cur), "the C++ driver (graph replay) differs from the operator composition"
    for st, l, c in traces:
        check_layer_against_oracle(ref, lws[l], c, dtype, parity_log, f"cfg2 M=2048 bf16 step {st} layer {l}")
    stack.close()


def test_config3_bands_on_two_lanes_worlds_are_independent(pkg, ref, parity_log):
    n_layers, worlds, per_world, dtype = 2, 4, 2048, torch.float16
    rows = worlds * per_world
    stack, lws = build_stack(pkg, ref, n_layers, rows, per_world, dtype)
    stack.set_lanes(2)
    x = torch.cat([ref.make_tokens(per_world, w, dtype) for w in range(worlds)]).to(DEV)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        y_all = stack.forward(x, use_graph=True)
        alone = [stack.forward(x[w * per_world:(w + 1) * per_world].contiguous()) for w in range(worlds)]
    stream.synchronize()
    assert pkg.poll_status() == 0
    for w in range(worlds):
        assert same(y_all[w * per_world:(w + 1) * per_world], alone[w]), f"world {w} depends on its neighbours"
    # world 0 operator by operator against the oracle
    Ls = [dev_layer(pkg, lw) for lw in lws]
    cur = x[:per_world].contiguous()
    for l in range(n_layers):
        t = {}
        cur = gpu_layer(pkg, cur, Ls[l], t)
        check_layer_against_oracle(ref, lws[l], {k: v.cpu() for k, v in t.items()}, dtype, parity_log,
                                   f"cfg3 world 0 fp16 layer {l}")
    assert same(alone[0], cur)
    stack.close()


def test_large_launch_takes_the_cta_pair_kernel_by_itself(pkg, ref):
    """M=16384, N=6144: 1536 pair tiles, far beyond two per SM, so the planner picks the CTA-pair kernel
    unforced; its accumulators and a fused 16-bit epilogue must equal the single-CTA kernel's bit for bit,
    and sampled accumulators the exact integer dot product (the reference probe's check,
    tools/profile/w8a8.cu:344-372)."""
    m, k, n = 16384, 2048, 6144
    g = torch.Generator().manual_seed(5)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    ad, bd = a.to(DEV), b.to(DEV)
    sx, sw = (torch.rand(m, generator=g) * 0.05 + 0.01).to(DEV), (torch.rand(n, generator=g) * 2e-4 + 1e-5).to(DEV)
    acc_pair = pkg.gemm_i8_i32(ad, bd)
    y_pair = pkg.linear(ad, sx, bd, sw, out_dtype=torch.float16)
    pkg.lib().b200_w8a8_set_pair_mma(2)  # never
    try:
        acc_single = pkg.gemm_i8_i32(ad, bd)
        y_single = pkg.linear(ad, sx, bd, sw, out_dtype=torch.float16)
    finally:
        pkg.lib().b200_w8a8_set_pair_mma(0)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    assert torch.equal(acc_pair, acc_single) and torch.equal(y_pair, y_single)
    acc = acc_pair.cpu()
    for i in range(256):  # evenly spaced samples, exact 64-bit dot products
        r, c = (i * 6151) % m, (i * 3571) % n
        assert int(acc[r, c]) == int((a[r].long() * b[c].long()).sum())


SKINNY = [(m, k, n) for (k, n) in [(2048, 2048), (2048, 8192), (8192, 2048)] for m in (16, 32, 64, 128)]


@pytest.mark.parametrize("m,k,n", SKINNY)
def test_config4_single_launch_planner_choice(pkg, ref, m, k, n):
    """The launch bench.py times for config 4: SLAB128 weights, no workspace, weights marked constant."""
    g = torch.Generator().manual_seed(m * 7 + k + n)
    qx, sx = ref.quantize_rows(torch.randn(m, k, generator=g))
    qw, sw = ref.quantize_weight(torch.randn(n, k, generator=g) * 0.02)
    packed = qw.view(n, k // 128, 128).permute(1, 0, 2).contiguous()
    want = ref.linear_w8a8(qx, sx, qw, sw, out_dtype=torch.float16)
    got = pkg.linear(qx.to(DEV), sx.to(DEV), packed.to(DEV), sw.to(DEV), n=n, w_layout=pkg.W_SLAB128,
                     out_dtype=torch.float16, const_weights=True)
    acc = pkg.gemm_i8_i32(qx.to(DEV), packed.to(DEV), n=n, w_layout=pkg.W_SLAB128)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    assert torch.equal(acc.cpu(), ref.gemm_i8_i32(qx, qw))
    assert same(got, want)


def test_config4_all_shapes_in_one_grouped_launch(pkg, ref):
    probs, wants = [], []
    for i, (m, k, n) in enumerate(SKINNY):
        g = torch.Generator().manual_seed(900 + i)
        qx, sx = ref.quantize_rows(torch.randn(m, k, generator=g))
        qw, sw = ref.quantize_weight(torch.randn(n, k, generator=g) * 0.02)
        packed = qw.view(n, k // 128, 128).permute(1, 0, 2).contiguous()
        probs.append(dict(x_i8=qx.to(DEV), x_scales=sx.to(DEV), w_i8=packed.to(DEV), w_scales=sw.to(DEV), n=n))
        wants.append(ref.linear_w8a8(qx, sx, qw, sw, out_dtype=torch.float16))
    outs = pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128, out_dtype=torch.float16, const_weights=True)
    outs2 = pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128, out_dtype=torch.float16)
    torch.cuda.synchronize()
    for a, b in zip(outs, outs2):
        assert same(a, b)
    assert pkg.poll_status() == 0
    for y, want in zip(outs, wants):
        assert same(y, want)


def test_config4_seventy_two_small_weight_linears_in_one_grouped_launch(pkg, ref):
    """The grouped call bench.py times on the 4 MB weights: 72 distinct 2048 -> 2048 linears at M=16 in one
    launch, each equal to the same linear launched alone and, for a sample, to the oracle."""
    m, k, n = 16, 2048, 2048
    g = torch.Generator().manual_seed(4242)
    qx, sx = ref.quantize_rows(torch.randn(m, k, generator=g))
    probs, hosts = [], []
    for i in range(72):
        qw = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
        sw = torch.rand(n, generator=g) * 2e-4 + 1e-5
        packed = qw.view(n, k // 128, 128).permute(1, 0, 2).contiguous()
        probs.append(dict(x_i8=qx.to(DEV), x_scales=sx.to(DEV), w_i8=packed.to(DEV), w_scales=sw.to(DEV), n=n))
        hosts.append((qw, sw))
    outs = pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128, out_dtype=torch.float16, const_weights=True)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    for i, (q, y) in enumerate(zip(probs, outs)):
        single = pkg.linear(q["x_i8"], q["x_scales"], q["w_i8"], q["w_scales"], n=n, w_layout=pkg.W_SLAB128,
                            out_dtype=torch.float16)
        assert same(y, single)
        if i % 24 == 0:
            assert same(y, ref.linear_w8a8(qx, sx, *hosts[i], out_dtype=torch.float16))
