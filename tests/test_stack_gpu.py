"""GPU parity of the linear-stack driver.

Three links: (1) every operator of a layer, run from Python on the GPU, agrees with the
oracle applied to the same inputs (exact except around the GELU, where the re-quantized
codes must still be exactly the oracle's quantization of the GPU's own fp32 hidden);
(2) the C++ driver equals that Python composition bit for bit (eager, graph, banded);
(3) end to end against the pure-CPU oracle the drift stays at the 16-bit rounding level."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
D, NQKV, HID = 256, 768, 1024


def dev_layer(pkg, lw):
    up = lambda qs: (qs[0].to(DEV), qs[1].to(DEV))
    return dict(qkv=up(lw.qkv), out=up(lw.out), ctrl=up(lw.ctrl), up=up(lw.up), down=up(lw.down),
                g_attn=lw.g_attn.to(DEV), g_ctrl=lw.g_ctrl.to(DEV), g_mlp=lw.g_mlp.to(DEV))


def gpu_layer(pkg, x, L, trace=None):
    e, d = x.dtype, x.shape[1]
    q1, s1 = pkg.rms_norm_quantize_rows(x, L["g_attn"], None, 1e-6, scale_is_mod=False)
    qkv = pkg.linear(q1, s1, *L["qkv"], out_dtype=e)
    q2, s2 = pkg.quantize_rows(qkv, cols=d)
    x1 = pkg.linear(q2, s2, *L["out"], residual=x, out_dtype=e)
    q3, s3 = pkg.rms_norm_quantize_rows(x1, L["g_ctrl"], None, 1e-6, scale_is_mod=False)
    x2 = pkg.linear(q3, s3, *L["ctrl"], residual=x1, out_dtype=e)
    q4, s4 = pkg.rms_norm_quantize_rows(x2, L["g_mlp"], None, 1e-6, scale_is_mod=False)
    h = pkg.linear(q4, s4, *L["up"], act=pkg.ACT_GELU_TANH, out_dtype=torch.float32)
    q5, s5 = pkg.quantize_rows(h)
    x3 = pkg.linear(q5, s5, *L["down"], residual=x2, out_dtype=e)
    if trace is not None:
        trace.update(x=x, q1=q1, s1=s1, qkv=qkv, q2=q2, s2=s2, x1=x1, q3=q3, s3=s3, x2=x2, q4=q4, s4=s4, h=h,
                     q5=q5, s5=s5, x3=x3)
    return x3


def same(a, b):
    return torch.equal(a.cpu().contiguous().view(torch.uint8), b.cpu().contiguous().view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_each_operator_of_a_layer_against_the_oracle_on_the_same_inputs(pkg, ref, dtype):
    lw = ref.make_layer(0, D, NQKV, HID)
    L = dev_layer(pkg, lw)
    x = ref.make_tokens(200, 0, dtype, D).to(DEV)
    t = {}
    gpu_layer(pkg, x, L, t)
    c = {k: v.cpu() for k, v in t.items()}
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
    _, _, h_ref = ref.linear_w8a8_requant(c["q4"], c["s4"], *lw.up, act=ref.ACT_GELU_TANH)
    # the kernel evaluates GELU(tanh) as v*sigmoid(2u) on the special-function unit: a few ulp from
    # the oracle's 0.5*v*(1+tanh(u)), whose own cancellation error for negative v is ~4e-7 absolute
    assert torch.allclose(c["h"], h_ref, rtol=4e-6, atol=1e-6)
    q, s = ref.quantize_rows(c["h"])  # the oracle's quantizer on the GPU's own fp32 hidden
    assert same(c["q5"], q) and same(c["s5"], s)
    assert same(c["x3"], ref.linear_w8a8(c["q5"], c["s5"], *lw.down, residual=c["x2"], out_dtype=dtype))


@pytest.mark.parametrize("fusion", [True, False])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,band,steps,graph,lanes", [(200, 0, 1, False, 1), (200, 128, 2, False, 1),
                                                         (333, 0, 2, True, 1), (16, 0, 1, True, 1),
                                                         (333, 64, 1, False, 2), (333, 96, 2, True, 2)])
def test_stack_driver_equals_operator_composition(pkg, ref, dtype, rows, band, steps, graph, lanes, fusion):
    """fusion=True: the quantizers that follow a linear run inside that linear's epilogue (six launches per
    layer plus the first norm); fusion=False: the ten-launch form.  Both must equal the composition."""
    n_layers = 3
    layers_fp32 = [ref.make_layer_fp32(l, D, NQKV, HID) for l in range(n_layers)]
    stack = pkg.LinearStack(D, NQKV, HID, n_layers, max_rows=rows, band_rows=band, dtype=dtype)
    for l, (ws, gs) in enumerate(layers_fp32):
        stack.set_layer(l, ws, gs, threads=4)
    stack.set_lanes(lanes)  # two lanes: alternate bands run on two streams
    stack.set_fusion(fusion)
    Ls = [dev_layer(pkg, ref.make_layer(l, D, NQKV, HID)) for l in range(n_layers)]
    x = ref.make_tokens(rows, 1, dtype, D).to(DEV)
    want = x
    for _ in range(steps):
        for L in Ls:
            want = gpu_layer(pkg, want, L)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        y = stack.forward(x, steps=steps, use_graph=graph)
        y2 = stack.forward(x, steps=steps, use_graph=graph)  # replay / rerun is deterministic
    stream.synchronize()
    assert pkg.poll_status() == 0
    assert same(y, want) and same(y2, want)
    per_band = (6 * n_layers * steps + 1) if fusion else 10 * n_layers * steps
    assert stack.launches_per_forward == per_band * (1 if band == 0 else -(-rows // band))
    # host entry point: pinned buffers in, pinned buffers out
    xh = x.cpu().pin_memory()
    yh = torch.empty_like(xh).pin_memory()
    stack.forward_host(xh, yh, steps=steps, use_graph=graph)
    assert same(yh, want)
    stack.close()


def test_stack_end_to_end_against_cpu_oracle(pkg, ref, parity_log):
    n_layers, rows = 2, 160
    stack = pkg.LinearStack(D, NQKV, HID, n_layers, max_rows=rows)
    layers = []
    for l in range(n_layers):
        ws, gs = ref.make_layer_fp32(l, D, NQKV, HID)
        stack.set_layer(l, ws, gs)
        layers.append(ref.make_layer(l, D, NQKV, HID))
    x = ref.make_tokens(rows, 2, torch.float16, D)
    want = ref.stack_forward(x, layers, steps=1)
    got = stack.forward(x.to(DEV)).cpu()
    ulp = ref.ulp_distance_f16(got, want)
    row = parity_log("stack output (2 layers, d=256) beyond 2 fp16 ulp of the pure-CPU oracle", int((ulp > 2).sum()),
                     ulp.numel(), max_ulp=int(ulp.max()), differing=int((ulp > 0).sum()))
    # a GELU ulp can move a re-quantized code across a tie; downstream that is a few 16-bit ulps.
    # Measured on B200: no element beyond 2 ulp, largest distance 1 ulp, 2 of 40 960 elements differ at all.
    assert row["mismatches"] == 0 and row["max_ulp"] <= 2 and row["differing"] <= 4
    assert float((got.float() - want.float()).abs().max()) <= 0.02 * float(want.float().abs().max())
    stack.close()


def test_stack_full_size_layers_properties(pkg, ref):
    """Real layer shapes (2048 / 6144 / 8192), 2 layers, M=512: graph replay equals eager, rows are
    independent (a row's result does not depend on which other rows are in the batch), and the
    first layer's QKV-side operators match the oracle exactly."""
    stack = pkg.LinearStack(max_rows=512, n_layers=2)
    lws = []
    for l in range(2):
        ws, gs = ref.make_layer_fp32(l)
        stack.set_layer(l, ws, gs)
        lws.append((ws, gs))
    x = ref.make_tokens(512, 0, torch.float16).to(DEV)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        y_eager = stack.forward(x)
        y_graph = stack.forward(x, use_graph=True)
        y_half = stack.forward(x[:256].contiguous())
    stream.synchronize()
    assert pkg.poll_status() == 0
    assert same(y_eager, y_graph)
    assert same(y_half, y_eager[:256])
    assert torch.isfinite(y_eager.float()).all()
    # oracle check of the first operators at full width (cheap on the CPU: one 512x2048x6144 GEMM)
    ws, gs = lws[0]
    q1, s1 = ref.rms_norm_quantize_rows(x.cpu(), gs[0], None, 1e-6, scale_is_mod=False)
    qw, sw = ref.quantize_weight(ws[0])
    want = ref.linear_w8a8(q1, s1, qw, sw, out_dtype=torch.float16)
    q1g, s1g = pkg.rms_norm_quantize_rows(x, gs[0].to(DEV), None, 1e-6, scale_is_mod=False)
    packed, swp = pkg.pack_weight(ws[0])
    got = pkg.linear(q1g, s1g, packed.to(DEV), swp.to(DEV), w_layout=pkg.W_SLAB128, out_dtype=torch.float16)
    assert same(q1g, q1) and same(got, want)
    stack.close()


def test_stack_loaded_from_a_packed_weight_file_equals_the_quantizing_loader(pkg, ref, tmp_path):
    """The offline file (written on the host without a GPU) and set_layer give the same device
    weights: identical forward output, and saving the resident weights reproduces the file."""
    n_layers, rows = 2, 160
    layers = [ref.make_layer_fp32(l, D, NQKV, HID) for l in range(n_layers)]
    path = tmp_path / "stack.w8a8"
    pkg.write_weight_file(path, D, NQKV, HID, layers, threads=4)
    a = pkg.LinearStack(D, NQKV, HID, n_layers, max_rows=rows)
    for l, (ws, gs) in enumerate(layers):
        a.set_layer(l, ws, gs, threads=4)
    b = pkg.LinearStack(D, NQKV, HID, n_layers, max_rows=rows)
    with pytest.raises(pkg.W8A8Error, match="before every layer was loaded"):
        b.forward(torch.zeros(rows, D, dtype=torch.float16, device=DEV))
    b.load_weights(path)
    x = ref.make_tokens(rows, 4, torch.float16, D).to(DEV)
    assert same(a.forward(x), b.forward(x))
    saved = tmp_path / "saved.w8a8"
    a.save_weights(saved)
    assert saved.read_bytes() == path.read_bytes()
    wrong = pkg.LinearStack(D, NQKV, HID, n_layers + 1, max_rows=rows)
    with pytest.raises(pkg.W8A8Error, match="the stack is"):
        wrong.load_weights(path)
    for s in (a, b, wrong):
        s.close()
