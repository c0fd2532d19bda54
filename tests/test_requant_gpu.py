"""The linear whose epilogue emits the next linear's A8 codes (b200_w8a8_linear_requant) against the
two-launch form it replaces (fused linear, then the stand-alone quantizer on the stored result) and
against the CPU oracle.  Codes and scales must be identical bit for bit: the fused kernel quantizes
the values it stores, the maximum is order-free and the fp64 sum of squares order-tolerant."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(m, k, n, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    x[:, :: max(k // 8, 1)] *= 20.0
    w = torch.randn(n, k, generator=g) * 0.02
    res = torch.randn(m, n, generator=g).to(dtype)
    gamma = 1.0 + 0.05 * torch.randn(n, generator=g)
    nbias = 0.1 * torch.randn(n, generator=g)
    bias = 0.01 * torch.randn(n, generator=g)
    gate = 1.0 + 0.1 * torch.randn(n, generator=g)
    return x, w, res, gamma, nbias, bias, gate


CASES = [
    # m, k, n, q_cols, dtype, mode, residual, act
    (512, 2048, 2048, 2048, torch.float16, "rms", True, 0),
    (2048, 2048, 2048, 2048, torch.bfloat16, "rms", True, 0),
    (300, 1024, 2048, 2048, torch.float16, "rms", True, 0),
    (512, 2048, 6144, 2048, torch.float16, "plain", False, 0),
    (640, 512, 768, 256, torch.bfloat16, "plain", False, 0),
    (96, 256, 256, 256, torch.float16, "rms", True, 0),
    (333, 1024, 1024, 1024, torch.float16, "rms", True, 0),
    (130, 512, 1536, 512, torch.float32, "rms", True, 0),
    (512, 2048, 2048, 2048, torch.float32, "rms", True, 0),
    (512, 8192, 2048, 2048, torch.float16, "rms", True, 0),
    (4736, 2048, 2048, 2048, torch.float16, "rms", True, 0),     # more row blocks than clusters: persistent loop
    (4736, 2048, 6144, 2048, torch.float16, "plain", False, 0),
    (64, 2048, 2048, 2048, torch.float32, "plain", False, 1),     # codes of silu(dequant + bias), nothing stored
]


@pytest.mark.parametrize("m,k,n,q_cols,dtype,mode,with_res,act", CASES)
def test_linear_requant_matches_two_launch_form(pkg, ref, m, k, n, q_cols, dtype, mode, with_res, act):
    dev = "cuda"
    x, w, res, gamma, nbias, bias, gate = _inputs(m, k, n, 1000 + m + n, dtype)
    qx, sx = pkg.quantize_rows(x.to(dev))
    packed, sw = pkg.pack_weight(w, layout=pkg.W_SLAB128)
    packed, sw = packed.to(dev), sw.to(dev)
    resd = res.to(dev) if with_res else None
    use_gate = gate.to(dev) if with_res else None
    use_bias = bias.to(dev) if act else None
    store = act == 0
    y2 = pkg.linear(qx, sx, packed, sw, n=n, w_layout=pkg.W_SLAB128, bias=use_bias, gate=use_gate, residual=resd,
                    act=act, out_dtype=dtype)
    if mode == "rms":
        q2, s2 = _rms(pkg, y2, q_cols, gamma, nbias, dev)
    else:
        q2, s2 = pkg.quantize_rows(y2, cols=q_cols)
    y1, q1, s1 = pkg.linear_requant(qx, sx, packed, sw, n=n, w_layout=pkg.W_SLAB128, bias=use_bias, gate=use_gate,
                                    residual=resd, act=act, out_dtype=dtype, store_out=store,
                                    q_mode=pkg.RQ_RMS if mode == "rms" else pkg.RQ_PLAIN, q_cols=q_cols,
                                    norm_scale=gamma[:q_cols].to(dev) if mode == "rms" else None, scale_is_mod=False,
                                    norm_bias=nbias[:q_cols].to(dev) if mode == "rms" else None, eps=1e-6)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    if store:
        assert torch.equal(y1, y2), "stored result differs from the plain fused linear"
    assert torch.equal(s1, s2), f"row scales differ in {(s1 != s2).sum().item()} of {m} rows"
    assert torch.equal(q1, q2), f"codes differ in {(q1 != q2).sum().item()} positions"


def _rms(pkg, y, q_cols, gamma, nbias, dev):
    rows = y.shape[0]
    q = torch.empty(rows, q_cols, dtype=torch.int8, device=dev)
    s = torch.empty(rows, dtype=torch.float32, device=dev)
    g, b = gamma[:q_cols].to(dev), nbias[:q_cols].to(dev)
    dt = {torch.float32: pkg.DT_F32, torch.float16: pkg.DT_F16, torch.bfloat16: pkg.DT_BF16}[y.dtype]
    rc = pkg.lib().b200_w8a8_rms_norm_quantize_rows(y.data_ptr(), dt, y.stride(0), g.data_ptr(), 0, b.data_ptr(),
                                                    q.data_ptr(), q_cols, s.data_ptr(), rows, q_cols, 1e-6,
                                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 0, pkg.lib().b200_w8a8_last_error()
    return q, s


def test_linear_requant_against_oracle(pkg, ref):
    """Small case end to end against the CPU oracle: out linear + residual, then RMSNorm + A8."""
    dev = "cuda"
    m, k, n = 200, 512, 512
    x, w, res, gamma, _, _, _ = _inputs(m, k, n, 7, torch.float16)
    qx_ref, sx_ref = ref.quantize_rows(x)
    qw_ref, sw_ref = ref.quantize_weight(w)
    y_ref = ref.linear_w8a8(qx_ref, sx_ref, qw_ref, sw_ref, residual=res, out_dtype=torch.float16)
    q_ref, s_ref = ref.rms_norm_quantize_rows(y_ref, gamma, None, 1e-6, scale_is_mod=False)
    packed, sw = pkg.pack_weight(w, layout=pkg.W_SLAB128)
    y, q, s = pkg.linear_requant(qx_ref.to(dev), sx_ref.to(dev), packed.to(dev), sw.to(dev), n=n,
                                 w_layout=pkg.W_SLAB128, residual=res.to(dev), out_dtype=torch.float16,
                                 q_mode=pkg.RQ_RMS, q_cols=n, norm_scale=gamma.to(dev), scale_is_mod=False, eps=1e-6)
    torch.cuda.synchronize()
    assert torch.equal(y.cpu(), y_ref)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu(), q_ref)


def test_linear_requant_wide_rows_take_the_two_launch_form(pkg, ref):
    """The MLP hidden (8192 columns = 32 tiles) is wider than a cluster: linear + GELU -> fp32 y, then the quantizer
    on y; without y that cannot be done and the call says so."""
    dev = "cuda"
    m, k, n = 64, 512, 8192
    x, w, _, _, _, _, _ = _inputs(m, k, n, 5, torch.float32)
    qx, sx = pkg.quantize_rows(x.to(dev))
    packed, sw = pkg.pack_weight(w, layout=pkg.W_SLAB128)
    packed, sw = packed.to(dev), sw.to(dev)
    y, q, s = pkg.linear_requant(qx, sx, packed, sw, n=n, w_layout=pkg.W_SLAB128, act=pkg.ACT_GELU_TANH,
                                 out_dtype=torch.float32, q_cols=n)
    y2 = pkg.linear(qx, sx, packed, sw, n=n, w_layout=pkg.W_SLAB128, act=pkg.ACT_GELU_TANH, out_dtype=torch.float32)
    q2, s2 = pkg.quantize_rows(y2)
    torch.cuda.synchronize()
    assert torch.equal(y, y2) and torch.equal(q, q2) and torch.equal(s, s2)
    qr, sr = ref.quantize_rows(y.cpu())  # the oracle's quantizer on the GPU's own hidden: exact
    assert torch.equal(q.cpu(), qr) and torch.equal(s.cpu(), sr)
    with pytest.raises(pkg.W8A8Error, match="needs y"):
        pkg.linear_requant(qx, sx, packed, sw, n=n, w_layout=pkg.W_SLAB128, act=pkg.ACT_GELU_TANH,
                           out_dtype=torch.float32, q_cols=n, store_out=False)


@pytest.mark.parametrize("m,k,n,q_cols", [(16, 512, 2304, 2048), (200, 256, 1312, 1024), (129, 1024, 512, 512)])
def test_linear_requant_modulation_form_ragged_groups_and_short_row_blocks(pkg, m, k, n, q_cols):
    """(1 + modulation) scale with a bias (the reference's AdaRMSNorm form), a last column group that is not a whole
    cluster of tiles (N is no multiple of q_cols or of 256), and row counts that leave a row block mostly empty."""
    dev = "cuda"
    x, w, res, gamma, nbias, bias, gate = _inputs(m, k, n, 77 + m, torch.float32)
    qx, sx = pkg.quantize_rows(x.to(dev))
    packed, sw = pkg.pack_weight(w, layout=pkg.W_SLAB128)
    packed, sw, resd = packed.to(dev), sw.to(dev), res.to(dev)
    mod = (gamma - 1.0)[:q_cols].to(dev)
    nb = nbias[:q_cols].to(dev)
    y2 = pkg.linear(qx, sx, packed, sw, n=n, w_layout=pkg.W_SLAB128, gate=gate.to(dev), residual=resd,
                    out_dtype=torch.float32)
    q2, s2 = pkg.rms_norm_quantize_rows(y2[:, :q_cols], mod, nb, 1.1920929e-07, scale_is_mod=True)
    y1, q1, s1 = pkg.linear_requant(qx, sx, packed, sw, n=n, w_layout=pkg.W_SLAB128, gate=gate.to(dev), residual=resd,
                                    out_dtype=torch.float32, q_mode=pkg.RQ_RMS, q_cols=q_cols, norm_scale=mod,
                                    scale_is_mod=True, norm_bias=nb, eps=1.1920929e-07)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    assert torch.equal(y1, y2) and torch.equal(s1, s2) and torch.equal(q1, q2)
