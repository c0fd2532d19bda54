"""GPU parity of the QKV linear whose epilogue is the reference's QKV consumer (per-head
RMSNorm + rotary embedding, head-major fp32 q/k/v).

The fused kernel must equal, bit for bit, the two-call form it replaces on the same inputs
(int8 GEMM to int32, then the stand-alone consumer); both are compared with the CPU oracle
within the few ulps by which the device's cosf/sinf differ from the host's."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_case(ref, T, K, Hq, Hkv, d, W, H, seed, bias=False):
    g = torch.Generator().manual_seed(seed)
    n = (Hq + 2 * Hkv) * d
    x = torch.randn(T, K, generator=g) * 1.5
    x[:, 3] *= 20.0  # an outlier channel, as in the stack's activations
    w = torch.randn(n, K, generator=g) * 0.03
    qx, sx = ref.quantize_rows(x)
    qw, sw = ref.quantize_weight(w)
    c = dict(qx=qx, sx=sx, qw=qw, sw=sw,
             xp=torch.randint(0, W, (T,), generator=g), yp=torch.randint(0, H, (T,), generator=g),
             tp=torch.randint(0, 64, (T,), generator=g), xy=torch.rand(d // 8, generator=g) * 6.0,
             inv_t=torch.rand(d // 2 - 2 * (d // 8), generator=g),
             bias=(torch.randn(n, generator=g) * 0.2) if bias else None)
    return c


def slab(w):
    n, k = w.shape
    return w.view(n, k // 128, 128).permute(1, 0, 2).contiguous()


def run_fused(pkg, c, Hq, Hkv, d, W, H, eps, layout_slab=False):
    dv = {k: (v.to(DEV) if v is not None else None) for k, v in c.items()}
    cos, sin = pkg.rope_tables(dv["xp"], dv["yp"], dv["tp"], dv["xy"], dv["inv_t"], d, W, H)
    w = slab(c["qw"]).to(DEV) if layout_slab else dv["qw"]
    out = pkg.linear_qkv_heads(dv["qx"], dv["sx"], w, dv["sw"], cos, sin, Hq, Hkv, d, eps, bias=dv["bias"],
                               w_layout=pkg.W_SLAB128 if layout_slab else pkg.W_ROW_MAJOR)
    assert pkg.poll_status() == 0
    return out


def run_two_calls(pkg, c, Hq, Hkv, d, W, H, eps):
    dv = {k: (v.to(DEV) if v is not None else None) for k, v in c.items()}
    acc = pkg.gemm_i8_i32(dv["qx"], dv["qw"])
    return pkg.qkv_rms_rope_dequant(acc, dv["sx"], dv["sw"], dv["xp"], dv["yp"], dv["tp"], dv["xy"], dv["inv_t"],
                                    Hq, Hkv, d, W, H, eps)


def same(a, b):
    return torch.equal(a.cpu().contiguous().view(torch.int32), b.cpu().contiguous().view(torch.int32))


def test_rope_tables_match_the_oracle_phases(pkg, ref):
    T, d, W, H = 333, 64, 16, 8
    c = make_case(ref, T, 128, 2, 1, d, W, H, seed=5)
    cos, sin = pkg.rope_tables(c["xp"].to(DEV), c["yp"].to(DEV), c["tp"].to(DEV), c["xy"].to(DEV),
                               c["inv_t"].to(DEV), d, W, H)
    phases = torch.stack([ref.rope_phase(p, c["xp"], c["yp"], c["tp"], c["xy"], c["inv_t"], W, H, d // 8)
                          for p in range(d // 2)], dim=1).to(torch.float32)
    assert torch.allclose(cos.cpu(), torch.cos(phases), rtol=0, atol=2e-6)
    assert torch.allclose(sin.cpu(), torch.sin(phases), rtol=0, atol=2e-6)


@pytest.mark.parametrize("T,K,Hq,Hkv,tile", [
    (96, 256, 8, 4, 0),       # N = 1024
    (200, 512, 3, 1, 0),      # N = 320: the last tile is ragged at a head boundary
    (333, 2048, 32, 16, 0),   # the reference's head counts, ragged rows
    (512, 2048, 32, 16, 128), (512, 2048, 32, 16, 256),
    (512, 2048, 32, 32, 0),   # N = 6144
    (2048, 2048, 32, 16, 0),  # enough tiles for the 256-wide default
    (17, 128, 1, 1, 0),
])
def test_fused_qkv_epilogue_equals_the_two_call_form(pkg, ref, T, K, Hq, Hkv, tile):
    d, W, H, eps = 64, 32, 16, 1e-6
    c = make_case(ref, T, K, Hq, Hkv, d, W, H, seed=T + Hq)
    pkg.lib().b200_w8a8_set_tile_width(tile)
    try:
        q, k, v = run_fused(pkg, c, Hq, Hkv, d, W, H, eps)
    finally:
        pkg.lib().b200_w8a8_set_tile_width(0)
    q2, k2, v2 = run_two_calls(pkg, c, Hq, Hkv, d, W, H, eps)
    assert same(q, q2) and same(k, k2) and same(v, v2)
    if T <= 512:
        acc = ref.gemm_i8_i32(c["qx"], c["qw"])
        qr, kr, vr = ref.qkv_fused_rms_rope_i32_dequant(acc, c["sx"], c["sw"], c["xp"], c["yp"], c["tp"], c["xy"],
                                                        c["inv_t"], Hq, Hkv, d, W, H, eps)
        assert torch.equal(v.cpu(), vr)
        assert torch.allclose(q.cpu(), qr, rtol=1e-5, atol=2e-6)
        assert torch.allclose(k.cpu(), kr, rtol=1e-5, atol=2e-6)


def test_fused_qkv_epilogue_with_bias_and_slab_weights(pkg, ref):
    T, K, Hq, Hkv, d, W, H, eps = 160, 1024, 6, 2, 64, 16, 8, 1e-5
    c = make_case(ref, T, K, Hq, Hkv, d, W, H, seed=11, bias=True)
    q, k, v = run_fused(pkg, c, Hq, Hkv, d, W, H, eps, layout_slab=True)
    q_rm, k_rm, v_rm = run_fused(pkg, c, Hq, Hkv, d, W, H, eps, layout_slab=False)
    assert same(q, q_rm) and same(k, k_rm) and same(v, v_rm)
    acc = ref.gemm_i8_i32(c["qx"], c["qw"])
    qr, kr, vr = ref.qkv_fused_rms_rope_i32_dequant(acc, c["sx"], c["sw"], c["xp"], c["yp"], c["tp"], c["xy"],
                                                    c["inv_t"], Hq, Hkv, d, W, H, eps, bias=c["bias"])
    assert torch.equal(v.cpu(), vr)
    assert torch.allclose(q.cpu(), qr, rtol=1e-5, atol=2e-6)
    assert torch.allclose(k.cpu(), kr, rtol=1e-5, atol=2e-6)


def test_fused_qkv_epilogue_rejects_what_it_cannot_run(pkg, ref):
    c = make_case(ref, 32, 128, 1, 1, 128, 16, 8, seed=3)
    with pytest.raises(pkg.W8A8Error, match="d_head = 64"):
        run_fused(pkg, c, 1, 1, 128, 16, 8, 1e-6)
    c = make_case(ref, 32, 128, 1, 1, 64, 16, 8, seed=3)
    dv = {k: (v.to(DEV) if v is not None else None) for k, v in c.items()}
    cos, sin = pkg.rope_tables(dv["xp"], dv["yp"], dv["tp"], dv["xy"], dv["inv_t"], 64, 16, 8)
    odd = torch.empty(32 * 32 + 1, dtype=torch.float32, device=DEV)[1:].view(32, 32)  # 4-byte aligned only
    odd.copy_(cos)
    with pytest.raises(pkg.W8A8Error, match="16-byte aligned"):
        pkg.linear_qkv_heads(dv["qx"], dv["sx"], dv["qw"], dv["sw"], odd, sin, 1, 1, 64, 1e-6)
    # empty batch: nothing to do
    e = torch.empty(0, 128, dtype=torch.int8, device=DEV)
    q, k, v = pkg.linear_qkv_heads(e, torch.empty(0, device=DEV), dv["qw"], dv["sw"], cos[:0], sin[:0], 1, 1, 64, 1e-6)
    assert q.shape == (1, 0, 64)
