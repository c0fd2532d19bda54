"""GPU parity of the grouped skinny linears: every problem of a group must equal, bit for bit,
the same linear run on its own (integer sums are exact in any order and the epilogue arithmetic
is the same code), and the CPU oracle within the usual bound."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def slab(w):
    n, k = w.shape
    return w.view(n, k // 128, 128).permute(1, 0, 2).contiguous()


def make_problem(ref, m, k, n, seed, out_dtype, bias, residual, use_slab):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    qx, sx = ref.quantize_rows(x)
    qw, sw = ref.quantize_weight(torch.randn(n, k, generator=g) * 0.02)
    q = dict(x_i8=qx.to(DEV), x_scales=sx.to(DEV), w_i8=(slab(qw) if use_slab else qw).to(DEV), w_scales=sw.to(DEV), n=n)
    host = dict(qx=qx, sx=sx, qw=qw, sw=sw, bias=None, residual=None)
    if bias:
        host["bias"] = torch.randn(n, generator=g) * 0.1
        q["bias"] = host["bias"].to(DEV)
    if residual:
        host["residual"] = torch.randn(m, n, generator=g).to(out_dtype)
        q["residual"] = host["residual"].to(DEV)
    return q, host


def same(a, b):
    return torch.equal(a.cpu().contiguous().view(torch.uint8), b.cpu().contiguous().view(torch.uint8))


@pytest.mark.parametrize("out_dtype,act,use_slab", [(torch.float16, 0, True), (torch.bfloat16, 0, False),
                                                    (torch.float32, 2, True), (torch.float16, 1, False)])
def test_grouped_equals_single_linears_and_the_oracle(pkg, ref, out_dtype, act, use_slab):
    shapes = [(16, 2048, 2048), (128, 2048, 2048), (1, 256, 320), (77, 512, 8192), (32, 8192, 2048), (100, 128, 36),
              (64, 2048, 520)]
    probs, hosts = [], []
    for i, (m, k, n) in enumerate(shapes):
        q, h = make_problem(ref, m, k, n, 100 + i, out_dtype, bias=i % 2 == 0, residual=i % 3 == 0, use_slab=use_slab)
        probs.append(q)
        hosts.append(h)
    layout = pkg.W_SLAB128 if use_slab else pkg.W_ROW_MAJOR
    outs = pkg.linear_grouped(probs, w_layout=layout, act=act, out_dtype=out_dtype)
    assert pkg.poll_status() == 0
    for q, h, y in zip(probs, hosts, outs):
        single = pkg.linear(q["x_i8"], q["x_scales"], q["w_i8"], q["w_scales"], n=q["n"], w_layout=layout,
                            bias=q.get("bias"), residual=q.get("residual"), act=act, out_dtype=out_dtype)
        assert same(y, single)
        want = ref.linear_w8a8(h["qx"], h["sx"], h["qw"], h["sw"], bias=h["bias"], residual=h["residual"], act=act,
                               out_dtype=out_dtype)
        if act == 0:
            assert same(y, want)
        else:
            assert torch.allclose(y.cpu().float(), want.float(), rtol=2e-3, atol=2e-3)


def test_grouped_more_problems_than_one_launch_holds(pkg, ref):
    """150 problems (three shapes, 50 weight sets each): more than the 72 one launch takes, cut into
    launches of about equal work."""
    probs = []
    for i in range(150):
        m, k, n = [(16, 2048, 2048), (128, 256, 1024), (64, 512, 768)][i % 3]
        q, _ = make_problem(ref, m, k, n, 500 + i, torch.float16, bias=False, residual=False, use_slab=True)
        probs.append(q)
    outs = pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128)
    outs2 = pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128)
    assert pkg.poll_status() == 0
    for q, y, y2 in zip(probs, outs, outs2):
        single = pkg.linear(q["x_i8"], q["x_scales"], q["w_i8"], q["w_scales"], n=q["n"], w_layout=pkg.W_SLAB128,
                            out_dtype=torch.float16)
        assert same(y, single) and same(y2, single)


def test_grouped_rejects_what_it_cannot_run(pkg, ref):
    q, _ = make_problem(ref, 129, 256, 256, 1, torch.float16, False, False, False)
    with pytest.raises(pkg.W8A8Error, match="M <= 128"):
        pkg.linear_grouped([q])
    q, _ = make_problem(ref, 16, 256, 256, 1, torch.float16, False, False, False)
    q["x_i8"] = q["x_i8"][:, :48].contiguous()  # K = 48
    with pytest.raises(pkg.W8A8Error, match="multiple of 32"):
        pkg.linear_grouped([q])
    assert pkg.linear_grouped([]) == []
