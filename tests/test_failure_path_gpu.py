"""The time-out path of the GEMM kernels, exercised without faulting anything: a test switch makes
the TMA producer leave out one operand tile, so the MMA issuer's bounded wait (limit lowered to a
few milliseconds) runs out, the kernel drains and returns, and the status word it left makes the
next operator call return 1 once -- the reference's "non-zero on any failure" convention
(src/world_cuda_ops.cu:28-42, 2856-2863).  The call after that must be healthy and exact."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _problem(m=256, k=512, n=512, seed=3):
    g = torch.Generator().manual_seed(seed)
    qx = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    qw = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    return qx, qw


@pytest.fixture
def short_waits(pkg):
    L = pkg.lib()
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    L.b200_w8a8_debug_set_wait_limit_ns(5_000_000)  # 5 ms instead of 2 s
    yield L
    L.b200_w8a8_debug_drop_operand_load(0)
    L.b200_w8a8_debug_force_plan(0, 0, 0)
    L.b200_w8a8_debug_set_wait_limit_ns(0)
    torch.cuda.synchronize()
    pkg.poll_status()  # leave the word clean for the tests that follow


def test_wait_that_runs_out_is_reported_once_then_healthy(pkg, ref, short_waits):
    L = short_waits
    qx, qw = _problem()
    want = ref.gemm_i8_i32(qx, qw)
    qxd, qwd = qx.to(DEV), qw.to(DEV)
    assert torch.equal(pkg.gemm_i8_i32(qxd, qwd).cpu(), want)
    L.b200_w8a8_debug_drop_operand_load(1)
    pkg.gemm_i8_i32(qxd, qwd)          # the launch itself succeeds; the kernel gives up after 5 ms
    torch.cuda.synchronize()           # returns: nothing hangs, the context stays usable
    with pytest.raises(pkg.W8A8Error, match="gave up a bounded wait.*status 102"):
        pkg.gemm_i8_i32(qxd, qwd)      # reported exactly once, by the next launching call
    assert torch.equal(pkg.gemm_i8_i32(qxd, qwd).cpu(), want)  # clean again, and exact
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0


def test_poll_status_reports_and_clears(pkg, short_waits):
    L = short_waits
    qx, qw = _problem(seed=4)
    L.b200_w8a8_debug_drop_operand_load(1)
    pkg.gemm_i8_i32(qx.to(DEV), qw.to(DEV))
    assert pkg.poll_status() == 102    # KS_TIMEOUT_SMEM_FULL: the MMA issuer waited for operands
    assert pkg.poll_status() == 0


def test_drop_in_operator_returns_one_after_a_timed_out_kernel(pkg, short_waits):
    """Through the reference-named path: the C-ABI call the wm_cuda_* wrappers forward to."""
    L = short_waits
    qx, qw = _problem(seed=5)
    qxd, qwd = qx.to(DEV), qw.to(DEV)
    acc = torch.empty(qx.shape[0], qw.shape[0], dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    L.b200_w8a8_debug_drop_operand_load(1)
    assert L.b200_w8a8_gemm_i8_i32(qxd.data_ptr(), qwd.data_ptr(), pkg.W_ROW_MAJOR, acc.data_ptr(), *qx.shape,
                                   qw.shape[0], st) == 0
    torch.cuda.synchronize()
    x = torch.randn(8, 64, device=DEV)
    q = torch.empty(8, 64, dtype=torch.int8, device=DEV)
    s = torch.empty(8, device=DEV)
    assert L.b200_w8a8_quantize_rows(x.data_ptr(), pkg.DT_F32, 64, q.data_ptr(), 64, s.data_ptr(), 8, 64, st) == 1
    assert b"bounded wait" in L.b200_w8a8_last_error()
    assert L.b200_w8a8_quantize_rows(x.data_ptr(), pkg.DT_F32, 64, q.data_ptr(), 64, s.data_ptr(), 8, 64, st) == 0


def test_row_quantizing_linear_times_out_cleanly(pkg, short_waits):
    """The cluster kernel: every CTA of every cluster loses its first tile and drains; no CTA is left
    waiting for the row statistics of another."""
    L = short_waits
    m, k, n = 256, 512, 512
    g = torch.Generator().manual_seed(6)
    qx = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).to(DEV)
    w = torch.randint(-127, 128, (n * k,), generator=g, dtype=torch.int8).to(DEV)
    sx, sw = torch.rand(m, device=DEV) * 1e-2, torch.rand(n, device=DEV) * 1e-3
    good = pkg.linear_requant(qx, sx, w, sw, n=n, w_layout=pkg.W_SLAB128, q_cols=n)
    L.b200_w8a8_debug_drop_operand_load(1)
    pkg.linear_requant(qx, sx, w, sw, n=n, w_layout=pkg.W_SLAB128, q_cols=n)
    assert pkg.poll_status() == 102
    again = pkg.linear_requant(qx, sx, w, sw, n=n, w_layout=pkg.W_SLAB128, q_cols=n)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(good, again))
    assert pkg.poll_status() == 0


@pytest.mark.parametrize("width", [128, 256])
def test_blockwise_linear_times_out_cleanly(pkg, ref, short_waits, width):
    """The 128 x 128 blockwise kernel: its MMA issuer gives up, the sixteen epilogue warps and the producer see the
    abort flag and drain, tensor memory is returned, and the next call is exact."""
    L = short_waits
    g = torch.Generator().manual_seed(6)
    m, k, n = 300, 512, 264
    x = torch.randn(m, k, generator=g)
    w = torch.randn(n, k, generator=g) * 0.03
    qx, sx = pkg.quantize_blocks128(x.to(DEV))
    packed, sw = pkg.pack_weight_blocks128(w)
    packed, sw = packed.to(DEV), sw.to(DEV)
    qx_ref, sx_ref = ref.quantize_blocks128(x)
    qw_ref, sw_ref = ref.quantize_blocks128(w)
    want = ref.linear_blocks128(qx_ref, sx_ref, qw_ref, sw_ref, out_dtype=torch.float16)
    L.b200_w8a8_debug_force_plan(width, 0, 0)
    L.b200_w8a8_debug_drop_operand_load(1)
    pkg.linear_blocks128(qx, sx, packed, sw, n=n)      # launches; every CTA loses its first A tile
    torch.cuda.synchronize()
    # the MMA issuer (waiting for operands, 102) and the epilogue warps (waiting for the accumulator, 104) run
    # out at about the same moment; whichever is first leaves its code
    with pytest.raises(pkg.W8A8Error, match="gave up a bounded wait.*status 10[24]"):
        pkg.linear_blocks128(qx, sx, packed, sw, n=n)
    y = pkg.linear_blocks128(qx, sx, packed, sw, n=n)
    L.b200_w8a8_debug_force_plan(0, 0, 0)
    torch.cuda.synchronize()
    assert pkg.poll_status() == 0
    assert torch.equal(y.cpu().view(torch.uint8), want.view(torch.uint8))
