"""The no-allocation linear (b200_w8a8_linear_static_scratch) against the ordinary entry point.

Some callers of this library cannot allocate device memory at the point where they need a
linear: they run under a memory budget fixed at start-up, or inside a loop or callback where
entering the allocator is not allowed.  For them the library carries its own split-K scratch.
This file is collected last on purpose, so a run that stops at the first failure has already
been through every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def codes(rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-127, 128, (rows, cols), generator=g, dtype=torch.int8)


@pytest.mark.parametrize("m,k,n,dtype", [(16, 2048, 2048, torch.float16), (128, 8192, 2048, torch.bfloat16),
                                         (100, 1024, 520, torch.float32)])
def test_static_scratch_linear_matches_the_allocating_entry_point_twice_in_a_row(pkg, ref, m, k, n, dtype):
    g = torch.Generator().manual_seed(m + n)
    a, b = codes(m, k, 21).to(DEV), codes(n, k, 22).to(DEV)
    sx = (torch.rand(m, generator=g) * 0.05 + 0.01).to(DEV)
    sw = (torch.rand(n, generator=g) * 2e-4 + 1e-5).to(DEV)
    bias = (torch.randn(n, generator=g) * 0.1).to(DEV)
    res = torch.randn(m, n, generator=g).to(dtype).to(DEV)
    want = pkg.linear(a, sx, b, sw, bias=bias, residual=res, out_dtype=dtype)  # existing entry point
    out1 = torch.empty(m, n, dtype=dtype, device=DEV)
    out2 = torch.empty(m, n, dtype=dtype, device=DEV)
    pkg.linear_static_scratch(a, sx, b, sw, bias=bias, residual=res, out=out1)
    torch.cuda.synchronize()
    # the first call fixes the footprint (module image, scratch address look-up); from then on a call
    # must leave the device's free memory exactly as it found it
    free_before = torch.cuda.mem_get_info()[0]
    pkg.linear_static_scratch(a, sx, b, sw, bias=bias, residual=res, out=out2)  # same scratch, second call
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the no-allocation entry point changed the free device memory"
    assert pkg.poll_status() == 0
    # both paths add the same integers and run the same fp32 epilogue: identical bits, no tolerance
    assert torch.equal(out1.view(torch.uint8), want.view(torch.uint8))
    assert torch.equal(out2.view(torch.uint8), want.view(torch.uint8))
    # and the CPU oracle agrees (no activation in this epilogue: exact)
    want_cpu = ref.linear_w8a8(a.cpu(), sx.cpu(), b.cpu(), sw.cpu(), bias=bias.cpu(), residual=res.cpu(), out_dtype=dtype)
    assert torch.equal(out1.cpu().view(torch.uint8), want_cpu.view(torch.uint8))


def test_static_scratch_linear_rejects_what_does_not_fit(pkg):
    cap = pkg.lib().b200_w8a8_linear_static_scratch_capacity()
    assert cap == 4096 + 8 * 1024 * 1024
    m, k, n = 2048, 2048, 2048  # two splits alone would need 32 MiB
    a, b = codes(m, k, 1).to(DEV), codes(n, k, 2).to(DEV)
    sx, sw = torch.ones(m, device=DEV), torch.ones(n, device=DEV)
    out = torch.empty(m, n, dtype=torch.float16, device=DEV)
    with pytest.raises(pkg.W8A8Error, match="built-in scratch holds"):
        pkg.linear_static_scratch(a, sx, b, sw, out=out)
    with pytest.raises(pkg.W8A8Error, match="K >= 512"):
        pkg.linear_static_scratch(a[:16, :256].contiguous(), sx[:16], b[:, :256].contiguous(), sw, out=out[:16])
