"""Generates tests/golden/w8a8_reference_golden.npz from the reference's own PyTorch helpers.

Run once on a machine that has the reference checkout:
    python tests/golden/make_golden.py /path/to/reference
(without an argument: $WORLDMODEL_REFERENCE_DIR, else a directory named `reference` beside this repository)
It imports tools/tests/test_w8a8_quantization.py from that checkout (the reference's
"PyTorch parity reference"), runs its private helpers `_symmetric_quantize_rows` and
`_w8a8_linear_reference` on seeded inputs and stores inputs and outputs.  Tests read only the
committed .npz, so they run where no reference checkout exists.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch


def load_reference(root: Path):
    path = root / "tools" / "tests" / "test_w8a8_quantization.py"
    spec = importlib.util.spec_from_file_location("ref_w8a8_policy", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    import os
    default = os.environ.get("WORLDMODEL_REFERENCE_DIR") or Path(__file__).resolve().parents[3] / "reference"
    root = Path(sys.argv[1] if len(sys.argv) > 1 else default)
    ref = load_reference(root)
    out = {"torch_version": np.array(torch.__version__)}

    # the reference's own four tests must hold for the module we just imported
    ref.test_w8a8_zero_rows_have_unit_scale_and_zero_codes()
    ref.test_w8a8_outer_scale_dequantization_matches_elementwise_formula()
    ref.test_w8a8_reference_quality_with_row_scale_variation_and_outliers()
    ref.test_waypoint_maximum_k_has_int32_accumulator_headroom()

    # case A: the reference's dequantization test inputs (seed 0x57A8, 17x128 . 33x128)
    torch.manual_seed(0x57A8)
    x = torch.randn(17, 128, dtype=torch.float32)
    w = torch.randn(33, 128, dtype=torch.float32)
    o, qx, qw, sx, sw, acc = ref._w8a8_linear_reference(x, w)
    out.update(a_x=x.numpy(), a_w=w.numpy(), a_out=o.numpy(), a_qx=qx.numpy(), a_qw=qw.numpy(),
               a_sx=sx.numpy(), a_sw=sw.numpy(), a_acc=acc.numpy())

    # case B: the reference's quality test inputs (seed 1234, 32x256x64, scale spread, outliers)
    torch.manual_seed(1234)
    m, k, n = 32, 256, 64
    x = torch.randn(m, k, dtype=torch.float32)
    w = torch.randn(n, k, dtype=torch.float32)
    x *= torch.exp2(torch.linspace(-1.5, 1.5, m))[:, None]
    w *= torch.exp2(torch.linspace(-1.0, 1.0, n))[:, None]
    x[1, k // 3] *= 10.0
    w[1, k // 5] *= -10.0
    o, qx, qw, sx, sw, acc = ref._w8a8_linear_reference(x, w)
    out.update(b_x=x.numpy(), b_w=w.numpy(), b_out=o.numpy(), b_qx=qx.numpy(), b_qw=qw.numpy(),
               b_sx=sx.numpy(), b_sw=sw.numpy(), b_acc=acc.numpy())

    # case C: zero rows (reference test 1) plus a ragged, non-multiple-of-anything width
    x = torch.zeros(3, 128, dtype=torch.float32)
    x[1] = torch.linspace(-2.0, 2.0, 128)
    q, s = ref._symmetric_quantize_rows(x)
    out.update(c_x=x.numpy(), c_q=q.numpy(), c_s=s.numpy())

    # case D: a slice of the config-0 distribution (fp16 tokens with x20 outlier channels,
    # N(0,0.02) fp16 weights), 64 x 2048 . 96 x 2048, fp32 up-cast before the reference call
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 2048, generator=g)
    x[:, list(range(0, 2048, 256))] *= 20.0
    x = x.to(torch.float16).to(torch.float32)
    w = (torch.randn(96, 2048, generator=g) * 0.02).to(torch.float16).to(torch.float32)
    o, qx, qw, sx, sw, acc = ref._w8a8_linear_reference(x, w)
    out.update(d_x=x.numpy().astype(np.float16), d_w=w.numpy().astype(np.float16), d_out=o.numpy(),
               d_qx=qx.numpy(), d_qw=qw.numpy(), d_sx=sx.numpy(), d_sw=sw.numpy(), d_acc=acc.numpy())

    # case E: K = 8192 worst case near the int32 headroom the reference asserts
    x = torch.full((2, 8192), 3.0)
    x[1, ::2] = -3.0
    w = torch.full((2, 8192), -0.5)
    o, qx, qw, sx, sw, acc = ref._w8a8_linear_reference(x, w)
    out.update(e_x=x.numpy(), e_w=w.numpy(), e_out=o.numpy(), e_qx=qx.numpy(), e_qw=qw.numpy(),
               e_sx=sx.numpy(), e_sw=sw.numpy(), e_acc=acc.numpy())

    dst = Path(__file__).with_name("w8a8_reference_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, dst.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
