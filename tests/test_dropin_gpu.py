"""Builds tests/dropin_sequence.cu against the shared library (it sees only the restated
reference operator header) and checks every buffer it dumps against the oracle."""
import shutil
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "dropin_sequence.cu"


def build_dropin(out_dir: Path, pkg) -> Path:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = out_dir / "dropin_sequence"
    lib_dir = pkg.LIB_PATH.parent
    r = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", f"-I{ROOT / 'include'}",
                        str(SRC), f"-L{lib_dir}", "-lb200_w8a8", f"-Xlinker=-rpath={lib_dir}", "-o", str(exe)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_dropin_sequence_links_against_the_library(tmp_path, pkg):
    """CPU-side: the reference-named operators resolve at link time with C++ linkage."""
    build_dropin(tmp_path, pkg)


def read_dump(path):
    raw = path.read_bytes()
    out, off = {}, 0
    while off < len(raw):
        nlen, nbytes = struct.unpack_from("<QQ", raw, off)
        off += 16
        name = raw[off:off + nlen].decode()
        off += nlen
        out[name] = raw[off:off + nbytes]
        off += nbytes
    return out


@pytest.mark.gpu
def test_dropin_sequence_matches_oracle(tmp_path, pkg, ref, parity_log):
    exe = build_dropin(tmp_path, pkg)
    out = tmp_path / "dump.bin"
    r = subprocess.run([str(exe), str(out)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    d = read_dump(out)
    T, D, KV, HID, HQ, HKV, DH, W, H = 96, 256, 128, 512, 4, 2, 64, 16, 6
    NQKV = D + 2 * KV
    eps = 1.1920929e-07
    f = lambda n, *shape: torch.from_numpy(np.frombuffer(d[n], dtype=np.float32).reshape(*shape).copy())
    i8 = lambda n, *shape: torch.from_numpy(np.frombuffer(d[n], dtype=np.int8).reshape(*shape).copy())
    i32 = lambda n, *shape: torch.from_numpy(np.frombuffer(d[n], dtype=np.int32).reshape(*shape).copy())
    i64 = lambda n: torch.from_numpy(np.frombuffer(d[n], dtype=np.int64).copy())
    same = lambda a, b: torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))

    tokens, attn = f("tokens", T, D), f("attn", T, D)
    q, s = ref.rms_norm_quantize_rows(tokens, f("s0", D), f("b0", D), eps, scale_is_mod=True)
    assert same(i8("q1", T, D), q) and same(f("sa1", T), s)
    assert same(i32("acc_qkv", T, NQKV), ref.gemm_i8_i32(q, i8("wqkv", NQKV, D)))
    qr, kr, vr = ref.qkv_fused_rms_rope_i32_dequant(i32("acc_qkv", T, NQKV), s, f("sqkv", NQKV), i64("xp"), i64("yp"),
                                                    i64("tp"), f("xy", DH // 8), f("invt", DH // 2 - 2 * (DH // 8)),
                                                    HQ, HKV, DH, W, H, eps)
    assert same(f("v", HKV, T, DH), vr)
    assert torch.allclose(f("q", HQ, T, DH), qr, rtol=1e-5, atol=2e-6)
    assert torch.allclose(f("k", HKV, T, DH), kr, rtol=1e-5, atol=2e-6)

    q, s = ref.quantize_rows(attn)
    assert same(i8("q2", T, D), q) and same(f("sa2", T), s)
    acc = ref.gemm_i8_i32(q, i8("wout", D, D))
    assert same(i32("acc_out", T, D), acc)
    after_attn = ref.dequant_gated_residual(acc, s, f("sout", D), tokens, f("g0", D))
    assert same(f("after_attn", T, D), after_attn)

    q, s = ref.rms_norm_quantize_rows(after_attn, None, None, eps)
    assert same(i8("q3", T, D), q) and same(f("sa3", T), s)
    acc = ref.gemm_i8_i32(q, i8("wfc1x", D, D))
    assert same(i32("acc_fc1x", T, D), acc)
    q4_ref, s4_ref = ref.dequant_silu_quantize_rows(acc, s, f("sfc1x", D), f("cond", D))
    q4, s4 = i8("q4", T, D), f("sa4", T)
    d4 = (q4.int() - q4_ref.int()).abs()
    row4 = parity_log("drop-in sequence: controller codes after SiLU (q4)", int((d4 != 0).sum()), d4.numel(),
                      max_step=int(d4.max()))
    assert torch.allclose(s4, s4_ref, rtol=2e-6) and int(d4.max()) <= 1 and row4["mismatches"] <= 1  # measured: 0 of 24 576
    acc = ref.gemm_i8_i32(q4, i8("wfc2x", D, D))  # continue from the GPU's own codes
    assert same(i32("acc_fc2x", T, D), acc)
    after_ctrl = ref.dequant_add_residual(acc, s4, f("sfc2x", D), after_attn)
    assert same(f("after_ctrl", T, D), after_ctrl)

    q, s = ref.rms_norm_quantize_rows(after_ctrl, f("s1", D), f("b1", D), eps, scale_is_mod=True)
    assert same(i8("q5", T, D), q) and same(f("sa5", T), s)
    acc = ref.gemm_i8_i32(q, i8("wfc1", HID, D))
    assert same(i32("acc_fc1", T, HID), acc)
    q6_ref, s6_ref = ref.dequant_silu_quantize_rows(acc, s, f("sfc1", HID), None)
    q6, s6 = i8("q6", T, HID), f("sa6", T)
    d6 = (q6.int() - q6_ref.int()).abs()
    row6 = parity_log("drop-in sequence: MLP codes after SiLU (q6)", int((d6 != 0).sum()), d6.numel(),
                      max_step=int(d6.max()))
    assert torch.allclose(s6, s6_ref, rtol=2e-6) and int(d6.max()) <= 1 and row6["mismatches"] <= 1  # measured: 0 of 49 152
    acc = ref.gemm_i8_i32(q6, i8("wfc2", D, HID))
    assert same(i32("acc_fc2", T, D), acc)
    assert same(f("next", T, D), ref.dequant_gated_residual(acc, s6, f("sfc2", D), after_ctrl, f("g1", D)))


@pytest.mark.gpu
def test_operators_from_two_host_threads_on_their_own_streams(pkg, ref):
    """The operators keep no per-call state outside their arguments: two host threads, each with its own stream,
    buffers and shapes, run quantizer + fused linear 40 times at once and both get the oracle's bits."""
    import threading

    results, errors = {}, []

    def worker(idx, m, k, n):
        try:
            g = torch.Generator().manual_seed(100 + idx)
            x = (torch.randn(m, k, generator=g) * 0.7).to(torch.float16)
            w = torch.randn(n, k, generator=g) * 0.02
            bias = torch.randn(n, generator=g) * 0.1
            packed, sw = pkg.pack_weight(w, layout=pkg.W_SLAB128)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                xd, pd, swd, bd = x.to("cuda"), packed.to("cuda"), sw.to("cuda"), bias.to("cuda")
                outs = []
                for _ in range(40):
                    q, s = pkg.quantize_rows(xd)
                    outs.append(pkg.linear(q, s, pd, swd, n=n, w_layout=pkg.W_SLAB128, bias=bd, out_dtype=torch.float16))
            stream.synchronize()
            qr, sr = ref.quantize_rows(x)
            qw, swr = ref.quantize_weight(w)
            want = ref.linear_w8a8(qr, sr, qw, swr, bias=bias, out_dtype=torch.float16)
            results[idx] = all(torch.equal(o.cpu().view(torch.uint8), want.view(torch.uint8)) for o in outs)
        except Exception as exc:  # surfaced in the main thread below
            errors.append(repr(exc))

    threads = [threading.Thread(target=worker, args=(0, 512, 2048, 2048)),
               threading.Thread(target=worker, args=(1, 48, 1024, 6144))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert results == {0: True, 1: True}
    assert pkg.poll_status() == 0
