"""CPU oracle for the W8A8 linear hot path of WorldDiT (TEST INFRASTRUCTURE ONLY).

This module restates, in plain PyTorch on the CPU, the arithmetic of the reference's
row/channel-wise int8 linears.  It is the checker the parity tests compare the CUDA
kernels against; it is never imported by the product library, which has no CPU path.

Parity pin: the functions below are checked against the reference's own PyTorch policy
test (tools/tests/test_w8a8_quantization.py) both by re-running that file's four known
answer tests and by golden vectors generated from the reference's private helpers
(tests/golden/make_golden.py).  The fused operators (RMSNorm->A8, dequant->act->A8,
dequant->residual, QKV dequant->RMS->RoPE, weight packing) have no PyTorch pin in the
reference; for those this file restates the cited kernel lines.  Their runnable pin is the
reference's own operator file compiled in place (oracle/build_reference_ops.py ->
oracle/_ref/, loaded by oracle/ref_cuda_ops.py): tests/test_reference_kernels_gpu.py runs
the reference's eight CUDA operators and this repository's kernels on the same inputs on
the same GPU (integer results bit for bit, floating-point results within the tolerance
that the reference's --use_fast_math build leaves).

Conventions fixed here (the reference is not self-consistent between its torch test,
its probe and its fast-math CUDA build):
  1. every input is up-cast to fp32 before any arithmetic;
  2. scale = amax / 127.0f   (IEEE fp32 division; torch test line 10), zero row -> 1;
  3. code  = clamp(round_half_even(x / scale), -127, 127)   (IEEE division; line 11);
  4. dequant = (float(acc) * s_row) * s_col, left to right in fp32, then + bias,
     activation, * gate, + residual, one final round-to-nearest-even at the store;
  5. GELU(tanh) and SiLU are evaluated in fp32;
  6. fused RMSNorm: sum of squares accumulated in fp64, inv_rms = fp32(1/sqrt(ss/K+eps))
     with correctly rounded fp64 sqrt and division, then separate fp32 multiplies/adds.

The 128 x 128 blockwise functions at the end of the file (`quantize_blocks128`,
`linear_blocks128`) are PARITY UNPINNED: the reference describes that rule in its notes
(docs/cuda_w8a8_optimization.md:319-321) but holds neither an implementation nor vectors for it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

ACT_NONE = 0
ACT_SILU = 1
ACT_GELU_TANH = 2


# --------------------------------------------------------------------------------------
# quantizers
# --------------------------------------------------------------------------------------
def quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric absmax int8.

    Follows tools/tests/test_w8a8_quantization.py:6-12 (`_symmetric_quantize_rows`);
    the CUDA counterpart it checks replaces src/world_cuda_ops.cu:94-125.
    """
    assert x.ndim == 2
    x = x.to(torch.float32)
    amax = x.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.round(x / scale[:, None]).clamp(-127, 127).to(torch.int8)
    return q, scale


def quantize_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-output-channel weight quantization: the same rule applied to rows of W[N,K].

    Follows src/world_cuda.cu:172-197 for structure (zero row -> scale 1, non-finite
    weights rejected) with the scale/rounding convention of quantize_rows.
    """
    if not torch.isfinite(w).all():
        raise ValueError("non-finite W8 weight")
    return quantize_rows(w)


def inv_rms_rows(x: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32(1 / sqrt(mean(x^2) + eps)) with the sum of squares carried in fp64."""
    xd = x.to(torch.float32).to(torch.float64)
    ss = (xd * xd).sum(dim=1)
    eps64 = float(torch.tensor(eps, dtype=torch.float32))
    v = ss / float(x.shape[1]) + eps64
    return (1.0 / torch.sqrt(v)).to(torch.float32)


def rms_norm_rows(x, scale_vec, bias, eps, scale_is_mod):
    """Normalised fp32 rows that the fused quantizer sees (before quantization).

    Operation order follows src/world_cuda_ops.cu:156-161: x*inv_rms, then the scale
    vector, then the bias.  `scale_is_mod` selects the reference's (1 + mod_scale[col])
    form; otherwise scale_vec is a plain gamma multiplier.
    """
    xf = x.to(torch.float32)
    v = xf * inv_rms_rows(xf, eps)[:, None]
    if scale_vec is not None:
        s = scale_vec.to(torch.float32)
        if scale_is_mod:
            s = torch.tensor(1.0, dtype=torch.float32) + s
        v = v * s[None, :]
    if bias is not None:
        v = v + bias.to(torch.float32)[None, :]
    return v


def rms_norm_quantize_rows(x, mod_scale=None, bias=None, eps=1e-6, scale_is_mod=True):
    """Fused (Ada)RMSNorm -> A8.  Replaces src/world_cuda_ops.cu:129-182."""
    return quantize_rows(rms_norm_rows(x, mod_scale, bias, eps, scale_is_mod))


# --------------------------------------------------------------------------------------
# GEMM and epilogues
# --------------------------------------------------------------------------------------
def gemm_i8_i32(qx: torch.Tensor, qw: torch.Tensor, exact_fast: bool = True) -> torch.Tensor:
    """acc[m,n] = sum_k int32(qx[m,k]) * int32(qw[n,k]).

    The reference expression is `qx.to(int32) @ qw.to(int32).T`
    (tools/tests/test_w8a8_quantization.py:18).  With exact_fast the same integers are
    produced through an fp64 matmul: every partial sum is an integer below 2^53, so the
    result is exact in any summation order and much faster on the CPU.
    """
    if exact_fast:
        return (qx.to(torch.float64) @ qw.to(torch.float64).T).to(torch.int32)
    return qx.to(torch.int32) @ qw.to(torch.int32).T


def silu(v: torch.Tensor) -> torch.Tensor:
    """v / (1 + exp(-v)) in fp32 (src/world_cuda_ops.cu:48-50)."""
    return v / (1.0 + torch.exp(-v))


def gelu_tanh(v: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(v, approximate="tanh")


def activation(v: torch.Tensor, act: int) -> torch.Tensor:
    if act == ACT_NONE:
        return v
    if act == ACT_SILU:
        return silu(v)
    if act == ACT_GELU_TANH:
        return gelu_tanh(v)
    raise ValueError(act)


def dequant(acc, row_scales, col_scales) -> torch.Tensor:
    """(float(acc) * s_row) * s_col (src/world_cuda_ops.cu:243)."""
    return (acc.to(torch.float32) * row_scales[:, None]) * col_scales[None, :]


def epilogue_f32(acc, row_scales, col_scales, bias=None, act=ACT_NONE, gate=None, residual=None):
    """dequant -> +bias -> act -> *gate -> +residual, all fp32, no final rounding."""
    v = dequant(acc, row_scales, col_scales)
    if bias is not None:
        v = v + bias.to(torch.float32)[None, :]
    v = activation(v, act)
    if gate is not None:
        v = v * gate.to(torch.float32)[None, :]
    if residual is not None:
        v = residual.to(torch.float32) + v
    return v


def linear_w8a8(qx, sx, qw, sw, bias=None, act=ACT_NONE, gate=None, residual=None,
                out_dtype=torch.float16):
    """Fused linear: int8 GEMM + epilogue + one RNE rounding at the store."""
    acc = gemm_i8_i32(qx, qw)
    return epilogue_f32(acc, sx, sw, bias, act, gate, residual).to(out_dtype)


def linear_w8a8_requant(qx, sx, qw, sw, bias=None, act=ACT_GELU_TANH):
    """Fused linear whose fp32 result is re-quantized per row for the next GEMM."""
    acc = gemm_i8_i32(qx, qw)
    h = epilogue_f32(acc, sx, sw, bias, act)
    q, s = quantize_rows(h)
    return q, s, h


def dequant_silu_quantize_rows(acc, in_row_scales, w_scales, bias=None, act=ACT_SILU):
    """src/world_cuda_ops.cu:187-227: dequant -> (+bias) -> SiLU -> row absmax -> A8."""
    return quantize_rows(epilogue_f32(acc, in_row_scales, w_scales, bias, act))


def dequant_gated_residual(acc, row_scales, col_scales, residual, gate):
    """src/world_cuda_ops.cu:229-245: residual + (acc*sA*sW) * gate."""
    return epilogue_f32(acc, row_scales, col_scales, None, ACT_NONE, gate, residual)


def dequant_add_residual(acc, row_scales, col_scales, residual):
    """src/world_cuda_ops.cu:247-262."""
    return epilogue_f32(acc, row_scales, col_scales, None, ACT_NONE, None, residual)


def rope_phase(pair_id, x_pos, y_pos, t_pos, xy, inv_t, width, height, d_xy):
    """src/world_cuda_ops.cu:61-80, vectorised over tokens for one pair index."""
    if pair_id < d_xy:
        x = (2.0 * x_pos.to(torch.float32) + 1.0) / float(width) - 1.0
        return x * xy[pair_id]
    if pair_id < 2 * d_xy:
        y = (2.0 * y_pos.to(torch.float32) + 1.0) / float(height) - 1.0
        return y * xy[pair_id - d_xy]
    return t_pos.to(torch.float32) * inv_t[pair_id - 2 * d_xy]


def qkv_fused_rms_rope_i32_dequant(acc, row_scales, w_scales, x_pos, y_pos, t_pos, xy, inv_t,
                                   n_heads, n_kv_heads, d_head, width, height, eps, bias=None):
    """src/world_cuda_ops.cu:1229-1305.  Returns head-major fp32 q[Hq,T,d], k, v[Hkv,T,d].
    `bias` (not in the reference, whose QKV linear has none) is added right after the dequantization."""
    T = acc.shape[0]
    q_dim, kv_dim = n_heads * d_head, n_kv_heads * d_head
    z = dequant(acc, row_scales, w_scales)
    if bias is not None:
        z = z + bias.to(torch.float32)[None, :]
    half, d_xy = d_head // 2, d_head // 8
    phases = torch.stack([rope_phase(p, x_pos, y_pos, t_pos, xy, inv_t, width, height, d_xy)
                          for p in range(half)], dim=1).to(torch.float32)  # [T, half]
    c, s = torch.cos(phases), torch.sin(phases)

    def heads(block, nh):
        zz = block.reshape(T, nh, d_head)
        ss = (zz.to(torch.float64) ** 2).sum(dim=2)
        inv = (1.0 / torch.sqrt(ss / d_head + float(torch.tensor(eps, dtype=torch.float32)))).to(torch.float32)
        zn = zz * inv[:, :, None]
        a, b = zn[:, :, 0::2], zn[:, :, 1::2]
        out = torch.empty_like(zn)
        out[:, :, :half] = a * c[:, None, :] - b * s[:, None, :]
        out[:, :, half:] = b * c[:, None, :] + a * s[:, None, :]
        return out.permute(1, 0, 2).contiguous()

    q = heads(z[:, :q_dim], n_heads)
    k = heads(z[:, q_dim:q_dim + kv_dim], n_kv_heads)
    v = z[:, q_dim + kv_dim:].reshape(T, n_kv_heads, d_head).permute(1, 0, 2).contiguous()
    return q, k, v


def w8a8_linear_reference(x: torch.Tensor, weight: torch.Tensor):
    """tools/tests/test_w8a8_quantization.py:15-20 (`_w8a8_linear_reference`), verbatim policy."""
    qx, sx = quantize_rows(x)
    qw, sw = quantize_rows(weight)
    acc = gemm_i8_i32(qx, qw, exact_fast=False)
    out = acc.float() * sx[:, None] * sw[None, :]
    return out, qx, qw, sx, sw, acc


# --------------------------------------------------------------------------------------
# synthetic workloads (the benchmark configurations) and the 24-layer linear stack
# --------------------------------------------------------------------------------------
D_MODEL = 2048
N_QKV = 6144
D_HIDDEN = 8192
OUTLIER_CHANNELS = tuple(range(0, D_MODEL, D_MODEL // 8))


def make_tokens(m: int, seed: int, dtype=torch.float16, d: int = D_MODEL) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, d, generator=g)
    x[:, list(range(0, d, d // 8))] *= 20.0
    return x.to(dtype)


def make_cfg0(m: int = 512, k: int = 2048, n: int = 6144):
    """Config 0: one QKV linear with bias, fp16 in/out, seed 0."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(m, k, generator=g)
    x[:, list(range(0, k, k // 8))] *= 20.0
    x = x.to(torch.float16)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.float16)
    bias = torch.randn(n, generator=g) * 0.01
    return x, w, bias


@dataclass
class LayerWeights:
    """int8 codes + fp32 per-channel scales of one layer, and its three fp32 gammas."""
    qkv: Tuple[torch.Tensor, torch.Tensor]
    out: Tuple[torch.Tensor, torch.Tensor]
    ctrl: Tuple[torch.Tensor, torch.Tensor]
    up: Tuple[torch.Tensor, torch.Tensor]
    down: Tuple[torch.Tensor, torch.Tensor]
    g_attn: torch.Tensor
    g_ctrl: torch.Tensor
    g_mlp: torch.Tensor


def make_layer_fp32(layer: int, d: int = D_MODEL, n_qkv: int = N_QKV, hidden: int = D_HIDDEN):
    """fp32 weights (already rounded through fp16) and gammas of one layer, seed 1000+layer."""
    g = torch.Generator().manual_seed(1000 + layer)
    shapes = [(n_qkv, d), (d, d), (d, d), (hidden, d), (d, hidden)]
    ws = [(torch.randn(n, k, generator=g) * 0.02).to(torch.float16).to(torch.float32) for n, k in shapes]
    gs = [1.0 + torch.randn(d, generator=g) * 0.05 for _ in range(3)]
    return ws, gs


def make_layer(layer: int, d: int = D_MODEL, n_qkv: int = N_QKV, hidden: int = D_HIDDEN) -> LayerWeights:
    ws, gs = make_layer_fp32(layer, d, n_qkv, hidden)
    q = [quantize_weight(w) for w in ws]
    return LayerWeights(q[0], q[1], q[2], q[3], q[4], gs[0], gs[1], gs[2])


def layer_forward(x: torch.Tensor, lw: LayerWeights, eps: float = 1e-6, trace: Optional[dict] = None):
    """One layer of the linear stack; x and the returned tensor share x's 16-bit dtype.

    Wiring (norm -> A8 -> GEMM -> epilogue, attention left out, controller linear as a
    residual branch like src/world_cuda.cu:2146-2153, MLP with a re-quantized hidden like
    src/world_cuda.cu:2249-2279):
      1 rmsnorm+quant(g_attn)  2 QKV linear -> e        3 quant of the first d columns
      4 out linear + residual  5 rmsnorm+quant(g_ctrl)  6 ctrl linear + residual
      7 rmsnorm+quant(g_mlp)   8 up linear -> GELU(tanh), fp32   9 quant of the fp32 hidden
      10 down linear + residual
    """
    e = x.dtype
    d = x.shape[1]
    q1, s1 = rms_norm_quantize_rows(x, lw.g_attn, None, eps, scale_is_mod=False)
    qkv = linear_w8a8(q1, s1, *lw.qkv, out_dtype=e)
    q2, s2 = quantize_rows(qkv[:, :d])
    x1 = linear_w8a8(q2, s2, *lw.out, residual=x, out_dtype=e)
    q3, s3 = rms_norm_quantize_rows(x1, lw.g_ctrl, None, eps, scale_is_mod=False)
    x2 = linear_w8a8(q3, s3, *lw.ctrl, residual=x1, out_dtype=e)
    q4, s4 = rms_norm_quantize_rows(x2, lw.g_mlp, None, eps, scale_is_mod=False)
    q5, s5, h = linear_w8a8_requant(q4, s4, *lw.up, act=ACT_GELU_TANH)
    x3 = linear_w8a8(q5, s5, *lw.down, residual=x2, out_dtype=e)
    if trace is not None:
        trace.update(q1=q1, s1=s1, qkv=qkv, q2=q2, s2=s2, x1=x1, q3=q3, s3=s3, x2=x2,
                     q4=q4, s4=s4, h=h, q5=q5, s5=s5, x3=x3)
    return x3


def stack_forward(x: torch.Tensor, layers: Sequence[LayerWeights], steps: int = 1, eps: float = 1e-6):
    for _ in range(steps):
        for lw in layers:
            x = layer_forward(x, lw, eps)
    return x


def stack_ops_per_row(d: int = D_MODEL, n_qkv: int = N_QKV, hidden: int = D_HIDDEN) -> int:
    """Algorithmic int8 ops per token row per layer: 2 * sum(N*K) over the five linears."""
    return 2 * (n_qkv * d + d * d + d * d + hidden * d + d * hidden)


# --------------------------------------------------------------------------------------
# 128 x 128 blockwise numerics (parity unpinned, see the module docstring)
# --------------------------------------------------------------------------------------
def quantize_blocks128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scale per 128 x 128 block: scale = max(amax, 1e-8) / 128, code = rne(x / scale) saturated to
    [-128, 127] (the rule docs/cuda_w8a8_optimization.md:319 of the reference quotes).  x [R, C] with C % 128 == 0;
    a ragged last block row takes its maximum over the rows that exist.  Returns (int8 [R, C], fp32 [ceil(R/128), C/128])."""
    assert x.ndim == 2 and x.shape[1] % 128 == 0
    x = x.to(torch.float32)
    rows, cols = x.shape
    rb = (rows + 127) // 128
    xp = torch.zeros(rb * 128, cols, dtype=torch.float32)
    xp[:rows] = x
    blocks = xp.view(rb, 128, cols // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = torch.clamp(amax, min=1e-8) / 128.0
    q = torch.round(blocks / scale[:, None, :, None]).clamp(-128, 127).to(torch.int8)
    return q.view(rb * 128, cols)[:rows].contiguous(), scale


def quantize_row_blocks128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The same rule on 1 x 128 groups: one scale per row and 128-wide K block.  Returns (int8 [R, C], fp32 [R, C/128])."""
    assert x.ndim == 2 and x.shape[1] % 128 == 0
    x = x.to(torch.float32)
    rows, cols = x.shape
    groups = x.view(rows, cols // 128, 128)
    scale = torch.clamp(groups.abs().amax(dim=2), min=1e-8) / 128.0
    q = torch.round(groups / scale[:, :, None]).clamp(-128, 127).to(torch.int8)
    return q.view(rows, cols).contiguous(), scale


def rms_norm_quantize_row_blocks128(x, mod_scale=None, bias=None, eps=1e-6, scale_is_mod=True):
    """Fused (Ada)RMSNorm (`rms_norm_rows`) -> 1 x 128 group codes."""
    return quantize_row_blocks128(rms_norm_rows(x, mod_scale, bias, eps, scale_is_mod))


def fma_f32(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """Correctly rounded fp32 fused multiply-add a * b + c for fp32 inputs whose product is exact in fp64 (here a is
    an integer of at most 22 bits).  The product is formed exactly in fp64; adding c rounds once to fp64 and the
    conversion to fp32 rounds a second time.  Two roundings differ from one only when the fp64 sum sits exactly
    halfway between two fp32 neighbours while the exact sum does not; the rounding error of the fp64 addition
    (TwoSum, exact) then says on which side the exact sum lies."""
    a64, b64, c64 = a.to(torch.float64), b.to(torch.float64), c.to(torch.float64)
    p = a64 * b64
    s = p + c64
    bb = s - p
    err = (p - (s - bb)) + (c64 - bb)            # s + err == p + c exactly
    r = s.to(torch.float32)
    d = s - r.to(torch.float64)                  # exact
    inf = torch.full_like(r, float("inf"))
    other = torch.where(d > 0, torch.nextafter(r, inf), torch.nextafter(r, -inf))
    tie = (d != 0) & ((other.to(torch.float64) - s) == d)
    toward_other = tie & (err != 0) & ((err > 0) == (d > 0))
    # on a tie with err pointing back to r's side, r is right only if round-to-even happened to pick that side:
    # it did pick r, so nothing to do; with err == 0 the tie is real and round-to-even is the IEEE answer
    return torch.where(toward_other, other, r)


def linear_blocks128(qx, sx, qw, sw, bias=None, out_dtype=torch.float16, act=ACT_NONE, gate=None,
                     residual=None, x_scale_per_row=False) -> torch.Tensor:
    """y = 0; for every K block in order y = fma(float(acc_kb), sx[r/128, kb] * sw[c/128, kb], y) in fp32 (the scale
    product rounded to fp32 first), then the epilogue of `epilogue_f32` (+ bias, activation, * gate, + residual) and one
    rounding to the output type.  acc_kb is the exact int32
    partial sum of one 128-wide K block (|acc_kb| <= 2^21, so an fp32 matmul of the codes is exact)."""
    m, k = qx.shape
    n = qw.shape[0]
    assert k % 128 == 0 and qw.shape[1] == k
    rows = torch.arange(m) if x_scale_per_row else torch.arange(m) // 128
    cols = torch.arange(n) // 128
    y = torch.zeros(m, n, dtype=torch.float32)
    for kb in range(k // 128):
        acc = qx[:, kb * 128:(kb + 1) * 128].to(torch.float32) @ qw[:, kb * 128:(kb + 1) * 128].to(torch.float32).T
        f = sx[rows, kb][:, None] * sw[cols, kb][None, :]
        y = fma_f32(acc, f.expand(m, n), y)
    if bias is not None:
        y = y + bias.to(torch.float32)[None, :]
    y = activation(y, act)
    if gate is not None:
        y = y * gate.to(torch.float32)[None, :]
    if residual is not None:
        y = residual.to(torch.float32) + y
    return y.to(out_dtype)


def sqnr_db(reference: torch.Tensor, value: torch.Tensor) -> float:
    err = value.double() - reference.double()
    return float(10.0 * torch.log10(reference.double().square().sum() / err.square().sum()))


def ulp_distance_f16(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in units of the last place between two fp16/bf16 tensors of equal dtype."""
    def key(t):
        i = t.view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(a) - key(b)).abs()
