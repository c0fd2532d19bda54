"""Python access to libb200_w8a8.so (the sm_100a W8A8 linear path) through its C ABI.

This is harness code for tests and benchmarks: it loads the shared library with ctypes,
declares the prototypes of include/b200_w8a8.h and offers thin helpers that pass
`torch.Tensor.data_ptr()` values.  There is no fallback of any kind: if the library has
not been built, importing `lib()` raises, and every wrapper raises `W8A8Error` when the C
function returns non-zero.

The directory name contains a dot, so it is not importable by name; load it with
`importlib.util.spec_from_file_location("worldmodel_cu_b200", ".../__init__.py")`
(see `__graft_entry__.load_package`).
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p, POINTER
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libb200_w8a8.so"

DT_F32, DT_F16, DT_BF16, DT_S32 = 0, 1, 2, 3
RQ_PLAIN, RQ_RMS = 1, 2
ACT_NONE, ACT_SILU, ACT_GELU_TANH = 0, 1, 2
W_ROW_MAJOR, W_SLAB128 = 0, 1


class W8A8Error(RuntimeError):
    pass


_PROTOTYPES = {
    "b200_w8a8_abi_version": (c_int, []),
    "b200_w8a8_last_error": (c_char_p, []),
    "b200_w8a8_poll_status": (c_int, [POINTER(c_int)]),
    "b200_w8a8_quantize_rows": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p]),
    "b200_w8a8_rms_norm_quantize_rows": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                                                 c_int64, c_void_p, c_int, c_int, c_float, c_void_p]),
    "b200_w8a8_dequant_act_quantize_rows": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                    c_int64, c_void_p, c_int, c_int, c_void_p]),
    "b200_w8a8_dequant_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                           c_int, c_int, c_void_p]),
    "b200_w8a8_qkv_rms_rope_dequant": (c_int, [c_void_p] * 11 + [c_int] * 6 + [c_float, c_void_p]),
    "b200_w8a8_linear_grouped": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_w8a8_linear_grouped_const_weights": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_w8a8_rope_tables": (c_int, [c_void_p] * 5 + [c_int] * 4 + [c_void_p] * 3),
    "b200_w8a8_linear_qkv_heads": (c_int, [c_void_p] * 3 + [c_int] + [c_void_p] * 7 + [c_int] * 5 + [c_float, c_void_p]),
    "b200_w8a8_gemm_i8_i32_can_implement": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int]),
    "b200_w8a8_gemm_i8_i32": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200_w8a8_selftest_mma_rate": (c_int, [c_int, POINTER(ctypes.c_double)]),
    "b200_w8a8_debug_set_wait_limit_ns": (None, [ctypes.c_ulonglong]),
    "b200_w8a8_debug_drop_operand_load": (None, [c_int]),
    "b200_w8a8_debug_force_plan": (None, [c_int, c_int, c_int]),
    "b200_w8a8_debug_one_slab_stages": (None, [c_int]),
    "b200_w8a8_linear_requant": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int64, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int,
                                         c_int, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int64, c_void_p,
                                         c_void_p]),
    "b200_w8a8_linear_requant_supported": (c_int, [c_int, c_int, c_int, c_int]),
    "b200_w8a8_set_tile_width": (None, [c_int]),
    "b200_w8a8_set_trace_buffer": (None, [c_void_p]),
    "b200_w8a8_set_pair_mma": (None, [c_int]),
    "b200_w8a8_set_overlapped_launch": (None, [c_int]),
    "b200_w8a8_linear_workspace_size": (c_size_t, [c_int, c_int, c_int]),
    "b200_w8a8_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                 c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "b200_w8a8_linear_const_weights": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_int64, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p,
                                               c_size_t, c_void_p]),
    "b200_w8a8_linear_static_scratch_capacity": (c_size_t, []),
    "b200_w8a8_linear_static_scratch": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_int64, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_w8a8_packed_weight_bytes": (c_size_t, [c_int, c_int, c_int]),
    "b200_w8a8_pack_weight_host": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int]),
    "b200_w8a8_pack_weight_blocks128_host": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int]),
    "b200_w8a8_quantize_blocks128": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_int,
                                             c_void_p]),
    "b200_w8a8_rms_norm_quantize_row_blocks128": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                                                          c_int64, c_void_p, c_int, c_int, c_float, c_void_p]),
    "b200_w8a8_linear_blocks128": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_int64, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200_w8a8_stack_create": (c_void_p, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float]),
    "b200_w8a8_stack_destroy": (None, [c_void_p]),
    "b200_w8a8_stack_set_layer": (c_int, [c_void_p, c_int] + [c_void_p] * 8 + [c_int]),
    "b200_w8a8_stack_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200_w8a8_stack_forward_host": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]),
    "b200_w8a8_stack_set_act_dtype": (c_int, [c_void_p, c_int]),
    "b200_w8a8_stack_set_lanes": (c_int, [c_void_p, c_int]),
    "b200_w8a8_stack_set_fusion": (c_int, [c_void_p, c_int]),
    "b200_w8a8_stack_device_bytes": (c_size_t, [c_void_p]),
    "b200_w8a8_stack_launches_per_forward": (ctypes.c_longlong, [c_void_p]),
    "b200_w8a8_layer_ctx_create": (c_void_p, [c_int] * 6 + [c_float, c_int]),
    "b200_w8a8_layer_ctx_destroy": (None, [c_void_p]),
    "b200_w8a8_layer_ctx_device_bytes": (c_size_t, [c_void_p]),
    "b200_w8a8_layer_qkv": (c_int, [c_void_p] * 8 + [c_int, c_void_p]),
    "b200_w8a8_layer_after_attention": (c_int, [c_void_p] * 5 + [c_int, c_void_p]),
    "b200_w8a8_weight_file_create": (c_void_p, [ctypes.c_char_p, c_int, c_int, c_int, c_int]),
    "b200_w8a8_weight_file_add_layer": (c_int, [c_void_p] + [c_void_p] * 8 + [c_int]),
    "b200_w8a8_weight_file_close": (c_int, [c_void_p]),
    "b200_w8a8_weight_file_info": (c_int, [ctypes.c_char_p] + [ctypes.POINTER(c_int)] * 4 + [c_int]),
    "b200_w8a8_stack_load_weights": (c_int, [c_void_p, ctypes.c_char_p]),
    "b200_w8a8_stack_save_weights": (c_int, [c_void_p, ctypes.c_char_p]),
}

_lib = None


def exported_symbols():
    """Names this module expects the library to export (every declaration of the C header)."""
    return sorted(_PROTOTYPES)


def lib() -> ctypes.CDLL:
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise W8A8Error(f"{LIB_PATH} is missing: run `python worldmodel.cu_b200/build.py` (needs nvcc); "
                            "there is no fallback path")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def _check(rc: int, what: str):
    if rc != 0:
        msg = lib().b200_w8a8_last_error()
        raise W8A8Error(f"{what} failed: {msg.decode() if msg else '?'}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _dt(t) -> int:
    import torch
    return {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16, torch.int32: DT_S32}[t.dtype]


def mma_rate(slabs_per_cta=16384) -> float:
    """Measured tcgen05 int8 MMA rate of the current device in TOP/s (see b200_w8a8_selftest_mma_rate)."""
    out = ctypes.c_double(0.0)
    _check(lib().b200_w8a8_selftest_mma_rate(slabs_per_cta, ctypes.byref(out)), "selftest_mma_rate")
    return out.value


def poll_status() -> int:
    st = c_int(0)
    _check(lib().b200_w8a8_poll_status(ctypes.byref(st)), "poll_status")
    return st.value


# ------------------------------------------------------------------ operators on CUDA tensors
def quantize_rows(x, cols=None):
    """x: [rows, >=cols] CUDA tensor (fp32/fp16/bf16), last dim contiguous.  Returns (q int8, scales)."""
    import torch
    rows = x.shape[0]
    cols = x.shape[1] if cols is None else cols
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(lib().b200_w8a8_quantize_rows(_ptr(x), _dt(x), x.stride(0), _ptr(q), cols, _ptr(s), rows, cols, _stream()),
           "quantize_rows")
    return q, s


def rms_norm_quantize_rows(x, vec_scale=None, bias=None, eps=1e-6, scale_is_mod=True):
    import torch
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(lib().b200_w8a8_rms_norm_quantize_rows(_ptr(x), _dt(x), x.stride(0), _ptr(vec_scale), int(scale_is_mod),
                                                  _ptr(bias), _ptr(q), cols, _ptr(s), rows, cols, eps, _stream()),
           "rms_norm_quantize_rows")
    return q, s


def dequant_act_quantize_rows(acc, in_row_scales, w_scales, bias=None, act=ACT_SILU, out_row_scales=None):
    import torch
    rows, cols = acc.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=acc.device)
    s = torch.empty(rows, dtype=torch.float32, device=acc.device) if out_row_scales is None else out_row_scales
    _check(lib().b200_w8a8_dequant_act_quantize_rows(_ptr(acc), acc.stride(0), _ptr(in_row_scales), _ptr(w_scales),
                                                     _ptr(bias), act, _ptr(q), cols, _ptr(s), rows, cols, _stream()),
           "dequant_act_quantize_rows")
    return q, s


def dequant_residual(acc, row_scales, col_scales, residual=None, gate=None, out_dtype=None):
    import torch
    rows, cols = acc.shape
    out_dtype = out_dtype or (residual.dtype if residual is not None else torch.float32)
    out = torch.empty(rows, cols, dtype=out_dtype, device=acc.device)
    _check(lib().b200_w8a8_dequant_residual(_ptr(acc), _ptr(row_scales), _ptr(col_scales), _ptr(residual),
                                            _dt(residual) if residual is not None else _dt(out), _ptr(gate),
                                            _ptr(out), _dt(out), rows, cols, _stream()), "dequant_residual")
    return out


def qkv_rms_rope_dequant(acc, row_scales, w_scales, x_pos, y_pos, t_pos, xy, inv_t, n_heads, n_kv_heads, d_head,
                         width, height, eps):
    import torch
    T = acc.shape[0]
    q = torch.empty(n_heads, T, d_head, dtype=torch.float32, device=acc.device)
    k = torch.empty(n_kv_heads, T, d_head, dtype=torch.float32, device=acc.device)
    v = torch.empty(n_kv_heads, T, d_head, dtype=torch.float32, device=acc.device)
    _check(lib().b200_w8a8_qkv_rms_rope_dequant(_ptr(acc), _ptr(row_scales), _ptr(w_scales), _ptr(q), _ptr(k), _ptr(v),
                                                _ptr(x_pos), _ptr(y_pos), _ptr(t_pos), _ptr(xy), _ptr(inv_t), T,
                                                n_heads, n_kv_heads, d_head, width, height, eps, _stream()),
           "qkv_rms_rope_dequant")
    return q, k, v


class _Problem(ctypes.Structure):
    """b200_w8a8_problem of include/b200_w8a8.h."""
    _fields_ = [("x_i8", c_void_p), ("x_scales", c_void_p), ("w_i8", c_void_p), ("w_scales", c_void_p),
                ("bias", c_void_p), ("residual", c_void_p), ("ldr", ctypes.c_int64), ("y", c_void_p),
                ("ldy", ctypes.c_int64), ("m", c_int), ("k", c_int), ("n", c_int)]


def linear_grouped(problems, w_layout=W_ROW_MAJOR, act=ACT_NONE, out_dtype=None, stream=None, const_weights=False):
    """Runs several independent skinny linears (M <= 128) in one launch.  `problems` is a list of dicts with
    keys x_i8, x_scales, w_i8, w_scales, n and optionally bias, residual, out; returns the list of outputs."""
    import torch
    out_dtype = out_dtype or torch.float16
    arr = (_Problem * len(problems))()
    outs = []
    for i, q in enumerate(problems):
        m, k = q["x_i8"].shape
        n = q["n"]
        res = q.get("residual")
        y = q.get("out")
        if y is None:
            y = torch.empty(m, n, dtype=out_dtype, device=q["x_i8"].device)
        outs.append(y)
        arr[i] = _Problem(_ptr(q["x_i8"]), _ptr(q["x_scales"]), _ptr(q["w_i8"]), _ptr(q["w_scales"]), _ptr(q.get("bias")),
                          _ptr(res), res.stride(0) if res is not None else 0, _ptr(y), y.stride(0), m, k, n)
    st = stream if stream is not None else _stream()
    fn = lib().b200_w8a8_linear_grouped_const_weights if const_weights else lib().b200_w8a8_linear_grouped
    _check(fn(ctypes.cast(arr, c_void_p), len(problems), w_layout, act, _dt(outs[0]) if outs else DT_F16, st),
           "linear_grouped")
    return outs


def rope_tables(x_pos, y_pos, t_pos, xy, inv_t, d_head, width, height):
    """cos / sin tables [T, d_head/2] of one frame's positions (see b200_w8a8_rope_tables)."""
    import torch
    T = x_pos.shape[0]
    c = torch.empty(T, d_head // 2, dtype=torch.float32, device=x_pos.device)
    s = torch.empty_like(c)
    _check(lib().b200_w8a8_rope_tables(_ptr(x_pos), _ptr(y_pos), _ptr(t_pos), _ptr(xy), _ptr(inv_t), T, d_head, width,
                                       height, _ptr(c), _ptr(s), _stream()), "rope_tables")
    return c, s


def linear_qkv_heads(x_i8, x_scales, w_i8, w_scales, rope_cos, rope_sin, n_heads, n_kv_heads, d_head, eps,
                     bias=None, w_layout=W_ROW_MAJOR):
    """QKV linear + per-head RMSNorm + rotary embedding in one kernel; returns head-major fp32 q, k, v."""
    import torch
    T, kdim = x_i8.shape
    q = torch.empty(n_heads, T, d_head, dtype=torch.float32, device=x_i8.device)
    k = torch.empty(n_kv_heads, T, d_head, dtype=torch.float32, device=x_i8.device)
    v = torch.empty(n_kv_heads, T, d_head, dtype=torch.float32, device=x_i8.device)
    _check(lib().b200_w8a8_linear_qkv_heads(_ptr(x_i8), _ptr(x_scales), _ptr(w_i8), w_layout, _ptr(w_scales), _ptr(bias),
                                            _ptr(rope_cos), _ptr(rope_sin), _ptr(q), _ptr(k), _ptr(v), T, kdim, n_heads,
                                            n_kv_heads, d_head, eps, _stream()), "linear_qkv_heads")
    return q, k, v


def gemm_i8_i32(x_i8, w_i8, n=None, w_layout=W_ROW_MAJOR):
    import torch
    m, k = x_i8.shape
    n = w_i8.shape[0] if n is None else n
    acc = torch.empty(m, n, dtype=torch.int32, device=x_i8.device)
    _check(lib().b200_w8a8_gemm_i8_i32(_ptr(x_i8), _ptr(w_i8), w_layout, _ptr(acc), m, k, n, _stream()), "gemm_i8_i32")
    return acc


def make_workspace(m, k, n, device="cuda"):
    """Zero-filled split-K scratch for (m, k, n), or None when the planner would not split.  The
    library keeps it zero-filled between launches, so one buffer can serve many calls in a row."""
    import torch
    nbytes = lib().b200_w8a8_linear_workspace_size(m, k, n)
    return torch.zeros(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def linear(x_i8, x_scales, w_i8, w_scales, n=None, w_layout=W_ROW_MAJOR, bias=None, gate=None, residual=None,
           act=ACT_NONE, out_dtype=None, out=None, workspace=None, const_weights=False):
    import torch
    m, k = x_i8.shape
    n = w_scales.shape[0] if n is None else n
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype or torch.float16, device=x_i8.device)
    ws_bytes, ws = 0, None
    if workspace is not None:
        ws, ws_bytes = workspace, workspace.numel() * workspace.element_size()
    fn = lib().b200_w8a8_linear_const_weights if const_weights else lib().b200_w8a8_linear
    _check(fn(_ptr(x_i8), _ptr(x_scales), _ptr(w_i8), w_layout, _ptr(w_scales), _ptr(bias),
              _ptr(gate), _ptr(residual), residual.stride(0) if residual is not None else 0,
              _ptr(out), _dt(out), out.stride(0), m, k, n, act, _ptr(ws), ws_bytes, _stream()), "linear")
    return out


def linear_requant(x_i8, x_scales, w_i8, w_scales, n=None, w_layout=W_ROW_MAJOR, bias=None, gate=None, residual=None,
                   act=ACT_NONE, out_dtype=None, store_out=True, q_mode=RQ_PLAIN, q_cols=None, norm_scale=None,
                   scale_is_mod=False, norm_bias=None, eps=1e-6):
    """The fused linear that also emits the next linear's A8 codes (see b200_w8a8_linear_requant).
    Returns (y or None, codes int8 [m, q_cols], scales fp32 [m])."""
    import torch
    m, k = x_i8.shape
    n = w_scales.shape[0] if n is None else n
    q_cols = n if q_cols is None else q_cols
    out_dtype = out_dtype or (residual.dtype if residual is not None else torch.float16)
    out = torch.empty(m, n, dtype=out_dtype, device=x_i8.device) if store_out else None
    dt = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}[out_dtype]
    q = torch.empty(m, q_cols, dtype=torch.int8, device=x_i8.device)
    qs = torch.empty(m, dtype=torch.float32, device=x_i8.device)
    _check(lib().b200_w8a8_linear_requant(_ptr(x_i8), _ptr(x_scales), _ptr(w_i8), w_layout, _ptr(w_scales), _ptr(bias),
                                          _ptr(gate), _ptr(residual), residual.stride(0) if residual is not None else 0,
                                          _ptr(out), dt, n, m, k, n, act, q_mode, q_cols, _ptr(norm_scale),
                                          int(scale_is_mod), _ptr(norm_bias), eps, _ptr(q), q_cols, _ptr(qs), _stream()),
           "linear_requant")
    return out, q, qs


def linear_static_scratch(x_i8, x_scales, w_i8, w_scales, n=None, w_layout=W_ROW_MAJOR, bias=None, gate=None,
                          residual=None, act=ACT_NONE, out=None):
    """The no-allocation entry point: `out` must be supplied, nothing is allocated on the way."""
    m, k = x_i8.shape
    n = w_scales.shape[0] if n is None else n
    _check(lib().b200_w8a8_linear_static_scratch(_ptr(x_i8), _ptr(x_scales), _ptr(w_i8), w_layout, _ptr(w_scales),
                                                 _ptr(bias), _ptr(gate), _ptr(residual),
                                                 residual.stride(0) if residual is not None else 0, _ptr(out),
                                                 _dt(out), out.stride(0), m, k, n, act, _stream()),
           "linear_static_scratch")
    return out


def pack_weight(w_f32_cpu, layout=W_SLAB128, threads=0):
    """Host fp32 [N,K] -> (int8 packed CPU tensor [N*K], fp32 scales [N])."""
    import torch
    w = w_f32_cpu.contiguous().to(torch.float32)
    n, k = w.shape
    nbytes = lib().b200_w8a8_packed_weight_bytes(n, k, layout)
    if nbytes == 0:
        raise W8A8Error(f"layout {layout} cannot hold N={n} K={k}")
    packed = torch.empty(nbytes, dtype=torch.int8)
    scales = torch.empty(n, dtype=torch.float32)
    _check(lib().b200_w8a8_pack_weight_host(w.data_ptr(), n, k, layout, packed.data_ptr(), scales.data_ptr(), threads),
           "pack_weight_host")
    return packed, scales


# ------------------------------------------------------------------ 128 x 128 blockwise numerics
def pack_weight_blocks128(w_f32_cpu, layout=W_SLAB128, threads=0):
    """Host fp32 [N,K] -> (int8 packed CPU tensor [N*K], fp32 block scales [ceil(N/128), K/128])."""
    import torch
    w = w_f32_cpu.contiguous().to(torch.float32)
    n, k = w.shape
    packed = torch.empty(n * k, dtype=torch.int8)
    scales = torch.empty((n + 127) // 128, max(k // 128, 1), dtype=torch.float32)
    _check(lib().b200_w8a8_pack_weight_blocks128_host(w.data_ptr(), n, k, layout, packed.data_ptr(), scales.data_ptr(),
                                                      threads), "pack_weight_blocks128_host")
    return packed, scales


def quantize_blocks128(x, block_rows=128):
    """x: [rows, cols] CUDA tensor (fp32/fp16/bf16), cols % 128 == 0.  Returns (codes int8, block scales
    [ceil(rows/128), cols/128]; with block_rows=1 one scale per row and K block, [rows, cols/128])."""
    import torch
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    s = torch.empty(rows if block_rows == 1 else (rows + 127) // 128, max(cols // 128, 1), dtype=torch.float32,
                    device=x.device)
    _check(lib().b200_w8a8_quantize_blocks128(_ptr(x), _dt(x), x.stride(0), _ptr(q), cols, _ptr(s), rows, cols,
                                              block_rows, _stream()), "quantize_blocks128")
    return q, s


def rms_norm_quantize_row_blocks128(x, vec_scale=None, bias=None, eps=1e-6, scale_is_mod=True):
    """Fused (Ada)RMSNorm -> codes with one scale per row and 128-wide K block.  Returns (int8 [rows, cols], fp32 [rows, cols/128])."""
    import torch
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    s = torch.empty(rows, max(cols // 128, 1), dtype=torch.float32, device=x.device)
    _check(lib().b200_w8a8_rms_norm_quantize_row_blocks128(_ptr(x), _dt(x), x.stride(0), _ptr(vec_scale), int(scale_is_mod),
                                                           _ptr(bias), _ptr(q), cols, _ptr(s), rows, cols, eps, _stream()),
           "rms_norm_quantize_row_blocks128")
    return q, s


def linear_blocks128(x_i8, x_block_scales, w_i8, w_block_scales, n, w_layout=W_SLAB128, bias=None, gate=None,
                     residual=None, act=ACT_NONE, out_dtype=None, out=None, x_block_rows=128):
    import torch
    m, k = x_i8.shape
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype or torch.float16, device=x_i8.device)
    _check(lib().b200_w8a8_linear_blocks128(_ptr(x_i8), _ptr(x_block_scales), _ptr(w_i8), w_layout, _ptr(w_block_scales),
                                            _ptr(bias), _ptr(gate), _ptr(residual),
                                            residual.stride(0) if residual is not None else 0, _ptr(out), _dt(out),
                                            out.stride(0), m, k, n, act, x_block_rows, _stream()), "linear_blocks128")
    return out


def write_weight_file(path, d_model, n_qkv, d_hidden, layers, threads=0):
    """Quantizes and packs `layers` (an iterable of (five fp32 CPU weights, three fp32 norm vectors),
    as LinearStack.set_layer takes them) into one packed-weight file.  Host only: needs no GPU."""
    layers = list(layers)
    w = lib().b200_w8a8_weight_file_create(str(path).encode(), d_model, n_qkv, d_hidden, len(layers))
    if not w:
        raise W8A8Error("weight_file_create failed: " + lib().b200_w8a8_last_error().decode())
    rc, msg = 0, ""
    for weights_fp32, gammas in layers:
        ws = [t.contiguous().float() for t in weights_fp32]
        gs = [t.contiguous().float() for t in gammas]
        rc = lib().b200_w8a8_weight_file_add_layer(w, *[t.data_ptr() for t in ws], *[t.data_ptr() for t in gs],
                                                   threads)
        if rc:
            msg = lib().b200_w8a8_last_error().decode()
            break
    rc_close = lib().b200_w8a8_weight_file_close(w)
    if rc:
        raise W8A8Error("weight_file_add_layer failed: " + msg)
    _check(rc_close, "weight_file_close")


def weight_file_info(path, verify=True):
    """Returns (d_model, n_qkv, d_hidden, n_layers) of a packed-weight file; raises if it is invalid."""
    vals = [c_int(0) for _ in range(4)]
    _check(lib().b200_w8a8_weight_file_info(str(path).encode(), *[ctypes.byref(v) for v in vals], int(verify)),
           "weight_file_info")
    return tuple(v.value for v in vals)


class _Layer(ctypes.Structure):
    """b200_w8a8_layer of include/b200_w8a8.h."""
    _fields_ = [(n, c_void_p) for n in ("w_qkv", "s_qkv", "w_out", "s_out", "w_ctrl_fc1", "s_ctrl_fc1", "w_ctrl_fc2",
                                        "s_ctrl_fc2", "w_fc1", "s_fc1", "w_fc2", "s_fc2", "mod_scale0", "mod_bias0",
                                        "gate0", "ctrl_cond", "mod_scale1", "mod_bias1", "gate1")]


class ReferenceLayerDriver:
    """The per-layer driver in the reference's parameterization (b200_w8a8_layer_*).  `layer` arguments are
    dicts of CUDA tensors keyed like the fields of b200_w8a8_layer; missing keys are NULL."""

    def __init__(self, max_tokens, d_model, n_heads, n_kv_heads, d_head, d_hidden, eps, w_layout=W_ROW_MAJOR):
        self.dims = (d_model, n_heads, n_kv_heads, d_head, d_hidden)
        self.handle = lib().b200_w8a8_layer_ctx_create(max_tokens, d_model, n_heads, n_kv_heads, d_head, d_hidden, eps,
                                                       w_layout)
        if not self.handle:
            raise W8A8Error("layer_ctx_create failed: " + lib().b200_w8a8_last_error().decode())

    @staticmethod
    def pack(layer):
        keep = dict(layer)  # keeps the tensors alive as long as the struct
        st = _Layer(**{n: _ptr(layer.get(n)) for n, _ in _Layer._fields_})
        st._keep = keep
        return st

    def qkv(self, layer, tokens, rope_cos, rope_sin):
        import torch
        d, hq, hkv, dh, _ = self.dims
        T = tokens.shape[0]
        q = torch.empty(hq, T, dh, dtype=torch.float32, device=tokens.device)
        k = torch.empty(hkv, T, dh, dtype=torch.float32, device=tokens.device)
        v = torch.empty(hkv, T, dh, dtype=torch.float32, device=tokens.device)
        st = layer if isinstance(layer, _Layer) else self.pack(layer)
        _check(lib().b200_w8a8_layer_qkv(self.handle, ctypes.byref(st), _ptr(tokens), _ptr(rope_cos), _ptr(rope_sin),
                                         _ptr(q), _ptr(k), _ptr(v), T, _stream()), "layer_qkv")
        return q, k, v

    def after_attention(self, layer, attn, tokens, out=None):
        import torch
        out = torch.empty_like(tokens) if out is None else out
        st = layer if isinstance(layer, _Layer) else self.pack(layer)
        _check(lib().b200_w8a8_layer_after_attention(self.handle, ctypes.byref(st), _ptr(attn), _ptr(tokens), _ptr(out),
                                                     tokens.shape[0], _stream()), "layer_after_attention")
        return out

    def close(self):
        if self.handle:
            lib().b200_w8a8_layer_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LinearStack:
    """Thin holder of a b200_w8a8_stack handle (see include/b200_w8a8.h)."""

    def __init__(self, d_model=2048, n_qkv=6144, d_hidden=8192, n_layers=24, max_rows=512, band_rows=0,
                 dtype=None, eps=1e-6):
        import torch
        self.dtype = dtype or torch.float16
        self.shape = (d_model, n_qkv, d_hidden, n_layers)
        self.max_rows = max_rows
        self.handle = lib().b200_w8a8_stack_create(d_model, n_qkv, d_hidden, n_layers, max_rows, band_rows,
                                                   DT_F16 if self.dtype == torch.float16 else DT_BF16, eps)
        if not self.handle:
            raise W8A8Error("stack_create failed: " + lib().b200_w8a8_last_error().decode())

    def set_layer(self, layer, weights_fp32, gammas, threads=0):
        """weights_fp32: five CPU fp32 tensors (qkv, out, ctrl, up, down); gammas: three fp32 vectors."""
        ws = [w.contiguous().float() for w in weights_fp32]
        gs = [g.contiguous().float() for g in gammas]
        _check(lib().b200_w8a8_stack_set_layer(self.handle, layer, *[w.data_ptr() for w in ws],
                                               *[g.data_ptr() for g in gs], threads), "stack_set_layer")

    def forward(self, x, y=None, steps=1, use_graph=False, stream=None):
        import torch
        y = torch.empty_like(x) if y is None else y
        st = stream if stream is not None else _stream()
        _check(lib().b200_w8a8_stack_forward(self.handle, x.data_ptr(), y.data_ptr(), x.shape[0], steps,
                                             int(use_graph), st), "stack_forward")
        return y

    def forward_host(self, x_host, y_host, steps=1, use_graph=False):
        _check(lib().b200_w8a8_stack_forward_host(self.handle, x_host.data_ptr(), y_host.data_ptr(), x_host.shape[0],
                                                  steps, int(use_graph)), "stack_forward_host")
        return y_host

    def load_weights(self, path):
        """Loads every layer from a packed-weight file (see write_weight_file)."""
        _check(lib().b200_w8a8_stack_load_weights(self.handle, str(path).encode()), "stack_load_weights")

    def save_weights(self, path):
        _check(lib().b200_w8a8_stack_save_weights(self.handle, str(path).encode()), "stack_save_weights")

    def set_lanes(self, lanes):
        _check(lib().b200_w8a8_stack_set_lanes(self.handle, lanes), "stack_set_lanes")

    def set_fusion(self, on):
        _check(lib().b200_w8a8_stack_set_fusion(self.handle, int(bool(on))), "stack_set_fusion")

    def set_dtype(self, dtype):
        import torch
        _check(lib().b200_w8a8_stack_set_act_dtype(self.handle, DT_F16 if dtype == torch.float16 else DT_BF16),
               "stack_set_act_dtype")
        self.dtype = dtype

    @property
    def device_bytes(self):
        return lib().b200_w8a8_stack_device_bytes(self.handle)

    @property
    def launches_per_forward(self):
        return lib().b200_w8a8_stack_launches_per_forward(self.handle)

    def close(self):
        if self.handle:
            lib().b200_w8a8_stack_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
