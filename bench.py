"""Benchmark of the W8A8 linear stack (the hot path) on B200.

    python bench.py --gpus N --steps K --warmup W            # this library, one JSON line
    python bench.py --impl reference --gpus N --steps K ...  # the reference arm

A step is one denoising pass of the 24-layer linear stack over the sharded config: 64
independent worlds x 2048 token rows (131 072 rows, d_model 2048, QKV 6144, MLP 8192, fp16
activations), the worlds dealt out over the N ranks with replicated weights and no collective on
the data path: strong scaling, time = max over ranks.  `value` is int8 tera-operations per
second over all GPUs with the tokens already resident in HBM, the median of `--repeats` timed
passes of K steps; `e2e` is the same metric through the host-buffer entry point with the H2D /
D2H copies inside the timed region.  At N = 1 `extras` adds the other configs (M=512 one pass,
M=2048 four chained passes in bf16, the skinny weight-bound linears, the QKV consumer epilogue).

`--impl reference` times the reference's own CUDA operators (its src/world_cuda_ops.cu compiled
where it lies into oracle/_ref/) in the reference's per-layer call order on the same rows, or,
when that library was not built, the CPU oracle port.  The CPU oracle under oracle/ is used only
by the `cpu_baseline` leg and by that arm; nothing measured as the product touches it.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

D_MODEL, N_QKV, D_HIDDEN, N_LAYERS = 2048, 6144, 8192, 24
LINEARS = [("qkv", N_QKV, D_MODEL), ("out", D_MODEL, D_MODEL), ("ctrl", D_MODEL, D_MODEL),
           ("up", D_HIDDEN, D_MODEL), ("down", D_MODEL, D_HIDDEN)]
OPS_PER_ROW_LAYER = 2 * sum(n * k for _, n, k in LINEARS)  # 109,051,904
WEIGHT_BYTES_LAYER = sum(n * k for _, n, k in LINEARS)     # 54,525,952
# DRAM read+write of the five GEMM launches of one layer from the committed ncu captures (profiles/)
NCU_DRAM_BYTES_PER_LAYER = {512: 69.6e6, 2048: 129.7e6, 8192: 668.5e6, 16384: 1521.6e6}
WORKLOADS = {
    # name: (rows per GPU, chained steps per bench step, activation dtype, band rows)
    "cfg1": (512, 1, "fp16", 0),
    "cfg2": (2048, 4, "bf16", 0),
    "cfg3": (None, 1, "fp16", 8192),    # 64 worlds x 2048 rows dealt over the ranks (strong scaling)
}
CFG3_WORLDS, CFG3_ROWS_PER_WORLD = 64, 2048


def layer_gemm_algorithmic_bytes(m: int, e: int = 2) -> int:
    """Bytes the five fused linears of one layer must move at M rows: A8 codes and W8 codes in, both scale
    vectors, the residual where there is one, and the result (e bytes per element; the up linear's hidden
    is fp32)."""
    total = 0
    for name, n, k in LINEARS:
        total += m * k + n * k + 4 * m + 4 * n
        total += (4 if name == "up" else e) * m * n
        if name in ("out", "ctrl", "down"):
            total += e * m * n
    return total


def workload_string(name: str, layers: int, worlds: int = CFG3_WORLDS) -> str:
    """The same text from both arms of the bench, so that their lines can be matched."""
    if name == "cfg3":
        return (f"cfg3: {layers}-layer W8A8 linear stack, {worlds} independent worlds x {CFG3_ROWS_PER_WORLD} rows = "
                f"{worlds * CFG3_ROWS_PER_WORLD} token rows dealt over the GPUs, d=2048, qkv 6144, mlp 8192, fp16")
    rows, chained, dt_name, _ = WORKLOADS[name]
    return (f"{name}: {layers}-layer W8A8 linear stack, M={rows} rows per GPU, {chained} chained pass(es) per step, "
            f"d=2048, qkv 6144, mlp 8192, {dt_name}")
SKINNY_SHAPES = [(2048, 2048), (2048, 8192), (8192, 2048)]  # (K, N) of config 4


def _load(name, path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_package():
    return _load("worldmodel_cu_b200", ROOT / "worldmodel.cu_b200" / "__init__.py")


def load_oracle():
    return _load("w8a8_ref", ROOT / "oracle" / "w8a8_ref.py")


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ------------------------------------------------------------------------------------------
# clock sampling (NVML, read-only) during the timed region
# ------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, device_index: int, period_s: float = 0.002):
        self.samples = []  # (t, sm_mhz, reasons_bitmask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = device_index
            if visible:
                try:
                    idx = int(visible.split(",")[device_index])
                except ValueError:
                    idx = device_index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    why = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    why = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, why))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1.0)

    def summary(self, t0: float, t1: float):
        if not self.nv:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml_unavailable"]}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        scope = "timed_region"
        if len(inside) < 3:  # region shorter than a few sampling periods: use every sample under load
            inside, scope = self.samples, "whole_run"
        mask = 0
        for s in inside:
            mask |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if mask & bit]
        return {"sm_mhz": statistics.median(s[1] for s in inside) if inside else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(inside), "scope": scope}


# ------------------------------------------------------------------------------------------
# CPU baseline: the oracle port on the host cores
# ------------------------------------------------------------------------------------------
def cpu_layer_seconds(ref, rows: int, layer_weights, x):
    """One layer of the stack through the oracle with the reference's own int32 matmul expression."""
    import torch
    orig = ref.gemm_i8_i32
    ref.gemm_i8_i32 = lambda qx, qw, exact_fast=True: orig(qx, qw, exact_fast=False)
    try:
        t0 = time.perf_counter()
        y = ref.layer_forward(x[:rows], layer_weights)
        dt = time.perf_counter() - t0
    finally:
        ref.gemm_i8_i32 = orig
    assert torch.isfinite(y.float()).all()
    return dt


def use_all_host_threads():
    """torchrun pins OMP_NUM_THREADS=1; the CPU arm should use every core the box offers."""
    import torch
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(max(n, 1))
    return torch.get_num_threads()


def run_cpu_baseline(budget_s: float = 15.0):
    """Times a bounded sample of the workload on the host: rows of one layer of one world."""
    import torch
    ref = load_oracle()
    cores = use_all_host_threads()
    lw = ref.make_layer(0)
    x = ref.make_tokens(512, 0, torch.float16)
    t_probe = cpu_layer_seconds(ref, 32, lw, x)
    rows = int(max(32, min(512, 32 * budget_s / max(t_probe, 1e-3))))
    rows -= rows % 32
    dt = cpu_layer_seconds(ref, rows, lw, x)
    tops = rows * OPS_PER_ROW_LAYER / dt / 1e12
    return {"value": tops, "unit": "TOP/s", "cores": cores, "kind": "port",
            "sample": f"1 of 24 layers of the stack on {rows} rows of world 0, oracle port with the reference's "
                      f"int32 matmul expression, {dt:.2f} s"}


# ------------------------------------------------------------------------------------------
# reference arm: the reference's own CUDA operators in its per-layer call order
# ------------------------------------------------------------------------------------------
class ReferenceCudaStack:
    """The reference's W8A8 operator sequence for the linears of a layer (src/world_cuda.cu:1819-2330 with
    attention left out, as in the stack): norm->A8, int8 GEMM into the int32 scratch, consumer / dequant
    kernels, on fp32 tokens, 24 distinct weight sets.  Launched one by one on the default stream, as the
    reference does (its operators take no stream)."""

    def __init__(self, rows, n_heads=32, d_head=64):
        import torch
        sys.path.insert(0, str(ROOT / "oracle"))
        import ref_cuda_ops as rk
        self.rk, self.rows = rk, rows
        dev = "cuda"
        d, nq, hid = D_MODEL, N_QKV, D_HIDDEN
        g = torch.Generator().manual_seed(11)
        rnd8 = lambda *shape: torch.randint(-127, 128, shape, dtype=torch.int8, device=dev)
        self.ws = {name: [rnd8(n, k) for _ in range(N_LAYERS)] for name, n, k in LINEARS}
        self.sw = {name: torch.rand(n, device=dev) * 1e-3 for name, n, k in LINEARS}
        self.x = torch.randn(rows, d, device=dev)
        self.x1, self.x2, self.x3 = (torch.empty_like(self.x) for _ in range(3))
        self.gamma = torch.randn(d, device=dev) * 0.05
        self.gate = torch.ones(d, device=dev)
        self.a8 = rnd8(rows, hid)
        self.sa = torch.rand(rows, device=dev) * 1e-2
        self.acc = torch.empty(rows, hid, dtype=torch.int32, device=dev)
        self.n_heads, self.d_head = n_heads, d_head
        self.n_kv = (nq // d_head - n_heads) // 2
        self.q = torch.empty(n_heads, rows, d_head, device=dev)
        self.k = torch.empty(self.n_kv, rows, d_head, device=dev)
        self.v = torch.empty(self.n_kv, rows, d_head, device=dev)
        self.pos = [torch.randint(0, hi, (rows,), generator=g).to(dev) for hi in (32, 16, 64)]
        self.xy = (torch.rand(d_head // 8, generator=g) * 6).to(dev)
        self.inv_t = torch.rand(d_head // 2 - 2 * (d_head // 8), generator=g).to(dev)

    def gemm(self, name, layer):
        n, k = next((n, k) for nm, n, k in LINEARS if nm == name)
        self.rk.call("gemm_i8_i32", self.a8, self.ws[name][layer], self.acc, self.rows, k, n)

    def layers(self, n_layers=N_LAYERS):
        rk, rows, d, nq, hid = self.rk, self.rows, D_MODEL, N_QKV, D_HIDDEN
        x, x1, x2, x3, a8, sa, acc, sw = self.x, self.x1, self.x2, self.x3, self.a8, self.sa, self.acc, self.sw
        for l in range(n_layers):
            rk.call("rms_norm_quantize_rows_i8", x, self.gamma, None, a8, sa, rows, d, 1e-6)
            self.gemm("qkv", l)
            rk.call("qkv_fused_rms_rope_i32_dequant", acc, sa, sw["qkv"], self.q, self.k, self.v, *self.pos, self.xy,
                    self.inv_t, rows, self.n_heads, self.n_kv, self.d_head, 32, 16, 1e-6)
            rk.call("quantize_rows_f32_i8", self.q, a8, sa, rows, d)  # stands in for the attention output [rows, d]
            self.gemm("out", l)
            rk.call("dequant_gated_residual_f32", acc, sa, sw["out"], x, self.gate, x1, rows, d)
            rk.call("rms_norm_quantize_rows_i8", x1, self.gamma, None, a8, sa, rows, d, 1e-6)
            self.gemm("ctrl", l)
            rk.call("dequant_add_residual_f32", acc, sa, sw["ctrl"], x1, x2, rows, d)
            rk.call("rms_norm_quantize_rows_i8", x2, self.gamma, None, a8, sa, rows, d, 1e-6)
            self.gemm("up", l)
            rk.call("dequant_silu_quantize_rows_i8", acc, sa, sw["up"], None, a8, sa, rows, hid)
            self.gemm("down", l)
            rk.call("dequant_gated_residual_f32", acc, sa, sw["down"], x2, self.gate, x3, rows, d)


    def layers_reference_wiring(self, n_layers=N_LAYERS):
        """The reference's real layer: six GEMMs (the controller branch is fc1 + cond -> SiLU -> fc2), sixteen
        launches, as world_cuda_runtime_step_rgb issues them (src/world_cuda.cu:1819-2330)."""
        rk, rows, d, nq, hid = self.rk, self.rows, D_MODEL, N_QKV, D_HIDDEN
        x, x1, x2, x3, a8, sa, acc, sw = self.x, self.x1, self.x2, self.x3, self.a8, self.sa, self.acc, self.sw
        for l in range(n_layers):
            rk.call("rms_norm_quantize_rows_i8", x, self.gamma, self.gamma, a8, sa, rows, d, 1e-6)
            self.gemm("qkv", l)
            rk.call("qkv_fused_rms_rope_i32_dequant", acc, sa, sw["qkv"], self.q, self.k, self.v, *self.pos, self.xy,
                    self.inv_t, rows, self.n_heads, self.n_kv, self.d_head, 32, 16, 1e-6)
            rk.call("quantize_rows_f32_i8", self.q, a8, sa, rows, d)  # stands in for the attention output [rows, d]
            self.gemm("out", l)
            rk.call("dequant_gated_residual_f32", acc, sa, sw["out"], x, self.gate, x1, rows, d)
            rk.call("rms_norm_quantize_rows_i8", x1, None, None, a8, sa, rows, d, 1e-6)
            self.gemm("ctrl", l)
            rk.call("dequant_silu_quantize_rows_i8", acc, sa, sw["ctrl"], self.gamma, a8, sa, rows, d)
            self.gemm("ctrl", (l + 1) % N_LAYERS)
            rk.call("dequant_add_residual_f32", acc, sa, sw["ctrl"], x1, x2, rows, d)
            rk.call("rms_norm_quantize_rows_i8", x2, self.gamma, self.gamma, a8, sa, rows, d, 1e-6)
            self.gemm("up", l)
            rk.call("dequant_silu_quantize_rows_i8", acc, sa, sw["up"], None, a8, sa, rows, hid)
            self.gemm("down", l)
            rk.call("dequant_gated_residual_f32", acc, sa, sw["down"], x2, self.gate, x3, rows, d)


def reference_cuda_available():
    import torch
    if not torch.cuda.is_available():
        return "no CUDA device"
    sys.path.insert(0, str(ROOT / "oracle"))
    import ref_cuda_ops as rk
    if not rk.available():
        return ("oracle/_ref/libworld_cuda_ops_ref.so is not built (needs the reference checkout and a CUTLASS "
                "header tree at build time)")
    return None


def event_ms(fn, reps):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def run_reference_arm(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    rows_w, chained, dt_name, _ = WORKLOADS[args.workload]
    total_rows = args.worlds * CFG3_ROWS_PER_WORLD if args.workload == "cfg3" else rows_w
    line = {"impl": "reference", "metric": "w8a8_linear_stack_int8_tops", "unit": "TOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "scaling": "strong" if args.workload == "cfg3" else "weak", "vs_baseline": None, "dtype": "s8",
            "data": "synthetic", "config": {"workload": workload_string(args.workload, args.layers, args.worlds)}}
    why_not = reference_cuda_available()
    if why_not is None:
        # The reference has no multi-GPU mode and no CPU implementation of this path: one process runs its
        # CUDA operators over the whole job on one GPU, in slices of 16 384 rows (its int32 scratch is
        # 4 * rows * 8192 bytes), every slice through all layers, `chained` times.
        torch.cuda.set_device(0)
        slice_rows = min(total_rows, 16384)
        n_slices = -(-total_rows // slice_rows)
        stack = ReferenceCudaStack(slice_rows)

        def step():
            for _ in range(n_slices * chained):
                stack.layers(args.layers)
        for _ in range(args.warmup):
            step()
        ms = event_ms(step, args.steps)
        ops = n_slices * slice_rows * OPS_PER_ROW_LAYER * args.layers * chained
        tops = ops / (ms * 1e-3) / 1e12
        sample = (f"the reference's own CUDA operators (src/world_cuda_ops.cu built with its --use_fast_math, CUTLASS "
                  f"Sm80 mma.sync GEMM) on ONE GPU: the whole job, {n_slices} slice(s) of {slice_rows} rows x "
                  f"{args.layers} layers x {chained} pass(es) per step, 14 eager launches per layer, fp32 tokens")
        line.update(value=tops, ms_per_step=ms, gpu_launches=int(14 * args.layers * n_slices * chained * args.steps),
                    cpu_baseline={"value": tops, "unit": "TOP/s", "cores": 1, "kind": "reference", "sample": sample},
                    e2e={"value": tops, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        try:
            line["cpu_port"] = run_cpu_baseline(10.0)
        except Exception as exc:
            line["cpu_port"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        print(json.dumps(line))
        return 0
    # no reference CUDA library on this box: the CPU oracle port on the host cores, a bounded sample per step
    ref = load_oracle()
    cores = use_all_host_threads()
    lw = ref.make_layer(0)
    x = ref.make_tokens(512, 0, torch.float16)
    t_probe = cpu_layer_seconds(ref, 32, lw, x)
    total = max(args.steps + args.warmup, 1)
    rows = int(max(32, min(512, 32 * (150.0 / total) / max(t_probe, 1e-3))))
    rows -= rows % 32
    for _ in range(args.warmup):
        cpu_layer_seconds(ref, rows, lw, x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_layer_seconds(ref, rows, lw, x)
    dt = time.perf_counter() - t0
    tops = args.steps * rows * OPS_PER_ROW_LAYER / dt / 1e12
    sample = (f"each step = 1 of {args.layers} layers on {rows} rows of world 0 (bounded sample of the workload), oracle "
              f"port with the reference's int32 matmul expression on {cores} host threads")
    line.update(value=tops, ms_per_step=dt / args.steps * 1e3, reference_cuda_unavailable=why_not,
                cpu_baseline={"value": tops, "unit": "TOP/s", "cores": cores, "kind": "port", "sample": sample},
                e2e={"value": tops, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------
def build_stack(pkg, ref, rows, band_rows, dtype, n_layers=N_LAYERS):
    t0 = time.perf_counter()
    stack = pkg.LinearStack(D_MODEL, N_QKV, D_HIDDEN, n_layers, max_rows=rows, band_rows=band_rows, dtype=dtype)
    for l in range(n_layers):
        ws, gs = ref.make_layer_fp32(l)  # seeded synthetic fp32 weights (host), quantized + packed by the library
        stack.set_layer(l, ws, gs)
    return stack, time.perf_counter() - t0


def time_steps(fn, steps, stream, barrier):
    """CUDA-event time of `steps` calls of fn on `stream`, bracketed by barrier + synchronize."""
    import torch
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(steps):
            fn()
        stop.record(stream)
    stop.synchronize()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    barrier()
    return start.elapsed_time(stop), t0, t1


def time_gemm_kernels(pkg, rows, stream, iters=3):
    """Average device time per launch of the dominant kernel (the tcgen05 GEMM), per linear shape,
    cycling through 24 distinct weight matrices per shape so that weights come from HBM as in the stack."""
    import torch
    res = {}
    dev = "cuda"
    for name, n, k in LINEARS:
        ws = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev) for _ in range(N_LAYERS)]
        sw = torch.rand(n, device=dev) * 1e-3
        a8 = torch.randint(-127, 128, (rows, k), dtype=torch.int8, device=dev)
        sx = torch.rand(rows, device=dev) * 1e-2
        residual = torch.randn(rows, n, device=dev).half() if n == D_MODEL else None
        out_dtype = torch.float32 if name == "up" else torch.float16
        out = torch.empty(rows, n, dtype=out_dtype, device=dev)
        act = pkg.ACT_GELU_TANH if name == "up" else pkg.ACT_NONE

        def run():
            for w in ws:
                pkg.linear(a8, sx, w, sw, n=n, w_layout=pkg.W_SLAB128, residual=residual, act=act, out=out,
                           const_weights=True)
        # replayed as a graph so that the device, not the Python launch rate, sets the pace
        with torch.cuda.stream(stream):
            run()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
        with torch.cuda.stream(stream):
            graph.replay()
        ms, _, _ = time_steps(graph.replay, iters, stream, lambda: None)
        res[name] = ms / (iters * N_LAYERS) * 1e-3  # seconds per launch
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="timed passes of --steps steps; the median is reported")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--worlds", type=int, default=CFG3_WORLDS,
                    help="cfg3 only: worlds of 2048 rows in the job (64 = the real workload; fewer for a small, "
                         "self-ending profiler capture)")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels one by one instead of replaying a graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary configs reported under `extras`")
    ap.add_argument("--layers", type=int, default=N_LAYERS, help="layers of the stack (24 = the real workload)")
    ap.add_argument("--band", type=int, default=-1, help="rows per band (default: the workload's own)")
    ap.add_argument("--lanes", type=int, default=0, help="streams that bands alternate over (default 2 for cfg3)")
    ap.add_argument("--pair-mma", type=int, default=0, choices=[0, 1, 2],
                    help="CTA-pair (cta_group::2) GEMM: 0 = the planner decides, 1 = wherever legal, 2 = never")
    ap.add_argument("--fusion", action="store_true",
                    help="let the linears with d_model outputs emit the next linear's codes from their epilogue "
                         "(six launches per layer instead of ten; measured slower, off by default)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)

    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)

    def max_over_ranks(v):
        if world == 1:
            return float(v)
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    pkg, ref = load_package(), load_oracle()
    pkg.lib().b200_w8a8_set_pair_mma(args.pair_mma)  # (lib() raises if the CUDA library is missing)
    peaks = measured_peaks()
    rows, chained, dt_name, band = WORKLOADS[args.workload]
    sharding = _load("w8a8_sharding", ROOT / "worldmodel.cu_b200" / "sharding.py")
    my_worlds = [rank]  # cfg1 / cfg2: one independent world per rank, seeded by its global id (weak scaling)
    if args.workload == "cfg3":
        my_worlds = sharding.world_seeds(args.worlds, world, rank)
        rows = len(my_worlds) * CFG3_ROWS_PER_WORLD
    if rows == 0:
        raise SystemExit(f"rank {rank} of {world} has no world to run: use at most {args.worlds} GPUs")
    dtype = torch.float16 if dt_name == "fp16" else torch.bfloat16
    use_graph = not args.no_graph
    if args.workload == "cfg3" and rows >= 32768:
        band = 16384  # bands as tall as still leaves every lane one: the CTA-pair GEMMs gain from more tiles per launch
    if args.band >= 0:
        band = args.band
    lanes = args.lanes if args.lanes > 0 else (2 if args.workload == "cfg3" else 1)

    want_extras = not args.no_extras and world == 1 and args.layers == N_LAYERS
    stack, setup_s = build_stack(pkg, ref, max(rows, 2048 if want_extras else rows), band, dtype, args.layers)
    stack.set_lanes(lanes)
    stack.set_fusion(args.fusion)
    # every world has its own seeded tokens; weights are replicated on every rank
    per_world = rows // len(my_worlds)
    x = torch.cat([ref.make_tokens(per_world, w, dtype) for w in my_worlds]).to("cuda")
    y = torch.empty_like(x)
    stream = torch.cuda.Stream()
    step = lambda: stack.forward(x, y, steps=chained, use_graph=use_graph, stream=stream.cuda_stream)

    sampler = ClockSampler(local_rank)
    sampler.start()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step()
    stream.synchronize()
    # `repeats` timed passes of exactly `steps` steps, each bracketed by barrier + synchronize, each the max over ranks
    pass_ms, t_first, t_last = [], None, None
    for _ in range(args.repeats):
        ms, t0, t1 = time_steps(step, args.steps, stream, barrier)
        pass_ms.append(max_over_ranks(ms))
        t_first = t0 if t_first is None else t_first
        t_last = t1
    clocks = sampler.summary(t_first, t_last)
    if pkg.poll_status() != 0:
        raise SystemExit("a GEMM kernel reported a bounded-wait timeout")
    ms = statistics.median(pass_ms)
    total_rows = rows * world if args.workload != "cfg3" else args.worlds * CFG3_ROWS_PER_WORLD
    job_ops_per_step = total_rows * OPS_PER_ROW_LAYER * args.layers * chained
    value = job_ops_per_step * args.steps / (ms * 1e-3) / 1e12
    launches = stack.launches_per_forward * args.steps

    # end to end through the host-buffer entry point (pinned host tokens in, pinned result out)
    xh = x.cpu().pin_memory()
    yh = torch.empty_like(xh).pin_memory()
    for _ in range(3):
        stack.forward_host(xh, yh, steps=chained, use_graph=use_graph)
    e2e_ms = []
    for _ in range(min(args.repeats, 3)):
        barrier()
        torch.cuda.synchronize()
        e0 = time.perf_counter()
        for _ in range(args.steps):
            stack.forward_host(xh, yh, steps=chained, use_graph=use_graph)
        e2e_ms.append(max_over_ranks((time.perf_counter() - e0) * 1e3))
        barrier()
    e_ms = statistics.median(e2e_ms)
    e2e_value = job_ops_per_step * args.steps / (e_ms * 1e-3) / 1e12
    io_bytes = rows * D_MODEL * 2

    if rank != 0:
        sampler.stop()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    # roofline of the dominant kernel (the tcgen05 GEMM), timed per launch with CUDA events at the
    # height the stack launches it with (one band of rows)
    launch_rows = min(rows, band) if band > 0 else rows
    per_launch = time_gemm_kernels(pkg, launch_rows, stream)
    gemm_ops = launch_rows * OPS_PER_ROW_LAYER
    gemm_s = sum(per_launch.values())
    int8_peak = 2.0 * peaks["bf16_tflops"]  # tcgen05 int8 issues at twice the bf16 rate
    achieved = gemm_ops / gemm_s / 1e12
    weight_gbs = WEIGHT_BYTES_LAYER / gemm_s / 1e9
    mma_burst, mma_sustained = pkg.mma_rate(16384), pkg.mma_rate(1 << 20)
    traffic = NCU_DRAM_BYTES_PER_LAYER.get(launch_rows)
    algo_bytes = layer_gemm_algorithmic_bytes(launch_rows)
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                "frac": achieved / int8_peak, "traffic": traffic,
                "traffic_note": "dram read+write summed over the five GEMM launches of one layer at this height (ncu, "
                                f"profiles/); algorithmic bytes of the same launches: {algo_bytes / 1e6:.1f} MB",
                "kernel": f"gemm_i8 (tcgen05 s8xs8->s32 + fused epilogue), five linears of a layer at M={launch_rows}",
                "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']}); nominal dense int8 4500",
                "frac_of_nominal_4500": achieved / 4500.0,
                "measured_int8_mma_tops": {"burst": mma_burst, "sustained": mma_sustained,
                                           "how": "b200_w8a8_selftest_mma_rate: one CTA per SM issuing tcgen05.mma "
                                                  "kind::i8 128x256x32 back to back, no loads, no epilogue"},
                "frac_of_measured_int8_mma": achieved / mma_burst,
                "frac_of_measured_int8_mma_sustained": achieved / mma_sustained,
                "weight_stream_gbs": weight_gbs, "weight_stream_frac_of_hbm": weight_gbs / peaks["hbm_gbs"],
                "us_per_launch": {k: v * 1e6 for k, v in per_launch.items()}}

    line = {"metric": "w8a8_linear_stack_int8_tops", "value": value, "unit": "TOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if args.workload == "cfg3" else "weak", "vs_baseline": None, "dtype": "s8",
            "data": "synthetic",
            "config": {"workload": workload_string(args.workload, args.layers, args.worlds),
                       "rows_per_gpu": rows, "layers": args.layers, "graph_replay": use_graph,
                       "band_rows": band, "lanes": lanes, "fused_quantizers": bool(args.fusion),
                       "l2": "no flush: each step streams 1.31 GB of int8 weights per band, 10x the 126 MB L2"},
            "timing": {"repeats": args.repeats, "ms_per_step_each": [m / args.steps for m in pass_ms],
                       "statistic": "median of the repeats; each repeat = K steps between barrier + synchronize, "
                                    "CUDA events, max over ranks"},
            "gpu_launches": int(launches), "clocks": clocks, "setup_s": setup_s,
            "e2e": {"value": e2e_value, "unit": "TOP/s", "ms_per_step": e_ms / args.steps,
                    "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes},
            "roofline": roofline}

    if want_extras:
        line["extras"] = run_extras(pkg, ref, stack, stream, peaks)
    sampler.stop()
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = run_cpu_baseline()
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_extras(pkg, ref, stack, stream, peaks):
    """Secondary configs on one GPU, each a short run with the same stack: config 1 (M=512, one pass, graph
    and eager, with the reference's CUDA operators at the same M beside it), config 2 (M=2048, four chained
    passes, bf16), config 4 (skinny linears) and the QKV consumer epilogue."""
    import torch
    out = {}
    stack.set_lanes(1)

    def timed(x, y, steps, use_graph, reps):
        fn = lambda: stack.forward(x, y, steps=steps, use_graph=use_graph, stream=stream.cuda_stream)
        with torch.cuda.stream(stream):
            for _ in range(3):
                fn()
        passes = [time_steps(fn, reps, stream, lambda: None)[0] / reps for _ in range(5)]
        return statistics.median(passes), passes

    # config 2: M=2048, 4 chained passes, bf16
    stack.set_dtype(torch.bfloat16)
    x = ref.make_tokens(2048, 0, torch.bfloat16).to("cuda")
    y = torch.empty_like(x)
    ms, passes = timed(x, y, 4, True, 5)
    tops = 2048 * OPS_PER_ROW_LAYER * N_LAYERS * 4 / (ms * 1e-3) / 1e12
    out["cfg2_m2048_4steps_bf16"] = {"ms_per_4_steps": ms, "ms_each": passes, "tops": tops,
                                     "frac_of_2x_measured_bf16": tops / (2 * peaks["bf16_tflops"]),
                                     "frac_of_nominal_4500": tops / 4500.0,
                                     "target": "<= 7.94 ms (60 % of 4500 TOP/s)"}
    # config 1: M=512, one pass, fp16: graph replay and eager launches
    stack.set_dtype(torch.float16)
    x = ref.make_tokens(512, 0, torch.float16).to("cuda")
    y = torch.empty_like(x)
    ms_graph, passes = timed(x, y, 1, True, 20)
    ms_eager, _ = timed(x, y, 1, False, 20)
    ops1 = 512 * OPS_PER_ROW_LAYER * N_LAYERS
    out["cfg1_m512_fp16"] = {"graph_ms_per_step": ms_graph, "graph_ms_each": passes, "eager_ms_per_step": ms_eager,
                             "graph_tops": ops1 / (ms_graph * 1e-3) / 1e12, "eager_tops": ops1 / (ms_eager * 1e-3) / 1e12}
    try:  # the reference's own CUDA operators at the same M, eager like the reference launches them
        why_not = reference_cuda_available()
        if why_not is None:
            rstack = ReferenceCudaStack(512)
            rstack.layers()
            ms_ref = event_ms(rstack.layers, 3)
            gemm_us = {}
            for name, _, _ in LINEARS:
                gemm_us[name] = event_ms(lambda name=name: [rstack.gemm(name, l) for l in range(N_LAYERS)], 3) / N_LAYERS * 1e3
            out["cfg1_m512_fp16"]["reference_cuda_ops"] = {"eager_ms_per_step": ms_ref, "tops": ops1 / (ms_ref * 1e-3) / 1e12,
                                                           "gemm_us": gemm_us, "launches_per_layer": 14}
            del rstack
        else:
            out["cfg1_m512_fp16"]["reference_cuda_ops"] = {"unavailable": why_not}
    except Exception as exc:  # a comparator must never cost the line
        out["cfg1_m512_fp16"]["reference_cuda_ops"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    out["cfg4_skinny"] = run_skinny(pkg, stream, peaks)
    out["qkv_heads_t512"] = run_qkv_heads(pkg, stream)
    try:
        out["blockwise_128x128_m8192"] = run_blockwise(pkg, stream)
    except Exception as exc:
        out["blockwise_128x128_m8192"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    try:
        out["reference_layer_t512"] = run_reference_layer(pkg, stream)
    except Exception as exc:
        out["reference_layer_t512"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    return out


def run_reference_layer(pkg, stream, tokens=512, n_heads=32, d_head=64):
    """The per-layer driver in the reference's parameterization (b200_w8a8_layer_qkv + _after_attention: AdaRMSNorm,
    head-major q/k/v with RoPE, gated residuals, controller branch, SiLU MLP, fp32 tokens; 13 launches per layer)
    over 24 distinct layers at T=512, next to the reference's own operators in the reference's own order
    (16 launches per layer) on the same GPU.  The q block stands in for the attention output in both."""
    import torch
    dev = "cuda"
    d, hid = D_MODEL, D_HIDDEN
    n_kv = (N_QKV // d_head - n_heads) // 2
    g = torch.Generator().manual_seed(21)
    rnd8 = lambda n, k: torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev)
    vec = lambda n, s=1e-3: torch.rand(n, device=dev) * s
    layers = []
    for _ in range(N_LAYERS):
        layers.append(dict(w_qkv=rnd8(N_QKV, d), s_qkv=vec(N_QKV), w_out=rnd8(d, d), s_out=vec(d), w_ctrl_fc1=rnd8(d, d),
                           s_ctrl_fc1=vec(d), w_ctrl_fc2=rnd8(d, d), s_ctrl_fc2=vec(d), w_fc1=rnd8(hid, d), s_fc1=vec(hid),
                           w_fc2=rnd8(d, hid), s_fc2=vec(d, 1e-4), mod_scale0=vec(d, 0.1), mod_bias0=vec(d, 0.1),
                           gate0=vec(d, 1.0), ctrl_cond=vec(d, 0.1), mod_scale1=vec(d, 0.1), mod_bias1=vec(d, 0.1),
                           gate1=vec(d, 1.0)))
    drv = pkg.ReferenceLayerDriver(tokens, d, n_heads, n_kv, d_head, hid, 1e-6, w_layout=pkg.W_SLAB128)
    packed = [drv.pack(L) for L in layers]
    pos = [torch.randint(0, hi, (tokens,), generator=g).to(dev) for hi in (32, 16, 64)]
    xy = (torch.rand(d_head // 8, generator=g) * 6).to(dev)
    inv_t = torch.rand(d_head // 2 - 2 * (d_head // 8), generator=g).to(dev)
    x = torch.randn(tokens, d, device=dev)
    bufs = [torch.empty_like(x), torch.empty_like(x)]
    q = torch.empty(n_heads, tokens, d_head, device=dev)
    k = torch.empty(n_kv, tokens, d_head, device=dev)
    v = torch.empty(n_kv, tokens, d_head, device=dev)
    L = pkg.lib()
    import ctypes
    with torch.cuda.stream(stream):
        cos, sin = pkg.rope_tables(*pos, xy, inv_t, d_head, 32, 16)

    def step():
        st = torch.cuda.current_stream().cuda_stream
        cur = x
        for i, pl in enumerate(packed):
            nxt = bufs[i & 1]
            rc = L.b200_w8a8_layer_qkv(drv.handle, ctypes.byref(pl), cur.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                       q.data_ptr(), k.data_ptr(), v.data_ptr(), tokens, st)
            rc |= L.b200_w8a8_layer_after_attention(drv.handle, ctypes.byref(pl), q.data_ptr(), cur.data_ptr(),
                                                    nxt.data_ptr(), tokens, st)
            assert rc == 0, L.b200_w8a8_last_error()
            cur = nxt

    with torch.cuda.stream(stream):
        step()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step()
    with torch.cuda.stream(stream):
        graph.replay()
    passes = [time_steps(graph.replay, 10, stream, lambda: None)[0] / 10 for _ in range(5)]
    eager = [time_steps(step, 10, stream, lambda: None)[0] / 10 for _ in range(3)]
    ops = tokens * 2 * (N_QKV * d + 3 * d * d + 2 * hid * d) * N_LAYERS
    out = {"graph_ms_per_step": statistics.median(passes), "eager_ms_per_step": statistics.median(eager),
           "launches_per_layer": 13, "tops_graph": ops / (statistics.median(passes) * 1e-3) / 1e12,
           "shape": f"T={tokens} d={d} heads {n_heads}/{n_kv} x {d_head} hidden {hid}, 24 layers, SLAB128 weights"}
    why_not = reference_cuda_available()
    if why_not is None:
        rstack = ReferenceCudaStack(tokens)
        rstack.layers_reference_wiring()
        ms_ref = event_ms(rstack.layers_reference_wiring, 3)
        out["reference_cuda_ops"] = {"eager_ms_per_step": ms_ref, "launches_per_layer": 16,
                                     "tops": ops / (ms_ref * 1e-3) / 1e12}
    else:
        out["reference_cuda_ops"] = {"unavailable": why_not}
    drv.close()
    return out


def run_blockwise(pkg, stream, rows=8192, n_weights=8):
    """The 128 x 128 blockwise numerics (block quantizer + linear with per-K-block fp32 accumulation) next to the
    row/channel rule (row quantizer + fused linear) on the layer's shapes at one band of rows, fp16 in and out,
    graph replay over several distinct weight matrices per shape."""
    import torch
    dev = "cuda"
    out = {"rows": rows}
    for name, k, n in (("qkv", D_MODEL, N_QKV), ("out", D_MODEL, D_MODEL), ("down", D_HIDDEN, D_MODEL)):
        x = torch.randn(rows, k, device=dev, dtype=torch.float16)
        y = torch.empty(rows, n, device=dev, dtype=torch.float16)
        wq = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev) for _ in range(n_weights)]
        sw_blk = torch.rand((n + 127) // 128, k // 128, device=dev) * 1e-4 + 1e-5
        sw_row = torch.rand(n, device=dev) * 1e-4 + 1e-5
        qb, sb = pkg.quantize_blocks128(x)
        qg, sg = pkg.quantize_blocks128(x, block_rows=1)
        qr, sr = pkg.quantize_rows(x)

        def lin_blocks():
            for w in wq:
                pkg.linear_blocks128(qb, sb, w, sw_blk, n=n, out=y)

        def lin_groups():  # 1 x 128 activation groups: a scale per token row and K block
            for w in wq:
                pkg.linear_blocks128(qg, sg, w, sw_blk, n=n, out=y, x_block_rows=1)

        def lin_rows():
            for w in wq:
                pkg.linear(qr, sr, w, sw_row, n=n, w_layout=pkg.W_SLAB128, out=y, const_weights=True)

        def quant_blocks():
            for _ in wq:
                pkg.lib().b200_w8a8_quantize_blocks128(x.data_ptr(), pkg.DT_F16, k, qb.data_ptr(), k, sb.data_ptr(), rows, k, 128,
                                                       torch.cuda.current_stream().cuda_stream)

        def quant_rows():
            for _ in wq:
                pkg.lib().b200_w8a8_quantize_rows(x.data_ptr(), pkg.DT_F16, k, qr.data_ptr(), k, sr.data_ptr(), rows, k,
                                                  torch.cuda.current_stream().cuda_stream)

        res = {}
        for key, run in (("blockwise_linear_us", lin_blocks), ("row_group_linear_us", lin_groups),
                         ("row_channel_linear_us", lin_rows),
                         ("block_quantizer_us", quant_blocks), ("row_quantizer_us", quant_rows)):
            with torch.cuda.stream(stream):
                run()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                run()
            with torch.cuda.stream(stream):
                graph.replay()
            ms, _, _ = time_steps(graph.replay, 5, stream, lambda: None)
            res[key] = ms / (5 * n_weights) * 1e3
        ops = 2.0 * rows * k * n
        res["blockwise_tops"] = ops / res["blockwise_linear_us"] * 1e-6
        res["row_channel_tops"] = ops / res["row_channel_linear_us"] * 1e-6
        out[f"{name}_{k}x{n}"] = res
    # fp16 activation quantizer + linear at M=128 on the reference model's four shapes: the quantity the reference's
    # notes time for a third-party blockwise kernel on other hardware (docs/cuda_w8a8_optimization.md:344-347)
    small = {}
    for name, k, n in (("qkv", D_MODEL, 4096), ("out", D_MODEL, D_MODEL), ("fc1", D_MODEL, D_HIDDEN), ("fc2", D_HIDDEN, D_MODEL)):
        x = torch.randn(128, k, device=dev, dtype=torch.float16)
        y = torch.empty(128, n, device=dev, dtype=torch.float16)
        wq = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev) for _ in range(n_weights)]
        sw_blk = torch.rand((n + 127) // 128, k // 128, device=dev) * 1e-4 + 1e-5
        qb = torch.empty(128, k, dtype=torch.int8, device=dev)
        sb = torch.empty(1, k // 128, device=dev)

        def quant_then_linear():
            st = torch.cuda.current_stream().cuda_stream
            for w in wq:
                pkg.lib().b200_w8a8_quantize_blocks128(x.data_ptr(), pkg.DT_F16, k, qb.data_ptr(), k, sb.data_ptr(), 128, k,
                                                       128, st)
                pkg.linear_blocks128(qb, sb, w, sw_blk, n=n, out=y)

        with torch.cuda.stream(stream):
            quant_then_linear()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            quant_then_linear()
        with torch.cuda.stream(stream):
            graph.replay()
        ms, _, _ = time_steps(graph.replay, 5, stream, lambda: None)
        small[f"{name}_{k}x{n}_us"] = ms / (5 * n_weights) * 1e3
    out["m128_quant_plus_linear"] = small
    return out


def run_qkv_heads(pkg, stream, tokens=512, n_heads=32, n_kv_heads=16, k=2048, d_head=64):
    """The QKV linear with the per-head RMSNorm + RoPE consumer as its epilogue against the two-call
    form it replaces (GEMM to int32, then the consumer kernel), the reference's head counts, 24 distinct
    weight matrices per graph so that weights stream from HBM."""
    import torch
    dev = "cuda"
    n = (n_heads + 2 * n_kv_heads) * d_head
    g = torch.Generator().manual_seed(7)
    ws = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev) for _ in range(N_LAYERS)]
    a8 = torch.randint(-127, 128, (tokens, k), generator=g, dtype=torch.int8).to(dev)
    sx = (torch.rand(tokens, generator=g) * 0.05 + 0.01).to(dev)
    sw = (torch.rand(n, generator=g) * 2e-4 + 1e-5).to(dev)
    pos = [torch.randint(0, hi, (tokens,), generator=g).to(dev) for hi in (32, 16, 64)]
    xy = (torch.rand(d_head // 8, generator=g) * 6).to(dev)
    inv_t = torch.rand(d_head // 2 - 2 * (d_head // 8), generator=g).to(dev)
    acc = torch.empty(tokens, n, dtype=torch.int32, device=dev)
    q = torch.empty(n_heads, tokens, d_head, device=dev)
    kk = torch.empty(n_kv_heads, tokens, d_head, device=dev)
    v = torch.empty(n_kv_heads, tokens, d_head, device=dev)
    L = pkg.lib()
    with torch.cuda.stream(stream):
        cos, sin = pkg.rope_tables(*pos, xy, inv_t, d_head, 32, 16)

    def fused():
        st = torch.cuda.current_stream().cuda_stream
        for w in ws:
            rc = L.b200_w8a8_linear_qkv_heads(a8.data_ptr(), sx.data_ptr(), w.data_ptr(), pkg.W_SLAB128, sw.data_ptr(),
                                              None, cos.data_ptr(), sin.data_ptr(), q.data_ptr(), kk.data_ptr(),
                                              v.data_ptr(), tokens, k, n_heads, n_kv_heads, d_head, 1e-6, st)
            assert rc == 0, L.b200_w8a8_last_error()

    def two_calls():
        st = torch.cuda.current_stream().cuda_stream
        for w in ws:
            rc = L.b200_w8a8_gemm_i8_i32(a8.data_ptr(), w.data_ptr(), pkg.W_SLAB128, acc.data_ptr(), tokens, k, n, st)
            rc |= L.b200_w8a8_qkv_rms_rope_dequant(acc.data_ptr(), sx.data_ptr(), sw.data_ptr(), q.data_ptr(),
                                                   kk.data_ptr(), v.data_ptr(), pos[0].data_ptr(), pos[1].data_ptr(),
                                                   pos[2].data_ptr(), xy.data_ptr(), inv_t.data_ptr(), tokens, n_heads,
                                                   n_kv_heads, d_head, 32, 16, 1e-6, st)
            assert rc == 0, L.b200_w8a8_last_error()

    out = {}
    for name, run in (("fused_us", fused), ("two_call_us", two_calls)):
        with torch.cuda.stream(stream):
            run()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
        with torch.cuda.stream(stream):
            graph.replay()
        ms, _, _ = time_steps(graph.replay, 5, stream, lambda: None)
        out[name] = ms / (5 * N_LAYERS) * 1e3
    out["shape"] = f"T={tokens} K={k} N={n} heads {n_heads}/{n_kv_heads} d_head {d_head}"
    return out


def run_skinny(pkg, stream, peaks, n_weights=72):
    """Config 4: M in {16, 32, 64, 128} rows against K x N int8 weights; a graph-replayed chain of 72 launches
    with 72 distinct weight matrices (1.2 GB, far beyond L2); reports weight bytes per second."""
    import torch
    dev = "cuda"
    out = {}
    for k, n in SKINNY_SHAPES:
        ws = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev) for _ in range(n_weights)]
        sw = torch.rand(n, device=dev) * 1e-3
        for m in (16, 32, 64, 128):
            a8 = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
            sx = torch.rand(m, device=dev) * 1e-2
            y = torch.empty(m, n, dtype=torch.float16, device=dev)

            def run():
                for w in ws:
                    pkg.linear(a8, sx, w, sw, n=n, w_layout=pkg.W_SLAB128, out=y, const_weights=True)
            with torch.cuda.stream(stream):
                run()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                run()
            with torch.cuda.stream(stream):
                graph.replay()
            ms, _, _ = time_steps(graph.replay, 3, stream, lambda: None)
            us = ms / (3 * n_weights) * 1e3
            gbs = (n * k + m * k + 2 * m * n) / us / 1e3
            # the same 72 linears as independent problems of one grouped call (72 problems fit one launch)
            ys = [torch.empty(m, n, dtype=torch.float16, device=dev) for _ in ws]
            probs = [dict(x_i8=a8, x_scales=sx, w_i8=w, w_scales=sw, n=n, out=yy) for w, yy in zip(ws, ys)]
            with torch.cuda.stream(stream):
                pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128, out_dtype=torch.float16, const_weights=True)
            stream.synchronize()
            ggraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(ggraph, stream=stream):
                pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128, out_dtype=torch.float16, const_weights=True)
            with torch.cuda.stream(stream):
                ggraph.replay()
            gms, _, _ = time_steps(ggraph.replay, 3, stream, lambda: None)
            gus = gms / (3 * n_weights) * 1e3
            ggbs = (n * k + m * k + 2 * m * n) / gus / 1e3
            out[f"m{m}_k{k}_n{n}"] = {"us_per_linear": us, "gb_per_s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                      "frac_of_8000": gbs / 8000.0,
                                      "grouped_us_per_linear": gus, "grouped_gb_per_s": ggbs,
                                      "grouped_frac_of_measured_hbm": ggbs / peaks["hbm_gbs"],
                                      "grouped_frac_of_8000": ggbs / 8000.0}
            del ys, probs
        del ws
    return out


if __name__ == "__main__":
    sys.exit(main())
