"""Benchmark of the W8A8 linear stack (the hot path) on B200.

    python bench.py --gpus N --steps K --warmup W            # this library, one JSON line
    python bench.py --impl reference --gpus N --steps K ...  # the CPU reference arm

A step is one denoising pass of the 24-layer linear stack over one batch of synthetic
tokens (the workload of the headline config: M=512 rows, d_model 2048, QKV 6144, MLP 8192,
fp16 activations).  `value` is int8 tera-operations per second over all GPUs with the
tokens already resident in HBM; `e2e` is the same metric through the host-buffer entry
point with the H2D / D2H copies inside the timed region.  With N > 1 every rank runs its
own independent world of the same size (rows shard across GPUs, no collective): weak
scaling, time = max over ranks.

The CPU oracle under oracle/ is used here only by the `cpu_baseline` leg and by
`--impl reference`; nothing measured as the product touches it.
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
NCU_DRAM_BYTES_PER_LAYER_M512 = 69.5e6
WORKLOADS = {
    # name: (rows per GPU, chained steps per bench step, activation dtype, band rows)
    "cfg1": (512, 1, "fp16", 0),
    "cfg2": (2048, 4, "bf16", 0),
    "cfg3": (None, 1, "fp16", 8192),    # 64 worlds x 2048 rows dealt over the ranks (strong scaling)
}
CFG3_WORLDS, CFG3_ROWS_PER_WORLD = 64, 2048
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
# reference arm / CPU baseline: the oracle port on the host cores
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


def small_layer_for_cpu(ref):
    return ref.make_layer(0)


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
    """Times a bounded sample of the headline workload on the host: rows of one layer."""
    import torch
    ref = load_oracle()
    cores = use_all_host_threads()
    lw = small_layer_for_cpu(ref)
    x = ref.make_tokens(512, 0, torch.float16)
    t_probe = cpu_layer_seconds(ref, 32, lw, x)
    rows = int(max(32, min(512, 32 * budget_s / max(t_probe, 1e-3))))
    rows -= rows % 32
    dt = cpu_layer_seconds(ref, rows, lw, x)
    tops = rows * OPS_PER_ROW_LAYER / dt / 1e12
    return {"value": tops, "unit": "TOP/s", "cores": cores, "kind": "port",
            "sample": f"1 of 24 layers of the stack on {rows} of 512 rows, oracle port with the reference's "
                      f"int32 matmul expression, {dt:.2f} s"}


def run_reference_arm(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    ref = load_oracle()
    cores = use_all_host_threads()
    lw = small_layer_for_cpu(ref)
    x = ref.make_tokens(512, 0, torch.float16)
    t_probe = cpu_layer_seconds(ref, 32, lw, x)
    total = max(args.steps + args.warmup, 1)
    per_step_budget = 150.0 / total
    rows = int(max(32, min(512, 32 * per_step_budget / max(t_probe, 1e-3))))
    rows -= rows % 32
    for _ in range(args.warmup):
        cpu_layer_seconds(ref, rows, lw, x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_layer_seconds(ref, rows, lw, x)
    dt = time.perf_counter() - t0
    tops = args.steps * rows * OPS_PER_ROW_LAYER / dt / 1e12
    sample = (f"each step = 1 of 24 layers on {rows} of 512 rows (bounded sample of the cfg1 stack), oracle port "
              f"with the reference's int32 matmul expression on {cores} host threads")
    line = {"impl": "reference", "metric": "w8a8_linear_stack_int8_tops", "value": tops, "unit": "TOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "config": {"workload": "cfg1: 24-layer W8A8 linear stack, M=512, d=2048, qkv 6144, mlp 8192, fp16"},
            "cpu_baseline": {"value": tops, "unit": "TOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tops, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    # Beside the CPU figure: the reference's own CUDA operators on this box's GPU, when they were built.
    try:
        line["reference_cuda_ops_same_gpu"] = (run_reference_cuda_ops() if torch.cuda.is_available()
                                               else {"unavailable": "no CUDA device"})
    except Exception as exc:  # a comparator must never cost the line
        line["reference_cuda_ops_same_gpu"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------
def build_stack(pkg, ref, rows, band_rows, dtype, n_layers=N_LAYERS):
    import torch
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
                pkg.linear(a8, sx, w, sw, n=n, w_layout=pkg.W_SLAB128, residual=residual, act=act, out=out)
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
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-graph", action="store_true", help="launch kernels one by one instead of replaying a graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary configs reported under `extras`")
    ap.add_argument("--layers", type=int, default=N_LAYERS, help="layers of the stack (24 = the real workload)")
    ap.add_argument("--band", type=int, default=-1, help="rows per band (default: the workload's own)")
    ap.add_argument("--lanes", type=int, default=0, help="streams that bands alternate over (default 2 for cfg3)")
    ap.add_argument("--fusion", action="store_true",
                    help="let the linears with d_model outputs emit the next linear's codes from their epilogue "
                         "(six launches per layer instead of ten; measured slower, off by default)")
    ap.add_argument("--only-gemms", type=int, default=0, metavar="ROWS",
                    help="run the five fused linears of one layer at ROWS rows for --steps rounds with distinct "
                         "weights and exit (a small, self-ending case for ncu captures)")
    ap.add_argument("--only-qkv-heads", type=int, default=0, metavar="TOKENS",
                    help="run the QKV linear with the RMSNorm + RoPE epilogue (heads 32/16 x 64) at TOKENS rows for "
                         "--steps rounds with distinct weights and exit (a small case for ncu captures)")
    ap.add_argument("--only-quant", type=int, default=0, metavar="ROWS",
                    help="run the three quantizers of a layer (RMSNorm->A8 of fp16 rows, A8 of the first 2048 of 6144 "
                         "fp16 columns, A8 of 8192 fp32 columns) at ROWS rows for --steps rounds and exit")
    ap.add_argument("--only-grouped", type=int, default=0, metavar="ROWS",
                    help="run one grouped call of 24 skinny linears (ROWS rows each, K=2048, N=8192, distinct weights) "
                         "for --steps rounds and exit (a small case for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

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

    pkg, ref = load_package(), load_oracle()
    pkg.lib()  # raises if the CUDA library is missing
    if args.only_gemms:
        return run_only_gemms(pkg, args.only_gemms, max(args.steps, 1))
    if args.only_qkv_heads:
        return run_only_qkv_heads(pkg, args.only_qkv_heads, max(args.steps, 1))
    if args.only_grouped:
        return run_only_grouped(pkg, args.only_grouped, max(args.steps, 1))
    if args.only_quant:
        return run_only_quant(pkg, args.only_quant, max(args.steps, 1))
    peaks = measured_peaks()
    rows, chained, dt_name, band = WORKLOADS[args.workload]
    sharding = _load("w8a8_sharding", ROOT / "worldmodel.cu_b200" / "sharding.py")
    my_worlds = [rank]  # weak scaling: one independent world per rank, seeded by its global id
    if args.workload == "cfg3":
        my_worlds = sharding.world_seeds(CFG3_WORLDS, world, rank)
        rows = len(my_worlds) * CFG3_ROWS_PER_WORLD
    dtype = torch.float16 if dt_name == "fp16" else torch.bfloat16
    use_graph = not args.no_graph
    if args.band >= 0:
        band = args.band
    lanes = args.lanes if args.lanes > 0 else (2 if args.workload == "cfg3" else 1)

    want_extras = not args.no_extras and world == 1 and args.workload == "cfg1" and args.layers == N_LAYERS
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
    ms, t0, t1 = time_steps(step, args.steps, stream, barrier)
    clocks = sampler.summary(t0, t1)
    if pkg.poll_status() != 0:
        raise SystemExit("a GEMM kernel reported a bounded-wait timeout")
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ops_per_step = rows * OPS_PER_ROW_LAYER * args.layers * chained
    total_rows = rows * world if args.workload != "cfg3" else CFG3_WORLDS * CFG3_ROWS_PER_WORLD
    job_ops_per_step = total_rows * OPS_PER_ROW_LAYER * args.layers * chained
    value = job_ops_per_step * args.steps / (ms * 1e-3) / 1e12
    launches = stack.launches_per_forward * args.steps

    # end to end through the host-buffer entry point (pinned host tokens in, pinned result out)
    xh = x.cpu().pin_memory()
    yh = torch.empty_like(xh).pin_memory()
    for _ in range(3):
        stack.forward_host(xh, yh, steps=chained, use_graph=use_graph)
    barrier()
    torch.cuda.synchronize()
    e0 = time.perf_counter()
    for _ in range(args.steps):
        stack.forward_host(xh, yh, steps=chained, use_graph=use_graph)
    e_ms = (time.perf_counter() - e0) * 1e3
    barrier()
    if world > 1:
        t = torch.tensor([e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e_ms = float(t.item())
    e2e_value = job_ops_per_step * args.steps / (e_ms * 1e-3) / 1e12
    io_bytes = rows * D_MODEL * 2

    if rank != 0:
        sampler.stop()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    # roofline of the dominant kernel (the tcgen05 GEMM), timed per launch with CUDA events
    per_launch = time_gemm_kernels(pkg, rows, stream)
    gemm_ops = rows * OPS_PER_ROW_LAYER
    gemm_s = sum(per_launch.values())
    int8_peak = 2.0 * peaks["bf16_tflops"]  # tcgen05 int8 issues at twice the bf16 rate
    achieved = gemm_ops / gemm_s / 1e12
    weight_gbs = WEIGHT_BYTES_LAYER / gemm_s / 1e9
    # DRAM bytes of the five launches of one layer from the committed ncu capture (profiles/), M=512 only
    traffic = NCU_DRAM_BYTES_PER_LAYER_M512 if rows == 512 else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                "frac": achieved / int8_peak, "traffic": traffic,
                "traffic_note": "dram read+write summed over the five GEMM launches of one layer (ncu, profiles/"
                                "gemm_i8_kernel_layer_m512.md); algorithmic bytes of the same launches: "
                                f"{(WEIGHT_BYTES_LAYER + rows * (4 * D_MODEL + D_HIDDEN) + 3 * rows * D_MODEL * 2) / 1e6:.1f} MB",
                "kernel": "gemm_i8_kernel (tcgen05 s8xs8->s32 + fused epilogue), five linears of a layer",
                "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']}); nominal dense int8 4500",
                "frac_of_nominal_4500": achieved / 4500.0,
                "weight_stream_gbs": weight_gbs, "weight_stream_frac_of_hbm": weight_gbs / peaks["hbm_gbs"],
                "us_per_launch": {k: v * 1e6 for k, v in per_launch.items()}}

    line = {"metric": "w8a8_linear_stack_int8_tops", "value": value, "unit": "TOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if args.workload == "cfg3" else "weak", "vs_baseline": None, "dtype": "s8",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: {args.layers}-layer W8A8 linear stack, M={rows} rows per GPU, "
                                   f"{chained} chained pass(es) per step, d=2048, qkv 6144, mlp 8192, {dt_name}",
                       "rows_per_gpu": rows, "layers": args.layers, "graph_replay": use_graph,
                       "band_rows": band, "lanes": lanes,
                       "l2": "no flush: each step streams 1.31 GB of int8 weights, 10x the 126 MB L2"},
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


def run_only_gemms(pkg, rows, rounds):
    import torch
    dev = "cuda"
    bufs = []
    for name, n, k in LINEARS:
        a8 = torch.randint(-127, 128, (rows, k), dtype=torch.int8, device=dev)
        ws = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev) for _ in range(rounds)]
        sx, sw = torch.rand(rows, device=dev) * 1e-2, torch.rand(n, device=dev) * 1e-3
        out = torch.empty(rows, n, dtype=torch.float32 if name == "up" else torch.float16, device=dev)
        res = torch.randn(rows, n, device=dev).half() if n == D_MODEL else None
        bufs.append((n, a8, ws, sx, sw, out, res, pkg.ACT_GELU_TANH if name == "up" else pkg.ACT_NONE))
    for i in range(rounds):
        for n, a8, ws, sx, sw, out, res, act in bufs:
            pkg.linear(a8, sx, ws[i], sw, n=n, w_layout=pkg.W_SLAB128, residual=res, act=act, out=out,
                       const_weights=True)
    torch.cuda.synchronize()
    print(json.dumps({"only_gemms_rows": rows, "rounds": rounds, "status": pkg.poll_status()}))
    return 0


def run_only_quant(pkg, rows, rounds):
    import torch
    dev = "cuda"
    x = torch.randn(rows, D_MODEL, device=dev).half()
    gamma = 1 + 0.05 * torch.randn(D_MODEL, device=dev)
    qkv = torch.randn(rows, N_QKV, device=dev).half()
    h = torch.randn(rows, D_HIDDEN, device=dev)
    for _ in range(rounds):
        pkg.rms_norm_quantize_rows(x, gamma, None, 1e-6, scale_is_mod=False)
        pkg.quantize_rows(qkv, cols=D_MODEL)
        pkg.quantize_rows(h)
    torch.cuda.synchronize()
    print(json.dumps({"only_quant_rows": rows, "rounds": rounds}))
    return 0


def run_only_grouped(pkg, rows, rounds, k=D_MODEL, n=D_HIDDEN, n_weights=N_LAYERS):
    import torch
    dev = "cuda"
    ws = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev) for _ in range(n_weights)]
    a8 = torch.randint(-127, 128, (rows, k), dtype=torch.int8, device=dev)
    sx, sw = torch.rand(rows, device=dev) * 1e-2, torch.rand(n, device=dev) * 1e-3
    probs = [dict(x_i8=a8, x_scales=sx, w_i8=w, w_scales=sw, n=n,
                  out=torch.empty(rows, n, dtype=torch.float16, device=dev)) for w in ws]
    for _ in range(rounds):
        pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128, out_dtype=torch.float16)
    torch.cuda.synchronize()
    print(json.dumps({"only_grouped_rows": rows, "rounds": rounds, "problems": n_weights, "status": pkg.poll_status()}))
    return 0


def run_only_qkv_heads(pkg, tokens, rounds, n_heads=32, n_kv_heads=16, d_head=64, k=D_MODEL):
    import torch
    dev = "cuda"
    n = (n_heads + 2 * n_kv_heads) * d_head
    g = torch.Generator().manual_seed(7)
    ws = [torch.randint(-127, 128, (n * k,), dtype=torch.int8, device=dev) for _ in range(rounds)]
    a8 = torch.randint(-127, 128, (tokens, k), dtype=torch.int8, device=dev)
    sx, sw = torch.rand(tokens, device=dev) * 1e-2, torch.rand(n, device=dev) * 1e-3
    pos = [torch.randint(0, hi, (tokens,), generator=g).to(dev) for hi in (32, 16, 64)]
    xy = (torch.rand(d_head // 8, generator=g) * 6).to(dev)
    inv_t = torch.rand(d_head // 2 - 2 * (d_head // 8), generator=g).to(dev)
    cos, sin = pkg.rope_tables(*pos, xy, inv_t, d_head, 32, 16)
    for w in ws:
        pkg.linear_qkv_heads(a8, sx, w.view(n, k), sw, cos, sin, n_heads, n_kv_heads, d_head, 1e-6,
                             w_layout=pkg.W_SLAB128)
    torch.cuda.synchronize()
    print(json.dumps({"only_qkv_heads_tokens": tokens, "rounds": rounds, "status": pkg.poll_status()}))
    return 0


def run_extras(pkg, ref, stack, stream, peaks):
    """Secondary configs, each a short run: the chained M=2048 bf16 config, graph vs eager at M=512."""
    import torch
    out = {}
    # config 2: M=2048, 4 chained passes, bf16
    stack.set_dtype(torch.bfloat16)
    x = ref.make_tokens(2048, 0, torch.bfloat16).to("cuda")
    y = torch.empty_like(x)
    fn = lambda: stack.forward(x, y, steps=4, use_graph=True, stream=stream.cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
    ms, _, _ = time_steps(fn, 5, stream, lambda: None)
    ops = 2048 * OPS_PER_ROW_LAYER * N_LAYERS * 4
    tops = ops * 5 / (ms * 1e-3) / 1e12
    out["cfg2_m2048_4steps_bf16"] = {"ms_per_4_steps": ms / 5, "tops": tops,
                                     "frac_of_2x_measured_bf16": tops / (2 * peaks["bf16_tflops"]),
                                     "frac_of_nominal_4500": tops / 4500.0}
    # config 1 without graph replay
    stack.set_dtype(torch.float16)
    x = ref.make_tokens(512, 0, torch.float16).to("cuda")
    y = torch.empty_like(x)
    fn = lambda: stack.forward(x, y, steps=1, use_graph=False, stream=stream.cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(3):
            fn()
    ms, _, _ = time_steps(fn, 20, stream, lambda: None)
    out["cfg1_eager_ms_per_step"] = ms / 20
    out["cfg4_skinny"] = run_skinny(pkg, stream, peaks)
    out["qkv_heads_t512"] = run_qkv_heads(pkg, stream)
    return out


def run_reference_cuda_ops(rows=512, n_heads=32, d_head=64):
    """The reference's own CUDA operators (src/world_cuda_ops.cu compiled into oracle/_ref/, its
    CUTLASS Sm80 mma.sync GEMM included) on this GPU: each of the five GEMM shapes into the int32
    scratch, and the reference's per-layer operator sequence for the linears (norm->A8, GEMM, consumer /
    dequant kernels; attention left out, as in the stack), with 24 distinct weight sets.  Launched one by
    one on the default stream like the reference does (its operators take no stream), timed with events."""
    import torch
    sys.path.insert(0, str(ROOT / "oracle"))
    import ref_cuda_ops as rk
    if not rk.available():
        return {"unavailable": "oracle/_ref/libworld_cuda_ops_ref.so is not built (needs the reference checkout "
                               "and a CUTLASS header tree at build time)"}
    dev = "cuda"
    d, nq, hid = D_MODEL, N_QKV, D_HIDDEN
    g = torch.Generator().manual_seed(11)
    rnd8 = lambda *shape: torch.randint(-127, 128, shape, dtype=torch.int8, device=dev)
    ws = {name: [rnd8(n, k) for _ in range(N_LAYERS)] for name, n, k in LINEARS}
    sw = {name: torch.rand(n, device=dev) * 1e-3 for name, n, k in LINEARS}
    x = torch.randn(rows, d, device=dev)
    x1, x2, x3 = (torch.empty_like(x) for _ in range(3))
    gamma = torch.randn(d, device=dev) * 0.05
    gate = torch.ones(d, device=dev)
    a8 = rnd8(rows, hid)
    sa = torch.rand(rows, device=dev) * 1e-2
    acc = torch.empty(rows, hid, dtype=torch.int32, device=dev)
    n_kv = (nq // d_head - n_heads) // 2
    q = torch.empty(n_heads, rows, d_head, device=dev)
    kk = torch.empty(n_kv, rows, d_head, device=dev)
    v = torch.empty(n_kv, rows, d_head, device=dev)
    pos = [torch.randint(0, hi, (rows,), generator=g).to(dev) for hi in (32, 16, 64)]
    xy = (torch.rand(d_head // 8, generator=g) * 6).to(dev)
    inv_t = torch.rand(d_head // 2 - 2 * (d_head // 8), generator=g).to(dev)

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3  # us

    out = {"gemm_us": {}}
    for name, n, k in LINEARS:
        def gemms(name=name, n=n, k=k):
            for w in ws[name]:
                rk.call("gemm_i8_i32", a8, w, acc, rows, k, n)
        out["gemm_us"][name] = timed(gemms, 3) / N_LAYERS

    def layers():
        for l in range(N_LAYERS):
            rk.call("rms_norm_quantize_rows_i8", x, gamma, None, a8, sa, rows, d, 1e-6)
            rk.call("gemm_i8_i32", a8, ws["qkv"][l], acc, rows, d, nq)
            rk.call("qkv_fused_rms_rope_i32_dequant", acc, sa, sw["qkv"], q, kk, v, *pos, xy, inv_t, rows, n_heads,
                    n_kv, d_head, 32, 16, 1e-6)
            rk.call("quantize_rows_f32_i8", q, a8, sa, rows, d)  # stands in for the attention output [rows, d]
            rk.call("gemm_i8_i32", a8, ws["out"][l], acc, rows, d, d)
            rk.call("dequant_gated_residual_f32", acc, sa, sw["out"], x, gate, x1, rows, d)
            rk.call("rms_norm_quantize_rows_i8", x1, gamma, None, a8, sa, rows, d, 1e-6)
            rk.call("gemm_i8_i32", a8, ws["ctrl"][l], acc, rows, d, d)
            rk.call("dequant_add_residual_f32", acc, sa, sw["ctrl"], x1, x2, rows, d)
            rk.call("rms_norm_quantize_rows_i8", x2, gamma, None, a8, sa, rows, d, 1e-6)
            rk.call("gemm_i8_i32", a8, ws["up"][l], acc, rows, d, hid)
            rk.call("dequant_silu_quantize_rows_i8", acc, sa, sw["up"], None, a8, sa, rows, hid)
            rk.call("gemm_i8_i32", a8, ws["down"][l], acc, rows, hid, d)
            rk.call("dequant_gated_residual_f32", acc, sa, sw["down"], x2, gate, x3, rows, d)
    us = timed(layers, 3)
    out["stack_ms_per_step"] = us / 1e3
    out["stack_tops"] = rows * OPS_PER_ROW_LAYER * N_LAYERS / (us * 1e-6) / 1e12
    out["launches_per_layer"] = 14
    out["note"] = (f"M={rows}, fp32 tokens, SiLU, gated residuals (the reference's operator set); eager launches on the "
                   "default stream, built with the reference's --use_fast_math")
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
            # the same 72 linears as independent problems of one grouped call (two launches of <= 48 problems)
            ys = [torch.empty(m, n, dtype=torch.float16, device=dev) for _ in ws]
            probs = [dict(x_i8=a8, x_scales=sx, w_i8=w, w_scales=sw, n=n, out=yy) for w, yy in zip(ws, ys)]
            with torch.cuda.stream(stream):
                pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128, out_dtype=torch.float16)
            stream.synchronize()
            ggraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(ggraph, stream=stream):
                pkg.linear_grouped(probs, w_layout=pkg.W_SLAB128, out_dtype=torch.float16)
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
