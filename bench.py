#!/usr/bin/env python
"""Benchmark of the NVFP4 linear-layer hot path (activation quantizer + tcgen05 GEMM).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload linear|mlp|sweep|gemv|gemmloop|pushloop] [--M ..] [--N ..] [--K ..]

Default workload: thor_fp4.Linear(8192, 8192, bias=False, out_dtype='bf16') on a
bf16 activation [8192, 8192] ~N(0,1) (M = N = K = 8192, the shape the headline
metric is quoted on); one step = quantize the activation + block-scaled GEMM.
Inputs rotate over buffers larger than L2.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "thor-fp4_b200"))
sys.path.insert(0, str(ROOT))

# The reference arm is CPU work on all host threads.  torchrun exports OMP_NUM_THREADS=1 to its workers when the
# variable is unset, which would pin the BLAS matmul of that arm to one thread: give it the cores before numpy loads.
if "--impl" in sys.argv[1:] and "reference" in sys.argv[1:]:
    try:
        _ncpu = len(os.sched_getaffinity(0))
    except AttributeError:
        _ncpu = os.cpu_count() or 1
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(_ncpu)

import numpy as np  # noqa: E402
import torch  # noqa: E402


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="linear", choices=["linear", "mlp", "sweep", "gemv", "gemmloop", "pushloop"])
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--N", type=int, default=8192)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--inter", type=int, default=28672, help="mlp workload: intermediate size")
    ap.add_argument("--reduce-dtype", default="f32", choices=["f32", "f16", "bf16"],
                    help="mlp workload on several ranks: type of the partial outputs that are all-reduced")
    ap.add_argument("--exchange", default="all_reduce", choices=["all_reduce", "reduce_scatter", "push", "copy"],
                    help="mlp workload on several ranks: how the partial outputs are exchanged")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-mlp", action="store_true", help="skip the SwiGLU-block measurement added to the line")
    ap.add_argument("--graph", action="store_true", help="accepted for older command lines: the captured block is always timed")
    ap.add_argument("--no-graph", action="store_true",
                    help="do not capture the SwiGLU block (with its NCCL all-reduce, and the push form) in a CUDA graph")
    ap.add_argument("--debug-mask", type=int, default=0, help="gemmloop workload: test-hook mask of the GEMM kernel (tfp4_set_debug)")
    ap.add_argument("--ablate", action="store_true",
                    help="time the GEMM with parts of the kernel switched off through the library's test hooks and print a table")
    ap.add_argument("--plain-launch", action="store_true",
                    help="A/B: plain stream order instead of programmatic dependent launches between the kernels")
    ap.add_argument("--profile", action="store_true",
                    help="short run for a profiler: no CPU leg, no end-to-end leg, no sustained-load clock sampling")
    args = ap.parse_args()
    if args.profile:
        args.no_cpu = args.no_e2e = True
    return args


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16": d["bf16_tflops"], "bf16_sustained": d.get("bf16_tflops_sustained"),
                "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU legs
METRIC = "NVFP4 Linear TFLOPS at M=N=K=8192 (% FP4 peak); act-quantize GB/s (% HBM)"
DTYPE = "nvfp4 (e2m1 codes, ue4m3 block scales), f32 accumulate"


class CpuLinear:
    """The reference's CPU emulation of one NVFP4 linear layer (fake-quantize the activation,
    FP32 matmul against the dequantized quantized weight: src/thor_fp4/quant.py:32-53 and
    src/thor_fp4/verify.py:91-100 in the reference project), through the oracle port.  The
    weight is quantized once outside the timed step, as the reference caches it."""

    def __init__(self, N: int, K: int, threads: int):
        from oracle import oracle as orc
        self.orc, self.threads, self.N, self.K = orc, threads, N, K
        rng = np.random.default_rng(0)
        w = (rng.random((N, K), dtype=np.float32) * 2 - 1) * np.float32(1.0 / np.sqrt(K))   # Kaiming-uniform(a=sqrt 5)
        ts = orc.two_level_scale(w)
        p, s = orc.quantize_nvfp4(w, ts, threads)
        self.wd_t = np.ascontiguousarray(orc.dequantize_nvfp4(p, s, ts, N, K, threads).T)
        self.rng = rng

    def make_input(self, M: int):
        x = self.rng.standard_normal((M, self.K), dtype=np.float32)
        return (x.view(np.uint32) & 0xFFFF0000).view(np.float32)      # bf16-representable

    def step(self, x):
        orc = self.orc
        p, s = orc.quantize_nvfp4(x, 1.0, self.threads)
        xd = orc.dequantize_nvfp4(p, s, 1.0, x.shape[0], self.K, self.threads)
        return xd @ self.wd_t


def cpu_baseline(args, sample_rows: int = 8192, budget_s: float = 10.0):
    from oracle import oracle as orc
    threads = orc.host_threads()
    M = min(args.M, sample_rows)
    lin = CpuLinear(args.N, args.K, threads)
    x = lin.make_input(M)
    lin.step(x[:64])
    reps, t0 = 0, time.perf_counter()
    while reps < 1 or (time.perf_counter() - t0 < budget_s and reps < 64):
        lin.step(x)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": 2.0 * M * args.N * args.K / dt / 1e12, "unit": "TFLOPS", "cores": threads, "kind": "port",
            "sample": f"oracle port (C quantize + dequantize, numpy FP32 matmul) on {M} of {args.M} activation rows, "
                      f"N={args.N}, K={args.K}; weight quantized once outside the timed steps; {reps} steps of {dt:.2f} s"}


def run_reference(args):
    """--impl reference: the reference's own CPU emulation of the path on all host threads (oracle port: the
    reference's torch code cannot travel to the GPU box).  Runs exactly --steps timed and --warmup untimed steps
    on all --M activation rows; only when that would take more than about four minutes (a calibration step on
    1024 rows decides) does a step shrink to a slab of the rows, and the line says so."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    threads = orc.host_threads()
    steps, warm = max(1, args.steps), max(0, args.warmup)
    lin = CpuLinear(args.N, args.K, threads)
    probe = lin.make_input(min(args.M, 1024))
    lin.step(probe[:64])
    t0 = time.perf_counter()
    lin.step(probe)
    per_row = (time.perf_counter() - t0) / probe.shape[0]
    budget_rows = int(240.0 / ((steps + warm) * per_row))
    M = args.M if budget_rows >= args.M else max(128, budget_rows // 128 * 128)
    n_in = n_inputs(args) if M == args.M else 2
    xs = [lin.make_input(M) for _ in range(n_in)]      # the same rotation over inputs as the GPU arm
    for i in range(warm):
        lin.step(xs[i % n_in])
    t0 = time.perf_counter()
    for i in range(steps):
        lin.step(xs[i % n_in])
    dt = (time.perf_counter() - t0) / steps
    val = 2.0 * M * args.N * args.K / dt / 1e12
    sample = (f"{M} of {args.M} activation rows per step, oracle port (C quantize + dequantize, numpy FP32 matmul), "
              f"weight quantized once outside the timed steps")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": config_dict(args, args.gpus),
        "cpu_baseline": {"value": val, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ablation(args):
    """GEMM alone on fixed NVFP4 operands with parts of gemm_duo_kernel switched off (tfp4_set_debug masks:
    1 no global stores, 2 no scale stores to tensor memory, 4 no MMAs, 8 no loads, 32 no look-ahead polls)."""
    import thor_fp4
    from thor_fp4 import _ext, ops
    torch.cuda.set_device(0)
    M, N, K = args.M, args.N, args.K
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda") * 0.02
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    L = _ext.device_lib()
    cases = [(0, "full"), (32, "no look-ahead polls"), (1, "no global stores"), (2, "no scale stores to tensor memory"),
             (8, "no loads"), (8 | 2 | 1, "MMAs + barrier protocol only"), (4 | 8 | 2 | 1, "barrier protocol only"), (0, "full again")]
    try:
        for mask, name in cases:
            L.tfp4_set_debug(mask)
            for _ in range(3):
                ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, "bf16")
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, "bf16")
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / args.steps * 1e3
            print(f"| {name} | {mask} | {us:.1f} | {2.0 * M * N * K / us / 1e6:.0f} |", flush=True)
    finally:
        L.tfp4_set_debug(0)
    if _ext.status() != 0:
        raise RuntimeError(f"device status word {_ext.status()}")


def run_sweep(args):
    """--workload sweep: the shape grids of the reference's benchmark configurations as a markdown table
    (layer = activation quantize + GEMM through thor_fp4.Linear; median of 3 rounds of --steps calls)."""
    import thor_fp4
    from thor_fp4 import ops
    torch.cuda.set_device(0)
    torch.manual_seed(0)

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        res = []
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b.record()
            torch.cuda.synchronize()
            res.append(a.elapsed_time(b) / n * 1e3)
        return float(np.median(res))

    def outliers(x, frac, mul):
        k = x.shape[1]
        ch = torch.randperm(k, device=x.device)[: max(1, int(k * frac))]
        x[:, ch] *= mul
        return x

    print("| layer (K -> N) | M | kind | us per call | TFLOPS | weight-stream GB/s | us per CUDA-graph replay |")
    print("|---|---|---|---|---|---|---|")
    grids = [((8192, 8192), [1, 2048, 8192], "bf16", False)]
    grids += [((k, n), [1, 16, 128, 2048, 8192], "f16", True)
              for (k, n) in ((4096, 5120), (5120, 20480), (20480, 5120), (8192, 28672), (28672, 8192))]
    for (K, N), Ms, od, bias in grids:
        lin = thor_fp4.Linear(K, N, bias=bias, out_dtype=od, device="cuda")
        if bias:
            with torch.no_grad():
                lin.bias.normal_(std=0.01)
        lin.refresh_weight()
        for M in Ms:
            x = outliers(torch.randn(M, K, device="cuda"), 0.005, 30.0).bfloat16()
            us = timed(lambda: lin(x), args.steps)
            wbytes = N * K * (0.5 + 1.0 / 16)
            rep = "-"
            if M <= 128:      # the same call replayed from a captured graph: device time without the eager host path
                g = thor_fp4.capture_module(lin, x)
                rep = f"{timed(lambda: g.graph.replay(), args.steps):.1f}"
                del g
            print(f"| {K} -> {N} | {M} | nvfp4 x nvfp4 ({lin.engine_kind}) | {us:.1f} | {2.0 * M * N * K / us / 1e6:.1f} | {wbytes / us / 1e3:.0f} | {rep} |",
                  flush=True)
        del lin
        torch.cuda.empty_cache()
    # the activation quantizer alone over sizes (inputs rotate over > 300 MB)
    for (R, K) in ((2048, 8192), (4096, 8192), (8192, 8192), (16384, 8192), (8192, 28672)):
        n = max(2, int(300e6 / (R * K * 2)) + 1)
        xq = [torch.randn(R, K, device="cuda").bfloat16() for _ in range(n)]
        pq = torch.zeros(ops.packed_bytes(R, K), dtype=torch.uint8, device="cuda")
        sq = torch.zeros(ops.scale_bytes(R, K), dtype=torch.uint8, device="cuda")
        cnt = [0]

        def qstep():
            ops.quantize_nvfp4(xq[cnt[0] % n], 1.0, pq, sq)
            cnt[0] += 1
        us = timed(qstep, args.steps)
        print(f"| quantize bf16 [{R}, {K}] | - | quant_nvfp4_kernel | {us:.1f} | - | {R * K * 2.5625 / us / 1e3:.0f} (algorithmic bytes) |", flush=True)
        if R == 16384:
            # the same shape with a per-tensor scale (a decimal one, whose products with 16-bit inputs land on
            # rounding boundaries, and an arbitrary one), and with FP32 input
            for dt, nm, bpe in ((torch.bfloat16, "bf16", 2.5625), (torch.float32, "f32", 4.5625)):
                xs = xq if dt == torch.bfloat16 else [t.float() for t in xq[:2]]
                for ts in (0.37, 0.3712345):
                    cnt[0] = 0

                    def qstep_ts():
                        ops.quantize_nvfp4(xs[cnt[0] % len(xs)], ts, pq, sq)
                        cnt[0] += 1
                    us = timed(qstep_ts, args.steps)
                    print(f"| quantize {nm} [{R}, {K}] ts={ts} | - | quant_nvfp4_kernel | {us:.1f} | - | {R * K * bpe / us / 1e3:.0f} (algorithmic bytes) |",
                          flush=True)
                # the QAT forward (quantize -> dequantize in one kernel, f32 output) on the same inputs
                yq = torch.empty(R, K, device="cuda")
                cnt[0] = 0

                def fq_step():
                    ops.fake_quantize_nvfp4(xs[cnt[0] % len(xs)], 0.3712345, yq)
                    cnt[0] += 1
                us = timed(fq_step, args.steps)
                print(f"| fake-quantize {nm} [{R}, {K}] ts=0.3712345 | - | fake_quant_nvfp4_kernel | {us:.1f} | - | {R * K * (bpe - 0.5625 + 4) / us / 1e3:.0f} (in + f32 out) |",
                      flush=True)
                del xs, yq
        del xq, pq, sq
        torch.cuda.empty_cache()
    # the MX quantizer (UE8M0 scale per 32 elements) on the activation shapes of the mixed-format path
    for (R, K) in ((4096, 8192), (16384, 8192)):
        n = max(2, int(300e6 / (R * K * 2)) + 1)
        xq = [torch.randn(R, K, device="cuda").bfloat16() for _ in range(n)]
        pq = torch.zeros(ops.mx_packed_bytes(R, K, "mxfp8"), dtype=torch.uint8, device="cuda")
        sq = torch.zeros(ops.mx_scale_bytes(R, K), dtype=torch.uint8, device="cuda")
        cnt = [0]

        def mx_step():
            ops.quantize_mx(xq[cnt[0] % n], "mxfp8", pq, sq)
            cnt[0] += 1
        us = timed(mx_step, args.steps)
        print(f"| quantize_mx mxfp8 bf16 [{R}, {K}] | - | quant_mx_kernel | {us:.1f} | - | {R * K * (2 + 1 + 1 / 32) / us / 1e3:.0f} (algorithmic bytes) |",
              flush=True)
        del xq, pq, sq
        torch.cuda.empty_cache()
    # batch-1 engines: exact-activation GEMV (one launch) against quantize + split-K GEMM
    for (K, N) in ((8192, 8192), (8192, 28672), (28672, 8192)):
        for eng in ("gemv", "cublaslt"):
            lin = thor_fp4.Linear(K, N, bias=False, out_dtype="bf16", device="cuda", engine=eng)
            lin.refresh_weight()
            for M in (1, 4, 8):
                x = torch.randn(M, K, device="cuda").bfloat16()
                us = timed(lambda: lin(x), max(args.steps, 50))
                wbytes = N * K * (0.5 + 1.0 / 16)
                print(f"| {K} -> {N} | {M} | engine={eng} ({lin.engine_kind}) | {us:.1f} | {2.0 * M * N * K / us / 1e6:.1f} | {wbytes / us / 1e3:.0f} |",
                      flush=True)
            del lin
            torch.cuda.empty_cache()
    # MXFP8 activations x MXFP4 weights against NVFP4 x NVFP4 on the same data
    M, K, N = 4096, 8192, 28672
    x = outliers(torch.randn(M, K, device="cuda"), 0.001, 50.0)
    w = torch.randn(N, K, device="cuda") * 0.02
    ref = x @ w.t()
    a8, w4 = thor_fp4.MXTensor.from_float(x, "mxfp8"), thor_fp4.MXTensor.from_float(w, "mxfp4")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    from thor_fp4 import _ext
    vmx = _ext.device_lib().tfc4_variant_index(thor_fp4.linear.resolve_mx8_variant(K).encode())
    us = timed(lambda: ops.gemm_mx(vmx, a8.packed, a8.sblk, w4.packed, w4.sblk, out, M, N, K), args.steps)
    err = ((out.float() - ref).norm() / ref.norm()).item()
    print(f"| {K} -> {N} | {M} | mxfp8 x mxfp4 (GEMM only) | {us:.1f} | {2.0 * M * N * K / us / 1e6:.1f} | rel. error vs fp32 matmul {err:.4f} |")
    an, wn = thor_fp4.NVFP4Tensor.from_float(x, 1.0), thor_fp4.NVFP4Tensor.from_float(w, None)
    us = timed(lambda: ops.gemm(an.packed, an.sblk, 1.0, wn.packed, wn.sblk, wn.tensor_scale, out, M, N, K, "bf16"), args.steps)
    err = ((out.float() - ref).norm() / ref.norm()).item()
    print(f"| {K} -> {N} | {M} | nvfp4 x nvfp4 (GEMM only) | {us:.1f} | {2.0 * M * N * K / us / 1e6:.1f} | rel. error vs fp32 matmul {err:.4f} |")


def run_gemv(args):
    """Exact-activation GEMV engine alone (ops.gemv on a resident NVFP4 weight), M = 1, 2, 4, 8; three weights
    in rotation so that every call streams its weight from HBM (3 x 37.7 MB at 8192 x 8192 stays under the L2
    size only for the smallest layer, stated per row)."""
    import thor_fp4
    from thor_fp4 import ops
    print("| layer (K -> N) | M | input | us per call | weight-stream GB/s | fraction of measured copy |")
    print("|---|---|---|---|---|---|")
    pk = peaks()
    for (K, N) in ((args.K, args.N),) if (args.K, args.N) != (8192, 8192) else ((8192, 8192), (8192, 28672), (28672, 8192)):
        Ws = [thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda") * 0.02) for _ in range(4)]
        for w in Ws:
            w.gemv_scales()
        for M in (1, 2, 4, 8):
            for dt, nm in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
                x = torch.randn(M, K, device="cuda").to(dt)
                out = torch.empty(M, N, device="cuda")
                for w in Ws:
                    ops.gemv(x, w, "f32", out=out)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(args.steps):
                    for w in Ws:
                        ops.gemv(x, w, "f32", out=out)
                b.record()
                torch.cuda.synchronize()
                us = a.elapsed_time(b) * 1e3 / (args.steps * len(Ws))
                gbs = N * K * 0.5625 / us / 1e3
                print(f"| {K} -> {N} | {M} | {nm} | {us:.1f} | {gbs:.0f} | {gbs / pk['hbm_gbs']:.2f} |", flush=True)
        del Ws
        torch.cuda.empty_cache()


def run_mlp(args):
    """--workload mlp: the NVFP4 SwiGLU block (hidden --K, intermediate --inter, --M tokens), tensor-parallel over the
    ranks: gate/up split by rows, down by columns, one all-reduce of the f32 partial outputs per step (strong scaling:
    the block is fixed, each rank holds 1/P of the intermediate dimension)."""
    import torch.distributed as dist
    from thor_fp4 import _ext
    from thor_fp4.parallel import TensorParallelGatedMLP
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    M, H, I = args.M, args.K, args.inter
    torch.manual_seed(1234 + rank)
    tp = TensorParallelGatedMLP(H, I, device=dev, reduce_dtype=args.reduce_dtype if world > 1 else "bf16", weight_std=0.02,
                                exchange=args.exchange)
    tp.local.refresh_weight()
    xs = [torch.randn(M, H, device=dev).bfloat16() for _ in range(2)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for i in range(max(3, args.warmup)):
        tp(xs[i % 2])
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    for i in range(args.steps):
        tp(xs[i % 2])
    b.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if _ext.status() != 0:
        raise RuntimeError(f"device status word {_ext.status()}")
    if rank == 0:
        ms = float(t[0]) / args.steps
        flop = 6.0 * M * H * I
        pk = peaks()
        print(json.dumps({
            "metric": "NVFP4 SwiGLU MLP block TFLOPS (hidden 8192, intermediate 28672, 16384 tokens)", "value": flop / (ms * 1e-3) / 1e12,
            "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": f"NVFP4 gated MLP: x bf16 [{M},{H}] -> quantize -> [Wg;Wu] GEMM ({2 * I // world} rows per rank) with "
                                   f"silu*up + NVFP4 quantize in its epilogue -> Wd GEMM (K = {I // world} per rank) -> "
                                   + (f"{args.reduce_dtype} partials, {tp.exchange_name()}" if world > 1 else "bf16 out"),
                       "tensor_parallel": world, "l2": "activations (268 MB) and weights (396 MB) exceed the 126 MB L2; inputs alternate between two buffers"},
            "per_gpu_frac_of_4x_bf16_burst": flop / world / (ms * 1e-3) / 1e12 / (4.0 * pk["bf16"]),
            "gpu_launches": 3 * args.steps, "clocks": clocks}))
    tp.close()
    if world > 1:
        dist.destroy_process_group()


def profile_traffic(name: str):
    """DRAM bytes per launch of a kernel, as recorded in its committed ncu summary under profiles/ (the line
    'dram_bytes_per_launch: <bytes> (<shape>)'); None when the summary or the line is missing."""
    import re
    f = ROOT / "profiles" / name
    if not f.exists():
        return None
    m = re.search(r"^dram_bytes_per_launch:\s*([0-9.eE+]+)", f.read_text(), re.M)
    return float(m.group(1)) if m else None


def same_box_gpu(xs, w, M, N, K, steps):
    """The reference's own GPU path for the same step on this GPU, outside the product's timed region: its two-kernel
    activation quantizer and its cuBLASLt NVFP4 GEMM (csrc/thor_fp4_core.cu:555-578,697-757 of the reference project,
    compiled unmodified for sm_100a into oracle/_ref by oracle/build_ref.sh), on the same activations and the same
    quantized weight.  A comparison figure only; nothing of it is on the product path."""
    import importlib.util
    from thor_fp4 import ops
    spec = importlib.util.spec_from_file_location("_refgpu", ROOT / "tests" / "refgpu.py")
    refgpu = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(refgpu)
    try:
        L = refgpu.lib()
    except OSError as e:
        return {"unavailable": f"unavailable on this box: {e}"}
    if L is None:
        return {"unavailable": "unavailable on this box: oracle/_ref/libthorfp4_ref_core.so was not shipped"}
    rc = L.tfp4_init(32 << 20)
    if rc != 0:
        return {"unavailable": f"unavailable on this box: reference tfp4_init rc={rc}"}
    dev = xs[0].device
    packed = torch.zeros(L.tfp4_packed_bytes(M, K), dtype=torch.uint8, device=dev)
    sblk = torch.zeros(L.tfp4_scale_bytes(M, K), dtype=torch.uint8, device=dev)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    st = lambda: torch.cuda.current_stream().cuda_stream

    def step(i, ev=None):
        x = xs[i % len(xs)]
        if ev:
            ev[0].record()
        r1 = L.tfp4_quant(x.data_ptr(), M, K, 2, 1.0, packed.data_ptr(), sblk.data_ptr(), st())
        if ev:
            ev[1].record()
        r2 = L.tfp4_gemm(packed.data_ptr(), sblk.data_ptr(), 1.0, w.packed.data_ptr(), w.sblk.data_ptr(),
                         float(w.tensor_scale), out.data_ptr(), M, N, K, 1, st())
        if ev:
            ev[2].record()
        return r1, r2
    r1, r2 = step(0)
    if r1 != 0 or r2 != 0:
        return {"unavailable": f"unavailable on this box: reference tfp4_quant rc={r1}, tfp4_gemm rc={r2}"}
    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    for i in range(steps):
        step(i, evs[i])
    torch.cuda.synchronize()
    q_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in evs]))
    g_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in evs]))
    t_ms = evs[0][0].elapsed_time(evs[-1][2]) / steps

    # the two GEMMs alone, back to back on the same operands: inside its own step the reference's GEMM follows two long
    # memory-bound kernels and finds a cooler, faster-clocked chip than a GEMM that fills most of its step
    def gemm_loop(call):
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            call()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps
    ref_loop = gemm_loop(lambda: L.tfp4_gemm(packed.data_ptr(), sblk.data_ptr(), 1.0, w.packed.data_ptr(), w.sblk.data_ptr(),
                                             float(w.tensor_scale), out.data_ptr(), M, N, K, 1, st()))
    out2 = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    ours_loop = gemm_loop(lambda: ops.gemm(packed, sblk, 1.0, w.packed, w.sblk, w.tensor_scale, out2, M, N, K, "bf16"))
    same_bits = bool(torch.equal(out, out2))
    return {"source": "the reference's csrc/thor_fp4_core.cu compiled for sm_100a (oracle/_ref): tfp4_quant (two kernels) + "
                      "tfp4_gemm (cuBLASLt NVFP4), same activations and quantized weight, same GPU, after the timed region",
            "steps": steps, "ms_per_step": t_ms, "step_tflops": 2.0 * M * N * K / (t_ms * 1e-3) / 1e12,
            "gemm_ms": g_ms, "gemm_tflops": 2.0 * M * N * K / (g_ms * 1e-3) / 1e12,
            "quant_ms": q_ms, "quant_gbs": M * K * (2 + 0.5 + 1.0 / 16) / (q_ms * 1e-3) / 1e9,
            "gemm_back_to_back": {"launches": steps, "reference_ms": ref_loop, "ours_ms": ours_loop,
                                  "outputs_bit_identical": same_bits,
                                  "note": "each GEMM alone in a loop on the reference quantizer's codes and scales"}}


def measure_mlp_block(args, dev, rank, world, steps):
    """BASELINE configuration 5 on the ranks of this run: the NVFP4 SwiGLU block (hidden 8192, intermediate 28672,
    16384 tokens, weights ~N(0, 0.02)), gate/up split by rows and down by columns over the ranks, one exchange of
    the partial outputs per block.  Every rank builds the same full weights from one seed and keeps its shard, so
    rank 0 can compare the sharded result with the unsharded block on the same input.  Device-timed, max over ranks."""
    import torch.distributed as dist
    from thor_fp4 import _ext
    from thor_fp4.fused import NVFP4GatedMLP
    from thor_fp4.parallel import TensorParallelGatedMLP
    M, H, I = 16384, 8192, args.inter
    g = torch.Generator(device=dev).manual_seed(4321)
    wg = torch.randn(I, H, device=dev, generator=g) * 0.02
    wu = torch.randn(I, H, device=dev, generator=g) * 0.02
    wd = torch.randn(H, I, device=dev, generator=g) * 0.02
    xs = [torch.randn(M, H, device=dev, generator=g).bfloat16() for _ in range(2)]
    reduce_dtype = args.reduce_dtype if world > 1 else "bf16"
    tp = TensorParallelGatedMLP(H, I, device=dev, reduce_dtype=reduce_dtype, weight_std=0.02)
    tp.load_full_weights(wg, wu, wd)
    tp.local.refresh_weight()
    err = None
    if rank == 0:
        full = NVFP4GatedMLP(H, I, device=dev, out_dtype="f32" if world > 1 else "bf16", weight_std=0.02)
        with torch.no_grad():
            full.w_gate.copy_(wg); full.w_up.copy_(wu); full.w_down.copy_(wd)
        ref = full(xs[0][:1024]).float().clone()
        del full
    del wg, wu, wd
    torch.cuda.empty_cache()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        for i in range(3):
            fn(i)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            fn(i)
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b) / n], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])
    y = tp(xs[0])
    torch.cuda.synchronize()
    if rank == 0:
        got = y[:1024].float()
        err = float((got - ref).norm() / ref.norm())
    ms = timed(lambda i: tp(xs[i % 2]), steps)
    ms_local = timed(lambda i: tp.local(xs[i % 2]), steps)          # the rank's GEMMs alone, nothing exchanged
    ms_xchg = None
    scatter = push = copy = None
    if world > 1:
        buf = torch.zeros(M, H, dtype={"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[reduce_dtype], device=dev)
        ms_xchg = timed(lambda i: dist.all_reduce(buf), steps)          # the exchange alone (NCCL all-reduce of the partials)
        del buf
        # the same block with the partial outputs reduce-scattered by token rows (each rank keeps M/P summed rows)
        name_ar = tp.exchange_name()
        tp.exchange = "reduce_scatter"
        ys = tp(xs[0])
        torch.cuda.synchronize()
        err_rs = None
        if rank == 0:
            rows = tp.owned_rows(M)
            rows = rows[rows < 1024].to(dev)
            err_rs = float((ys[: rows.numel()].float() - ref[rows]).norm() / ref[rows].norm()) if rows.numel() else None
        ms_rs = timed(lambda i: tp(xs[i % 2]), steps)
        scatter = {"exchange": tp.exchange_name(), "ms_per_block": ms_rs, "tflops": 6.0 * M * H * I / (ms_rs * 1e-3) / 1e12,
                   "rel_error_vs_unsharded_block": err_rs,
                   "note": "every rank ends with its M/P token rows of the output, fully summed"}
        # and with the transfer inside the down projection (TMA stores into the owners' staging buffers, local sum)
        tp.exchange = "push"
        try:
            yp = tp(xs[0])          # the set-up (CUDA IPC) succeeds or fails on all ranks together
            torch.cuda.synchronize()
            err_p = None
            if rank == 0:
                err_p = float((yp[:1024].float() - ref).norm() / ref.norm())
            ms_p = timed(lambda i: tp(xs[i % 2]), steps)
            push = {"exchange": tp.exchange_name(), "ms_per_block": ms_p, "tflops": 6.0 * M * H * I / (ms_p * 1e-3) / 1e12,
                    "rel_error_vs_unsharded_block": err_p,
                    "nvlink_bytes_sent_per_rank": (world - 1) * (M // world) * H * (4 if reduce_dtype == "f32" else 2)}
            if reduce_dtype == "f32":
                # the same exchange with 16-bit partials: half the bytes over NVLink, each partial rounded once before the
                # sum (f16: 2^-12 relative, needs the partials inside the f16 range; bf16: 2^-9)
                for pd in ("f16", "bf16"):
                    tp.local.out_dtype = pd
                    try:
                        yb = tp(xs[0])
                        torch.cuda.synchronize()
                        err_b = float((yb[:1024].float() - ref).norm() / ref.norm()) if rank == 0 else None
                        ms_b = timed(lambda i: tp(xs[i % 2]), steps)
                        push[pd + "_partials"] = {"ms_per_block": ms_b, "tflops": 6.0 * M * H * I / (ms_b * 1e-3) / 1e12,
                                                  "rel_error_vs_unsharded_block": err_b,
                                                  "nvlink_bytes_sent_per_rank": (world - 1) * (M // world) * H * 2}
                    finally:
                        tp.local.out_dtype = "f32"
        except RuntimeError as e:
            push = {"unavailable": str(e)[:300]}
        tp.close()
        # and with the transfer on the copy engines beside the next token chunk's GEMMs
        tp.exchange = "copy"
        try:
            yc = tp(xs[0])
            torch.cuda.synchronize()
            err_c = None
            if rank == 0:
                rows = tp.owned_rows(M)
                rows = rows[rows < 1024].to(dev)
                err_c = float((yc[: rows.numel()].float() - ref[rows]).norm() / ref[rows].norm()) if rows.numel() else None
            ms_c = timed(lambda i: tp(xs[i % 2]), steps)
            copy = {"exchange": tp.exchange_name(), "ms_per_block": ms_c, "tflops": 6.0 * M * H * I / (ms_c * 1e-3) / 1e12,
                    "rel_error_vs_unsharded_block": err_c}
        except RuntimeError as e:
            copy = {"unavailable": str(e)[:300]}
        tp.close()
        tp.exchange = "all_reduce"
    # the per-rank block captured in a CUDA graph and replayed (the form the benchmark configuration names): one rank
    # -> the three kernels; several ranks -> the block with its NCCL all-reduce (the configuration's own form) and the
    # push form, whose staging set alternates from call to call: two blocks in a row are captured, so that a replay
    # leaves the alternation where it found it
    graph = None
    if not args.no_graph:
        def capture(exchange, blocks):
            tp.exchange = exchange
            xg = xs[0].clone()
            for _ in range(2):
                tp(xg)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(blocks):
                    yg = tp(xg)
            ms_g = timed(lambda i: g.replay(), steps) / blocks
            name = tp.exchange_name() if world > 1 else None
            del g, yg
            return {"exchange": name, "ms_per_block": ms_g, "tflops": 6.0 * M * H * I / (ms_g * 1e-3) / 1e12,
                    "blocks_per_graph": blocks}
        try:
            if world == 1:
                graph = capture("all_reduce", 1)
            else:
                graph = capture("all_reduce", 1)
                try:
                    graph["push"] = capture("push", 2)
                    torch.cuda.synchronize()
                    if dist.is_initialized():
                        dist.barrier()
                    tp.close()
                except Exception as e:  # noqa: BLE001
                    graph["push"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        except Exception as e:  # noqa: BLE001
            graph = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        tp.exchange = "all_reduce"
    if _ext.status() != 0:
        raise RuntimeError(f"device status word {_ext.status()}")
    flop = 6.0 * M * H * I
    res = {"workload": f"NVFP4 SwiGLU block, hidden {H}, intermediate {I}, {M} tokens bf16, weights ~N(0,0.02); gate/up "
                       f"rows and down columns split over {world} rank(s)",
           "tensor_parallel": world, "scaling": "strong", "steps": steps, "ms_per_block": ms,
           "tflops": flop / (ms * 1e-3) / 1e12, "ms_local_gemms_only": ms_local,
           "exchange": name_ar if world > 1 else None, "reduce_dtype": reduce_dtype if world > 1 else None,
           "ms_exchange_alone": ms_xchg,
           "exchange_share": (None if world == 1 else max(0.0, 1.0 - ms_local / ms)),
           "rel_error_vs_unsharded_block": err,
           "reduce_scatter": scatter, "push": push, "copy": copy, "cuda_graph": graph,
           "fused_epilogue": bool(getattr(tp.local, "fuse_epilogue", False))}
    del tp, xs
    torch.cuda.empty_cache()
    return res


def run_gemmloop(args):
    """--workload gemmloop: the NVFP4 GEMM alone on fixed operands (--M/--N/--K, bf16 out; --debug-mask switches parts
    of the kernel off through the library's test hooks), timed two ways: bursts of 20 launches after a pause (the clock
    the power cap allows a short run) and a seconds-long loop (the last 1000 of 4000 launches)."""
    import thor_fp4
    from thor_fp4 import _ext, ops
    M, N, K = args.M, args.N, args.K
    L = _ext.core()
    torch.manual_seed(0)
    a = thor_fp4.NVFP4Tensor.from_float(torch.randn(M, K, device="cuda"), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda") * 0.02, None)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    call = lambda: ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, "bf16")

    def loop(n_warm, n):
        for _ in range(n_warm):
            call()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            call()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3
    L.tfp4_set_debug(args.debug_mask)
    try:
        bursts = []
        for _ in range(3):
            time.sleep(0.5)
            bursts.append(loop(3, 20))
        sustained = loop(3000, 1000)
    finally:
        L.tfp4_set_debug(0)
        L.tfp4_clear_status()
    print(json.dumps({"workload": f"NVFP4 GEMM {M} x {N} x {K}, bf16 out, fixed operands", "debug_mask": args.debug_mask,
                      "burst_of_20_us": [round(t, 2) for t in bursts], "sustained_us": round(sustained, 2),
                      "burst_tflops": 2.0 * M * N * K / (min(bursts) * 1e-6) / 1e12}))


def run_pushloop(args):
    """--workload pushloop (under torchrun, one rank per GPU): the push GEMM alone - 16384 tokens x 8192 features, K = --K
    per rank, partial rows stored into the owning ranks' staging buffers - for f32, f16 and bf16 partials, beside the same
    GEMM with a local output; max over ranks, NVLink bytes leaving a rank per second."""
    import torch.distributed as dist
    import thor_fp4
    from thor_fp4 import _ext, ops
    from thor_fp4.parallel import _PushStaging
    rank, local, world = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    L = _ext.device_lib()
    M, H, I = 16384, 8192, (args.K if args.K != 8192 else 28672 // world)
    torch.manual_seed(rank)
    a = thor_fp4.NVFP4Tensor.from_float(torch.randn(M, I, device=dev), 1.0)
    w = thor_fp4.NVFP4Tensor.from_float(torch.randn(H, I, device=dev) * 0.02, None)

    def timed(fn, n=10):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])
    res = {"workload": f"push GEMM {M} x {H} x {I} per rank, {world} ranks"}
    rows = M // world
    for od, dt in (("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)):
        out = torch.empty(M, H, dtype=dt, device=dev)
        ms_local = timed(lambda: ops.gemm(a.packed, a.sblk, 1.0, w.packed, w.sblk, w.tensor_scale, out, M, H, I, od))
        stg = _PushStaging(None, world, rank, rows, H, dt, dev)

        def push():
            rc = L.tfp4_gemm_push(a.packed.data_ptr(), a.sblk.data_ptr(), 1.0, w.packed.data_ptr(), w.sblk.data_ptr(),
                                  float(w.tensor_scale), stg.dest[0], world, rows, (rank + 1) % world, M, H, I,
                                  _ext.OUT_DTYPE[od], _ext.stream())
            assert rc == 0
        ms_push = timed(push)
        ys = torch.empty(rows, H, dtype=dt, device=dev)
        ms_sum = timed(lambda: L.tfp4_sum_slots(stg.local_set[0], world, rows, H, _ext.IN_DTYPE[dt], ys.data_ptr(),
                                                _ext.OUT_DTYPE[od], _ext.stream()))
        sent = (world - 1) * rows * H * (4 if od == "f32" else 2)
        res[od] = {"ms_local_output": ms_local, "ms_push": ms_push, "ms_sum_slots": ms_sum,
                   "nvlink_gbs_out_per_rank": sent / (ms_push * 1e-3) / 1e9}
        torch.cuda.synchronize()
        dist.barrier()
        stg.close()
        del out, ys
    if rank == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


def n_inputs(args):
    """Input buffers a run rotates over so that together they exceed the 126 MB L2 (> 256 MB of bf16 activations)."""
    return max(2, int(np.ceil(300e6 / (args.M * args.K * 2))))


def config_dict(args, world):
    return {"workload": workload_name(args), "replicas": world,
            "l2": f"inputs rotate over {n_inputs(args)} buffers of {args.M * args.K * 2 / 1e6:.0f} MB (> 126 MB L2)"}


def workload_name(args):
    return (f"thor_fp4.Linear({args.K},{args.N},bias=False,out_dtype=bf16), activation bf16 [{args.M},{args.K}] ~N(0,1), "
            "weight Kaiming-uniform fp32 quantized once (two-level NVFP4); step = activation quantize + block-scaled GEMM")


# --------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch.distributed as dist
    import thor_fp4
    from thor_fp4 import _ext, ops

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=4))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    M, N, K = args.M, args.N, args.K
    pk = peaks()
    torch.manual_seed(1234 + rank)
    lin = thor_fp4.Linear(K, N, bias=False, out_dtype="bf16").to(dev)
    lin.refresh_weight()
    w = lin._weight_fp4
    # inputs larger than L2 (126 MB): rotate over buffers totalling > 256 MB
    n_in = n_inputs(args)
    xs = [torch.randn(M, K, device=dev).bfloat16() for _ in range(n_in)]
    packed = torch.zeros(ops.packed_bytes(M, K), dtype=torch.uint8, device=dev)
    sblk = torch.zeros(ops.scale_bytes(M, K), dtype=torch.uint8, device=dev)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

    def step(i, ev=None):
        x = xs[i % n_in]
        if ev is not None:
            ev[0].record()
        ops.quantize_nvfp4(x, 1.0, packed, sblk)
        if ev is not None:
            ev[1].record()
        ops.gemm(packed, sblk, 1.0, w.packed, w.sblk, w.tensor_scale, out, M, N, K, "bf16")
        if ev is not None:
            ev[2].record()

    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # per-kernel events on every fourth timed step: an event between the two launches of a step turns their
    # programmatic dependent launch into plain stream order, so the other steps run as the library chains them
    ev_every = 4 if args.steps >= 8 else 1
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] if i % ev_every == 0 else None
           for i in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record()
    for i in range(args.steps):
        step(i, evs[i])
    t_end.record()
    barrier()
    total_ms = t_begin.elapsed_time(t_end)
    # the timed region lasts a few milliseconds, less than one nvidia-smi sample: keep the identical
    # step running (untimed) until the sampler has seen about half a second of this load
    t_load = time.perf_counter()
    i = args.steps
    while not args.profile and time.perf_counter() - t_load < 0.5:
        for _ in range(20):
            step(i)
            i += 1
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["note"] = "sampled every 20 ms during the timed steps and 0.5 s more of the same step"
    q_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in evs if e is not None]))
    g_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in evs if e is not None]))
    if _ext.status() != 0:
        raise RuntimeError(f"device status word {_ext.status()}: a GEMM wait expired")

    # ---------------- what a plain device copy reaches in the quantizer's place: the same loop with the quantizer
    # replaced by a copy that moves the quantizer's algorithmic bytes (half read, half written), right behind the GEMM,
    # i.e. at the SM / L2 clock the power cap leaves after it and with the GEMM's output lines still dirty in L2
    in_step_copy = None
    if not args.profile:
        q_bytes_i = int(M * K * (2 + 0.5 + 1.0 / 16))
        half = (q_bytes_i // 2 + 255) // 256 * 256
        srcs = [xs[j].view(torch.uint8).reshape(-1)[:half] for j in range(min(n_in, 3))]
        dstc = torch.empty(half, dtype=torch.uint8, device=dev)
        n_c = max(8, min(args.steps, 40))
        cev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_c)]
        for i in range(3 + n_c):
            if i >= 3:
                cev[i - 3][0].record()
            dstc.copy_(srcs[i % len(srcs)])
            if i >= 3:
                cev[i - 3][1].record()
            ops.gemm(packed, sblk, 1.0, w.packed, w.sblk, w.tensor_scale, out, M, N, K, "bf16")
        torch.cuda.synchronize()
        c_ms = float(np.mean([a.elapsed_time(b) for a, b in cev]))
        in_step_copy = {"bytes_moved": 2 * half, "avg_ms": c_ms, "gbs": 2 * half / (c_ms * 1e-3) / 1e9,
                        "note": "torch copy_ of half the quantizer's algorithmic bytes (read + write = the same total) timed "
                                "between the GEMMs of the same loop"}
        del dstc, srcs

    # ---------------- the activation quantizer alone on [16384, 8192] bf16 (the larger of the metric's two shapes)
    q_large = None
    if not args.profile:
        RL, KL = 16384, 8192
        xl = [torch.randn(RL, KL, device=dev).bfloat16() for _ in range(2)]     # 2 x 268 MB > L2
        pl_ = torch.zeros(ops.packed_bytes(RL, KL), dtype=torch.uint8, device=dev)
        sl_ = torch.zeros(ops.scale_bytes(RL, KL), dtype=torch.uint8, device=dev)
        for i in range(3):
            ops.quantize_nvfp4(xl[i % 2], 1.0, pl_, sl_)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_q = max(10, args.steps)
        a.record()
        for i in range(n_q):
            ops.quantize_nvfp4(xl[i % 2], 1.0, pl_, sl_)
        b.record()
        torch.cuda.synchronize()
        ql_ms = a.elapsed_time(b) / n_q
        ql_bytes = RL * KL * (2 + 0.5 + 1.0 / 16)
        q_large = {"shape": [RL, KL], "in_dtype": "bf16", "avg_launch_ms": ql_ms, "achieved": ql_bytes / (ql_ms * 1e-3) / 1e9,
                   "unit": "GB/s", "algorithmic_bytes_per_launch": ql_bytes}
        del xl, pl_, sl_

    # ---------------- end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        hx = [torch.randn(M, K).bfloat16().pin_memory() for _ in range(2)]
        hy = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        dx = [torch.empty(M, K, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        dy = [torch.empty(M, N, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        # as many steps as the device-timed region (at most 50): the pipeline's fill and drain - one upload and one download
        # that overlap nothing - are part of the timed region and weigh 1/n of a transfer each
        n_e2e = max(4, min(args.steps, 50))
        # Every step copies its input from pinned host memory and its result back; the copies of neighbouring steps
        # run on their own streams (PCIe is full duplex), so a step costs the slowest of upload, layer and download.
        main, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def e2e_step(i):
            k = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_done[k])          # the layer of step i-2 has consumed this input buffer
                dx[k].copy_(hx[k], non_blocking=True)
                ev_in[k].record(s_in)
            main.wait_event(ev_in[k])
            if i >= 2:
                main.wait_event(ev_out[k])               # the download of step i-2 has left this result buffer
            dy[k].copy_(lin(dx[k]))                      # the layer returns its reused buffer: keep a copy for the download
            ev_done[k].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[k])
                hy[k].copy_(dy[k], non_blocking=True)
                ev_out[k].record(s_out)

        def e2e_drain():
            main.wait_stream(s_in)
            main.wait_stream(s_out)
        for i in range(2):
            e2e_step(i)
        e2e_drain()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n_e2e):
            e2e_step(i + 2)
        e2e_drain()
        b.record()
        barrier()
        e2e_ms = a.elapsed_time(b) / n_e2e
    else:
        e2e_ms = None

    # ---------------- the reference's own GPU kernels on this GPU, same operands (rank 0, outside every timed region)
    same_box = None
    if rank == 0 and not args.profile:
        same_box = same_box_gpu(xs, w, M, N, K, max(5, min(args.steps, 20)))
    barrier()
    # ---------------- the sharded configuration (SwiGLU block over the ranks of this run)
    mlp = None
    if not args.profile and not args.no_mlp:
        del xs, packed, sblk, out
        torch.cuda.empty_cache()
        mlp = measure_mlp_block(args, dev, rank, world, max(3, min(args.steps, 10)))

    t = torch.tensor([total_ms, e2e_ms or 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_max = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_step = total_ms / args.steps
    flop = 2.0 * M * N * K
    value = world * flop / (ms_step * 1e-3) / 1e12
    gemm_tflops = flop / (g_ms * 1e-3) / 1e12
    q_bytes = M * K * (2 + 0.5 + 1.0 / 16)
    q_gbs = q_bytes / (q_ms * 1e-3) / 1e9
    fp4_peak = 4.0 * pk["bf16"]
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": config_dict(args, world),
        "roofline": {"bound": "tensor", "kernel": "gemm_duo_kernel (tcgen05 cta_group::2 NVFP4 block-scaled GEMM, 256x256 tiles)",
                     "achieved": gemm_tflops, "peak": fp4_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp4_peak,
                     "peak_note": f"4 x {pk['src']} bf16 burst ({pk['bf16']}); no FP4 peak is measured on this pool",
                     "frac_of_nominal_9000": gemm_tflops / 9000.0,
                     # dram__bytes_read + dram__bytes_write of one launch at 8192^3, read from the committed ncu summary
                     "traffic": profile_traffic("gemm_duo_kernel_8192.md") if (M, N, K) == (8192, 8192, 8192) else None,
                     "avg_launch_ms": g_ms},
        "roofline_quantizer": {"bound": "hbm", "kernel": "quant_nvfp4_kernel", "achieved": q_gbs,
                               "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": q_gbs / pk["hbm_gbs"],
                               "peak_note": f"{pk['src']} copy bandwidth",
                               # one ncu capture of this kernel on [8192, 8192] bf16, read from the committed summary
                               "traffic": profile_traffic("quant_nvfp4_kernel.md") if (args.M, args.K) == (8192, 8192) else None,
                               "avg_launch_ms": q_ms,
                               "algorithmic_bytes_per_launch": q_bytes,
                               "note": "inside the step, on [8192, 8192]; 'alone_large' is the same kernel timed alone on [16384, 8192]",
                               "alone_large": (dict(q_large, frac=q_large["achieved"] / pk["hbm_gbs"]) if q_large else None),
                               "in_step_copy": (dict(in_step_copy, quantizer_vs_copy=q_gbs / in_step_copy["gbs"])
                                                if in_step_copy else None)},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
    }
    if e2e_ms is not None:
        line["e2e"] = {"value": world * flop / (e2e_max * 1e-3) / 1e12, "unit": "TFLOPS",
                       "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                       "ms_per_step": e2e_max,
                       "api": "thor_fp4.Linear.forward, pinned host buffers; upload, layer and download of neighbouring steps overlap on three streams"}
    if same_box is not None:
        same_box["ours_gemm_ms"], same_box["ours_quant_ms"], same_box["ours_ms_per_step"] = g_ms, q_ms, ms_step
        line["same_box_gpu"] = same_box
    if mlp is not None:
        line["tp_mlp"] = mlp
    if not args.no_cpu and world == 1:      # the CPU baseline is a single-GPU-run item
        line["cpu_baseline"] = cpu_baseline(args)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the engine has no CPU fallback (use --impl reference for the CPU arm)")
    if args.plain_launch:
        from thor_fp4 import _ext
        _ext.core().tfp4_set_dependent_launch(0)
    if args.ablate:
        run_ablation(args)
        return
    if args.workload == "sweep":
        run_sweep(args)
        return
    if args.workload == "gemv":
        run_gemv(args)
        return
    if args.workload == "gemmloop":
        run_gemmloop(args)
        return
    if args.workload == "pushloop":
        run_pushloop(args)
        return
    if args.workload == "mlp":
        if args.M == 8192 and args.K == 8192 and args.N == 8192:
            args.M = 16384          # the block's own default batch
        run_mlp(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
