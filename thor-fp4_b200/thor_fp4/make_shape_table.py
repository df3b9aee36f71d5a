"""Regenerate shape_table.json for the GPU this runs on: per (N, K) layer shape and batch size, the time
of the NVFP4 layer call (activation quantize + GEMM through thor_fp4.Linear) against torch's bf16
F.linear, which is what convert(policy="auto") weighs.  Method after the reference's
benchmarks/bench_gemm.py:110-167: one second of warm-up, CUDA events, median of 5 rounds of 20 calls,
the two candidates alternating.

usage: python thor-fp4_b200/thor_fp4/make_shape_table.py [out.json]   (default: the package's shape_table.json)
"""
import json
import statistics
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import thor_fp4  # noqa: E402

SHAPES = [(256, 256), (512, 512), (1024, 1024), (1280, 1280), (2048, 2048), (4096, 4096), (8192, 8192),
          (5120, 4096), (20480, 5120), (5120, 20480), (28672, 8192), (8192, 28672)]     # (N, K)
BATCHES = [1, 16, 128, 4096]


def _time(fn, rounds=5, iters=20):
    res = []
    for _ in range(rounds):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        res.append(a.elapsed_time(b) / iters)
    return statistics.median(res)


def main():
    out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("shape_table.json")
    dev = torch.device("cuda")
    t0 = time.perf_counter()
    spin = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
    while time.perf_counter() - t0 < 1.0:       # clocks up
        spin @ spin
    torch.cuda.synchronize()
    shapes = {}
    for N, K in SHAPES:
        lin = thor_fp4.Linear(K, N, bias=False, out_dtype="bf16", device=dev)
        lin.refresh_weight()
        wb = lin.weight.detach().to(torch.bfloat16)
        rows = {}
        for M in BATCHES:
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            for _ in range(3):
                lin(x)
                torch.nn.functional.linear(x, wb)
            fp4 = _time(lambda: lin(x))
            bf = _time(lambda: torch.nn.functional.linear(x, wb))
            rows[str(M)] = {"fp4_ms": round(fp4, 5), "bf16_ms": round(bf, 5), "fp4_wins": bool(fp4 < bf)}
            print(f"N={N:6d} K={K:6d} M={M:5d}: fp4 {fp4 * 1e3:8.1f} us   bf16 {bf * 1e3:8.1f} us   {'fp4' if fp4 < bf else 'bf16'}",
                  flush=True)
        shapes[f"{N}x{K}"] = rows
        del lin, wb
        torch.cuda.empty_cache()
    # crossover: the smallest square shape from which FP4 wins at the table's decision batch (4096)
    squares = sorted((int(k.split("x")[0]) for k in shapes if k.split("x")[0] == k.split("x")[1]))
    cross = squares[-1]
    for n in reversed(squares):
        if shapes[f"{n}x{n}"]["4096"]["fp4_wins"]:
            cross = n
        else:
            break
    table = {
        "_comment": "Per-shape FP4-vs-BF16 decisions for convert(policy='auto'): keys \"<N>x<K>\", one row per batch size with "
                    "the layer-call times in ms (activation quantize included); decisions are taken at batch 4096. "
                    f"Measured with make_shape_table.py on {torch.cuda.get_device_name(0)}.",
        "crossover": {"min_k": cross, "min_n": cross},
        "shapes": shapes,
    }
    out_path.write_text(json.dumps(table, indent=1) + "\n")
    print(f"wrote {out_path} (crossover {cross})")


if __name__ == "__main__":
    main()
