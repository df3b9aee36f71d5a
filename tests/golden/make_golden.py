"""Generate tests/golden/ref_fakequant.npz from the reference's own Python code.

Runs on CPU in a container that has the thor-fp4 checkout; imports the
reference's torch fake quantizers (src/thor_fp4/quant.py:25-81) and records, for
seeded inputs shaped after the reference's own quantizer tests
(tests/test_quant.py:13-61) and after the benchmark configurations, the inputs
and the values the reference returns.  The CPU oracle and the CUDA library are
then checked against these vectors without the reference being present.

usage: python tests/golden/make_golden.py [reference-checkout]   (default: $THOR_FP4_REFERENCE)
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch

# the checkout: first argument, else THOR_FP4_REFERENCE, else a directory `reference` beside this repository
ref = Path(sys.argv[1] if len(sys.argv) > 1
           else os.environ.get("THOR_FP4_REFERENCE", str(Path(__file__).resolve().parents[3] / "reference")))
sys.path.insert(0, str(ref / "src"))
from thor_fp4.quant import mx_fake_quant, nvfp4_fake_quant, two_level_scale  # noqa: E402

out = {}
torch.manual_seed(0)

# tests/test_quant.py:13-22 -- randn * linspace(0.001, 3, K), block-only and two-level
for K in (320, 1024, 2048):
    x = torch.randn(8, K) * torch.linspace(0.001, 3, K)
    out[f"nv_K{K}_x"] = x.numpy()
    out[f"nv_K{K}_block_ts"] = np.float64(1.0)
    out[f"nv_K{K}_block_y"] = nvfp4_fake_quant(x, 1.0).numpy()
    ts = two_level_scale(x)
    out[f"nv_K{K}_two_ts"] = np.float64(ts)
    out[f"nv_K{K}_two_y"] = nvfp4_fake_quant(x, ts).numpy()

# tests/test_quant.py:25-32 -- all-zero blocks
x = torch.zeros(8, 128)
x[:, :64] = torch.randn(8, 64)
out["nv_zero_x"] = x.numpy()
out["nv_zero_y"] = nvfp4_fake_quant(x).numpy()

# tests/test_quant.py:35-42 -- 16-bit inputs (stored as raw bit patterns)
for name, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
    x = torch.randn(16, 256).to(dt)
    out[f"nv_{name}_xbits"] = x.view(torch.int16).numpy().view(np.uint16)
    out[f"nv_{name}_y"] = nvfp4_fake_quant(x.float()).numpy()

# tests/test_quant.py:51-61 -- known-answer tie vector
x = torch.zeros(1, 64)
x[0, :4] = torch.tensor([0.25, 0.6, 2.6, -6.0])
out["nv_tie_x"] = x.numpy()
out["nv_tie_y"] = nvfp4_fake_quant(x).numpy()

# wide dynamic range + outlier channels (benchmark configuration 3: 0.5 % of K channels x30)
x = torch.randn(8, 4096)
ch = torch.randperm(4096)[:20]
x[:, ch] *= 30
x = x.bfloat16()
out["nv_outlier_xbits"] = x.view(torch.int16).numpy().view(np.uint16)
out["nv_outlier_y"] = nvfp4_fake_quant(x.float()).numpy()
ts = two_level_scale(x.float())
out["nv_outlier_two_ts"] = np.float64(ts)
out["nv_outlier_two_y"] = nvfp4_fake_quant(x.float(), ts).numpy()

# MX formats (src/thor_fp4/quant.py:56-81)
for K in (512, 320):
    x = torch.randn(16, K) * torch.linspace(0.01, 4, K)
    out[f"mx_K{K}_x"] = x.numpy()
    for kind in ("mxfp4", "mxfp8"):
        out[f"mx_K{K}_{kind}_y"] = mx_fake_quant(x, kind).numpy()

# benchmark configuration 1, a slab: act bf16 ~N(0,1), weight ~N(0,0.02), two-level
# per-tensor scales on both, dequantize + FP32 matmul (src/thor_fp4/verify.py:91-100)
x = torch.randn(8, 4096).bfloat16()
w = torch.randn(8, 4096) * 0.02
tsx, tsw = two_level_scale(x.float()), two_level_scale(w)
xd, wd = nvfp4_fake_quant(x.float(), tsx), nvfp4_fake_quant(w, tsw)
out["cfg1_xbits"] = x.view(torch.int16).numpy().view(np.uint16)
out["cfg1_w"] = w.numpy()
out["cfg1_tsx"] = np.float64(tsx)
out["cfg1_tsw"] = np.float64(tsw)
out["cfg1_out"] = (xd @ wd.t()).numpy()

dst = Path(__file__).resolve().parent / "ref_fakequant.npz"
np.savez_compressed(dst, **out)
print(f"wrote {dst} ({dst.stat().st_size} bytes, {len(out)} arrays)")
