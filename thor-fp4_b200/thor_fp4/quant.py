"""Torch-side quantizer arithmetic: fake quantizers, the two-level scale, PTQ
calibration and QAT wrappers (API of src/thor_fp4/quant.py:15-148 in the reference
project).  Device-agnostic torch code used by tests, verify() and QAT; the
inference path never calls it.  The QAT forward (STE) runs the fused device kernel on CUDA tensors.

Value semantics follow the device kernels: block scale = UE4M3 round trip of
amax * (1/6) / ts (that operand order), codes = nearest e2m1 with midpoint ties
going up in magnitude, blocks whose scale encodes to zero return zeros.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = [
    "nvfp4_fake_quant", "mx_fake_quant", "STE", "qat", "QATLinear", "qat_linear",
    "QATSequential", "calibrate_linear", "two_level_scale",
]

_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_CUTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def two_level_scale(x: torch.Tensor) -> float:
    """Per-tensor scale of the two-level NVFP4 recipe: amax / (6 * 448), floored at 1e-30."""
    return max(x.abs().amax().item() / (6.0 * 448.0), 1e-30)


def _snap_e2m1(q: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 value with ties up in magnitude; sign of q kept (zero stays +)."""
    grid = torch.tensor(_GRID, dtype=torch.float32, device=q.device)
    cuts = torch.tensor(_CUTS, dtype=torch.float32, device=q.device)
    mag = q.abs().clamp_max(6.0)
    idx = torch.bucketize(mag, cuts, right=True)
    return torch.where(q < 0, -grid[idx], grid[idx])


def nvfp4_fake_quant(x: torch.Tensor, tensor_scale: float = 1.0, blk: int = 16) -> torch.Tensor:
    """quantize -> dequantize with the NVFP4 arithmetic of the device quantizer."""
    shp = x.shape
    v = x.reshape(-1, blk).float()
    amax = v.abs().amax(dim=1, keepdim=True)
    pre = (amax * (1.0 / 6.0) / tensor_scale).clamp_max(448.0)   # the device cast saturates
    sf = pre.to(torch.float8_e4m3fn).to(torch.float32)
    ds = sf * tensor_scale
    q = v / ds.clamp_min(1e-30)
    out = _snap_e2m1(q) * ds
    return torch.where(ds > 0, out, torch.zeros_like(out)).reshape(shp)


def mx_fake_quant(x: torch.Tensor, kind: str = "mxfp4", blk: int = 32) -> torch.Tensor:
    """MX fake quant: UE8M0 scale per 32 = nearest power of two of amax/maxval with
    midpoint ties up; e2m1 (ties up) or e4m3 (RNE, saturating) codes."""
    assert kind in ("mxfp4", "mxfp8")
    shp = x.shape
    v = x.reshape(-1, blk).float()
    amax = v.abs().amax(dim=1, keepdim=True)
    r = amax / (6.0 if kind == "mxfp4" else 448.0)
    _, e = torch.frexp(r)
    lo = torch.ldexp(torch.ones_like(r), e - 1)
    code = torch.where(r - lo < 2 * lo - r, e - 1, e).clamp(-127, 127)
    ds = torch.ldexp(torch.ones_like(r), code)
    q = v / ds.clamp_min(1e-30)
    if kind == "mxfp4":
        out = _snap_e2m1(q) * ds
    else:
        out = q.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).to(torch.float32) * ds
    return torch.where((ds > 0) & (amax > 0), out, torch.zeros_like(out)).reshape(shp)


class STE(torch.autograd.Function):
    """Fake-quantized forward, identity gradient.  On a CUDA tensor the forward is one fused kernel
    (ops.fake_quantize_nvfp4, same values as nvfp4_fake_quant); on CPU the torch arithmetic above."""

    @staticmethod
    def forward(ctx, x, tensor_scale=1.0):
        if x.is_cuda and x.dtype in (torch.float32, torch.float16, torch.bfloat16) and x.numel() % 16 == 0:
            from . import ops
            return ops.fake_quantize_nvfp4(x, float(tensor_scale))
        return nvfp4_fake_quant(x, tensor_scale)

    @staticmethod
    def backward(ctx, g):
        return g, None


def qat(x: torch.Tensor, tensor_scale: float = 1.0) -> torch.Tensor:
    return STE.apply(x, tensor_scale)


class QATLinear(nn.Linear):
    """nn.Linear whose weight and input are NVFP4-fake-quantized with a straight-through
    gradient; two_level=True recomputes the weight's per-tensor scale each forward."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, two_level: bool = False):
        super().__init__(in_features, out_features, bias=bias)
        self.two_level = two_level

    def forward(self, x):
        wts = two_level_scale(self.weight) if self.two_level else 1.0
        return F.linear(qat(x), qat(self.weight, wts), self.bias)


def qat_linear(l: nn.Linear, two_level: bool = False) -> QATLinear:
    q = QATLinear(l.in_features, l.out_features, l.bias is not None, two_level)
    with torch.no_grad():
        q.weight.copy_(l.weight)
        if l.bias is not None:
            q.bias.copy_(l.bias)
    return q


class QATSequential(nn.Sequential):
    def __init__(self, *layers: nn.Module, two_level: bool = False):
        super().__init__(*[qat_linear(m, two_level) if isinstance(m, nn.Linear) else m for m in layers])


@torch.no_grad()
def calibrate_linear(layer: nn.Linear, inputs, method: str = "amax") -> float:
    xs = inputs if isinstance(inputs, list) else [inputs]
    amax = max((x.abs().amax().item() for x in xs), default=0.0)
    return amax / (6.0 * 448.0) if method == "amax" else 1.0
