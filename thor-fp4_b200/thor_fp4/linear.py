"""thor_fp4.Linear -- the nn.Linear drop-in on the sm_100a engine (interface of
src/thor_fp4/linear.py:89-279 in the reference project).

State: fp32 master ``weight`` / ``bias`` parameters; a lazily built quantized weight
(``_weight_fp4``: NVFP4Tensor, or MXTensor for the MXFP8-activation engine) that is
dropped whenever the module is moved or reset; per-(M, dtype) activation buffers
(codes, scale bytes, output) that are reused on every call, which is what makes a
warmed layer allocation-free and CUDA-graph capturable.  The returned tensor is that
reused output buffer.

Engines (strings of the reference keep parsing; ``engine_kind`` stays observable):
  'cublaslt' -> kind 'lt' : activation quantizer + tcgen05 NVFP4 GEMM (the default path);
  'gemv'     -> kind 'gv' : register-dequant GEMV, M <= 8, exact activations;
  'cutlass' / 'cutlass:<nvfp4 variant>' -> kind 'nv': same GEMM through the variant registry;
  'cutlass:mx8' / 'cutlass:<mxfp8xfp4 variant>' -> kind 'mx8': MXFP8 activations x MXFP4 weights.
Difference from the reference: the bias is added to the FP32 accumulator inside the
GEMM epilogue (one rounding) instead of afterwards in the output dtype (two).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import _ext, ops
from .ops import MXTensor, NVFP4Tensor

__all__ = ["Linear", "resolve_mx8_variant"]

_OPS_QUANT, _OPS_GEMM = ops.quantize_nvfp4, ops.gemm     # to notice when a caller has replaced them

_DEFAULT_NV_VARIANTS = ["nvfp4_128x256x256_c2x1", "nvfp4_128x128x256_c1"]
_MX8_SMALL_K = ["mxfp8xfp4_128x128x128_c2x1", "mxfp8xfp4_128x128x256_c1"]
_MX8_BIG_K = ["mxfp8xfp4_128x256x128_c2x1", "mxfp8xfp4_128x128x256_c1"]


def _variant_names() -> list[str]:
    L = _ext.cutlass()
    return [bytes(L.tfc4_variant_name(i)).decode() for i in range(L.tfc4_n_variants())]


def resolve_mx8_variant(K: int | None = None) -> str:
    """Name of the MXFP8-activation variant used for in_features=K."""
    names = _variant_names()
    for c in (_MX8_SMALL_K if (K is not None and K <= 2048) else _MX8_BIG_K):
        if c in names:
            return c
    for n in names:
        if n.startswith("mxfp8xfp4"):
            return n
    raise RuntimeError("no mxfp8xfp4 variant in the library")


def _resolve_engine(engine: str, K: int | None = None):
    """engine string -> (kind, variant index); kind in {'lt', 'gv', 'nv', 'mx8'}."""
    if engine == "cublaslt":
        return "lt", -1
    if engine == "gemv":
        return "gv", -1
    L = _ext.cutlass()
    if engine == "cutlass":
        names = _variant_names()
        name = next((c for c in _DEFAULT_NV_VARIANTS if c in names),
                    next(n for n in names if n.startswith("nvfp4_")))
    elif engine == "cutlass:mx8":
        name = resolve_mx8_variant(K)
    elif engine.startswith("cutlass:"):
        name = engine.split(":", 1)[1]
    else:
        raise ValueError(f"unknown engine {engine!r}")
    idx = L.tfc4_variant_index(name.encode())
    if idx < 0:
        raise ValueError(f"unknown cutlass variant {name!r}")
    return ("mx8" if name.startswith("mxfp8") else "nv"), idx


class Linear(nn.Module):
    """y = quant(x) @ quant(W)^T (+ bias) on the FP4 tensor cores.

    Args follow the reference: in_features (K, multiple of 64), out_features (N >= 8,
    multiple of 8), bias, out_dtype 'f16' | 'bf16' | 'f32', tensor_scale (None = two-level
    recipe from the weight amax, 1.0 = block scales only), act_tensor_scale (1.0 or a
    calibrated static value), engine (see module docstring)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 device=None, dtype=None, out_dtype: str = "f16",
                 tensor_scale: float | None = None, act_tensor_scale: float = 1.0,
                 engine: str = "cublaslt"):
        super().__init__()
        if in_features % 64 != 0:
            raise ValueError(f"in_features={in_features}: NVFP4 needs K % 64 == 0 "
                             "(keep such layers in BF16 - see thor_fp4.convert)")
        if out_features < 8 or out_features % 8 != 0:
            raise ValueError(f"out_features={out_features}: NVFP4 needs N >= 8 and N % 8 == 0")
        self.in_features, self.out_features = in_features, out_features
        self.engine_kind, self.engine_variant = _resolve_engine(engine, in_features)
        if self.engine_kind == "mx8" and in_features % 128 != 0:
            raise ValueError(f"in_features={in_features}: the MXFP8 engine needs K % 128 == 0")
        if self.engine_kind in ("nv", "mx8"):
            out_dtype = "bf16"     # the variant registry's output type, as in the reference
        if out_dtype not in _ext.OUT_DTYPE:
            raise ValueError(f"out_dtype={out_dtype!r}: pick 'f16' | 'bf16' | 'f32'")
        self.out_dtype = out_dtype
        self.act_tensor_scale = float(act_tensor_scale)
        self._tensor_scale_requested = tensor_scale
        self._weight_fp4: NVFP4Tensor | MXTensor | None = None
        _ = dtype
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, device=device))
        else:
            self.register_parameter("bias", None)
        self._act_bufs: dict = {}
        self._gemv_outs: dict = {}
        self.reset_parameters()

    # ------------------------------------------------------------------ lifecycle
    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        if self.bias is not None:
            nn.init.zeros_(self.bias)
        self._weight_fp4 = None

    def _apply(self, fn, recurse=True):
        self._weight_fp4 = None
        self._act_bufs = {}
        self._gemv_outs = {}
        return super()._apply(fn, recurse)

    def _load_from_state_dict(self, *args, **kwargs):
        self._weight_fp4 = None
        return super()._load_from_state_dict(*args, **kwargs)

    def refresh_weight(self):
        """Re-quantize the master weight (call after in-place weight edits)."""
        w = self.weight.detach().contiguous().float()
        if self.engine_kind == "mx8":
            self._weight_fp4 = MXTensor.from_float(w, "mxfp4")
        else:
            self._weight_fp4 = NVFP4Tensor.from_float(w, self._tensor_scale_requested)
        return self

    # ------------------------------------------------------------------ quantized checkpoint
    def quantized_state(self) -> dict:
        """The layer as the GEMM sees it: NVFP4 weight (codes, scale tiles, per-tensor scale), bias and the
        activation scale.  About 3.6x smaller than the FP32 state_dict; restoring it re-quantizes nothing."""
        if self.engine_kind == "mx8":
            raise RuntimeError("quantized_state covers NVFP4 weights; this layer holds an MXFP4 weight")
        if self._weight_fp4 is None:
            self.refresh_weight()
        return {"weight_fp4": self._weight_fp4.state_dict(),
                "bias": None if self.bias is None else self.bias.detach(),
                "act_tensor_scale": float(self.act_tensor_scale), "out_dtype": self.out_dtype}

    def load_quantized_state(self, state: dict):
        """Install a quantized_state(): the codes are used as they are; the FP32 master weight becomes their
        dequantized value (re-quantizing it with the stored per-tensor scale gives the same scale bytes and values
        back; a value that had rounded to a negative zero comes back as a positive zero code)."""
        if self.engine_kind == "mx8":
            raise RuntimeError("load_quantized_state covers NVFP4 weights; this layer holds an MXFP4 weight")
        w = NVFP4Tensor.from_state_dict(state["weight_fp4"], device=self.weight.device)
        if tuple(w.shape) != (self.out_features, self.in_features):
            raise ValueError(f"checkpoint weight is {tuple(w.shape)}, layer is {(self.out_features, self.in_features)}")
        if (state.get("bias") is None) != (self.bias is None):
            raise ValueError("checkpoint and layer disagree on having a bias")
        with torch.no_grad():
            self.weight.copy_(w.dequantize())
            if self.bias is not None:
                self.bias.copy_(state["bias"].to(self.bias.device))
        self.act_tensor_scale = float(state.get("act_tensor_scale", self.act_tensor_scale))
        self._tensor_scale_requested = w.tensor_scale
        self._weight_fp4 = w
        return self

    def _bias_f32(self):
        b = self.bias
        if b is None:
            return None
        b = b.detach()
        return b if (b.dtype == torch.float32 and b.is_contiguous()) else b.float().contiguous()

    def _out_buffer(self, cache: dict, key, M: int, device):
        out = cache.get(key)
        if out is None:
            out = torch.empty(M, self.out_features, dtype=_ext.OUT_TORCH[self.out_dtype], device=device)
            cache[key] = out
        return out

    # ------------------------------------------------------------------ forward
    def forward(self, x):
        with torch.no_grad():
            if self._weight_fp4 is None:
                self.refresh_weight()
            w = self._weight_fp4
            M = x.shape[0]
            N, K = self.out_features, self.in_features
            packed_in = hasattr(x, "packed") and hasattr(x, "sblk")
            if packed_in:
                dt = "mx8act"
            else:
                x = x.detach() if x.requires_grad else x
                if not x.is_contiguous():
                    x = x.contiguous()
                dt = x.dtype
                if dt not in _ext.IN_DTYPE:
                    x, dt = x.float(), torch.float32
            key = (M, dt)

            if self.engine_kind == "gv":
                if M > 8:
                    raise RuntimeError(f"engine='gemv' serves M <= 8 (got {M}); use engine='cublaslt'")
                out = self._out_buffer(self._gemv_outs, key, M, x.device)
                ops.gemv(x, w, self.out_dtype, out=out)
                if self.bias is not None:
                    out += self.bias.to(out.dtype)
                return out

            if packed_in and self.engine_kind == "mx8":
                # already-packed MXFP8 activations (output of a fused layer): no quantize pass
                out = self._out_buffer(self._gemv_outs, key, M, x.packed.device)
                ops.gemm_mx(self.engine_variant, x.packed, x.sblk, w.packed, w.sblk, out, M, N, K, 1.0)
                if self.bias is not None:
                    out += self.bias.to(out.dtype)
                return out

            bufs = self._act_bufs.get(key)
            if bufs is None:
                if self.engine_kind == "mx8":
                    pb, sb = ops.mx_packed_bytes(M, K, "mxfp8"), ops.mx_scale_bytes(M, K)
                else:
                    pb, sb = ops.packed_bytes(M, K), ops.scale_bytes(M, K)
                bufs = (torch.zeros(pb, dtype=torch.uint8, device=x.device),
                        torch.zeros(sb, dtype=torch.uint8, device=x.device),
                        torch.empty(M, N, dtype=_ext.OUT_TORCH[self.out_dtype], device=x.device))
                self._act_bufs[key] = bufs
            packed, sblk, out = bufs
            if self.engine_kind == "lt":
                if ops.quantize_nvfp4 is _OPS_QUANT and ops.gemm is _OPS_GEMM:
                    # both steps in one foreign call (small batches are bound by per-call host cost); the
                    # two-call form below stays for callers that wrap or replace ops.quantize_nvfp4 / ops.gemm
                    b = self._bias_f32()
                    rc = _ext.device_lib().tfp4_linear(
                        x.data_ptr(), M, K, _ext.IN_DTYPE[dt], self.act_tensor_scale, packed.data_ptr(), sblk.data_ptr(),
                        w.packed.data_ptr(), w.sblk.data_ptr(), w.tensor_scale, b.data_ptr() if b is not None else None,
                        out.data_ptr(), N, _ext.OUT_DTYPE[self.out_dtype], _ext.stream())
                    assert rc == 0, f"tfp4_linear rc={rc}"
                    return out
                ops.quantize_nvfp4(x, self.act_tensor_scale, packed, sblk)
                ops.gemm(packed, sblk, self.act_tensor_scale, w.packed, w.sblk, w.tensor_scale,
                         out, M, N, K, self.out_dtype, bias=self._bias_f32())
                return out
            if self.engine_kind == "nv":
                ops.quantize_nvfp4(x, self.act_tensor_scale, packed, sblk)
                ops.gemm_mx(self.engine_variant, packed, sblk, w.packed, w.sblk, out, M, N, K,
                            self.act_tensor_scale * w.tensor_scale)
            else:
                ops.quantize_mx(x, "mxfp8", packed, sblk)
                ops.gemm_mx(self.engine_variant, packed, sblk, w.packed, w.sblk, out, M, N, K, 1.0)
            if self.bias is not None:
                out += self.bias.to(out.dtype)
            return out

    def extra_repr(self) -> str:
        ts = (self._weight_fp4.tensor_scale
              if self._weight_fp4 is not None and hasattr(self._weight_fp4, "tensor_scale")
              else self._tensor_scale_requested)
        eng = {"lt": "cublaslt", "gv": "gemv"}.get(self.engine_kind, f"cutlass:{self.engine_variant}")
        return (f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}, "
                f"out_dtype={self.out_dtype}, tensor_scale={ts}, engine={eng}")

    def fp4_weight_nbytes(self) -> int:
        """Bytes of the resident weight (codes + block scales)."""
        return self.in_features * self.out_features // 2 + self.out_features * (self.in_features // 16)
