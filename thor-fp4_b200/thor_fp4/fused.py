"""MLP chains whose activations stay quantized between layers (API of
src/thor_fp4/fused.py:34-249 in the reference project, plus the NVFP4 SwiGLU block).

MX8Act / FusedLinear / GatedMLP / mx8_chain keep the reference semantics for MXFP8
activations: a hidden layer returns act(x @ W^T + bias) already packed as MXFP8
codes + UE8M0 scales, which the next layer consumes without a quantize pass.
NVFP4GatedMLP is the NVFP4 SwiGLU block down(silu(gate x) * up x): x is quantized
once for both wide GEMMs and the product h is re-quantized to NVFP4 for the down
projection.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _ext, ops
from .linear import Linear, resolve_mx8_variant
from .ops import NVFP4Tensor

__all__ = ["MX8Act", "FusedLinear", "GatedMLP", "mx8_chain", "NVFP4GatedMLP"]


class MX8Act:
    """Row-major (M, K) activations resident in MXFP8 (e4m3 codes + tile-layout UE8M0 scales)."""

    def __init__(self, packed: torch.Tensor, sblk: torch.Tensor, shape):
        self.packed, self.sblk, self.shape = packed, sblk, tuple(shape)

    def nbytes(self) -> int:
        M, K = self.shape
        return M * (K + K // 32)

    def dequant(self) -> torch.Tensor:
        """-> f32 (M, K), un-scattering the scale tiles in torch."""
        M, K = self.shape
        S = K // 32
        assert S % 4 == 0, "dequant assumes K % 128 == 0"
        dev = self.packed.device
        codes = self.packed[: M * K].view(M, K).view(torch.float8_e4m3fn).float()
        r = torch.arange(M, device=dev)[:, None]
        s = torch.arange(S, device=dev)[None, :]
        idx = ((r // 128) * (S // 4) + s // 4) * 512 + 16 * (r % 32) + 4 * ((r % 128) // 32) + s % 4
        sb = self.sblk.view(-1)[idx.reshape(-1)].view(M, S).to(torch.int32)
        sf = torch.ldexp(torch.ones(M, S, device=dev), sb - 127)
        return (codes.view(M, S, 32) * sf.unsqueeze(-1)).reshape(M, K)

    def rows(self, a: int, b: int) -> "MX8Act":
        """Rows [a, b) as views (a must be a multiple of 128)."""
        M, K = self.shape
        assert a % 128 == 0, "slices must be 128-row aligned"
        s0 = ops.mx_scale_bytes(a, K) if a else 0
        return MX8Act(self.packed[a * K:a * K + ops.mx_packed_bytes(b - a, K, "mxfp8")],
                      self.sblk[s0:s0 + ops.mx_scale_bytes(b - a, K)], (b - a, K))


_ACTS = {"gelu": F.gelu, "silu": F.silu, "ident": lambda t: t}
_ACT_CODE = {"ident": 0, "gelu": 1, "silu": 2}


class FusedLinear(nn.Module):
    """MXFP8 in -> act(x @ W_mxfp4^T + bias) -> MXFP8 out.  A plain tensor input is
    quantized once on entry.  Output buffers are reused per batch size."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 variant: str | None = None, device=None, max_chunk: int = 0, act: str = "gelu"):
        super().__init__()
        if in_features % 128 != 0:
            raise ValueError(f"in_features={in_features}: the fused epilogue needs K % 128 == 0")
        if out_features % 32 != 0:
            raise ValueError(f"out_features={out_features}: the SF store needs N % 32 == 0")
        if act not in _ACTS:
            raise ValueError(f"act={act!r}: pick 'gelu' | 'silu' | 'ident'")
        L = _ext.fused()
        if variant is None:      # the reference's default pick: the first registered variant of this activation
            names = [bytes(L.tfc4f_variant_name(i)).decode() for i in range(L.tfc4f_n_variants())]
            variant = next((n for n in names if n.startswith(f"mx8out_{act}_128x128x256")), names[0])
        self.variant_idx = L.tfc4f_variant_index(variant.encode())
        if self.variant_idx < 0:
            raise ValueError(f"unknown fused variant {variant!r}")
        self.variant = variant
        # the plain GEMM variant of the unfused (checker) path
        self._plain_idx = _ext.cutlass().tfc4_variant_index(resolve_mx8_variant(in_features).encode())
        self.act = act
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, device=device))
        else:
            self.register_parameter("bias", None)
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        self._w: ops.MXTensor | None = None
        self._bufs: dict = {}
        self.max_chunk = max_chunk
        self.fuse_epilogue = True     # False: GEMM, then bias + activation + quantizer as separate passes (the checker's path)

    def _apply(self, fn, recurse=True):
        self._w, self._bufs = None, {}
        return super()._apply(fn, recurse)

    def refresh_weight(self):
        self._w = ops.MXTensor.from_float(self.weight.detach().contiguous().float(), "mxfp4")
        return self

    def forward(self, x):
        with torch.no_grad():
            if self._w is None:
                self.refresh_weight()
            K, N = self.in_features, self.out_features
            if isinstance(x, MX8Act):
                M, act_in = x.shape[0], x
                assert x.shape[1] == K
                dev = x.packed.device
            else:
                xc = x.detach().contiguous()
                if xc.dtype not in _ext.IN_DTYPE:
                    xc = xc.float()
                M, dev = xc.shape[0], xc.device
            bufs = self._bufs.get(M)
            if bufs is None:
                bufs = {
                    "in": MX8Act(torch.zeros(ops.mx_packed_bytes(M, K, "mxfp8"), dtype=torch.uint8, device=dev),
                                 torch.zeros(ops.mx_scale_bytes(M, K), dtype=torch.uint8, device=dev), (M, K)),
                    "out": MX8Act(torch.zeros(ops.mx_packed_bytes(M, N, "mxfp8"), dtype=torch.uint8, device=dev),
                                  torch.zeros(ops.mx_scale_bytes(M, N), dtype=torch.uint8, device=dev), (M, N)),
                }
                self._bufs[M] = bufs
            if not isinstance(x, MX8Act):
                act_in = bufs["in"]
                ops.quantize_mx(xc, "mxfp8", act_in.packed, act_in.sblk)
            out = bufs["out"]
            if self.fuse_epilogue:
                # bias, activation and MXFP8 re-quantization in the GEMM's epilogue: one kernel, no (M, N) tensor
                b = self.bias.detach().float().contiguous() if self.bias is not None else self._zero_bias(dev)
                ops.gemm_mx8_out(self.variant_idx, act_in.packed, act_in.sblk, self._w.packed, self._w.sblk, b,
                                 out.packed, out.sblk, M, N, K, 1.0)
                return out
            acc = bufs.get("acc")
            if acc is None:
                acc = bufs["acc"] = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            ops.gemm_mx(self._plain_idx, act_in.packed, act_in.sblk, self._w.packed, self._w.sblk, acc, M, N, K, 1.0)
            b = self.bias.detach().float().contiguous() if self.bias is not None else None
            rc = _ext.device_lib().tfp4_act_quant_mx8(
                acc.data_ptr(), b.data_ptr() if b is not None else None, M, N, _ext.IN_DTYPE[acc.dtype],
                _ACT_CODE[self.act], out.packed.data_ptr(), out.sblk.data_ptr(), _ext.stream())
            assert rc == 0, f"tfp4_act_quant_mx8 rc={rc}"
            return out

    def _zero_bias(self, dev):
        z = self._bufs.get("zero_bias")
        if z is None:
            z = self._bufs["zero_bias"] = torch.zeros(self.out_features, dtype=torch.float32, device=dev)
        return z

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}, "
                f"variant={self.variant}, act={self.act}")


class GatedMLP(nn.Module):
    """MXFP8 SwiGLU block down(silu(gate(x)) * up(x)); d_model % 128 == 0, d_ff % 32 == 0."""

    def __init__(self, d_model: int, d_ff: int, device=None):
        super().__init__()
        self.gate = FusedLinear(d_model, d_ff, bias=True, act="silu", device=device)
        self.up = FusedLinear(d_model, d_ff, bias=True, act="ident", device=device)
        self.down = Linear(d_ff, d_model, bias=True, engine="cutlass:mx8").to(device)
        self._h: dict[int, MX8Act] = {}

    def _apply(self, fn, recurse=True):
        self._h = {}
        return super()._apply(fn, recurse)

    def forward(self, x):
        with torch.no_grad():
            g, u = self.gate(x), self.up(x)
            M = g.shape[0]
            h = self._h.get(M)
            if h is None:
                dev = g.packed.device
                h = MX8Act(torch.zeros(ops.mx_packed_bytes(M, g.shape[1], "mxfp8"), dtype=torch.uint8, device=dev),
                           torch.zeros(ops.mx_scale_bytes(M, g.shape[1]), dtype=torch.uint8, device=dev), g.shape)
                self._h[M] = h
            ops.mx8_mul(g, u, h.packed, h.sblk)
            return self.down(h)


def mx8_chain(*dims: int, variant: str | None = None, device=None) -> nn.Sequential:
    """dims[0] -> ... -> dims[-1]: FusedLinear hidden layers, MXFP8-engine Linear last."""
    mods = []
    for i in range(len(dims) - 1):
        if i < len(dims) - 2:
            mods.append(FusedLinear(dims[i], dims[i + 1], bias=True, variant=variant, device=device))
        else:
            mods.append(Linear(dims[i], dims[i + 1], bias=True, engine="cutlass:mx8").to(device))
    return nn.Sequential(*mods)


class NVFP4GatedMLP(nn.Module):
    """NVFP4 SwiGLU block: y = down( nvfp4( silu(x Wg^T) * (x Wu^T) ) ), no biases.

    x is quantized once; gate and up run as ONE GEMM over the stacked weight whose epilogue computes
    silu(gate) * up in FP32 and quantizes h to NVFP4 straight into the down projection's operand
    buffers (tfp4_swiglu_gemm: no (M, 2I) tensor is written).  h is quantized with act_tensor_scale 1
    (dynamic block scales only, so shards of the intermediate dimension quantize independently).
    Buffers are cached per batch size; the warmed block is capturable.

    fuse_epilogue = False selects the three-kernel form (gate/up GEMM to bf16, one-pass silu*up +
    quantize kernel, down GEMM; with fuse_activation = False the middle step is torch elementwise ops
    + the plain quantizer): the path the tests check the fused one against."""

    def __init__(self, hidden: int, intermediate: int, device=None, out_dtype: str = "bf16",
                 weight_std: float | None = None):
        super().__init__()
        if hidden % 64 or intermediate % 64:
            raise ValueError("hidden and intermediate must be multiples of 64")
        self.hidden, self.intermediate, self.out_dtype = hidden, intermediate, out_dtype
        self.w_gate = nn.Parameter(torch.empty(intermediate, hidden, device=device))
        self.w_up = nn.Parameter(torch.empty(intermediate, hidden, device=device))
        self.w_down = nn.Parameter(torch.empty(hidden, intermediate, device=device))
        for w in (self.w_gate, self.w_up, self.w_down):
            if weight_std is None:
                nn.init.kaiming_uniform_(w, a=5 ** 0.5)
            else:
                nn.init.normal_(w, std=weight_std)
        self.tensor_scales: tuple | None = None   # optional (ts_gate_up, ts_down) override
        self.fuse_epilogue = True                 # False: separate kernels between the GEMMs (the checker's path)
        self.fuse_activation = True               # unfused path only: False = torch elementwise + plain quantizer
        self._q = None
        self._q_layout = None
        self._bufs: dict = {}

    def _apply(self, fn, recurse=True):
        self._q, self._bufs = None, {}
        return super()._apply(fn, recurse)

    def refresh_weight(self):
        """Quantize the weights: the gate/up stack in the row order of the selected path (blocks of 16 alternating
        for the fused epilogue, gate half then up half otherwise); the per-tensor scale covers the whole stack."""
        wg, wu = self.w_gate.detach().float(), self.w_up.detach().float()
        wgu = ops.interleave16(wg, wu) if self.fuse_epilogue else torch.cat([wg, wu], dim=0).contiguous()
        ts = self.tensor_scales or (None, None)
        self._q = (NVFP4Tensor.from_float(wgu, ts[0]),
                   NVFP4Tensor.from_float(self.w_down.detach().float().contiguous(), ts[1]))
        self._q_layout = self.fuse_epilogue
        return self

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None, down: bool = True):
        """down=False stops after the hidden tensor and returns its buffers (codes, scale tiles), for callers that run
        the down projection themselves (the tensor-parallel block's push exchange)."""
        with torch.no_grad():
            if self._q is None or self._q_layout != self.fuse_epilogue:
                self.refresh_weight()
            wgu, wd = self._q
            H, I = self.hidden, self.intermediate
            x = x.detach()
            if not x.is_contiguous():
                x = x.contiguous()
            if x.dtype not in _ext.IN_DTYPE:
                x = x.float()
            M = x.shape[0]
            key = (M, x.dtype)
            b = self._bufs.get(key)
            if b is None:
                dev = x.device
                b = {
                    "xp": torch.zeros(ops.packed_bytes(M, H), dtype=torch.uint8, device=dev),
                    "xs": torch.zeros(ops.scale_bytes(M, H), dtype=torch.uint8, device=dev),
                    "hp": torch.zeros(ops.packed_bytes(M, I), dtype=torch.uint8, device=dev),
                    "hs": torch.zeros(ops.scale_bytes(M, I), dtype=torch.uint8, device=dev),
                    "y": torch.empty(M, H, dtype=_ext.OUT_TORCH[self.out_dtype], device=dev),
                }
                self._bufs[key] = b
            ops.quantize_nvfp4(x, 1.0, b["xp"], b["xs"])
            if self.fuse_epilogue:
                ops.swiglu_gemm(b["xp"], b["xs"], 1.0, wgu, M, b["hp"], b["hs"])
            else:
                gu = b.get("gu")
                if gu is None:
                    gu = b["gu"] = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=x.device)
                ops.gemm(b["xp"], b["xs"], 1.0, wgu.packed, wgu.sblk, wgu.tensor_scale, gu, M, 2 * I, H, "bf16")
                if self.fuse_activation:
                    # silu(gate) * up and the re-quantization of h in one pass over the GEMM output
                    ops.swiglu_quantize_nvfp4(gu, b["hp"], b["hs"])
                else:
                    h = (F.silu(gu[:, :I].float()) * gu[:, I:].float()).to(torch.bfloat16)
                    ops.quantize_nvfp4(h, 1.0, b["hp"], b["hs"])
            if not down:
                return b["hp"], b["hs"]
            y = out if out is not None else b["y"]
            ops.gemm(b["hp"], b["hs"], 1.0, wd.packed, wd.sblk, wd.tensor_scale, y, M, H, I, self.out_dtype)
            return y
