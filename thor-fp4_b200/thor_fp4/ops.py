"""Functional NVFP4 / MX ops over the C ABI (interface of src/thor_fp4/ops.py:16-246
in the reference project).

All buffers are torch-owned uint8 tensors sized by the *_bytes helpers (rows
padded to 128, scale columns to 4).  The quantizers write the padding rows of
the last 128-row tile as zeros themselves, so buffers may come from
torch.empty as well as torch.zeros; steady-state calls allocate nothing and
can be captured into CUDA graphs.
"""
from __future__ import annotations

import torch

from . import _ext

__all__ = [
    "pad_rows", "packed_bytes", "scale_bytes", "mx_packed_bytes", "mx_scale_bytes",
    "quantize_nvfp4", "fake_quantize_nvfp4", "quantize_mx", "mx8_mul", "dequantize_nvfp4", "block_scales",
    "gemm", "gemm_mx", "gemv", "NVFP4Tensor", "MXTensor", "interleave16", "swiglu_gemm", "gemm_mx8_out",
]


def pad_rows(R: int) -> int:
    return int(_ext.core().tfp4_pad_rows(R))


def packed_bytes(R: int, K: int) -> int:
    return int(_ext.core().tfp4_packed_bytes(R, K))


def scale_bytes(R: int, K: int) -> int:
    return int(_ext.core().tfp4_scale_bytes(R, K))


def mx_packed_bytes(R: int, K: int, kind: str) -> int:
    return int(_ext.core().tfp4_mx_packed_bytes(R, K, 0 if kind == "mxfp4" else 1))


def mx_scale_bytes(R: int, K: int) -> int:
    return int(_ext.core().tfp4_mx_scale_bytes(R, K))


def _check_2d_cuda(x: torch.Tensor):
    assert x.ndim == 2 and x.is_cuda and x.is_contiguous(), "expected a contiguous 2-D cuda tensor"


def quantize_nvfp4(x: torch.Tensor, tensor_scale: float = 1.0,
                   packed: torch.Tensor | None = None,
                   sblk: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Row-major (R, K) f32/f16/bf16 cuda tensor -> (packed codes, tile-layout scale bytes)."""
    L = _ext.device_lib()
    _check_2d_cuda(x)
    R, K = x.shape
    assert K % 64 == 0, f"K={K} must be a multiple of 64 (scale tiles are 4 scale columns wide)"
    if packed is None:
        packed = torch.zeros(packed_bytes(R, K), dtype=torch.uint8, device=x.device)
    if sblk is None:
        sblk = torch.zeros(scale_bytes(R, K), dtype=torch.uint8, device=x.device)
    rc = L.tfp4_quant(x.data_ptr(), R, K, _ext.IN_DTYPE[x.dtype], float(tensor_scale),
                      packed.data_ptr(), sblk.data_ptr(), _ext.stream())
    assert rc == 0, f"tfp4_quant rc={rc}"
    return packed, sblk


def swiglu_quantize_nvfp4(gu: torch.Tensor, packed: torch.Tensor | None = None,
                          sblk: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """gu = (R, 2*I) f16/bf16 output of the stacked gate/up GEMM -> NVFP4 codes and scale tiles of
    h = silu(gu[:, :I]) * gu[:, I:] (FP32 math, h held in gu's dtype, per-tensor scale 1), in one pass."""
    L = _ext.device_lib()
    _check_2d_cuda(gu)
    assert gu.dtype in (torch.float16, torch.bfloat16), "stacked gate/up tensor must be f16 or bf16"
    R, two_i = gu.shape
    I = two_i // 2
    assert two_i == 2 * I and I % 64 == 0, f"intermediate size {I} must be a multiple of 64"
    if packed is None:
        packed = torch.zeros(packed_bytes(R, I), dtype=torch.uint8, device=gu.device)
    if sblk is None:
        sblk = torch.zeros(scale_bytes(R, I), dtype=torch.uint8, device=gu.device)
    rc = L.tfp4_swiglu_quant(gu.data_ptr(), R, I, _ext.IN_DTYPE[gu.dtype], packed.data_ptr(), sblk.data_ptr(),
                             _ext.stream())
    assert rc == 0, f"tfp4_swiglu_quant rc={rc}"
    return packed, sblk


def interleave16(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Stack two (I, K) weights as (2I, K) with rows alternating in blocks of 16: gate rows j..j+15, up rows j..j+15,
    gate rows j+16.., ...  This is the row order swiglu_gemm wants: a 32-column chunk of the gate/up GEMM's output then
    holds one 16-element quantization block of gate values and the matching block of up values."""
    I, K = w_gate.shape
    assert w_up.shape == (I, K) and I % 16 == 0, "intermediate size must be a multiple of 16"
    return torch.stack([w_gate.reshape(I // 16, 16, K), w_up.reshape(I // 16, 16, K)], dim=1).reshape(2 * I, K).contiguous()


def swiglu_gemm(packedA: torch.Tensor, sblkA: torch.Tensor, tsA: float, w: "NVFP4Tensor", M: int,
                h_packed: torch.Tensor | None = None, h_sblk: torch.Tensor | None = None):
    """Gate/up GEMM with silu(gate) * up and the NVFP4 quantization of h in its epilogue (tfp4_swiglu_gemm).
    w: the NVFP4 stack interleave16(Wg, Wu) of shape (2I, K).  Returns (codes, scale tiles) of h (M, I), quantized with
    per-tensor scale 1: the A operand of the down projection.  No (M, 2I) tensor is written."""
    L = _ext.device_lib()
    N, K = w.shape
    I = N // 2
    assert N % 128 == 0, f"intermediate size {I} must be a multiple of 64"
    if h_packed is None:
        h_packed = torch.zeros(packed_bytes(M, I), dtype=torch.uint8, device=packedA.device)
    if h_sblk is None:
        h_sblk = torch.zeros(scale_bytes(M, I), dtype=torch.uint8, device=packedA.device)
    rc = L.tfp4_swiglu_gemm(packedA.data_ptr(), sblkA.data_ptr(), float(tsA), w.packed.data_ptr(), w.sblk.data_ptr(),
                            float(w.tensor_scale), h_packed.data_ptr(), h_sblk.data_ptr(), M, N, K, _ext.stream())
    assert rc == 0, f"tfp4_swiglu_gemm rc={rc}"
    return h_packed, h_sblk


def gemm_mx8_out(variant: int, packedA: torch.Tensor, sblkA: torch.Tensor, packedB: torch.Tensor, sblkB: torch.Tensor,
                 bias: torch.Tensor, d_packed: torch.Tensor, d_sblk: torch.Tensor, M: int, N: int, K: int,
                 alpha: float = 1.0) -> None:
    """tfc4f_gemm: MXFP8 (M, K) x MXFP4 (N, K) with bias[n], the variant's activation and the MXFP8 re-quantization of
    the output in the epilogue; d_packed (>= M*N bytes) and d_sblk (tfc4f_sfd_bytes) receive codes and scale tiles."""
    L = _ext.device_lib()
    assert bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous()
    rc = L.tfc4f_gemm(variant, packedA.data_ptr(), sblkA.data_ptr(), packedB.data_ptr(), sblkB.data_ptr(), bias.data_ptr(),
                      d_packed.data_ptr(), d_sblk.data_ptr(), M, N, K, float(alpha), _ext.stream())
    assert rc == 0, f"tfc4f_gemm rc={rc}"


_FQ_OUT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def fake_quantize_nvfp4(x: torch.Tensor, tensor_scale: float = 1.0, out: torch.Tensor | None = None,
                        out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """dequantize(quantize(x)) in one kernel, no codes stored: the values of quant.nvfp4_fake_quant
    (src/thor_fp4/quant.py:32-53 of the reference project) for a CUDA tensor of any shape whose element
    count is a multiple of 16 (consecutive 16-element blocks of the flattened tensor)."""
    assert x.is_cuda, "fake_quantize_nvfp4 needs a CUDA tensor"
    L = _ext.device_lib()
    if x.dtype not in _ext.IN_DTYPE:
        x = x.float()
    x = x.contiguous()
    assert x.numel() % 16 == 0, "element count must be a multiple of 16"
    if out is None:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    assert out.is_cuda and out.is_contiguous() and out.numel() == x.numel() and out.dtype in _FQ_OUT
    rc = L.tfp4_fake_quant(x.data_ptr(), x.numel(), _ext.IN_DTYPE[x.dtype], float(tensor_scale),
                           out.data_ptr(), _FQ_OUT[out.dtype], _ext.stream())
    assert rc == 0, f"tfp4_fake_quant failed ({rc})"
    return out


def quantize_mx(x: torch.Tensor, kind: str = "mxfp4",
                packed: torch.Tensor | None = None,
                sblk: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """MX quantize: 'mxfp4' (e2m1 codes) or 'mxfp8' (e4m3 codes), UE8M0 scale per 32."""
    L = _ext.device_lib()
    assert kind in ("mxfp4", "mxfp8")
    _check_2d_cuda(x)
    R, K = x.shape
    assert K % 64 == 0, f"K={K} must be a multiple of 64"
    if packed is None:
        packed = torch.zeros(mx_packed_bytes(R, K, kind), dtype=torch.uint8, device=x.device)
    if sblk is None:
        sblk = torch.zeros(mx_scale_bytes(R, K), dtype=torch.uint8, device=x.device)
    rc = L.tfp4_quant_mx(x.data_ptr(), R, K, _ext.IN_DTYPE[x.dtype], 0 if kind == "mxfp4" else 1,
                         packed.data_ptr(), sblk.data_ptr(), _ext.stream())
    assert rc == 0, f"tfp4_quant_mx rc={rc}"
    return packed, sblk


def mx8_mul(a, b, packed: torch.Tensor | None = None, sblk: torch.Tensor | None = None):
    """h = a * b for two MXFP8 tensors of the same (R, K), K % 128 == 0; ceil-pow2 scales."""
    L = _ext.device_lib()
    R, K = a.shape
    assert tuple(b.shape) == (R, K), f"mx8_mul shape mismatch {a.shape} vs {b.shape}"
    assert K % 128 == 0, f"K={K} must be a multiple of 128 (atom alignment)"
    dev = a.packed.device
    if packed is None:
        packed = torch.zeros(mx_packed_bytes(R, K, "mxfp8"), dtype=torch.uint8, device=dev)
    if sblk is None:
        sblk = torch.zeros(mx_scale_bytes(R, K), dtype=torch.uint8, device=dev)
    rc = L.tfp4_mx8_mul(a.packed.data_ptr(), a.sblk.data_ptr(), b.packed.data_ptr(), b.sblk.data_ptr(),
                        packed.data_ptr(), sblk.data_ptr(), R, K, _ext.stream())
    assert rc == 0, f"tfp4_mx8_mul rc={rc}"
    return packed, sblk


def dequantize_nvfp4(packed: torch.Tensor, sblk: torch.Tensor, tensor_scale: float,
                     R: int, K: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """NVFP4 buffers -> plain f32 (R, K) (operand builder of verify()'s reference path)."""
    L = _ext.device_lib()
    if out is None:
        out = torch.empty(R, K, dtype=torch.float32, device=packed.device)
    rc = L.tfp4_dequant_f32(packed.data_ptr(), sblk.data_ptr(), float(tensor_scale), R, K,
                            out.data_ptr(), _ext.stream())
    assert rc == 0, f"tfp4_dequant_f32 rc={rc}"
    return out


def block_scales(sblk: torch.Tensor, R: int, K: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Tile-layout UE4M3 bytes -> decoded f32 (R, K/16), without the per-tensor scale."""
    L = _ext.device_lib()
    if out is None:
        out = torch.empty(R, K // 16, dtype=torch.float32, device=sblk.device)
    rc = L.tfp4_scales_f32(sblk.data_ptr(), R, K, out.data_ptr(), _ext.stream())
    assert rc == 0, f"tfp4_scales_f32 rc={rc}"
    return out


_TORCH_NAME = {"f16": "float16", "bf16": "bfloat16", "f32": "float32"}


def gemm(packedA: torch.Tensor, sblkA: torch.Tensor, tsA: float,
         packedB: torch.Tensor, sblkB: torch.Tensor, tsB: float,
         out: torch.Tensor, M: int, N: int, K: int, out_dtype: str = "f16",
         bias: torch.Tensor | None = None) -> None:
    """out (M, N) row-major = (tsA*tsB) * A(M, K) @ B(N, K)^T (+ bias[n]), NVFP4 operands.

    `bias` (f32, N elements) is an addition over the reference signature: it is added
    to the FP32 accumulator before the single cast to `out_dtype`."""
    L = _ext.device_lib()
    assert out.is_contiguous() and out.numel() == M * N and str(out.dtype).endswith(_TORCH_NAME[out_dtype])
    if bias is None:
        rc = L.tfp4_gemm(packedA.data_ptr(), sblkA.data_ptr(), float(tsA),
                         packedB.data_ptr(), sblkB.data_ptr(), float(tsB),
                         out.data_ptr(), M, N, K, _ext.OUT_DTYPE[out_dtype], _ext.stream())
    else:
        assert bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous()
        rc = L.tfp4_gemm_bias(packedA.data_ptr(), sblkA.data_ptr(), float(tsA),
                              packedB.data_ptr(), sblkB.data_ptr(), float(tsB), bias.data_ptr(),
                              out.data_ptr(), M, N, K, _ext.OUT_DTYPE[out_dtype], _ext.stream())
    assert rc == 0, f"tfp4_gemm rc={rc}"


def gemm_mx(variant: int, packedA: torch.Tensor, sblkA: torch.Tensor,
            packedB: torch.Tensor, sblkB: torch.Tensor, out: torch.Tensor,
            M: int, N: int, K: int, alpha: float = 1.0) -> None:
    """tfc4_gemm: bf16 out = alpha * A @ B^T through a named variant (NVFP4 or MXFP8 x MXFP4)."""
    L = _ext.device_lib()
    assert out.is_contiguous() and out.numel() == M * N and out.dtype == torch.bfloat16
    rc = L.tfc4_gemm(variant, packedA.data_ptr(), sblkA.data_ptr(), packedB.data_ptr(), sblkB.data_ptr(),
                     out.data_ptr(), M, N, K, float(alpha), _ext.stream())
    assert rc == 0, f"tfc4_gemm rc={rc}"


def gemv(x: torch.Tensor, w: "NVFP4Tensor", out_dtype: str = "f32",
         out: torch.Tensor | None = None) -> torch.Tensor:
    """out (M, N) = x (M, K) @ dequant(w)^T for M <= 8: exact activations, FP32 accumulation."""
    L = _ext.device_lib()
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    _check_2d_cuda(x)
    assert 1 <= M <= 8, f"gemv serves M <= 8 (got {M})"
    if out is None:
        out = torch.empty(M, N, dtype=_ext.OUT_TORCH[out_dtype], device=x.device)
    rc = L.tfp4_gemv(x.data_ptr(), M, K, _ext.IN_DTYPE[x.dtype],
                     w.packed.data_ptr(), w.gemv_scales().data_ptr(), float(w.tensor_scale),
                     out.data_ptr(), N, _ext.OUT_DTYPE[out_dtype], _ext.stream())
    assert rc == 0, f"tfp4_gemv rc={rc}"
    return out


class NVFP4Tensor:
    """A row-major (R, K) tensor resident in NVFP4: codes + block scales + per-tensor scale."""

    def __init__(self, packed: torch.Tensor, sblk: torch.Tensor, tensor_scale: float,
                 shape: tuple[int, int]):
        self.packed, self.sblk = packed, sblk
        self.tensor_scale, self.shape = float(tensor_scale), tuple(shape)
        self._gemv_scales: torch.Tensor | None = None

    def gemv_scales(self) -> torch.Tensor:
        """Block scales un-scattered to plain (R, K/16) bytes (cached)."""
        if self._gemv_scales is None:
            R, K = self.shape
            out = torch.empty(R, K // 16, dtype=torch.uint8, device=self.packed.device)
            rc = _ext.device_lib().tfp4_scales_gemv(self.sblk.data_ptr(), R, K, out.data_ptr(), _ext.stream())
            assert rc == 0, f"tfp4_scales_gemv rc={rc}"
            self._gemv_scales = out
        return self._gemv_scales

    @classmethod
    def from_float(cls, x: torch.Tensor, tensor_scale: float | None = None):
        """tensor_scale=None: two-level recipe amax/(6*448) (floor 1e-30); 1.0: block scales only."""
        assert x.ndim == 2 and x.is_contiguous()
        x = x.float() if x.dtype != torch.float32 else x
        if tensor_scale is None:
            tensor_scale = max(x.abs().amax().item() / (6.0 * 448.0), 1e-30)
        packed, sblk = quantize_nvfp4(x, tensor_scale)
        return cls(packed, sblk, tensor_scale, tuple(x.shape))

    def dequantize(self) -> torch.Tensor:
        R, K = self.shape
        return dequantize_nvfp4(self.packed, self.sblk, self.tensor_scale, R, K)

    def matmul_t(self, w: "NVFP4Tensor", out_dtype: str = "f16",
                 out: torch.Tensor | None = None) -> torch.Tensor:
        """(M, K) @ (N, K)^T -> (M, N); self is the activation-side operand."""
        M, K = self.shape
        N, K2 = w.shape
        assert K == K2
        if out is None:
            out = torch.empty(M, N, dtype=_ext.OUT_TORCH[out_dtype], device=self.packed.device)
        gemm(self.packed, self.sblk, self.tensor_scale, w.packed, w.sblk, w.tensor_scale,
             out, M, N, K, out_dtype)
        return out

    def nbytes(self) -> int:
        R, K = self.shape
        return R * K // 2 + R * (K // 16)

    # ---- row slices: views into the same code and scale buffers (no copy) ----
    def rows(self, start: int, stop: int | None = None) -> "NVFP4Tensor":
        """Rows [start, stop) as a tensor over the same buffers.  Codes are row-major and scale tiles cover
        128 rows each, so a slice that starts on a multiple of 128 is a pointer offset into both buffers
        (how a resident library is swept chunk by chunk).  The last tile of the slice may hold rows of the
        parent past `stop`; consumers read only `stop - start` rows of results."""
        R, K = self.shape
        stop = R if stop is None else stop
        assert 0 <= start < stop <= R, f"bad row range [{start}, {stop}) of {R}"
        assert start % 128 == 0, "a row slice must start on a multiple of 128 (scale tiles are 128 rows tall)"
        n = stop - start
        tile_bytes = ((K // 16 + 3) // 4) * 512                 # scale bytes per 128-row tile
        p = self.packed[start * (K // 2): (start + pad_rows_host(n)) * (K // 2)]
        sb = self.sblk[(start // 128) * tile_bytes: ((start + pad_rows_host(n)) // 128) * tile_bytes]
        return NVFP4Tensor(p, sb, self.tensor_scale, (n, K))

    def row_chunks(self, rows_per_chunk: int):
        """Iterate (first_row, slice) over consecutive row slices; rows_per_chunk % 128 == 0."""
        assert rows_per_chunk > 0 and rows_per_chunk % 128 == 0
        for r0 in range(0, self.shape[0], rows_per_chunk):
            yield r0, self.rows(r0, min(self.shape[0], r0 + rows_per_chunk))

    # ---- checkpoint: the quantized tensor as it sits in memory ----
    FORMAT = "nvfp4/e2m1-low-nibble-first/ue4m3-tiles-128x4/v1"

    def state_dict(self) -> dict:
        """Codes, scale tiles, per-tensor scale and shape: everything a GEMM needs, no FP32 copy."""
        return {"format": self.FORMAT, "shape": tuple(self.shape), "tensor_scale": float(self.tensor_scale),
                "packed": self.packed, "sblk": self.sblk}

    @classmethod
    def from_state_dict(cls, state: dict, device=None) -> "NVFP4Tensor":
        if state.get("format") != cls.FORMAT:
            raise ValueError(f"not an NVFP4 tensor checkpoint: format={state.get('format')!r}")
        R, K = (int(v) for v in state["shape"])
        packed, sblk = state["packed"], state["sblk"]
        want_p, want_s = pad_rows_host(R) * (K // 2), (pad_rows_host(R) // 128) * ((K // 16 + 3) // 4) * 512
        if (packed.dtype != torch.uint8 or sblk.dtype != torch.uint8 or K % 64 != 0
                or packed.numel() != want_p or sblk.numel() != want_s):
            raise ValueError(f"NVFP4 checkpoint buffers do not match shape ({R}, {K}): "
                             f"{packed.numel()} code bytes (want {want_p}), {sblk.numel()} scale bytes (want {want_s})")
        if device is not None:
            packed, sblk = packed.to(device), sblk.to(device)
        return cls(packed.contiguous(), sblk.contiguous(), float(state["tensor_scale"]), (R, K))

    def save(self, path) -> None:
        torch.save({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in self.state_dict().items()}, path)

    @classmethod
    def load(cls, path, device=None) -> "NVFP4Tensor":
        return cls.from_state_dict(torch.load(path, map_location="cpu", weights_only=True), device)


def pad_rows_host(R: int) -> int:
    """Rows padded to whole 128-row scale tiles (host arithmetic, same value as pad_rows)."""
    return (int(R) + 127) // 128 * 128


class MXTensor:
    """A row-major (R, K) tensor in an MX format ('mxfp4' or 'mxfp8')."""

    def __init__(self, packed: torch.Tensor, sblk: torch.Tensor, kind: str, shape):
        self.packed, self.sblk, self.kind, self.shape = packed, sblk, kind, tuple(shape)

    @classmethod
    def from_float(cls, x: torch.Tensor, kind: str = "mxfp4"):
        assert x.ndim == 2 and x.is_contiguous()
        packed, sblk = quantize_mx(x.float(), kind)
        return cls(packed, sblk, kind, x.shape)

    def nbytes(self) -> int:
        R, K = self.shape
        return R * (K // 2 if self.kind == "mxfp4" else K) + R * (K // 32)
