"""numpy front end of the CPU oracle (oracle/nvfp4_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline legs.  The product package never imports it.

All tensors are numpy arrays; 16-bit inputs must be widened to float32 by the
caller (exact, and what the device kernels do on load).  Heavy routines are
split into row ranges and run on a thread pool (ctypes drops the GIL).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liboracle.so"
_lib = None

_u8p = ctypes.POINTER(ctypes.c_uint8)
_f32p = ctypes.POINTER(ctypes.c_float)
_i64 = ctypes.c_int64


def build() -> Path:
    """Compile the C oracle in place (gcc only; no GPU toolchain needed)."""
    src = _HERE / "nvfp4_oracle.c"
    if not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-Wall", "-shared",
                        "-o", str(_LIB_PATH), str(src), "-lm"], check=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = ctypes.CDLL(str(_LIB_PATH))
        L.orc_e2m1_enc.argtypes = [ctypes.c_float]; L.orc_e2m1_enc.restype = ctypes.c_uint8
        L.orc_e2m1_dec.argtypes = [ctypes.c_uint8]; L.orc_e2m1_dec.restype = ctypes.c_float
        L.orc_e4m3_enc.argtypes = [ctypes.c_float]; L.orc_e4m3_enc.restype = ctypes.c_uint8
        L.orc_ue4m3_enc.argtypes = [ctypes.c_float]; L.orc_ue4m3_enc.restype = ctypes.c_uint8
        L.orc_e4m3_dec.argtypes = [ctypes.c_uint8]; L.orc_e4m3_dec.restype = ctypes.c_float
        L.orc_ue8m0_enc.argtypes = [ctypes.c_float]; L.orc_ue8m0_enc.restype = ctypes.c_uint8
        L.orc_ue8m0_enc_ceil.argtypes = [ctypes.c_float]; L.orc_ue8m0_enc_ceil.restype = ctypes.c_uint8
        L.orc_sf_index.argtypes = [_i64, _i64, _i64]; L.orc_sf_index.restype = _i64
        for name in ("orc_pad_rows",):
            getattr(L, name).argtypes = [_i64]; getattr(L, name).restype = _i64
        for name in ("orc_packed_bytes", "orc_scale_bytes", "orc_mx_scale_bytes"):
            getattr(L, name).argtypes = [_i64, _i64]; getattr(L, name).restype = _i64
        L.orc_mx_packed_bytes.argtypes = [_i64, _i64, ctypes.c_int]; L.orc_mx_packed_bytes.restype = _i64
        L.orc_quant_nvfp4_rows.argtypes = [_f32p, _i64, _i64, _i64, ctypes.c_float, _u8p, _u8p]
        L.orc_quant_nvfp4_rows.restype = ctypes.c_int
        L.orc_quant_mx_rows.argtypes = [_f32p, _i64, _i64, _i64, ctypes.c_int, _u8p, _u8p]
        L.orc_quant_mx_rows.restype = ctypes.c_int
        L.orc_quant_mx8_ceil_rows.argtypes = [_f32p, _i64, _i64, _i64, _u8p, _u8p]
        L.orc_quant_mx8_ceil_rows.restype = ctypes.c_int
        L.orc_mx8_mul.argtypes = [_u8p, _u8p, _u8p, _u8p, _u8p, _u8p, _i64, _i64]
        L.orc_mx8_mul.restype = ctypes.c_int
        L.orc_dequant_nvfp4_rows.argtypes = [_u8p, _u8p, ctypes.c_float, _i64, _i64, _i64, _f32p]
        L.orc_dequant_nvfp4_rows.restype = None
        L.orc_dequant_mx.argtypes = [_u8p, _u8p, ctypes.c_int, _i64, _i64, _f32p]
        L.orc_dequant_mx.restype = None
        L.orc_scales_f32.argtypes = [_u8p, _i64, _i64, _f32p]; L.orc_scales_f32.restype = None
        L.orc_scales_gemv.argtypes = [_u8p, _i64, _i64, _u8p]; L.orc_scales_gemv.restype = None
        L.orc_gemm_f64acc_rows.argtypes = [_f32p, _f32p, _f32p, ctypes.c_float, _i64, _i64, _i64, _i64, _f32p]
        L.orc_gemm_f64acc_rows.restype = None
        for name in ("orc_det_exp2", "orc_det_rcp", "orc_det_silu", "orc_det_gelu"):
            getattr(L, name).argtypes = [ctypes.c_float]; getattr(L, name).restype = ctypes.c_float
        L.orc_silu_mul.argtypes = [_f32p, _f32p, _i64, _f32p]; L.orc_silu_mul.restype = None
        L.orc_bias_act_rows.argtypes = [_f32p, _f32p, ctypes.c_int, _i64, _i64, _i64, _f32p]
        L.orc_bias_act_rows.restype = None
        _lib = L
    return _lib


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:  # pragma: no cover
        return max(1, os.cpu_count() or 1)


def _u8(a):
    return a.ctypes.data_as(_u8p)


def _f32(a):
    return a.ctypes.data_as(_f32p)


def _ranges(R: int, threads: int, align: int = 1):
    threads = max(1, min(threads, R))
    step = -(-R // threads)
    step = -(-step // align) * align
    return [(r0, min(R, r0 + step)) for r0 in range(0, R, step)]


def _run(fn, ranges, threads):
    if len(ranges) <= 1 or threads <= 1:
        for r in ranges:
            fn(*r)
        return
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(lambda r: fn(*r), ranges))


# --------------------------------------------------------------------------- sizes
def pad_rows(R): return int(lib().orc_pad_rows(R))
def packed_bytes(R, K): return int(lib().orc_packed_bytes(R, K))
def scale_bytes(R, K): return int(lib().orc_scale_bytes(R, K))
def mx_packed_bytes(R, K, kind): return int(lib().orc_mx_packed_bytes(R, K, 0 if kind in (0, "mxfp4") else 1))
def mx_scale_bytes(R, K): return int(lib().orc_mx_scale_bytes(R, K))


def two_level_scale(x: np.ndarray) -> float:
    """amax/(6*448) in Python double, floored at 1e-30 (src/thor_fp4/quant.py:25-29)."""
    return max(float(np.abs(x.astype(np.float32)).max()) / (6.0 * 448.0), 1e-30)


# --------------------------------------------------------------------------- quantize
def quantize_nvfp4(x: np.ndarray, ts: float = 1.0, threads: int = 1):
    """(R,K) float32 -> (packed uint8[packed_bytes], sblk uint8[scale_bytes])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, K = x.shape
    packed = np.zeros(packed_bytes(R, K), np.uint8)
    sblk = np.zeros(scale_bytes(R, K), np.uint8)
    L = lib()
    rcs = []

    def go(r0, r1):
        rcs.append(L.orc_quant_nvfp4_rows(_f32(x), r0, r1, K, ctypes.c_float(ts), _u8(packed), _u8(sblk)))
    _run(go, _ranges(R, threads), threads)
    if any(rcs):
        raise ValueError(f"orc_quant_nvfp4 rc={rcs}")
    return packed, sblk


def quantize_mx(x: np.ndarray, kind="mxfp4", threads: int = 1):
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, K = x.shape
    k = 0 if kind in (0, "mxfp4") else 1
    packed = np.zeros(mx_packed_bytes(R, K, k), np.uint8)
    sblk = np.zeros(mx_scale_bytes(R, K), np.uint8)
    L = lib()
    rcs = []

    def go(r0, r1):
        rcs.append(L.orc_quant_mx_rows(_f32(x), r0, r1, K, k, _u8(packed), _u8(sblk)))
    _run(go, _ranges(R, threads), threads)
    if any(rcs):
        raise ValueError(f"orc_quant_mx rc={rcs}")
    return packed, sblk


def mx8_mul(ap, as_, bp, bs, R, K):
    op = np.zeros(mx_packed_bytes(R, K, 1), np.uint8)
    os_ = np.zeros(mx_scale_bytes(R, K), np.uint8)
    rc = lib().orc_mx8_mul(_u8(ap), _u8(as_), _u8(bp), _u8(bs), _u8(op), _u8(os_), R, K)
    if rc:
        raise ValueError(f"orc_mx8_mul rc={rc}")
    return op, os_


# --------------------------------------------------------------------------- dequantize
def dequantize_nvfp4(packed, sblk, ts, R, K, threads: int = 1):
    out = np.empty((R, K), np.float32)
    L = lib()
    _run(lambda r0, r1: L.orc_dequant_nvfp4_rows(_u8(packed), _u8(sblk), ctypes.c_float(ts), r0, r1, K, _f32(out)),
         _ranges(R, threads), threads)
    return out


def quantize_mx8_ceil(x: np.ndarray):
    """(R,K) float32 -> MXFP8 codes and UE8M0 scale tiles with the ceil-pow2 block scale (fused-epilogue recipe)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, K = x.shape
    packed = np.zeros(mx_packed_bytes(R, K, 1), np.uint8)
    sblk = np.zeros(mx_scale_bytes(R, K), np.uint8)
    rc = lib().orc_quant_mx8_ceil_rows(_f32(x), 0, R, K, _u8(packed), _u8(sblk))
    if rc:
        raise ValueError(f"orc_quant_mx8_ceil rc={rc}")
    return packed, sblk


def dequantize_mx(packed, sblk, kind, R, K):
    out = np.empty((R, K), np.float32)
    lib().orc_dequant_mx(_u8(packed), _u8(sblk), 0 if kind in (0, "mxfp4") else 1, R, K, _f32(out))
    return out


def scales_f32(sblk, R, K):
    out = np.empty((R, K // 16), np.float32)
    lib().orc_scales_f32(_u8(sblk), R, K, _f32(out))
    return out


def scales_gemv(sblk, R, K):
    out = np.empty((R, K // 16), np.uint8)
    lib().orc_scales_gemv(_u8(sblk), R, K, _u8(out))
    return out


def sf_index(r, s, S):
    return int(lib().orc_sf_index(r, s, S))


def nvfp4_fake_quant(x: np.ndarray, ts: float = 1.0) -> np.ndarray:
    """quantize -> dequantize; what src/thor_fp4/quant.py:32-53 returns."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, K = x.shape
    p, s = quantize_nvfp4(x, ts)
    return dequantize_nvfp4(p, s, ts, R, K)


def mx_fake_quant(x: np.ndarray, kind="mxfp4") -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    R, K = x.shape
    p, s = quantize_mx(x, kind)
    return dequantize_mx(p, s, kind, R, K)


# --------------------------------------------------------------------------- activations of the fused epilogues
_ACT = {"ident": 0, "gelu": 1, "silu": 2, 0: 0, 1: 1, 2: 2}


def silu_mul(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """silu(g) * u in float32 with the library's reproducible silu (the hidden value of the SwiGLU block)."""
    g = np.ascontiguousarray(g, np.float32)
    u = np.ascontiguousarray(u, np.float32)
    out = np.empty_like(g)
    lib().orc_silu_mul(_f32(g), _f32(u), g.size, _f32(out))
    return out


def bias_act(x: np.ndarray, bias, act, threads: int = 1) -> np.ndarray:
    """act(x + bias[col]) in float32; act 'ident' | 'gelu' | 'silu' (the library's reproducible forms)."""
    x = np.ascontiguousarray(x, np.float32)
    R, N = x.shape
    out = np.empty_like(x)
    b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
    L = lib()
    _run(lambda r0, r1: L.orc_bias_act_rows(_f32(x), _f32(b) if b is not None else None, _ACT[act], r0, r1, N, _f32(out)),
         _ranges(R, threads), threads)
    return out


def deinterleave16(gu: np.ndarray):
    """Columns of the stacked gate/up GEMM whose weight rows alternate in blocks of 16 (16 gate features, the 16
    matching up features, ...) -> (gate, up), each (R, N/2)."""
    R, N = gu.shape
    v = gu.reshape(R, N // 32, 2, 16)
    return np.ascontiguousarray(v[:, :, 0, :]).reshape(R, N // 2), np.ascontiguousarray(v[:, :, 1, :]).reshape(R, N // 2)


# --------------------------------------------------------------------------- GEMM emulation
def gemm_f64acc(A, B, bias=None, alpha: float = 1.0, threads: int = 1):
    """alpha * A @ B.T (+bias) with double accumulation; A (M,K), B (N,K) float32."""
    A = np.ascontiguousarray(A, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    M, K = A.shape
    N = B.shape[0]
    out = np.empty((M, N), np.float32)
    bp = _f32(np.ascontiguousarray(bias, np.float32)) if bias is not None else None
    L = lib()
    _run(lambda m0, m1: L.orc_gemm_f64acc_rows(_f32(A), _f32(B), bp, ctypes.c_float(alpha), m0, m1, N, K, _f32(out)),
         _ranges(M, threads), threads)
    return out


def linear_nvfp4(x, w, ts_x=1.0, ts_w=None, bias=None, threads: int = 1, f32_matmul: bool = False):
    """The reference's emulation of one NVFP4 linear layer (src/thor_fp4/verify.py:91-100):
    quantize both operands, dequantize, FP32 matmul out = xd @ wd.T, + bias in f32.

    f32_matmul=True uses numpy's float32 BLAS matmul (the timed CPU baseline);
    otherwise the double-accumulating C loop (the strict checker)."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    if ts_w is None:
        ts_w = two_level_scale(w)
    xp, xs = quantize_nvfp4(x, ts_x, threads)
    wp, ws = quantize_nvfp4(w, ts_w, threads)
    xd = dequantize_nvfp4(xp, xs, ts_x, *x.shape, threads=threads)
    wd = dequantize_nvfp4(wp, ws, ts_w, *w.shape, threads=threads)
    if f32_matmul:
        out = xd @ wd.T
        if bias is not None:
            out = out + np.asarray(bias, np.float32)
        return out
    return gemm_f64acc(xd, wd, bias, 1.0, threads)
