"""Test helper: ctypes handle on the reference project's own core library compiled for
sm_100a (oracle/_ref/libthorfp4_ref_core.so, built by oracle/build_ref.sh).  Used only
as a byte-level checker and as the same-box baseline; returns None when absent."""
import ctypes
from pathlib import Path

import torch

_PATH = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libthorfp4_ref_core.so"
_lib = None
c_void, i64, c_int, c_float = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float


def lib():
    global _lib
    if _lib is None:
        if not _PATH.exists():
            return None
        L = ctypes.CDLL(str(_PATH))
        L.tfp4_init.argtypes = [ctypes.c_size_t]; L.tfp4_init.restype = c_int
        L.tfp4_packed_bytes.argtypes = [i64, i64]; L.tfp4_packed_bytes.restype = i64
        L.tfp4_scale_bytes.argtypes = [i64, i64]; L.tfp4_scale_bytes.restype = i64
        L.tfp4_mx_packed_bytes.argtypes = [i64, i64, c_int]; L.tfp4_mx_packed_bytes.restype = i64
        L.tfp4_mx_scale_bytes.argtypes = [i64, i64]; L.tfp4_mx_scale_bytes.restype = i64
        L.tfp4_quant.argtypes = [c_void, i64, i64, c_int, c_float, c_void, c_void, c_void]; L.tfp4_quant.restype = c_int
        L.tfp4_quant_mx.argtypes = [c_void, i64, i64, c_int, c_int, c_void, c_void, c_void]; L.tfp4_quant_mx.restype = c_int
        L.tfp4_mx8_mul.argtypes = [c_void] * 6 + [i64, i64, c_void]; L.tfp4_mx8_mul.restype = c_int
        L.tfp4_gemm.argtypes = [c_void, c_void, c_float, c_void, c_void, c_float, c_void, i64, i64, i64, c_int, c_void]
        L.tfp4_gemm.restype = c_int
        L.tfp4_dequant_f32.argtypes = [c_void, c_void, c_float, i64, i64, c_void, c_void]; L.tfp4_dequant_f32.restype = c_int
        _lib = L
    return _lib


_IN = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def quant(x: torch.Tensor, ts: float = 1.0):
    L = lib()
    R, K = x.shape
    packed = torch.zeros(L.tfp4_packed_bytes(R, K), dtype=torch.uint8, device=x.device)
    sblk = torch.zeros(L.tfp4_scale_bytes(R, K), dtype=torch.uint8, device=x.device)
    rc = L.tfp4_quant(x.data_ptr(), R, K, _IN[x.dtype], ts, packed.data_ptr(), sblk.data_ptr(), _stream())
    assert rc == 0, rc
    return packed, sblk


def quant_mx(x: torch.Tensor, kind: str):
    L = lib()
    R, K = x.shape
    k = 0 if kind == "mxfp4" else 1
    packed = torch.zeros(L.tfp4_mx_packed_bytes(R, K, k), dtype=torch.uint8, device=x.device)
    sblk = torch.zeros(L.tfp4_mx_scale_bytes(R, K), dtype=torch.uint8, device=x.device)
    rc = L.tfp4_quant_mx(x.data_ptr(), R, K, _IN[x.dtype], k, packed.data_ptr(), sblk.data_ptr(), _stream())
    assert rc == 0, rc
    return packed, sblk


def gemm(pA, sA, tsA, pB, sB, tsB, out, M, N, K, out_dtype):
    """cuBLASLt NVFP4 through the reference's own tfp4_gemm; returns its rc."""
    L = lib()
    return L.tfp4_gemm(pA.data_ptr(), sA.data_ptr(), tsA, pB.data_ptr(), sB.data_ptr(), tsB,
                       out.data_ptr(), M, N, K, {"f16": 0, "bf16": 1, "f32": 2}[out_dtype], _stream())
