"""ctypes binding to libthorfp4_b200.so, the sm_100a engine.

Mirrors the loader interface of the reference binding (src/thor_fp4/_ext.py:103-147
there): ``core()``, ``cutlass()``, ``fused()``, ``stream()`` and the dtype maps.
One shared library serves all three roles.  There is no CPU fallback: if the
library cannot be loaded (or built with nvcc) every op raises.
"""
from __future__ import annotations

import ctypes
import importlib.util
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
_ROOT = _PKG.parent
LIB_PATH = _ROOT / "build" / "libthorfp4_b200.so"

c_void = ctypes.c_void_p
i64 = ctypes.c_int64
c_int = ctypes.c_int
c_float = ctypes.c_float

# name -> (restype, argtypes); also the list the symbol-export test walks
SIGNATURES = {
    "tfp4_init": (c_int, [ctypes.c_size_t]),
    "tfp4_cublaslt_version": (ctypes.c_size_t, []),
    "tfp4_pad_rows": (i64, [i64]),
    "tfp4_packed_bytes": (i64, [i64, i64]),
    "tfp4_scale_bytes": (i64, [i64, i64]),
    "tfp4_mx_packed_bytes": (i64, [i64, i64, c_int]),
    "tfp4_mx_scale_bytes": (i64, [i64, i64]),
    "tfp4_quant": (c_int, [c_void, i64, i64, c_int, c_float, c_void, c_void, c_void]),
    "tfp4_quant_mx": (c_int, [c_void, i64, i64, c_int, c_int, c_void, c_void, c_void]),
    "tfp4_mx8_mul": (c_int, [c_void, c_void, c_void, c_void, c_void, c_void, i64, i64, c_void]),
    "tfp4_gemm": (c_int, [c_void, c_void, c_float, c_void, c_void, c_float, c_void, i64, i64, i64, c_int, c_void]),
    "tfp4_gemm_bias": (c_int, [c_void, c_void, c_float, c_void, c_void, c_float, c_void, c_void,
                               i64, i64, i64, c_int, c_void]),
    "tfp4_linear": (c_int, [c_void, i64, i64, c_int, c_float, c_void, c_void, c_void, c_void, c_float, c_void, c_void,
                            i64, c_int, c_void]),
    "tfp4_act_quant_mx8": (c_int, [c_void, c_void, i64, i64, c_int, c_int, c_void, c_void, c_void]),
    "tfp4_swiglu_quant": (c_int, [c_void, i64, i64, c_int, c_void, c_void, c_void]),
    "tfp4_fake_quant": (c_int, [c_void, i64, c_int, c_float, c_void, c_int, c_void]),
    "tfp4_gemm_noalloc": (c_int, [c_void, c_void, c_float, c_void, c_void, c_float, c_void, c_void,
                                  i64, i64, i64, c_int, c_void]),
    "tfp4_gemm_noalloc_status": (c_int, [c_int]),
    "tfp4_gemm_noalloc_capacity": (ctypes.c_size_t, []),
    "tfp4_gemv": (c_int, [c_void, i64, i64, c_int, c_void, c_void, c_float, c_void, i64, c_int, c_void]),
    "tfp4_scales_gemv": (c_int, [c_void, i64, i64, c_void, c_void]),
    "tfp4_dequant_f32": (c_int, [c_void, c_void, c_float, i64, i64, c_void, c_void]),
    "tfp4_scales_f32": (c_int, [c_void, i64, i64, c_void, c_void]),
    "tfc4_n_variants": (c_int, []),
    "tfc4_variant_name": (ctypes.c_char_p, [c_int]),
    "tfc4_variant_index": (c_int, [ctypes.c_char_p]),
    "tfc4_gemm": (c_int, [c_int, c_void, c_void, c_void, c_void, c_void, i64, i64, i64, c_float, c_void]),
    "tfc4_gemm_ex": (c_int, [c_int, c_void, c_void, c_void, c_void, c_void, c_void, i64, i64, i64, c_float, c_int, c_void]),
    "tfc4f_n_variants": (c_int, []),
    "tfc4f_variant_name": (ctypes.c_char_p, [c_int]),
    "tfc4f_variant_index": (c_int, [ctypes.c_char_p]),
    "tfc4f_sfd_bytes": (i64, [i64, i64]),
    "tfc4f_gemm": (c_int, [c_int, c_void, c_void, c_void, c_void, c_void, c_void, c_void, i64, i64, i64, c_float, c_void]),
    "tfp4_swiglu_gemm": (c_int, [c_void, c_void, c_float, c_void, c_void, c_float, c_void, c_void, i64, i64, i64, c_void]),
    "tfp4_gemm_push": (c_int, [c_void, c_void, c_float, c_void, c_void, c_float, ctypes.POINTER(c_void), c_int, i64, c_int,
                               i64, i64, i64, c_int, c_void]),
    "tfp4_sum_slots": (c_int, [c_void, c_int, i64, i64, c_int, c_void, c_int, c_void]),
    "tfp4_peer_alloc": (c_int, [ctypes.c_size_t, ctypes.POINTER(c_void), ctypes.c_char_p]),
    "tfp4_peer_open": (c_int, [ctypes.c_char_p, ctypes.POINTER(c_void)]),
    "tfp4_peer_close": (c_int, [c_void]),
    "tfp4_peer_copy": (c_int, [c_void, c_void, ctypes.c_size_t, c_void]),
    "tfp4_peer_free": (c_int, [c_void]),
    "tfp4_status": (c_int, []),
    "tfp4_clear_status": (None, []),
    "tfp4_plan_stats": (None, [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]),
    "tfp4_set_token_tile": (None, [c_int]),
    "tfp4_set_pair_mode": (None, [c_int]),
    "tfp4_set_dependent_launch": (None, [c_int]),
    "tfp4_set_splits": (None, [c_int]),
    "tfp4_set_debug": (None, [c_int]),
    "tfp4_set_raster": (None, [c_int]),
    "tfp4_set_quant_tile_rows": (None, [c_int]),
    "tfp4_debug_stats": (c_int, [ctypes.POINTER(ctypes.c_uint64), c_int]),
}

_lib = None
_inited = False


def _build():
    spec = importlib.util.spec_from_file_location("_thorfp4_b200_build", _ROOT / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def core():
    """The loaded library with argtypes declared (no device call is made here)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            try:
                _build()
            except Exception as e:  # noqa: BLE001
                raise RuntimeError(
                    f"thor_fp4: {LIB_PATH} is missing and could not be built with nvcc ({e}); "
                    "this package has no CPU fallback") from e
        L = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def device_lib():
    """core() plus the one-time per-process device initialisation."""
    global _inited
    L = core()
    if not _inited:
        if not torch.cuda.is_available():
            raise RuntimeError("thor_fp4: a CUDA device (sm_100a) is required; there is no CPU fallback")
        rc = L.tfp4_init(0)
        if rc != 0:
            raise RuntimeError(f"tfp4_init rc={rc}")
        _inited = True
    return L


def cutlass():
    """The reference keeps its own tensor-core kernels in a second, optional library;
    here the tfc4_* registry lives in the one library, so this never returns None."""
    return core()


def fused():
    """The reference keeps its fused-epilogue GEMMs (tfc4f_*) in a third, optional library; here they live in the
    one library, so this never returns None."""
    return core()


def cublaslt_version() -> int:
    return int(core().tfp4_cublaslt_version())


def stream() -> int:
    # the raw handle of the current stream without building a torch.cuda.Stream object (called on every launch)
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def status() -> int:
    return int(device_lib().tfp4_status())


def plan_stats() -> tuple[int, int]:
    h, m = ctypes.c_uint64(0), ctypes.c_uint64(0)
    core().tfp4_plan_stats(ctypes.byref(h), ctypes.byref(m))
    return int(h.value), int(m.value)


IN_DTYPE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
OUT_DTYPE = {"f16": 0, "bf16": 1, "f32": 2}
OUT_TORCH = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
