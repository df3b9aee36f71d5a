"""thor_fp4 on B200: NVFP4 linear layers on the sm_100a tensor cores, behind the
thor-fp4 Python API.

    import thor_fp4, torch
    lin = thor_fp4.Linear(4096, 4096).cuda()
    y = lin(torch.randn(256, 4096, device="cuda"))       # quantize + tcgen05 FP4 GEMM
    model = thor_fp4.convert(model, policy="auto")
    rep = thor_fp4.verify(model, x)
    g = thor_fp4.capture_module(model, x)
"""
__version__ = "0.1.0+b200"

from . import ops
from ._ext import cublaslt_version
from .linear import Linear
from .ops import NVFP4Tensor, MXTensor, gemm, gemv, quantize_nvfp4, quantize_mx, dequantize_nvfp4
from .quant import (QATLinear, QATSequential, calibrate_linear, mx_fake_quant,
                    nvfp4_fake_quant, qat, two_level_scale)
from .convert import auto_decision, calibrate, convert, load_shape_table
from .verify import ReferenceLinear, VerifyReport, verify, verify_linear
from .graphs import Graphed, capture_module
from .fused import FusedLinear, GatedMLP, MX8Act, mx8_chain, NVFP4GatedMLP
from .parallel import TensorParallelGatedMLP, shard_rows, shard_cols

__all__ = [
    "Linear", "NVFP4Tensor", "MXTensor", "ops",
    "quantize_nvfp4", "quantize_mx", "dequantize_nvfp4", "gemm", "gemv",
    "nvfp4_fake_quant", "mx_fake_quant", "qat", "two_level_scale",
    "QATLinear", "QATSequential", "calibrate_linear",
    "convert", "calibrate", "auto_decision", "load_shape_table",
    "verify", "verify_linear", "VerifyReport", "ReferenceLinear",
    "Graphed", "capture_module",
    "FusedLinear", "GatedMLP", "MX8Act", "mx8_chain", "NVFP4GatedMLP",
    "TensorParallelGatedMLP", "shard_rows", "shard_cols",
    "cublaslt_version", "__version__",
]
