"""The allocation-free GEMM entry point (tfp4_gemm_noalloc), for hosts that may not allocate device
or pinned memory when they call the library - a server whose device memory was handed out entirely at
start-up, a plug-in running under someone else's allocator, a loop that cannot take the device-wide
synchronisation an allocation implies.  Its
scratch (status word, split-K partial sums) is a fixed array inside the library, shared by all calls.

Checked through the C ABI against the ordinary entry point (tfp4_gemm_bias) on two calls in a row,
with split K active and inactive, and for the refusal of shapes whose partial sums do not fit.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import pytest
import torch

gpu = pytest.mark.gpu


def _call(fn, a, b, bias, out, M, N, K, od):
    from thor_fp4 import _ext
    return fn(a.packed.data_ptr(), a.sblk.data_ptr(), ctypes.c_float(a.tensor_scale),
              b.packed.data_ptr(), b.sblk.data_ptr(), ctypes.c_float(b.tensor_scale),
              bias.data_ptr() if bias is not None else None, out.data_ptr(), M, N, K,
              _ext.OUT_DTYPE[od], _ext.stream())


@gpu
@pytest.mark.parametrize("shape,od", [((16, 512, 8192), "bf16"), ((1, 256, 4096), "f32"), ((300, 264, 1024), "f16")])
def test_noalloc_matches_regular_entry_twice(shape, od):
    import thor_fp4
    from thor_fp4 import _ext
    L = _ext.device_lib()
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M + K)
    bias = torch.randn(N, device="cuda", generator=g) * 0.01
    w = thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda", generator=g) * 0.02, None)
    for rep in range(2):                                  # two calls in a row share the scratch
        x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
        ref = torch.empty(M, N, dtype=_ext.OUT_TORCH[od], device="cuda")
        got = torch.full((M, N), float("nan"), dtype=_ext.OUT_TORCH[od], device="cuda")
        assert _call(L.tfp4_gemm_bias, a, w, bias, ref, M, N, K, od) == 0
        mem = torch.cuda.memory_allocated()
        assert _call(L.tfp4_gemm_noalloc, a, w, bias, got, M, N, K, od) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == mem
        assert L.tfp4_gemm_noalloc_status(0) == 0
        diff = (got.float() - ref.float()).pow(2).mean().sqrt() / ref.float().pow(2).mean().sqrt()
        assert diff.item() < 1e-6, (rep, diff.item())    # same kernels, same split: equal to rounding noise


@gpu
def test_noalloc_refuses_partial_sums_beyond_the_fixed_array():
    import thor_fp4
    from thor_fp4 import _ext
    L = _ext.device_lib()
    M, N, K = 128, 8192, 8192
    assert L.tfp4_gemm_noalloc_capacity() == (16 << 20) - (16 << 10)
    a = thor_fp4.NVFP4Tensor.from_float(torch.randn(M, K, device="cuda"), 1.0)
    w = thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda") * 0.02, None)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    L.tfp4_set_splits(8)                                  # 8 x 128 x 8192 x 4 bytes = 32 MiB of partial sums
    try:
        assert _call(L.tfp4_gemm_noalloc, a, w, None, out, M, N, K, "bf16") == -7
    finally:
        L.tfp4_set_splits(0)
    assert _call(L.tfp4_gemm_noalloc, a, w, None, out, M, N, K, "bf16") == 0   # automatic split (2) fits
    ref = torch.empty_like(out)
    assert _call(L.tfp4_gemm_bias, a, w, None, ref, M, N, K, "bf16") == 0
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
