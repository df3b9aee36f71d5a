"""The allocation-free GEMM entry point (tfp4_gemm_noalloc), for hosts that may not allocate device
or pinned memory when they call the library - a server whose device memory was handed out entirely at
start-up, a plug-in running under someone else's allocator, a loop that cannot take the device-wide
synchronisation an allocation implies.  Its scratch (status word, split-K partial sums) is a fixed
array inside the library, shared by all calls.

Checked through the C ABI against the ordinary entry point (tfp4_gemm_bias) and against the CPU oracle
on two calls in a row, with split K active and inactive; the "allocates nothing" claim is checked on the
driver's own free-memory counter (cudaMemGetInfo) in a fresh process, where no earlier call has warmed
anything; a forced K split whose partial sums do not fit is refused (an automatic one holds the cut tiles'
columns only, at most one wave of CTAs of them, which always fits); the sticky status word in the array is set and reset through the bounded-wait test hook.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as orc

gpu = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _call(fn, a, b, bias, out, M, N, K, od):
    from thor_fp4 import _ext
    return fn(a.packed.data_ptr(), a.sblk.data_ptr(), ctypes.c_float(a.tensor_scale),
              b.packed.data_ptr(), b.sblk.data_ptr(), ctypes.c_float(b.tensor_scale),
              bias.data_ptr() if bias is not None else None, out.data_ptr(), M, N, K,
              _ext.OUT_DTYPE[od], _ext.stream())


@gpu
@pytest.mark.parametrize("shape,od", [((16, 512, 8192), "bf16"), ((1, 256, 4096), "f32"), ((300, 264, 1024), "f16"),
                                      ((128, 20480, 5120), "bf16")])
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
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]              # the driver's counter: sees cudaMalloc, not only torch's pool
        assert _call(L.tfp4_gemm_noalloc, a, w, bias, got, M, N, K, od) == 0
        torch.cuda.synchronize()
        if rep == 1:                                      # (the first call of a shape may load kernels lazily)
            assert torch.cuda.mem_get_info()[0] == free0
        assert L.tfp4_gemm_noalloc_status(0) == 0
        diff = (got.float() - ref.float()).pow(2).mean().sqrt() / ref.float().pow(2).mean().sqrt()
        assert diff.item() < 1e-6, (rep, diff.item())    # same kernels, same split: equal to rounding noise
    # the last result against the CPU oracle on sampled columns (all columns for the small layers)
    cols = np.arange(N) if N <= 1024 else np.linspace(0, N - 1, 512).astype(np.int64)
    ad = orc.dequantize_nvfp4(a.packed.cpu().numpy(), a.sblk.cpu().numpy(), 1.0, M, K)
    bd = orc.dequantize_nvfp4(w.packed.cpu().numpy(), w.sblk.cpu().numpy(), w.tensor_scale, N, K,
                              threads=orc.host_threads())[cols]
    want = orc.gemm_f64acc(ad, bd, bias.cpu().numpy()[cols], 1.0, threads=orc.host_threads())
    have = got.float().cpu().numpy()[:, cols]
    err = np.linalg.norm(have - want) / np.linalg.norm(want)
    assert err < (1e-3 if od == "f32" else 3e-3), err


@gpu
def test_noalloc_forced_split_beyond_the_array_is_refused_automatic_split_fits():
    import thor_fp4
    from thor_fp4 import _ext
    L = _ext.device_lib()
    M, N, K = 128, 8192, 8192
    assert L.tfp4_gemm_noalloc_capacity() == (16 << 20) - (16 << 10)
    a = thor_fp4.NVFP4Tensor.from_float(torch.randn(M, K, device="cuda"), 1.0)
    w = thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda") * 0.02, None)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    L.tfp4_set_splits(8)                                  # asked for: 8 x 128 x 8192 x 4 bytes = 32 MiB of partial sums
    try:
        assert _call(L.tfp4_gemm_noalloc, a, w, None, out, M, N, K, "bf16") == -7
    finally:
        L.tfp4_set_splits(0)
    assert _call(L.tfp4_gemm_noalloc, a, w, None, out, M, N, K, "bf16") == 0   # the automatic split fits
    ref = torch.empty_like(out)
    assert _call(L.tfp4_gemm_bias, a, w, None, ref, M, N, K, "bf16") == 0
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


@gpu
def test_noalloc_status_word_is_sticky_and_resettable():
    """The bounded waits of a kernel launched through this entry report to the status word inside the fixed array
    (the regular entry's pinned word stays untouched).  The test hook makes the waits run out after ~10 ms."""
    import thor_fp4
    from thor_fp4 import _ext
    L = _ext.device_lib()
    M, N, K = 512, 512, 1024
    a = thor_fp4.NVFP4Tensor.from_float(torch.randn(M, K, device="cuda"), 1.0)
    w = thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda") * 0.02, None)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    assert L.tfp4_gemm_noalloc_status(0) == 0
    try:
        L.tfp4_set_debug(512)
        assert _call(L.tfp4_gemm_noalloc, a, w, None, out, M, N, K, "bf16") == 0
        torch.cuda.synchronize()                         # returns: nothing hangs
    finally:
        L.tfp4_set_debug(0)
    assert 1 <= L.tfp4_gemm_noalloc_status(0) <= 10      # the role whose wait ran out first; still set
    assert 1 <= L.tfp4_gemm_noalloc_status(1) <= 10      # read and reset
    assert L.tfp4_gemm_noalloc_status(0) == 0
    assert _ext.status() == 0                            # the regular entry's word was never involved
    ref = torch.empty_like(out)
    assert _call(L.tfp4_gemm_noalloc, a, w, None, out, M, N, K, "bf16") == 0
    assert _call(L.tfp4_gemm_bias, a, w, None, ref, M, N, K, "bf16") == 0
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


_FRESH = textwrap.dedent('''
    import ctypes, sys
    sys.path.insert(0, r"{root}/thor-fp4_b200")
    import torch
    import thor_fp4
    from thor_fp4 import _ext
    L = _ext.device_lib()
    torch.manual_seed(0)
    cases = []
    for (M, N, K) in ((16, 512, 8192), (128, 20480, 5120), (300, 264, 1024)):      # split K, uneven cut, two-CTA kernel
        a = thor_fp4.NVFP4Tensor.from_float(torch.randn(M, K, device="cuda"), 1.0)
        w = thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda") * 0.02, None)
        out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        cases.append((a, w, out, M, N, K))
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for rep in range(2):
        for (a, w, out, M, N, K) in cases:          # the very first GEMMs of this process
            rc = L.tfp4_gemm_noalloc(a.packed.data_ptr(), a.sblk.data_ptr(), ctypes.c_float(1.0), w.packed.data_ptr(),
                                     w.sblk.data_ptr(), ctypes.c_float(w.tensor_scale), None, out.data_ptr(), M, N, K,
                                     1, _ext.stream())
            assert rc == 0, rc
    torch.cuda.synchronize()
    free1 = torch.cuda.mem_get_info()[0]
    assert L.tfp4_gemm_noalloc_status(0) == 0
    for (a, w, out, M, N, K) in cases:
        ref = a.dequantize() @ w.dequantize().t()
        err = ((out.float() - ref).norm() / ref.norm()).item()
        assert err < 3e-3, err
    print("FREE", free0, free1)
''')


@gpu
def test_noalloc_first_gemms_of_a_fresh_process_leave_free_memory_unchanged():
    """A fresh process with every kernel loaded at start-up (CUDA_MODULE_LOADING=EAGER, so that lazy loading of a
    kernel's code cannot be mistaken for an allocation): the free device memory the driver reports is the same
    before and after the first GEMMs the process ever runs, all through the allocation-free entry."""
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER")
    r = subprocess.run([sys.executable, "-c", _FRESH.format(root=str(ROOT))], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith("FREE")][-1].split()
    assert int(line[1]) == int(line[2]), f"free device memory changed across the calls: {line[1]} -> {line[2]}"
