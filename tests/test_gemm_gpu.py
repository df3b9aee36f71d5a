"""GPU parity of the tcgen05 block-scaled GEMM through the C ABI: against the oracle's
dequantize-then-matmul emulation (double accumulation) within 1e-3 relative Frobenius
error - the tolerance the task states - with f32 output, and against the same
emulation rounded to the output dtype for f16 / bf16."""
import numpy as np
import pytest
import torch

from conftest import rrms
from oracle import oracle as orc
import refgpu

gpu = pytest.mark.gpu
TOL = 1e-3   # relative Frobenius error, the stated bound


def _operands(M, N, K, seed=0, outliers=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", generator=g)
    if outliers:
        ch = torch.randperm(K, device="cuda", generator=g)[: max(1, K // 200)]
        x[:, ch] *= 30
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    return x.bfloat16(), w


def _oracle_out(a, b, bias=None):
    M, K = a.shape
    N = b.shape[0]
    ad = orc.dequantize_nvfp4(a.packed.cpu().numpy(), a.sblk.cpu().numpy(), a.tensor_scale, M, K)
    bd = orc.dequantize_nvfp4(b.packed.cpu().numpy(), b.sblk.cpu().numpy(), b.tensor_scale, N, K)
    return orc.gemm_f64acc(ad, bd, bias, 1.0, threads=orc.host_threads())


def _fro(got, ref):
    return float(np.linalg.norm(got.astype(np.float64) - ref) / np.linalg.norm(ref))


@gpu
@pytest.mark.parametrize("shape", [(1, 128, 64), (3, 136, 192), (17, 512, 1024), (128, 128, 256),
                                   (255, 384, 832), (300, 264, 2048), (512, 1024, 4096)])
@pytest.mark.parametrize("bn", [0, 32, 64, 128, 192, 256])
@pytest.mark.parametrize("pair", [0, 2])
def test_gemm_matches_oracle_f32(shape, bn, pair):
    import thor_fp4
    from thor_fp4 import _ext
    M, N, K = shape
    x, w = _operands(M, N, K, seed=M + N)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    _ext.core().tfp4_set_token_tile(bn)
    _ext.core().tfp4_set_pair_mode(pair)
    try:
        out = a.matmul_t(b, out_dtype="f32")
        torch.cuda.synchronize()
    finally:
        _ext.core().tfp4_set_token_tile(0)
        _ext.core().tfp4_set_pair_mode(-1)
    assert _ext.status() == 0
    assert _fro(out.cpu().numpy(), _oracle_out(a, b)) < TOL


@gpu
@pytest.mark.parametrize("shape", [(129, 64, 64), (256, 256, 256), (257, 72, 320), (300, 264, 2048), (640, 776, 1088),
                                   (1000, 520, 2112), (2048, 1024, 4096)])
@pytest.mark.parametrize("od", ["bf16", "f16", "f32"])
def test_two_cta_kernel_equals_single_cta_kernel(shape, od):
    """The 256x256 two-CTA kernel (TMA-store epilogue, token rows on the MMA's M side) against the
    single-CTA kernel on the same operands: same products, same K order, so equal bits; ragged M,
    N and K tails, bias, all output types."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = shape
    x, w = _operands(M, N, K, seed=M + K, outliers=True)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    bias = torch.randn(N, device="cuda") * 0.01
    outs = []
    L = _ext.core()
    try:
        for mode in (0, 2):
            L.tfp4_set_pair_mode(mode)
            L.tfp4_set_splits(1)
            out = torch.full((M, N), float("nan"), dtype=_ext.OUT_TORCH[od], device="cuda")
            ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, od, bias=bias)
            torch.cuda.synchronize()
            outs.append(out)
    finally:
        L.tfp4_set_pair_mode(-1)
        L.tfp4_set_splits(0)
    assert _ext.status() == 0
    assert torch.equal(outs[0], outs[1])


@gpu
@pytest.mark.parametrize("od,eps", [("f16", 2.0 ** -11), ("bf16", 2.0 ** -8), ("f32", 0.0)])
def test_gemm_out_dtypes_and_bias(od, eps):
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = 200, 136, 640
    x, w = _operands(M, N, K, seed=5, outliers=True)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    bias = torch.randn(N, device="cuda") * 0.01
    out = torch.empty(M, N, dtype=_ext.OUT_TORCH[od], device="cuda")
    ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, od, bias=bias)
    ref = torch.from_numpy(_oracle_out(a, b, bias.cpu().numpy()))
    got = out.float().cpu()
    # one rounding of the exact value to the output dtype: half an ulp relative, plus accumulation noise
    assert ((got - ref).abs() <= (eps + 2e-6) * ref.abs() + 1e-6 * ref.abs().max()).all()
    assert _fro(got.numpy(), ref.to(_ext.OUT_TORCH[od]).float().numpy().astype(np.float64)) < TOL


@gpu
def test_gemm_reference_test_shape_all_dtypes():
    # reference tests/test_quant.py:87-99
    import thor_fp4
    M, N, K = 256, 512, 1024
    a = thor_fp4.NVFP4Tensor.from_float(torch.randn(M, K, device="cuda") * 0.5, 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda") * 0.3, 1.0)
    ref = a.dequantize() @ b.dequantize().t()
    for od in ("f16", "bf16", "f32"):
        assert rrms(a.matmul_t(b, out_dtype=od), ref) < 2e-3


@gpu
def test_gemm_deterministic_and_matches_cublaslt_when_available():
    import thor_fp4
    M, N, K = 384, 512, 2048
    x, w = _operands(M, N, K, seed=11)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    o1 = a.matmul_t(b, out_dtype="bf16").clone()
    o2 = a.matmul_t(b, out_dtype="bf16").clone()
    assert torch.equal(o1, o2)
    if refgpu.lib() is not None:
        refgpu.lib().tfp4_init(32 << 20)
        o3 = torch.empty_like(o1)
        if refgpu.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, o3, M, N, K, "bf16") == 0:
            torch.cuda.synchronize()
            assert rrms(o1, o3) < 2e-3


@gpu
def test_gemm_rejects_bad_shapes():
    import thor_fp4
    from thor_fp4 import _ext, ops
    L = _ext.device_lib()
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    out = torch.zeros(64 * 64, dtype=torch.float32, device="cuda")
    args = lambda M, N, K: (buf.data_ptr(), buf.data_ptr(), 1.0, buf.data_ptr(), buf.data_ptr(), 1.0,
                            out.data_ptr(), M, N, K, 2, _ext.stream())
    assert L.tfp4_gemm(*args(8, 64, 48)) == -3
    assert L.tfp4_gemm(*args(8, 12, 64)) == -6
    assert L.tfp4_gemm(*args(0, 64, 64)) == -6
    assert L.tfp4_gemv(buf.data_ptr(), 9, 64, 0, buf.data_ptr(), buf.data_ptr(), 1.0, out.data_ptr(), 64, 2, _ext.stream()) == -6


@gpu
def test_gemm_full_size_properties():
    """M = N = K = 8192 (the headline shape): the CPU oracle would take minutes, so check
    (a) a random sample of output rows against the oracle, (b) the whole output against
    torch's FP32 matmul of the device-dequantized operands."""
    import thor_fp4
    M = N = K = 8192
    x, w = _operands(M, N, K, seed=3)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    out = a.matmul_t(b, out_dtype="f32")
    ref = a.dequantize() @ b.dequantize().t()
    assert rrms(out, ref) < TOL
    rows = [0, 1, 4095, 8191]
    ad = orc.dequantize_nvfp4(a.packed.cpu().numpy(), a.sblk.cpu().numpy(), 1.0, M, K)[rows]
    bd = orc.dequantize_nvfp4(b.packed.cpu().numpy(), b.sblk.cpu().numpy(), b.tensor_scale, N, K, threads=orc.host_threads())
    sample = orc.gemm_f64acc(ad, bd, None, 1.0, threads=orc.host_threads())
    assert _fro(out[rows].cpu().numpy(), sample) < TOL


@gpu
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("NK", [(512, 1024), (320, 640), (4096, 256), (8, 64)])
def test_gemv_matches_dequant_reference(M, NK):
    # reference tests/test_gemv.py:16-29
    import thor_fp4
    N, K = NK
    w = thor_fp4.NVFP4Tensor.from_float(torch.randn(N, K, device="cuda") * 0.3)
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        x = torch.randn(M, K, device="cuda").to(dt)
        y = thor_fp4.gemv(x, w, "f32")
        assert rrms(y, x.float() @ w.dequantize().t()) < 1e-5
    with pytest.raises(AssertionError):
        thor_fp4.gemv(torch.randn(9, K, device="cuda"), w)


@gpu
@pytest.mark.parametrize("shape", [(64, 256, 512), (300, 384, 1024), (4, 128, 128)])
def test_mx8_gemm_matches_fake_quant(shape):
    # reference tests/test_cutlass.py:39-50 (bound 2e-2 there; the kernel here is exact to bf16 rounding)
    import thor_fp4
    M, N, K = shape
    lin = thor_fp4.Linear(K, N, bias=False, engine="cutlass:mx8").cuda()
    assert lin.engine_kind == "mx8" and lin.out_dtype == "bf16"
    x = torch.randn(M, K, device="cuda")
    y = lin(x)
    ref = thor_fp4.mx_fake_quant(x, "mxfp8") @ thor_fp4.mx_fake_quant(lin.weight.detach(), "mxfp4").t()
    assert rrms(y, ref) < 4e-3


@gpu
def test_starved_wait_gives_up_and_library_recovers():
    """Every device-side wait is bounded.  The test hook 512 makes the producer warps of the two-CTA kernel signal
    nothing and shortens the limit to ~10 ms: the consumers' waits run out, the kernel tears down in order (tensor
    memory freed, both CTAs of each pair leave together), the status word records which role gave up, the next call
    is refused with -8, and after tfp4_clear_status the same operands give the right answer again."""
    import ctypes
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = 512, 512, 1024
    x, w = _operands(M, N, K, seed=9)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    L = _ext.core()

    def raw_gemm():
        return L.tfp4_gemm(a.packed.data_ptr(), a.sblk.data_ptr(), ctypes.c_float(1.0), b.packed.data_ptr(),
                           b.sblk.data_ptr(), ctypes.c_float(b.tensor_scale), out.data_ptr(), M, N, K,
                           _ext.OUT_DTYPE["bf16"], _ext.stream())
    try:
        L.tfp4_set_pair_mode(2)
        L.tfp4_set_debug(512)
        assert raw_gemm() == 0                   # the launch itself succeeds
        torch.cuda.synchronize()                 # returns: nothing hangs
        assert 1 <= _ext.status() <= 10          # code of the role whose wait ran out first
        assert raw_gemm() == -8                  # refused until the status word is cleared
    finally:
        L.tfp4_set_debug(0)
        L.tfp4_clear_status()
    assert _ext.status() == 0
    assert raw_gemm() == 0
    torch.cuda.synchronize()
    L.tfp4_set_pair_mode(0)
    try:
        ref = torch.empty_like(out)
        ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, ref, M, N, K, "bf16")
        torch.cuda.synchronize()
    finally:
        L.tfp4_set_pair_mode(-1)
    assert torch.equal(out, ref)


@gpu
@pytest.mark.parametrize("shape", [(129, 64, 128), (256, 256, 256), (300, 264, 1152), (1000, 520, 2176), (2048, 1024, 4096)])
def test_mx8_two_cta_kernel_equals_single_cta_kernel(shape):
    """MXFP8 x MXFP4 on the 256x256 two-CTA kernel against the single-CTA kernel: equal bits, and both
    within bf16 rounding of the fake-quantized product."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = shape
    x = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.05
    a, b = thor_fp4.MXTensor.from_float(x, "mxfp8"), thor_fp4.MXTensor.from_float(w, "mxfp4")
    L = _ext.core()
    v = L.tfc4_variant_index(thor_fp4.linear.resolve_mx8_variant(K).encode())
    outs = []
    try:
        for mode in (0, 2):
            L.tfp4_set_pair_mode(mode)
            L.tfp4_set_splits(1)
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.gemm_mx(v, a.packed, a.sblk, b.packed, b.sblk, out, M, N, K)
            torch.cuda.synchronize()
            outs.append(out)
    finally:
        L.tfp4_set_pair_mode(-1)
        L.tfp4_set_splits(0)
    assert _ext.status() == 0
    assert torch.equal(outs[0], outs[1])
    ref = thor_fp4.mx_fake_quant(x, "mxfp8") @ thor_fp4.mx_fake_quant(w, "mxfp4").t()
    assert rrms(outs[1], ref) < 4e-3


@gpu
@pytest.mark.parametrize("shape", [(1, 256, 4096), (17, 512, 8192), (128, 384, 2048), (100, 136, 2304)])
@pytest.mark.parametrize("splits", [0, 2, 4, 7])
@pytest.mark.parametrize("od", ["f32", "bf16"])
def test_gemm_split_k_matches_oracle(shape, splits, od):
    """Small batches split K over otherwise idle SMs (f32 partial tiles + a reduction kernel)."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = shape
    x, w = _operands(M, N, K, seed=K + M)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    bias = torch.randn(N, device="cuda") * 0.01
    out = torch.empty(M, N, dtype=_ext.OUT_TORCH[od], device="cuda")
    _ext.core().tfp4_set_splits(splits)
    try:
        ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, od, bias=bias)
        torch.cuda.synchronize()
        again = out.clone()
        ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, od, bias=bias)
        torch.cuda.synchronize()
    finally:
        _ext.core().tfp4_set_splits(0)
    assert _ext.status() == 0
    assert torch.equal(out, again)          # fixed summation order
    ref = _oracle_out(a, b, bias.cpu().numpy())
    assert _fro(out.float().cpu().numpy(), ref) < (TOL if od == "f32" else 3e-3)


@gpu
@pytest.mark.parametrize("M", [1, 16, 100])
@pytest.mark.parametrize("od", ["f32", "bf16"])
def test_gemm_uneven_split_whole_and_cut_tiles(M, od):
    """More output tiles than SMs (160 weight tiles): the tiles that fill a whole wave stay whole, the remaining
    ones are cut along K.  The result must equal the never-split and the all-tiles-cut runs up to the f32
    summation order, be repeatable, and carry the bias exactly once on both kinds of tile."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    N, K = 20480, 5120
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    a = thor_fp4.NVFP4Tensor.from_float(x, 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    del w
    bias = torch.randn(N, device="cuda", generator=g)
    outs = {}
    try:
        for mode in (0, 0, 1, -1):
            _ext.core().tfp4_set_splits(mode)
            out = torch.full((M, N), float("nan"), dtype=_ext.OUT_TORCH[od], device="cuda")
            ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, od, bias=bias)
            torch.cuda.synchronize()
            outs.setdefault(mode, []).append(out)
    finally:
        _ext.core().tfp4_set_splits(0)
    assert _ext.status() == 0
    assert torch.equal(outs[0][0], outs[0][1])
    tol = 2e-6 if od == "f32" else 3e-3
    for mode in (1, -1):
        d = (outs[0][0].float() - outs[mode][0].float()).norm() / outs[mode][0].float().norm()
        assert d.item() < tol, (mode, d.item())
    assert torch.isfinite(outs[0][0].float()).all()
    # first (whole) and last (cut) weight tiles against the dequantized reference
    ref = a.dequantize() @ b.dequantize().t() + bias
    for cols in (slice(0, 256), slice(N - 256, N)):
        d = (outs[0][0][:, cols].float() - ref[:, cols]).norm() / ref[:, cols].norm()
        assert d.item() < (1e-4 if od == "f32" else 5e-3)


@gpu
@pytest.mark.parametrize("M", [64, 2048])
@pytest.mark.parametrize("od", ["f16", "f32"])
def test_gemm_bias_reads_stay_inside_the_vector(M, od):
    """Out-of-bounds bait (the reference's tests/test_fused.py:142-177 places 8192 NaNs right behind its bias
    vector at M > N): the bias handed to the GEMM is the first N floats of a buffer whose every other float is
    NaN, before and after; both epilogues (single-CTA / split-K at M = 64, two-CTA at M = 2048) must stay finite,
    also with N % 32 != 0 where the last column chunk is ragged."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    for N in (1024, 1000):
        K = 512
        x, w = _operands(M, N, K, seed=M + N)
        a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
        b = thor_fp4.NVFP4Tensor.from_float(w, None)
        buf = torch.full((8192 + N + 8192,), float("nan"), device="cuda")
        bias = buf[8192:8192 + N]
        bias.copy_(torch.randn(N, device="cuda") * 0.5)
        out = torch.empty(M, N, dtype=_ext.OUT_TORCH[od], device="cuda")
        ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, od, bias=bias)
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all(), "NaN bait leaked in: out-of-bounds bias read"
        ref = _oracle_out(a, b, bias.cpu().numpy())
        assert _fro(out.float().cpu().numpy(), ref) < (TOL if od == "f32" else 3e-3)


@gpu
@pytest.mark.parametrize("shape", [(1300, 1104, 512), (2048, 768, 256), (700, 2600, 320)])
def test_tile_order_does_not_change_a_bit(shape):
    """The two-CTA kernel walks its output tiles either with the token tiles fastest or in bands of gm token tiles
    (chosen by the host from the L2 footprint for large activations): every order must give the same bits, also when
    the last band is short (6 or 9 token tiles in bands of 4 or 5) and when a band is wider than the matrix."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = shape
    x, w = _operands(M, N, K, seed=N)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    bias = torch.randn(N, device="cuda") * 0.01
    L = _ext.core()
    outs = {}
    try:
        for gm in (-1, 1, 2, 4, 5, 64):
            L.tfp4_set_raster(gm)
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, "bf16", bias=bias)
            torch.cuda.synchronize()
            outs[gm] = out
    finally:
        L.tfp4_set_raster(0)
    assert _ext.status() == 0
    assert torch.isfinite(outs[-1].float()).all()
    for gm, out in outs.items():
        assert torch.equal(out, outs[-1]), f"gm={gm}"


@gpu
@pytest.mark.parametrize("od", ["f32", "bf16"])
def test_slow_epilogue_does_not_change_a_bit(od):
    """Several tiles per CTA pair and an epilogue that holds the accumulator ~40k cycles per tile (test hook 64): the
    main loop then runs into a full pipeline at every tile - all operand stages, scale stages and scale slots filled,
    every producer parked - and restarts in a burst.  The hand-offs between the roles (scale stage back to its
    producer, slot to the loaders, accumulator to the MMA issuer) must hold in that regime too: same bits."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = 8192, 4096, 3584
    x, w = _operands(M, N, K, seed=5)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    L = _ext.core()
    L.tfp4_set_pair_mode(2)
    outs = []
    try:
        for dbg in (0, 64, 64 | 32):
            L.tfp4_set_debug(dbg)
            out = torch.full((M, N), float("nan"), dtype=_ext.OUT_TORCH[od], device="cuda")
            ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, od)
            torch.cuda.synchronize()
            outs.append(out)
    finally:
        L.tfp4_set_debug(0)
        L.tfp4_set_pair_mode(-1)
    assert _ext.status() == 0
    assert torch.isfinite(outs[0].float()).all()
    assert torch.equal(outs[1], outs[0]) and torch.equal(outs[2], outs[0])


@gpu
def test_slow_epilogue_does_not_change_a_bit_mx8():
    """The same stalled-pipeline regime for the MXFP8 x MXFP4 instantiation (one scale atom per part and K block)."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = 8192, 2048, 2048
    x = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.05
    a, b = thor_fp4.MXTensor.from_float(x, "mxfp8"), thor_fp4.MXTensor.from_float(w, "mxfp4")
    L = _ext.core()
    v = L.tfc4_variant_index(thor_fp4.linear.resolve_mx8_variant(K).encode())
    outs = []
    try:
        L.tfp4_set_pair_mode(2)
        for dbg in (0, 64):
            L.tfp4_set_debug(dbg)
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.gemm_mx(v, a.packed, a.sblk, b.packed, b.sblk, out, M, N, K)
            torch.cuda.synchronize()
            outs.append(out)
    finally:
        L.tfp4_set_debug(0)
        L.tfp4_set_pair_mode(-1)
    assert _ext.status() == 0
    assert torch.isfinite(outs[0].float()).all()
    assert torch.equal(outs[0], outs[1])


@gpu
def test_repeated_launches_give_the_same_bits():
    """Fifty launches of a shape with several tiles per CTA pair, each output compared with the first: a hand-off between
    the kernel's roles that held only most of the time would show up here as a launch that differs."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = 8192, 4096, 3584
    x, w = _operands(M, N, K, seed=21)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    first = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, first, M, N, K, "f32")
    out = torch.empty_like(first)
    differing = 0
    for _ in range(50):
        out.fill_(float("nan"))
        ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, "f32")
        differing += int(not torch.equal(out, first))
    assert _ext.status() == 0
    assert differing == 0
