"""Parity at the benchmark configurations' own shapes, through the public API and the C ABI.

The CPU oracle's double-accumulating GEMM would take minutes on these sizes, so each case checks
  (a) a seeded sample of output rows x columns against the oracle (operands dequantized by the oracle
      from the very bytes the device holds, products accumulated in double), and
  (b) the whole output against an FP32 matmul of the device-dequantized operands.
f32 outputs are held to the stated relative Frobenius bound 1e-3; f16 / bf16 outputs to "the exact
value rounded once to the output type" (half an ulp relative, plus FP32 accumulation noise).
"""
import numpy as np
import pytest
import torch

from conftest import rrms
from oracle import oracle as orc

gpu = pytest.mark.gpu
TOL = 1e-3
HALF_ULP = {"f16": 2.0 ** -11, "bf16": 2.0 ** -8, "f32": 0.0}


def _outlier_channels(x, frac, mul, gen):
    k = x.shape[1]
    ch = torch.randperm(k, device=x.device, generator=gen)[: max(1, int(k * frac))]
    x[:, ch] *= mul
    return x


def _sample(n, count, gen):
    if n <= count:
        return np.arange(n)
    idx = torch.randperm(n, generator=gen)[:count].sort().values.numpy()
    idx[0], idx[-1] = 0, n - 1          # always the first and the last row / column
    return idx


def _fro(got, ref):
    return float(np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-30))


def _assert_rounded_once(got, ref, od, K=640):
    """got (output dtype, widened) equals ref (f32 from double accumulation) rounded once to the output type.
    The slack beside the half ulp is the FP32 accumulation noise of the tensor cores, a random walk over K."""
    got, ref = torch.as_tensor(got).float(), torch.as_tensor(ref).float()
    bound = (HALF_ULP[od] + 2e-6) * ref.abs() + 1e-6 * max(1.0, (K / 640.0) ** 0.5) * ref.abs().max()
    bad = (got - ref).abs() > bound
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} elements off by more than one rounding"


# ------------------------------------------------------------------------------------------ config 1
@gpu
def test_config1_cpu_runnable_emulation_full():
    """bf16 [256, 4096] ~N(0,1) with a two-level activation scale amax/(6*448), W [4096, 4096] ~N(0,0.02),
    FP32 output, no bias, seed 0: every output element against the oracle's emulation of the layer."""
    import thor_fp4
    from thor_fp4 import ops
    torch.manual_seed(0)
    M, K, N = 256, 4096, 4096
    x = torch.randn(M, K).bfloat16()
    w = torch.randn(N, K) * 0.02
    ts_x = orc.two_level_scale(x.float().numpy())
    ts_w = orc.two_level_scale(w.numpy())
    a = thor_fp4.NVFP4Tensor.from_float(x.cuda().float(), ts_x)
    b = thor_fp4.NVFP4Tensor.from_float(w.cuda(), None)
    assert b.tensor_scale == pytest.approx(ts_w, rel=1e-7)
    # codes and scale bytes of both operands: bit-exact with the oracle's quantizer
    xp, xs = orc.quantize_nvfp4(x.float().numpy(), ts_x, orc.host_threads())
    wp, ws = orc.quantize_nvfp4(w.numpy(), b.tensor_scale, orc.host_threads())
    assert np.array_equal(a.packed.cpu().numpy(), xp) and np.array_equal(a.sblk.cpu().numpy(), xs)
    assert np.array_equal(b.packed.cpu().numpy(), wp) and np.array_equal(b.sblk.cpu().numpy(), ws)
    out = torch.empty(M, N, device="cuda")
    ops.gemm(a.packed, a.sblk, a.tensor_scale, b.packed, b.sblk, b.tensor_scale, out, M, N, K, "f32")
    ref = orc.linear_nvfp4(x.float().numpy(), w.numpy(), ts_x, b.tensor_scale, None, threads=orc.host_threads())
    assert _fro(out.cpu().numpy(), ref) < TOL
    # the same layer through the module API
    lin = thor_fp4.Linear(K, N, bias=False, out_dtype="f32", act_tensor_scale=ts_x, device="cuda")
    with torch.no_grad():
        lin.weight.copy_(w)
    lin.refresh_weight()
    assert torch.equal(lin(x.cuda()), out)


# ------------------------------------------------------------------------------------------ config 3
_GRID = [(4096, 5120), (5120, 20480), (20480, 5120), (8192, 28672), (28672, 8192)]
_weights = {}


def _layer(K, N):
    """One quantized weight per (K, N), with its oracle dequantization (cached over the M cases)."""
    import thor_fp4
    if (K, N) not in _weights:
        _weights.clear()                         # one layer resident at a time
        g = torch.Generator(device="cuda").manual_seed(K + N)
        w = (torch.rand(N, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5      # Kaiming-uniform(a = sqrt 5)
        b = thor_fp4.NVFP4Tensor.from_float(w, None)
        del w
        bias = torch.randn(N, device="cuda", generator=g) * 0.01
        bd = orc.dequantize_nvfp4(b.packed.cpu().numpy(), b.sblk.cpu().numpy(), b.tensor_scale, N, K,
                                  threads=orc.host_threads())
        _weights[(K, N)] = (b, bias, bd)
    return _weights[(K, N)]


@gpu
@pytest.mark.parametrize("M", [1, 16, 128, 2048])        # varies fastest: one weight serves its four batch sizes
@pytest.mark.parametrize("KN", _GRID)
def test_config3_feed_forward_grid_f16_bias_outliers(KN, M):
    """Feed-forward shape sweep: activations ~N(0,1) with 0.5% of the K channels x30, bias ~N(0,0.01), f16 out."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    K, N = KN
    b, bias, bd = _layer(K, N)
    g = torch.Generator(device="cuda").manual_seed(M + K)
    x = _outlier_channels(torch.randn(M, K, device="cuda", generator=g), 0.005, 30.0, g).bfloat16()
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, out, M, N, K, "f16", bias=bias)
    torch.cuda.synchronize()
    assert _ext.status() == 0
    cg = torch.Generator().manual_seed(N + M)
    rows, cols = _sample(M, 24, cg), _sample(N, 384, cg)
    ad = orc.dequantize_nvfp4(a.packed.cpu().numpy(), a.sblk.cpu().numpy(), 1.0, M, K)[rows]
    ref = orc.gemm_f64acc(ad, bd[cols], bias.cpu().numpy()[cols], 1.0, threads=orc.host_threads())
    got = out.cpu()[rows][:, cols]
    _assert_rounded_once(got, ref, "f16", K)
    # every element: FP32 matmul of the device-dequantized operands (its own summation noise ~1e-6), f16 rounding on top
    full = a.dequantize() @ b.dequantize().t() + bias
    assert rrms(out, full) < 4e-4
    assert torch.isfinite(out.float()).all()


@gpu
def test_config3_largest_batch_through_linear():
    """M = 8192 on the widest layer of the grid, through thor_fp4.Linear (bias, f16)."""
    import thor_fp4
    K, N, M = 8192, 28672, 8192
    b, bias, bd = _layer(K, N)
    g = torch.Generator(device="cuda").manual_seed(77)
    x = _outlier_channels(torch.randn(M, K, device="cuda", generator=g), 0.005, 30.0, g).bfloat16()
    lin = thor_fp4.Linear(K, N, bias=True, out_dtype="f16", device="cuda")
    lin.load_quantized_state({"weight_fp4": b.state_dict(), "bias": bias})     # the codes are used as they are
    out = lin(x)
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    cg = torch.Generator().manual_seed(5)
    rows, cols = _sample(M, 16, cg), _sample(N, 256, cg)
    ad = orc.dequantize_nvfp4(a.packed.cpu().numpy(), a.sblk.cpu().numpy(), 1.0, M, K,
                              threads=orc.host_threads())[rows]
    ref = orc.gemm_f64acc(ad, bd[cols], bias.cpu().numpy()[cols], 1.0, threads=orc.host_threads())
    _assert_rounded_once(out.cpu()[rows][:, cols], ref, "f16", K)
    _weights.clear()


# ------------------------------------------------------------------------------------------ config 4
@gpu
def test_config4_mxfp8_act_mxfp4_weight_full_shape():
    """[4096, 8192] MXFP8 activations (0.1% outlier channels x50) x [28672, 8192] MXFP4 weights, bf16 out:
    the sampled outputs are the exact product of the dequantized operands rounded once to bf16, and the
    NVFP4 x NVFP4 product of the same data is compared alongside."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, K, N = 4096, 8192, 28672
    g = torch.Generator(device="cuda").manual_seed(4)
    x = _outlier_channels(torch.randn(M, K, device="cuda", generator=g), 0.001, 50.0, g)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    a8, w4 = thor_fp4.MXTensor.from_float(x, "mxfp8"), thor_fp4.MXTensor.from_float(w, "mxfp4")
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    v = _ext.device_lib().tfc4_variant_index(thor_fp4.linear.resolve_mx8_variant(K).encode())
    ops.gemm_mx(v, a8.packed, a8.sblk, w4.packed, w4.sblk, out, M, N, K)
    torch.cuda.synchronize()
    assert _ext.status() == 0
    cg = torch.Generator().manual_seed(44)
    rows, cols = _sample(M, 24, cg), _sample(N, 384, cg)
    ad = orc.dequantize_mx(a8.packed.cpu().numpy(), a8.sblk.cpu().numpy(), "mxfp8", M, K)[rows]
    bd = orc.dequantize_mx(w4.packed.cpu().numpy(), w4.sblk.cpu().numpy(), "mxfp4", N, K)[cols]
    ref = orc.gemm_f64acc(ad, bd, None, 1.0, threads=orc.host_threads())
    _assert_rounded_once(out.cpu()[rows][:, cols], ref, "bf16", K)
    # against the unquantized product: both formats, same data (the comparison the configuration asks for)
    exact = (x[rows] @ w.t())[:, cols].cpu()
    e_mx = ((out.cpu()[rows][:, cols].float() - exact).norm() / exact.norm()).item()
    an, wn = thor_fp4.NVFP4Tensor.from_float(x, 1.0), thor_fp4.NVFP4Tensor.from_float(w, None)
    outn = an.matmul_t(wn, out_dtype="bf16")
    e_nv = ((outn.cpu()[rows][:, cols].float() - exact).norm() / exact.norm()).item()
    assert e_mx < 0.2 and e_nv < 0.2, (e_mx, e_nv)       # quantization error of 4-bit weights, not a parity bound


@gpu
@pytest.mark.parametrize("shape", [(64, 256, 512), (300, 384, 1024), (4, 128, 128), (1000, 520, 2176)])
def test_mx_gemm_is_exact_product_rounded_once(shape):
    """MXFP8 x MXFP4 at small shapes, every element: the oracle's double-accumulated product of the dequantized
    operands, rounded once to bf16 (both kernels: small batches take the single-CTA one)."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    a8, w4 = thor_fp4.MXTensor.from_float(x, "mxfp8"), thor_fp4.MXTensor.from_float(w, "mxfp4")
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    v = _ext.device_lib().tfc4_variant_index(thor_fp4.linear.resolve_mx8_variant(K).encode())
    ops.gemm_mx(v, a8.packed, a8.sblk, w4.packed, w4.sblk, out, M, N, K)
    torch.cuda.synchronize()
    ad = orc.dequantize_mx(a8.packed.cpu().numpy(), a8.sblk.cpu().numpy(), "mxfp8", M, K)
    bd = orc.dequantize_mx(w4.packed.cpu().numpy(), w4.sblk.cpu().numpy(), "mxfp4", N, K)
    ref = orc.gemm_f64acc(ad, bd, None, 1.0, threads=orc.host_threads())
    _assert_rounded_once(out.cpu(), ref, "bf16", K)
