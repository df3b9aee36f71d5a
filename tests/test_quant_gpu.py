"""GPU parity of the quantizers, called through the C ABI (thor_fp4.ops -> ctypes):
raw code and scale bytes must equal the CPU oracle's, the golden vectors made from the
reference's fake quantizers, and - when oracle/_ref holds the reference's own library
built for sm_100a - the bytes the reference's kernels write on the same GPU."""
import numpy as np
import pytest
import torch

from conftest import bits_to_torch
from oracle import oracle as orc
import refgpu

gpu = pytest.mark.gpu


def _adversarial(R, K, dt):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(R, K, device=dev, generator=g) * torch.logspace(-3, 2, K, device=dev)
    x[0, :64] = 0.0
    x[1, :32] = -0.0
    x[2, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0,
                              -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0], device=dev)
    x[3, :16] = 1e-6
    x[3, 3] = -1e-6                                   # block scale underflows to zero
    x[4, :16] = torch.tensor([0.0] * 5 + [-0.0, 1e-4, -1e-4] + [0.0] * 8, device=dev)
    x[5, 0], x[5, 17], x[5, 33] = float("inf"), float("-inf"), float("nan")
    x[6, :64] = 3000.0 * torch.randn(64, device=dev, generator=g)   # block scale saturates at 448
    if dt == torch.float32:
        x[8, :8] = torch.tensor([1e-45, -1e-45, 1e-40, -1e-40, 1e-38, -1e-38, 3e-39, -3e-39], device=dev)
        x[8, 8:16] = 100.0
        x[9, :16] = torch.tensor([1e-42, -1e-42] * 8, device=dev)
    return x.to(dt).contiguous()


def _check_nv(x, ts, with_ref=True):
    import thor_fp4
    R, K = x.shape
    p, s = thor_fp4.quantize_nvfp4(x, ts)
    torch.cuda.synchronize()
    po, so = orc.quantize_nvfp4(x.float().cpu().numpy(), ts, threads=orc.host_threads())
    assert np.array_equal(p.cpu().numpy(), po), "codes differ from the oracle"
    assert np.array_equal(s.cpu().numpy(), so), "scale bytes differ from the oracle"
    if with_ref and refgpu.lib() is not None:
        pr, sr = refgpu.quant(x, ts)
        torch.cuda.synchronize()
        assert torch.equal(p, pr), "codes differ from the reference's kernel"
        assert torch.equal(s, sr), "scale bytes differ from the reference's kernel"


@gpu
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(300, 1024), (64, 320), (1, 64), (129, 4096), (17, 192)])
@pytest.mark.parametrize("ts", [1.0, "two_level", 3.7, 2.0 ** -7, 1e-30])
def test_nvfp4_bytes_bit_exact(dt, shape, ts):
    R, K = shape
    x = _adversarial(max(R, 16), K, dt)[:R].contiguous()
    if ts == "two_level":
        xf = x.float()
        ts = max(xf[torch.isfinite(xf)].abs().max().item() / (6.0 * 448.0), 1e-30)
    _check_nv(x, float(ts))


@gpu
@pytest.mark.parametrize("K", [320, 1024, 2048])
@pytest.mark.parametrize("mode", ["block", "two"])
def test_golden_fake_quant_vectors(golden, K, mode):
    # reference tests/test_quant.py:13-22: device quantize -> device dequantize == fake quantizer
    import thor_fp4
    x = torch.from_numpy(golden[f"nv_K{K}_x"]).cuda()
    ts = float(golden[f"nv_K{K}_{mode}_ts"])
    p, s = thor_fp4.quantize_nvfp4(x, ts)
    d = thor_fp4.dequantize_nvfp4(p, s, ts, *x.shape)
    assert torch.equal(d.cpu(), torch.from_numpy(golden[f"nv_K{K}_{mode}_y"]))
    assert torch.equal(d, thor_fp4.nvfp4_fake_quant(x, ts))


@gpu
@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_golden_16bit_inputs(golden, kind):
    import thor_fp4
    x = bits_to_torch(golden[f"nv_{kind}_xbits"], kind, "cuda")
    p, s = thor_fp4.quantize_nvfp4(x)
    d = thor_fp4.dequantize_nvfp4(p, s, 1.0, *x.shape)
    assert torch.equal(d.cpu(), torch.from_numpy(golden[f"nv_{kind}_y"]))


@gpu
def test_golden_zero_blocks_tie_and_outliers(golden):
    import thor_fp4
    for key, kind in (("nv_zero", None), ("nv_tie", None), ("nv_outlier", "bf16")):
        x = (torch.from_numpy(golden[f"{key}_x"]).cuda() if kind is None
             else bits_to_torch(golden[f"{key}_xbits"], kind, "cuda"))
        p, s = thor_fp4.quantize_nvfp4(x)
        d = thor_fp4.dequantize_nvfp4(p, s, 1.0, *x.shape)
        assert torch.equal(d.cpu(), torch.from_numpy(golden[f"{key}_y"])), key
    x = bits_to_torch(golden["nv_outlier_xbits"], "bf16", "cuda")
    ts = float(golden["nv_outlier_two_ts"])
    p, s = thor_fp4.quantize_nvfp4(x, ts)
    d = thor_fp4.dequantize_nvfp4(p, s, ts, *x.shape)
    assert torch.equal(d.cpu(), torch.from_numpy(golden["nv_outlier_two_y"]))


@gpu
def test_pad_rows_are_zeroed_even_in_dirty_buffers():
    import thor_fp4
    from thor_fp4 import ops
    R, K = 130, 256
    x = torch.randn(R, K, device="cuda")
    packed = torch.full((ops.packed_bytes(R, K),), 0xA5, dtype=torch.uint8, device="cuda")
    sblk = torch.full((ops.scale_bytes(R, K),), 0xA5, dtype=torch.uint8, device="cuda")
    thor_fp4.quantize_nvfp4(x, 1.0, packed, sblk)
    po, so = orc.quantize_nvfp4(x.cpu().numpy(), 1.0)
    assert np.array_equal(packed.cpu().numpy(), po) and np.array_equal(sblk.cpu().numpy(), so)


@gpu
def test_guard_bands_untouched():
    import thor_fp4
    from thor_fp4 import ops
    R, K = 100, 320
    pb, sb = ops.packed_bytes(R, K), ops.scale_bytes(R, K)
    big_p = torch.full((pb + 512,), 0x5A, dtype=torch.uint8, device="cuda")
    big_s = torch.full((sb + 512,), 0x5A, dtype=torch.uint8, device="cuda")
    thor_fp4.quantize_nvfp4(torch.randn(R, K, device="cuda").half(), 1.0, big_p[256:256 + pb], big_s[256:256 + sb])
    for buf, n in ((big_p, pb), (big_s, sb)):
        assert (buf[:256] == 0x5A).all() and (buf[256 + n:] == 0x5A).all()


@gpu
def test_rejects_bad_k_and_dtypes():
    import thor_fp4
    with pytest.raises(AssertionError, match="multiple of 64"):
        thor_fp4.quantize_nvfp4(torch.randn(8, 48, device="cuda"))


@gpu
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(300, 1024), (64, 320), (5, 128)])
@pytest.mark.parametrize("kind", ["mxfp4", "mxfp8"])
def test_mx_bytes_bit_exact(dt, shape, kind):
    import thor_fp4
    R, K = shape
    x = _adversarial(max(R, 16), K, dt)[:R].contiguous()
    p, s = thor_fp4.quantize_mx(x, kind)
    torch.cuda.synchronize()
    po, so = orc.quantize_mx(x.float().cpu().numpy(), kind)
    per = K // 2 if kind == "mxfp4" else K
    assert np.array_equal(s.cpu().numpy(), so)
    assert np.array_equal(p.cpu().numpy()[: R * per], po[: R * per])
    if refgpu.lib() is not None:
        pr, sr = refgpu.quant_mx(x, kind)
        assert torch.equal(s, sr) and torch.equal(p[: R * per], pr[: R * per])


@gpu
def test_mx_golden(golden):
    import thor_fp4
    from thor_fp4.fused import MX8Act
    x = torch.from_numpy(golden["mx_K512_x"]).cuda()
    p, s = thor_fp4.quantize_mx(x, "mxfp8")
    d = MX8Act(p, s, x.shape).dequant()
    assert torch.equal(d.cpu(), torch.from_numpy(golden["mx_K512_mxfp8_y"]))
    for K in (512, 320):
        x = golden[f"mx_K{K}_x"]
        for kind in ("mxfp4", "mxfp8"):
            p, s = thor_fp4.quantize_mx(torch.from_numpy(x).cuda(), kind)
            d = orc.dequantize_mx(p.cpu().numpy(), s.cpu().numpy(), kind, *x.shape)
            assert np.array_equal(d, golden[f"mx_K{K}_{kind}_y"])


@gpu
def test_mx8_mul_bit_exact():
    import thor_fp4
    from thor_fp4 import ops
    R, K = 200, 512
    a = thor_fp4.MXTensor.from_float(torch.randn(R, K, device="cuda") * 3, "mxfp8")
    b = thor_fp4.MXTensor.from_float(torch.randn(R, K, device="cuda") * 0.1, "mxfp8")
    p, s = ops.mx8_mul(a, b)
    torch.cuda.synchronize()
    po, so = orc.mx8_mul(a.packed.cpu().numpy(), a.sblk.cpu().numpy(), b.packed.cpu().numpy(), b.sblk.cpu().numpy(), R, K)
    assert np.array_equal(p.cpu().numpy()[: R * K], po[: R * K])
    assert np.array_equal(s.cpu().numpy(), so)


@gpu
def test_dequant_and_scale_unscatter_match_oracle():
    import thor_fp4
    from thor_fp4 import ops
    R, K = 300, 1024        # crosses 128-row tiles (reference tests/test_gemv.py:64-77)
    torch.manual_seed(3)
    t = thor_fp4.NVFP4Tensor.from_float(torch.randn(R, K, device="cuda"), None)
    pn, sn = t.packed.cpu().numpy(), t.sblk.cpu().numpy()
    assert np.array_equal(t.dequantize().cpu().numpy(), orc.dequantize_nvfp4(pn, sn, t.tensor_scale, R, K))
    assert np.array_equal(ops.block_scales(t.sblk, R, K).cpu().numpy(), orc.scales_f32(sn, R, K))
    assert np.array_equal(t.gemv_scales().cpu().numpy(), orc.scales_gemv(sn, R, K))
    sf = ops.block_scales(t.sblk, R, K)
    assert 200.0 < sf.max().item() <= 448.0
    assert t.nbytes() == R * K // 2 + R * (K // 16)


@gpu
def test_full_size_round_trip_properties():
    """At the benchmark's size the oracle is too slow; use size-independent properties:
    idempotence (re-quantizing the dequantized tensor reproduces the scale bytes and the
    dequantized values; codes may differ only in the sign of zeros) and agreement with
    the torch fake quantizer on a slab."""
    import thor_fp4
    R, K = 8192, 8192
    x = torch.randn(R, K, device="cuda").bfloat16()
    p, s = thor_fp4.quantize_nvfp4(x)
    d = thor_fp4.dequantize_nvfp4(p, s, 1.0, R, K)
    p2, s2 = thor_fp4.quantize_nvfp4(d)
    assert torch.equal(s, s2)
    assert torch.equal(thor_fp4.dequantize_nvfp4(p2, s2, 1.0, R, K), d)
    assert torch.equal(thor_fp4.nvfp4_fake_quant(x[:256].float()), d[:256])


# --------------------------------------------------------------------------- fused fake quantizer (QAT forward)
@gpu
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("ts", [1.0, "two_level", 0.37, 3.7, 2.0 ** -7])
def test_fake_quant_kernel_equals_oracle_and_torch_chain(dt, ts):
    # one kernel against (a) the CPU oracle's quantize -> dequantize and (b) the torch restatement of the
    # reference's fake quantizer (src/thor_fp4/quant.py:32-53) on the same tensor; bit-exact (-0 == +0)
    import thor_fp4
    from thor_fp4 import ops
    x = _adversarial(300, 1024, dt)
    x[5, 0], x[5, 17], x[5, 33] = 1.0, -2.0, 0.5          # the fake quantizer is defined on finite data
    if ts == "two_level":
        ts = max(x.float().abs().max().item() / (6.0 * 448.0), 1e-30)
    y = ops.fake_quantize_nvfp4(x, float(ts))
    torch.cuda.synchronize()
    assert y.dtype == torch.float32 and y.shape == x.shape
    yo = orc.nvfp4_fake_quant(x.float().cpu().numpy(), float(ts))
    assert torch.equal(y.cpu(), torch.from_numpy(yo)), "differs from the oracle"
    assert torch.equal(y, thor_fp4.nvfp4_fake_quant(x, float(ts))), "differs from the torch chain"


@gpu
@pytest.mark.parametrize("K", [320, 1024, 2048])
@pytest.mark.parametrize("mode", ["block", "two"])
def test_fake_quant_kernel_golden_vectors(golden, K, mode):
    from thor_fp4 import ops
    x = torch.from_numpy(golden[f"nv_K{K}_x"]).cuda()
    ts = float(golden[f"nv_K{K}_{mode}_ts"])
    assert torch.equal(ops.fake_quantize_nvfp4(x, ts).cpu(), torch.from_numpy(golden[f"nv_K{K}_{mode}_y"]))


@gpu
def test_fake_quant_kernel_shapes_outputs_and_errors():
    import thor_fp4
    from thor_fp4 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(3, 5, 48, device="cuda", generator=g)              # any shape, flat 16-element blocks
    y = ops.fake_quantize_nvfp4(x, 0.5)
    assert torch.equal(y, thor_fp4.nvfp4_fake_quant(x, 0.5))
    xb = x.bfloat16()
    yb = ops.fake_quantize_nvfp4(xb, 1.0, out_dtype=torch.bfloat16)     # per-tensor scale 1: values fit bf16 exactly
    assert yb.dtype == torch.bfloat16 and torch.equal(yb.float(), thor_fp4.nvfp4_fake_quant(xb, 1.0))
    big = torch.randn(1 << 22, device="cuda", generator=g) * 4.0         # several grid-stride rounds, ragged tail
    big = big[: (1 << 22) - 16 * 37]
    assert torch.equal(ops.fake_quantize_nvfp4(big, 1.3), thor_fp4.nvfp4_fake_quant(big, 1.3))
    assert ops.fake_quantize_nvfp4(torch.zeros(0, 16, device="cuda")).numel() == 0
    with pytest.raises(AssertionError):
        ops.fake_quantize_nvfp4(torch.zeros(3, 5, device="cuda"))


@gpu
def test_qat_forward_uses_the_kernel_and_gradient_is_straight_through():
    # reference tests/test_qat.py pattern: fake-quantized forward, identity backward
    import thor_fp4
    from thor_fp4 import quant
    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 32).cuda()
    q = quant.qat_linear(lin, two_level=True).cuda()
    x = torch.randn(8, 64, device="cuda", requires_grad=True)
    y = q(x)
    wts = quant.two_level_scale(q.weight)
    want = torch.nn.functional.linear(quant.nvfp4_fake_quant(x.detach()), quant.nvfp4_fake_quant(q.weight.detach(), wts), q.bias)
    assert torch.equal(y, want)
    y.sum().backward()
    assert x.grad is not None and q.weight.grad is not None
    assert torch.allclose(q.weight.grad, x.detach().new_ones(8, 32).t() @ quant.nvfp4_fake_quant(x.detach()))
    v = torch.randn(4, 32, device="cuda", requires_grad=True)
    quant.qat(v, 0.7).backward(torch.full_like(v, 2.0))
    assert torch.equal(v.grad, torch.full_like(v, 2.0))
