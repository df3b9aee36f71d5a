"""CPU tier: the oracle against the reference's own vectors (tests/golden/ref_fakequant.npz,
made by tests/golden/make_golden.py from the reference's torch fake quantizers) and
against the format's known answers.  No GPU, no reference checkout needed."""
import numpy as np
import pytest
import torch

from conftest import bits_to_f32
from oracle import oracle as orc


@pytest.mark.parametrize("K", [320, 1024, 2048])
@pytest.mark.parametrize("mode", ["block", "two"])
def test_nvfp4_matches_reference_fake_quant(golden, K, mode):
    x = golden[f"nv_K{K}_x"]
    ts = float(golden[f"nv_K{K}_{mode}_ts"])
    assert np.array_equal(orc.nvfp4_fake_quant(x, ts), golden[f"nv_K{K}_{mode}_y"])


def test_zero_blocks(golden):
    y = orc.nvfp4_fake_quant(golden["nv_zero_x"])
    assert np.array_equal(y, golden["nv_zero_y"])
    assert np.abs(y[:, 64:]).max() == 0.0


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_16bit_inputs(golden, kind):
    x = bits_to_f32(golden[f"nv_{kind}_xbits"], kind)
    assert np.array_equal(orc.nvfp4_fake_quant(x), golden[f"nv_{kind}_y"])


def test_tie_vector_known_answer(golden):
    # reference tests/test_quant.py:51-61: [0.25, 0.6, 2.6, -6.0] -> [0.5, 0.5, 3.0, -6.0]
    y = orc.nvfp4_fake_quant(golden["nv_tie_x"])
    assert np.array_equal(y, golden["nv_tie_y"])
    assert y[0, :4].tolist() == [0.5, 0.5, 3.0, -6.0]


def test_outlier_channels(golden):
    x = bits_to_f32(golden["nv_outlier_xbits"], "bf16")
    assert np.array_equal(orc.nvfp4_fake_quant(x), golden["nv_outlier_y"])
    ts = float(golden["nv_outlier_two_ts"])
    assert np.array_equal(orc.nvfp4_fake_quant(x, ts), golden["nv_outlier_two_y"])


@pytest.mark.parametrize("K", [512, 320])
@pytest.mark.parametrize("kind", ["mxfp4", "mxfp8"])
def test_mx_matches_reference_fake_quant(golden, K, kind):
    assert np.array_equal(orc.mx_fake_quant(golden[f"mx_K{K}_x"], kind), golden[f"mx_K{K}_{kind}_y"])


def test_config1_slab_matches_reference_emulation(golden):
    x = bits_to_f32(golden["cfg1_xbits"], "bf16")
    out = orc.linear_nvfp4(x, golden["cfg1_w"], float(golden["cfg1_tsx"]), float(golden["cfg1_tsw"]))
    ref = golden["cfg1_out"]
    assert np.abs(out - ref).max() <= 1e-5 * np.abs(ref).max()


def test_two_level_scale_range():
    # reference tests/test_quant.py:72-75: largest block scale lands in (200, 448]
    x = np.random.default_rng(1).standard_normal((128, 512)).astype(np.float32)
    p, s = orc.quantize_nvfp4(x, orc.two_level_scale(x))
    sf = orc.scales_f32(s, 128, 512)
    assert 200.0 < sf.max() <= 448.0


def test_e2m1_edge_codes():
    L = orc.lib()
    inf, nan = float("inf"), float("nan")
    cases = {nan: 0x7, -inf: 0xF, inf: 0x7, -0.1: 0x8, -0.0: 0x0, 1.25: 0x3, 2.5: 0x5, 5.0: 0x7,
             0.25: 0x1, 0.2499999: 0x0, 0.75: 0x2, 1.75: 0x4, 3.5: 0x6, -6.5: 0xF}
    for v, code in cases.items():
        assert L.orc_e2m1_enc(v) == code, (v, code)


def test_e4m3_encode_all_codes_round_trip_and_rne():
    L = orc.lib()
    vals = [L.orc_e4m3_dec(b) for b in range(0x7F)]
    for b, v in enumerate(vals):
        assert L.orc_e4m3_enc(v) == b
    t = torch.rand(20000, dtype=torch.float32) * 460.0
    ref = t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([L.orc_e4m3_enc(float(v)) for v in t.numpy()], np.uint8)
    assert np.array_equal(got, ref)
    assert L.orc_e4m3_enc(1e9) == 0x7E and L.orc_e4m3_enc(float("inf")) == 0x7E
    assert L.orc_e4m3_enc(2.0 ** -10) == 0 and L.orc_e4m3_enc(2.0 ** -10 * 1.01) == 1


def test_ue8m0_rules():
    L = orc.lib()
    assert L.orc_ue8m0_enc(1.0) == 127 and L.orc_ue8m0_enc(1.49) == 127 and L.orc_ue8m0_enc(1.5) == 128
    assert L.orc_ue8m0_enc(0.0) == 0 and L.orc_ue8m0_enc(-1.0) == 0
    assert L.orc_ue8m0_enc_ceil(1.0) == 127 and L.orc_ue8m0_enc_ceil(1.0001) == 128


def test_zero_scale_block_raw_bytes():
    # amax*(1/6) <= 2^-10 encodes scale 0; x/0 gives +-inf or NaN -> magnitude code 7
    x = np.zeros((1, 64), np.float32)
    x[0, :4] = [1e-6, -1e-6, 0.0, -0.0]
    p, s = orc.quantize_nvfp4(x, 1.0)
    assert s[orc.sf_index(0, 0, 4)] == 0
    assert p[0] == 0xF7 and p[1] == 0x77
    assert np.abs(orc.dequantize_nvfp4(p, s, 1.0, 1, 64)).max() == 0.0


def test_layout_index_and_sizes():
    S = 64
    seen = {orc.sf_index(r, s, S) for r in range(300) for s in range(S)}
    assert len(seen) == 300 * S and max(seen) < orc.scale_bytes(300, 1024)
    assert orc.sf_index(0, 0, S) == 0 and orc.sf_index(1, 0, S) == 16 and orc.sf_index(32, 0, S) == 4
    assert orc.sf_index(0, 1, S) == 1 and orc.sf_index(0, 4, S) == 512 and orc.sf_index(128, 0, S) == (S // 4) * 512
    assert orc.packed_bytes(5, 128) == 128 * 64 and orc.scale_bytes(5, 128) == 128 * 8
    assert orc.mx_packed_bytes(64, 512, "mxfp8") == 128 * 512 and orc.mx_scale_bytes(64, 512) == 128 * 16


def test_rejects_bad_k():
    with pytest.raises(ValueError):
        orc.quantize_nvfp4(np.zeros((8, 48), np.float32))


def test_exact16_fast_path_equivalence_exhaustive():
    """The device quantizer's 16-bit fast path replaces RN(x/ds) by x * rb,
    rb = RN(1/ds) * (1 + 2^-21), and converts with round-to-nearest-even.  Check on every
    finite bf16 and f16 magnitude x every positive UE4M3 scale that the code equals the
    reference rule (threshold compares on the IEEE quotient, ties up)."""
    cuts = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    scales = torch.arange(1, 0x7F, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    for dt in (torch.bfloat16, torch.float16):
        bits = torch.arange(0, 0x7F80 if dt == torch.bfloat16 else 0x7C00, dtype=torch.int32).to(torch.int16)
        x = bits.view(dt).float()[:, None]
        for chunk in scales.split(16):
            ds = chunk[None, :]
            ref = torch.bucketize((x / ds).clamp_max(6.0), cuts, right=True)
            rb = (1.0 / ds) * (1.0 + 2.0 ** -21)
            y = (x * rb).clamp_max(6.0)
            # round-to-nearest-even onto the e2m1 grid
            lo = torch.bucketize(y, grid, right=True) - 1
            hi = (lo + 1).clamp_max(7)
            dlo, dhi = y - grid[lo], grid[hi] - y
            fast = torch.where(dhi < dlo, hi, lo)
            tie = (dhi == dlo) & (hi != lo)
            fast = torch.where(tie, torch.where(lo % 2 == 0, lo, hi), fast)
            assert torch.equal(fast, ref), str(dt)
            assert not tie.any()


def test_mx8_ceil_scale_quantizer_against_torch_float8():
    """Ceil-pow2 block scale (the reference's fused-epilogue / mx8_mul recipe, csrc/thor_fp4_core.cu:612-652):
    scale byte = smallest power of two >= amax/448, codes = e4m3(x / scale) - so nothing saturates, and the
    codes equal torch's float8_e4m3fn cast of the scaled values."""
    import torch
    rng = np.random.default_rng(7)
    R, K = 200, 256
    x = (rng.standard_normal((R, K)) * np.exp(rng.uniform(-6, 6, (R, 1)))).astype(np.float32)
    x[3, :32] = 0.0                                   # an all-zero block
    x[5, 40] = 448.0 * 4                              # amax exactly on a power of two times 448
    p, s = orc.quantize_mx8_ceil(x)
    d = orc.dequantize_mx(p, s, "mxfp8", R, K)
    blocks = x.reshape(R, K // 32, 32)
    amax = np.abs(blocks).max(-1)
    dblocks = d.reshape(R, K // 32, 32)
    nz = amax > 0
    scale = np.where(nz, 2.0 ** np.ceil(np.log2(np.where(nz, amax, 1.0) / 448.0)), 1.0)
    want = torch.from_numpy((blocks / scale[..., None]).astype(np.float32)).to(torch.float8_e4m3fn).float().numpy() * scale[..., None]
    assert np.array_equal(dblocks[nz], want[nz].astype(np.float32))
    assert np.all(np.abs(dblocks) <= 448.0 * scale[..., None])
    assert not dblocks[3, 0].any()
    # within half an e4m3 step (2^-4 relative) of the input wherever the input is not tiny next to its block's amax
    big = np.abs(blocks) > amax[..., None] * 2.0 ** -6
    assert np.max(np.abs(dblocks - blocks)[big] / np.abs(blocks)[big]) <= 2.0 ** -4 + 1e-7


def test_reproducible_activations_are_silu_and_gelu():
    """The activations of the fused epilogues are defined by this build (the reference's live in un-vendored CUTLASS
    and are pinned only by tolerances): built from correctly rounded FP32 operations so that CPU and GPU agree bit for
    bit.  Here: they are silu and gelu to FP32 working accuracy, and well behaved at the edges."""
    import math
    L = orc.lib()
    xs = np.concatenate([np.linspace(-30, 30, 4001), np.array([0.0, -0.0, 1e-30, -1e-30, 88.0, -88.0, 1e4, -1e4])]).astype(np.float32)
    for x in xs:
        x = float(x)
        s_ref = x / (1.0 + math.exp(-x)) if x > -700 else 0.0
        g_ref = 0.5 * x * (1.0 + math.erf(x / math.sqrt(2.0)))
        s, g = L.orc_det_silu(x), L.orc_det_gelu(x)
        assert abs(s - s_ref) <= 3e-6 * abs(s_ref) + 1e-30, (x, s, s_ref)
        assert abs(g - g_ref) <= 5e-7 * max(1.0, abs(x)), (x, g, g_ref)
    assert L.orc_det_exp2(0.0) == 1.0 and L.orc_det_exp2(3.0) == 8.0 and L.orc_det_exp2(-2.0) == 0.25
    assert abs(L.orc_det_rcp(3.0) - 1.0 / 3.0) < 1e-7
    assert math.isnan(L.orc_det_silu(float("nan"))) and L.orc_det_silu(float("inf")) == float("inf")
    g = np.array([[1.0, -2.0, 0.5, 30.0]], np.float32)
    u = np.array([[2.0, 3.0, -4.0, 0.1]], np.float32)
    h = orc.silu_mul(g, u)
    assert np.allclose(h, (g / (1 + np.exp(-g))) * u, rtol=2e-6)
    gu = np.arange(2 * 64, dtype=np.float32).reshape(2, 64)
    gate, up = orc.deinterleave16(gu)
    assert gate[0, :16].tolist() == list(range(16)) and up[0, :16].tolist() == list(range(16, 32))
    assert gate[0, 16:].tolist() == list(range(32, 48)) and up[1, 16:].tolist() == list(range(64 + 48, 128))
