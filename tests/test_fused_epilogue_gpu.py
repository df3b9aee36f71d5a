"""GPU parity of the GEMMs that quantize their own output in the epilogue, through the C ABI.

tfp4_swiglu_gemm (gate/up GEMM -> silu(gate) * up -> NVFP4 codes + UE4M3 scale tiles of h) and tfc4f_gemm (MXFP8 x
MXFP4 GEMM -> bias + gelu / silu / identity -> MXFP8 codes + UE8M0 scale tiles) are checked BYTE FOR BYTE: the same
kernel run with a plain FP32 output exposes the accumulator values, and the CPU oracle applies to them the recipe the
epilogue implements (reproducible activations of oracle/nvfp4_oracle.c, then the reference's quantizer arithmetic).
The reference pins its fused epilogues only by tolerances (tests/test_fused.py:73-76 of the reference project: 0.05 for
a layer, 0.12 for the gated block); those bounds are kept as a second check against float references.
"""
import ctypes

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import rrms
from oracle import oracle as orc

gpu = pytest.mark.gpu


def _f32_gemm_nv(a, w, M):
    """FP32 output of the NVFP4 GEMM with the K order of the two-CTA kernel (no split K)."""
    from thor_fp4 import ops, _ext
    N, K = w.shape
    out = torch.empty(M, N, device="cuda")
    L = _ext.core()
    L.tfp4_set_splits(1)
    try:
        ops.gemm(a.packed, a.sblk, 1.0, w.packed, w.sblk, w.tensor_scale, out, M, N, K, "f32")
        torch.cuda.synchronize()
    finally:
        L.tfp4_set_splits(0)
    return out


@gpu
@pytest.mark.parametrize("M,I,K", [(300, 192, 512), (128, 64, 256), (1000, 1024, 1024), (17, 128, 320), (256, 4096, 256),
                                   (129, 320, 64)])
def test_swiglu_gemm_bytes_match_oracle(M, I, K):
    import thor_fp4
    from thor_fp4 import ops, _ext
    g = torch.Generator(device="cuda").manual_seed(M + I + K)
    x = torch.randn(M, K, device="cuda", generator=g)
    x[:, ::97] *= 20.0                                            # outlier channels: a wide range of gate values
    wg = torch.randn(I, K, device="cuda", generator=g) * 0.08
    wu = torch.randn(I, K, device="cuda", generator=g) * 0.08
    a = thor_fp4.NVFP4Tensor.from_float(x.bfloat16().float(), 1.0)
    w = thor_fp4.NVFP4Tensor.from_float(ops.interleave16(wg, wu), None)
    # garbage-filled outputs: every byte the call owns must be written, nothing beyond
    hp = torch.full((ops.packed_bytes(M, I) + 64,), 0xEE, dtype=torch.uint8, device="cuda")
    hs = torch.full((ops.scale_bytes(M, I) + 64,), 0xEE, dtype=torch.uint8, device="cuda")
    ops.swiglu_gemm(a.packed, a.sblk, 1.0, w, M, hp, hs)
    torch.cuda.synchronize()
    assert _ext.status() == 0
    gu = _f32_gemm_nv(a, w, M).cpu().numpy()
    gate, up = orc.deinterleave16(gu)
    h = orc.silu_mul(gate, up)
    p_ref, s_ref = orc.quantize_nvfp4(h, 1.0, threads=orc.host_threads())
    got_p, got_s = hp.cpu().numpy(), hs.cpu().numpy()
    assert np.array_equal(got_p[:-64], p_ref), f"{int((got_p[:-64] != p_ref).sum())} code bytes differ"
    assert np.array_equal(got_s[:-64], s_ref), f"{int((got_s[:-64] != s_ref).sum())} scale bytes differ"
    assert (got_p[-64:] == 0xEE).all() and (got_s[-64:] == 0xEE).all()
    # and h is what the float block computes, to quantization accuracy
    hq = orc.dequantize_nvfp4(got_p[:-64], got_s[:-64], 1.0, M, I)
    ref = (F.silu(torch.from_numpy(gate)) * torch.from_numpy(up)).numpy()
    assert np.linalg.norm(hq - ref) / np.linalg.norm(ref) < 0.12


@gpu
def test_swiglu_gemm_full_size_slab():
    """The block of the benchmark configuration (hidden 8192, intermediate 28672) on a 256-token slab, stage by stage:
    gate/up accumulators against the oracle's double-accumulated product (sampled), h bytes against the oracle applied
    to the accumulators (all 256 x 28672), down projection against the oracle's product of the dequantized h (sampled)."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    from thor_fp4.fused import NVFP4GatedMLP
    M, H, I = 256, 8192, 28672
    torch.manual_seed(5)
    mlp = NVFP4GatedMLP(H, I, device="cuda", out_dtype="bf16", weight_std=0.02)
    x = torch.randn(M, H, device="cuda").bfloat16()
    y = mlp(x).clone()
    torch.cuda.synchronize()
    assert _ext.status() == 0
    wgu, wd = mlp._q
    b = mlp._bufs[(M, torch.bfloat16)]
    a = thor_fp4.NVFP4Tensor(b["xp"], b["xs"], 1.0, (M, H))
    gu = _f32_gemm_nv(a, wgu, M)
    # (a) accumulators: sampled columns of the interleaved stack
    cols = np.linspace(0, 2 * I - 1, 384).astype(np.int64)
    ad = orc.dequantize_nvfp4(b["xp"].cpu().numpy(), b["xs"].cpu().numpy(), 1.0, M, H)
    wdq = orc.dequantize_nvfp4(wgu.packed.cpu().numpy(), wgu.sblk.cpu().numpy(), wgu.tensor_scale, 2 * I, H,
                               threads=orc.host_threads())[cols]
    ref = orc.gemm_f64acc(ad, wdq, None, 1.0, threads=orc.host_threads())
    got = gu.cpu().numpy()[:, cols]
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 1e-3
    # (b) h: every byte
    gate, up = orc.deinterleave16(gu.cpu().numpy())
    p_ref, s_ref = orc.quantize_nvfp4(orc.silu_mul(gate, up), 1.0, threads=orc.host_threads())
    assert np.array_equal(b["hp"].cpu().numpy(), p_ref)
    assert np.array_equal(b["hs"].cpu().numpy(), s_ref)
    # (c) down projection: sampled outputs are the exact product rounded once to bf16
    hd = orc.dequantize_nvfp4(p_ref, s_ref, 1.0, M, I, threads=orc.host_threads())
    ocols = np.linspace(0, H - 1, 256).astype(np.int64)
    wdd = orc.dequantize_nvfp4(wd.packed.cpu().numpy(), wd.sblk.cpu().numpy(), wd.tensor_scale, H, I,
                               threads=orc.host_threads())[ocols]
    yref = torch.from_numpy(orc.gemm_f64acc(hd, wdd, None, 1.0, threads=orc.host_threads()))
    ygot = y.float().cpu()[:, ocols]
    bound = (2.0 ** -8 + 2e-6) * yref.abs() + 8e-6 * yref.abs().max()
    assert ((ygot - yref).abs() <= bound).all()


@gpu
@pytest.mark.parametrize("M", [64, 200, 640])
def test_gated_block_fused_epilogue_tracks_unfused_and_float(M):
    import thor_fp4
    from thor_fp4.fused import NVFP4GatedMLP
    H, I = 256, 512
    torch.manual_seed(3)
    mlp = NVFP4GatedMLP(H, I, device="cuda", out_dtype="f32", weight_std=0.05)
    x = torch.randn(M, H, device="cuda").bfloat16()
    y = mlp(x).clone()
    assert torch.equal(mlp(x), y)                              # repeatable
    mlp.fuse_epilogue = False
    y_kernel = mlp(x).clone()                                  # GEMM -> bf16 -> one-pass silu*up + quantize -> GEMM
    mlp.fuse_activation = False
    y_torch = mlp(x).clone()
    # the unfused forms round gate, up and h to bf16 first: about one h value in a hundred lands on the other side of an
    # e2m1 threshold (a 25-50 % step for that value), a few percent of the output's norm; torch's silu vs the
    # reproducible one moves far fewer
    assert rrms(y, y_kernel) < 8e-2 and rrms(y_kernel, y_torch) < 2e-2
    q = lambda t, ts=1.0: thor_fp4.nvfp4_fake_quant(t.float(), ts)
    xq = q(x)
    ts_gu = max(thor_fp4.two_level_scale(mlp.w_gate.detach()), thor_fp4.two_level_scale(mlp.w_up.detach()))
    gate = xq @ q(mlp.w_gate.detach(), ts_gu).t()
    up = xq @ q(mlp.w_up.detach(), ts_gu).t()
    ref = q(F.silu(gate) * up) @ q(mlp.w_down.detach(), thor_fp4.two_level_scale(mlp.w_down.detach())).t()
    assert rrms(y, ref) < 0.05


# ------------------------------------------------------------------------------------------ MXFP8-out epilogue
ACTS = {"ident": F.silu, "gelu": F.gelu, "silu": F.silu}


def _tfc4f(L, name, a8, w4, bias, M, N, K, d=None, sfd=None):
    from thor_fp4 import _ext
    v = L.tfc4f_variant_index(name.encode())
    assert v >= 0
    if d is None:
        d = torch.zeros(M * N, dtype=torch.uint8, device="cuda")
    if sfd is None:
        sfd = torch.zeros(int(L.tfc4f_sfd_bytes(M, N)), dtype=torch.uint8, device="cuda")
    rc = L.tfc4f_gemm(v, a8.packed.data_ptr(), a8.sblk.data_ptr(), w4.packed.data_ptr(), w4.sblk.data_ptr(),
                      bias.data_ptr() if bias is not None else None, d.data_ptr(), sfd.data_ptr(), M, N, K,
                      ctypes.c_float(1.0), _ext.stream())
    return rc, d, sfd


@gpu
@pytest.mark.parametrize("act", ["gelu", "silu", "ident"])
@pytest.mark.parametrize("M,N,K", [(256, 1024, 512), (300, 384, 256), (17, 128, 128), (1000, 640, 1152)])
def test_tfc4f_gemm_bytes_match_oracle(act, M, N, K):
    import thor_fp4
    from thor_fp4 import _ext
    L = _ext.device_lib()
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.1
    bias = torch.randn(N, device="cuda", generator=g)
    a8, w4 = thor_fp4.MXTensor.from_float(x, "mxfp8"), thor_fp4.MXTensor.from_float(w, "mxfp4")
    name = {"gelu": "mx8out_gelu_128x128x256_c1", "silu": "mx8out_silu_128x256x256_c2x1", "ident": "mx8out_ident_128x128x256_c1"}[act]
    d = torch.full((M * N + 64,), 0xEE, dtype=torch.uint8, device="cuda")
    sfd = torch.zeros(int(L.tfc4f_sfd_bytes(M, N)), dtype=torch.uint8, device="cuda")
    rc, d, sfd = _tfc4f(L, name, a8, w4, bias, M, N, K, d, sfd)
    assert rc == 0
    torch.cuda.synchronize()
    assert _ext.status() == 0
    # the accumulators: the same kernel with a plain FP32 output
    acc = torch.empty(M, N, device="cuda")
    vp = L.tfc4_variant_index(thor_fp4.linear.resolve_mx8_variant(K).encode())
    L.tfp4_set_splits(1)
    try:
        assert L.tfc4_gemm_ex(vp, a8.packed.data_ptr(), a8.sblk.data_ptr(), w4.packed.data_ptr(), w4.sblk.data_ptr(), None,
                              acc.data_ptr(), M, N, K, ctypes.c_float(1.0), 2, _ext.stream()) == 0
        torch.cuda.synchronize()
    finally:
        L.tfp4_set_splits(0)
    yv = orc.bias_act(acc.cpu().numpy(), bias.cpu().numpy(), act, threads=orc.host_threads())
    p_ref, s_ref = orc.quantize_mx8_ceil(yv)
    got_d, got_s = d.cpu().numpy(), sfd.cpu().numpy()
    assert np.array_equal(got_d[:M * N], p_ref[:M * N]), f"{int((got_d[:M * N] != p_ref[:M * N]).sum())} code bytes differ"
    assert (got_d[M * N:] == 0xEE).all()                      # D holds exactly M * N bytes: nothing behind it is touched
    assert np.array_equal(got_s, s_ref), f"{int((got_s != s_ref).sum())} scale bytes differ"
    # the reference's own bound against the float layer
    dec = orc.dequantize_mx(np.concatenate([got_d[:M * N], np.zeros(orc.mx_packed_bytes(M, N, 1) - M * N, np.uint8)]),
                            got_s, "mxfp8", M, N)
    fn = {"gelu": F.gelu, "silu": F.silu, "ident": (lambda t: t)}[act]
    ref = fn(thor_fp4.mx_fake_quant(x, "mxfp8") @ thor_fp4.mx_fake_quant(w, "mxfp4").t() + bias).cpu().numpy()
    assert np.linalg.norm(dec - ref) / np.linalg.norm(ref) < 0.05


@gpu
def test_tfc4f_gemm_argument_checks_and_registry():
    # codes of csrc/fused_kernels.cu:423-445 in the reference project
    import thor_fp4
    from thor_fp4 import _ext
    L = _ext.device_lib()
    names = [bytes(L.tfc4f_variant_name(i)).decode() for i in range(L.tfc4f_n_variants())]
    assert len(names) == 8 and all(n.startswith("mx8out_") for n in names)
    assert sum(n.startswith("mx8out_gelu_") for n in names) == 4
    assert L.tfc4f_variant_index(b"nope") == -1 and L.tfc4f_variant_name(99) is None
    assert L.tfc4f_sfd_bytes(300, 1024) == 384 * 32 and L.tfc4f_sfd_bytes(128, 96) == 128 * 4
    a8 = thor_fp4.MXTensor.from_float(torch.randn(64, 256, device="cuda"), "mxfp8")
    w4 = thor_fp4.MXTensor.from_float(torch.randn(128, 256, device="cuda"), "mxfp4")
    bias = torch.zeros(128, device="cuda")
    assert _tfc4f(L, names[0], a8, w4, None, 64, 128, 256)[0] == -5          # bias is required
    v = L.tfc4f_variant_index(names[0].encode())
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    args = lambda var, N, K: (var, a8.packed.data_ptr(), a8.sblk.data_ptr(), w4.packed.data_ptr(), w4.sblk.data_ptr(),
                              bias.data_ptr(), buf.data_ptr(), buf.data_ptr(), 64, N, K, ctypes.c_float(1.0), _ext.stream())
    assert L.tfc4f_gemm(*args(99, 128, 256)) == -1
    assert L.tfc4f_gemm(*args(v, 128, 192)) == -3
    assert L.tfc4f_gemm(*args(v, 100, 256)) == -4


@gpu
def test_tfc4f_gemm_bias_reads_stay_inside_the_vector_at_large_m():
    """The reference's regression test (tests/test_fused.py:142-177): M > N, the bias is a view whose trailing 8192
    floats are NaN bait - and here the floats in front of it as well."""
    import thor_fp4
    from thor_fp4 import _ext
    L = _ext.device_lib()
    torch.manual_seed(4)
    M, K, N = 2048, 512, 1024
    x = torch.randn(M, K, device="cuda")
    w = (torch.rand(N, K, device="cuda") * 2 - 1) / K ** 0.5
    a8, w4 = thor_fp4.MXTensor.from_float(x, "mxfp8"), thor_fp4.MXTensor.from_float(w, "mxfp4")
    buf = torch.full((8192 + N + 8192,), float("nan"), device="cuda")
    bias = buf[8192:8192 + N]
    bias.copy_(torch.randn(N, device="cuda") * 0.5)
    rc, d, sfd = _tfc4f(L, "mx8out_gelu_128x128x256_c1", a8, w4, bias, M, N, K)
    assert rc == 0
    torch.cuda.synchronize()
    dec = orc.dequantize_mx(np.concatenate([d.cpu().numpy(), np.zeros(orc.mx_packed_bytes(M, N, 1) - M * N, np.uint8)]),
                            sfd.cpu().numpy(), "mxfp8", M, N)
    assert np.isfinite(dec).all(), "NaN bait leaked in: out-of-bounds bias read"
    ref = F.gelu(thor_fp4.mx_fake_quant(x, "mxfp8") @ thor_fp4.mx_fake_quant(w, "mxfp4").t() + bias).cpu().numpy()
    assert np.linalg.norm(dec - ref) / np.linalg.norm(ref) < 0.1


@gpu
def test_act_quant_mx8_bias_reads_stay_inside_the_vector():
    from thor_fp4 import _ext, ops
    R, N = 2048, 1024
    acc = (torch.randn(R, N, device="cuda") * 2).bfloat16()
    buf = torch.full((8192 + N + 8192,), float("nan"), device="cuda")
    bias = buf[8192:8192 + N]
    bias.copy_(torch.randn(N, device="cuda"))
    packed = torch.zeros(ops.mx_packed_bytes(R, N, "mxfp8"), dtype=torch.uint8, device="cuda")
    sblk = torch.zeros(ops.mx_scale_bytes(R, N), dtype=torch.uint8, device="cuda")
    assert _ext.device_lib().tfp4_act_quant_mx8(acc.data_ptr(), bias.data_ptr(), R, N, 2, 1, packed.data_ptr(),
                                                sblk.data_ptr(), _ext.stream()) == 0
    torch.cuda.synchronize()
    dec = orc.dequantize_mx(packed.cpu().numpy(), sblk.cpu().numpy(), "mxfp8", R, N)
    assert np.isfinite(dec).all()


# ------------------------------------------------------------------------------------------ push epilogue (one GPU)
@gpu
@pytest.mark.parametrize("od", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("M,N,K,owners", [(512, 384, 1024, 2), (1024, 1000, 512, 4), (768, 256, 256, 8), (300, 264, 512, 2),
                                          (8192, 2048, 1024, 8)])
def test_gemm_push_fills_every_owners_staging_rows(od, M, N, K, owners):
    """tfp4_gemm_push on one GPU: the 'owners' are buffers of this process, so the destination logic (which 32-row
    block goes to which owner, at which row of its slot) is checked without NVLink: owner o must hold exactly the rows
    [o * rows, (o + 1) * rows) of the plain GEMM's output, bit for bit, and nothing outside its slot is touched."""
    import thor_fp4
    from thor_fp4 import ops, _ext
    L = _ext.device_lib()
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    a = thor_fp4.NVFP4Tensor.from_float(x.float(), 1.0)
    b = thor_fp4.NVFP4Tensor.from_float(w, None)
    dt = _ext.OUT_TORCH[od]
    rows = -(-M // owners)
    rows = -(-rows // 32) * 32                                   # rows per owner: a multiple of 32 covering M
    stage = [torch.full((rows + 8, N), 7.0, dtype=dt, device="cuda") for _ in range(owners)]
    dest = (ctypes.c_void_p * owners)(*[t.data_ptr() for t in stage])
    L.tfp4_set_splits(1)
    try:
        rc = L.tfp4_gemm_push(a.packed.data_ptr(), a.sblk.data_ptr(), ctypes.c_float(1.0), b.packed.data_ptr(), b.sblk.data_ptr(),
                              ctypes.c_float(b.tensor_scale), dest, owners, rows, (M + N) % owners, M, N, K, _ext.OUT_DTYPE[od],
                              _ext.stream())
        assert rc == 0
        ref = torch.empty(M, N, dtype=dt, device="cuda")
        L.tfp4_set_pair_mode(2)                                  # the same kernel for the plain output
        ops.gemm(a.packed, a.sblk, 1.0, b.packed, b.sblk, b.tensor_scale, ref, M, N, K, od)
        torch.cuda.synchronize()
    finally:
        L.tfp4_set_splits(0)
        L.tfp4_set_pair_mode(-1)
    assert _ext.status() == 0
    for o in range(owners):
        have = max(0, min(rows, M - o * rows))
        assert torch.equal(stage[o][:have], ref[o * rows: o * rows + have]), f"owner {o}"
        assert (stage[o][have:] == 7.0).all(), f"owner {o}: rows beyond its share were written"
    # and the owner-side sum over staged partials
    slots = torch.stack([t[:rows] for t in stage[:2]]).contiguous()
    for out_dt, code in ((torch.float32, 2), (torch.bfloat16, 1)):
        out = torch.empty(rows, N, dtype=out_dt, device="cuda")
        if (rows * N) % 8 == 0:
            assert L.tfp4_sum_slots(slots.data_ptr(), 2, rows, N, _ext.IN_DTYPE[dt], out.data_ptr(), code, _ext.stream()) == 0
            torch.cuda.synchronize()
            want = (slots[0].float() + slots[1].float()).to(out_dt)
            assert torch.equal(out, want)


@gpu
def test_gemm_push_argument_checks():
    from thor_fp4 import _ext
    L = _ext.device_lib()
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    dest = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    args = lambda n, rows, od: (buf.data_ptr(), buf.data_ptr(), ctypes.c_float(1.0), buf.data_ptr(), buf.data_ptr(), ctypes.c_float(1.0),
                                dest, n, rows, 0, 64, 64, 64, od, _ext.stream())
    assert L.tfp4_gemm_push(*args(2, 48, 2)) == -7        # rows per owner not a multiple of 32
    assert L.tfp4_gemm_push(*args(2, 16 * 2, 7)) == -7    # no such output type
    assert L.tfp4_gemm_push(*args(1, 32, 2)) == -7        # one owner of 32 rows does not cover 64 tokens
    assert L.tfp4_gemm_push(*args(9, 32, 2)) == -7        # more owners than the kernel's map table holds
