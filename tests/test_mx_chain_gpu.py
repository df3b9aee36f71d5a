"""GPU checks of the MXFP8 chain: the one-pass bias + activation + MXFP8 quantize kernel against the oracle's MX
quantizer applied to the same activation values, FusedLinear with that epilogue against its unfused form, and the MX
gated block / chain against fake-quantized float references within the bounds the reference's own tests use
(tests/test_fused.py:73-76 of the reference project: 0.05 for one fused layer, 0.12 for the gated block)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as orc

gpu = pytest.mark.gpu
ACTS = {"ident": (0, lambda t: t), "gelu": (1, F.gelu), "silu": (2, F.silu)}


@gpu
@pytest.mark.parametrize("act", ["ident", "gelu", "silu"])
@pytest.mark.parametrize("R,N", [(300, 256), (128, 1152), (1000, 384)])
def test_act_quant_mx8_matches_oracle_on_same_values(act, R, N):
    from thor_fp4 import _ext, ops
    g = torch.Generator(device="cuda").manual_seed(R + N)
    acc = (torch.randn(R, N, device="cuda", generator=g) * 3.0).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g)
    packed = torch.zeros(ops.mx_packed_bytes(R, N, "mxfp8"), dtype=torch.uint8, device="cuda")
    sblk = torch.zeros(ops.mx_scale_bytes(R, N), dtype=torch.uint8, device="cuda")
    code, fn = ACTS[act]
    rc = _ext.device_lib().tfp4_act_quant_mx8(acc.data_ptr(), bias.data_ptr(), R, N, _ext.IN_DTYPE[acc.dtype], code,
                                              packed.data_ptr(), sblk.data_ptr(), _ext.stream())
    assert rc == 0
    torch.cuda.synchronize()
    # the activations are built from correctly rounded operations that the oracle repeats: bytes are equal
    y = orc.bias_act(acc.float().cpu().numpy(), bias.cpu().numpy(), act)
    p_ref, s_ref = orc.quantize_mx8_ceil(y)
    got_p, got_s = packed.cpu().numpy(), sblk.cpu().numpy()
    assert np.array_equal(got_s, s_ref)
    assert np.array_equal(got_p, p_ref)
    # and they are gelu / silu: the float library's values quantize to nearly the same tensor
    d_got = orc.dequantize_mx(got_p, got_s, "mxfp8", R, N)
    d_flt = orc.dequantize_mx(*orc.quantize_mx8_ceil(fn(acc.float().cpu() + bias.float().cpu()).numpy()), "mxfp8", R, N)
    assert np.linalg.norm(d_got - d_flt) / np.linalg.norm(d_flt) < 2e-3


@gpu
@pytest.mark.parametrize("act", ["gelu", "silu", "ident"])
def test_fused_linear_epilogue_equals_unfused_and_tracks_float(act):
    from thor_fp4.fused import FusedLinear
    torch.manual_seed(1)
    lin = FusedLinear(512, 768, bias=True, act=act, device="cuda")
    with torch.no_grad():
        lin.bias.normal_(std=0.1)
    x = torch.randn(300, 512, device="cuda")
    out = lin(x)
    fused = out.dequant().clone()
    lin.fuse_epilogue = False
    unfused = lin(x).dequant().clone()
    lin.fuse_epilogue = True
    # the unfused form rounds the accumulator to bf16 before the epilogue arithmetic: some e4m3 codes move by one step
    assert ((fused - unfused).norm() / unfused.norm()).item() < 3e-2
    import thor_fp4
    q8, q4 = (lambda t: thor_fp4.mx_fake_quant(t, "mxfp8")), (lambda t: thor_fp4.mx_fake_quant(t, "mxfp4"))
    ref = ACTS[act][1](q8(x) @ q4(lin.weight.detach()).t() + lin.bias.detach())
    assert ((fused - ref).norm() / ref.norm()).item() < 0.05


@gpu
def test_mx_gated_block_and_chain_track_float():
    from thor_fp4.fused import GatedMLP, mx8_chain
    torch.manual_seed(2)
    mlp = GatedMLP(256, 512, device="cuda")
    x = torch.randn(200, 256, device="cuda")
    y = mlp(x).float()
    import thor_fp4
    q8, q4 = (lambda t: thor_fp4.mx_fake_quant(t, "mxfp8")), (lambda t: thor_fp4.mx_fake_quant(t, "mxfp4"))
    xq = q8(x)
    g = F.silu(xq @ q4(mlp.gate.weight.detach()).t() + mlp.gate.bias.detach())
    u = xq @ q4(mlp.up.weight.detach()).t() + mlp.up.bias.detach()
    ref = (g * u) @ q4(mlp.down.weight.detach()).t() + mlp.down.bias.detach()     # hidden tensors are MXFP8 with ceil scales: no saturation to model
    assert ((y - ref).norm() / ref.norm()).item() < 0.12
    chain = mx8_chain(256, 512, 384, device="cuda")
    yc = chain(x).float()
    h = F.gelu(xq @ q4(chain[0].weight.detach()).t() + chain[0].bias.detach())
    refc = h @ q4(chain[1].weight.detach()).t() + chain[1].bias.detach()
    assert ((yc - refc).norm() / refc.norm()).item() < 0.12
