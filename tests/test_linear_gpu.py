"""thor_fp4.Linear / convert / calibrate / verify / capture_module on the GPU: the same
behaviours the reference's own tests pin (tests/test_linear.py, test_verify.py,
test_convert.py, test_graphs_cascade.py, test_gemv.py there), against this engine."""
import os

import pytest
import torch
import torch.nn as nn

from conftest import rrms

gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("M", [1, 3, 5, 8, 17, 128, 255, 300])
def test_linear_matches_fake_quant(M):
    import thor_fp4
    lin = thor_fp4.Linear(1024, 512, bias=True).cuda()
    with torch.no_grad():
        lin.bias.normal_(std=0.05)
    x = torch.randn(M, 1024, device="cuda")
    y = lin(x)
    assert y.shape == (M, 512) and y.dtype == torch.float16
    ts = lin._weight_fp4.tensor_scale
    ref = (thor_fp4.nvfp4_fake_quant(x, 1.0) @ thor_fp4.nvfp4_fake_quant(lin.weight.detach(), ts).t()
           + lin.bias.float())
    assert rrms(y, ref) < 1e-3


@gpu
@pytest.mark.parametrize("od,dt", [("f16", torch.float16), ("bf16", torch.bfloat16), ("f32", torch.float32)])
def test_linear_output_dtypes(od, dt):
    import thor_fp4
    lin = thor_fp4.Linear(256, 128, out_dtype=od).cuda()
    assert lin(torch.randn(16, 256, device="cuda")).dtype == dt


@gpu
def test_linear_input_layouts_and_dtypes():
    import thor_fp4
    lin = thor_fp4.Linear(256, 128).cuda()
    base = torch.randn(16, 256, device="cuda")
    ref = lin(base).float().clone()
    buf = torch.empty(16, 512, device="cuda")
    xt = buf[:, :256]
    xt.copy_(base)
    assert not xt.is_contiguous()
    assert rrms(lin(xt), ref) < 1e-3
    for dt in (torch.float16, torch.bfloat16, torch.float64):
        assert lin(base.to(dt)).shape == (16, 128)


def test_linear_constraints():
    import thor_fp4
    with pytest.raises(ValueError, match="% 64"):
        thor_fp4.Linear(300, 128)
    with pytest.raises(ValueError, match="N >= 8"):
        thor_fp4.Linear(128, 4)
    with pytest.raises(ValueError, match="N % 8"):
        thor_fp4.Linear(128, 12)
    with pytest.raises(ValueError, match="unknown engine"):
        thor_fp4.Linear(128, 16, engine="nope")
    assert thor_fp4.Linear(128, 16, engine="gemv").engine_kind == "gv"
    assert thor_fp4.Linear(128, 16, engine="cutlass").engine_kind == "nv"
    assert thor_fp4.Linear(128, 16, engine="cutlass:mx8").engine_kind == "mx8"
    assert thor_fp4.Linear(128, 16, engine="cutlass:nvfp4_128x128x256_c1").out_dtype == "bf16"


@gpu
def test_linear_weight_lifecycle_and_determinism():
    import thor_fp4
    lin = thor_fp4.Linear(256, 128).cuda()
    x = torch.randn(8, 256, device="cuda")
    y1 = lin(x).clone()
    assert torch.equal(lin(x), y1)
    with torch.no_grad():
        lin.weight.mul_(2.0)
    lin.refresh_weight()
    y2 = lin(x).clone()
    assert torch.allclose(y2.float(), y1.float() * 2, rtol=0.02, atol=1e-3)
    lin2 = thor_fp4.Linear(256, 128).cuda()
    lin2.load_state_dict(lin.state_dict())
    assert torch.equal(lin2(x), y2)
    out = lin(torch.randn(8, 256, device="cuda", requires_grad=True))
    assert out.requires_grad is False
    big = thor_fp4.Linear(2048, 512).cuda()
    assert big.fp4_weight_nbytes() == 2048 * 512 // 2 + 512 * 128


@gpu
@pytest.mark.parametrize("M", [1, 4, 8])
def test_linear_gemv_engine(M):
    import thor_fp4
    lin = thor_fp4.Linear(640, 320, bias=True, out_dtype="f32", engine="gemv").cuda()
    x = torch.randn(M, 640, device="cuda")
    ref = x @ lin.refresh_weight()._weight_fp4.dequantize().t() + lin.bias.float()
    assert rrms(lin(x), ref) < 1e-5
    with pytest.raises(RuntimeError, match="M <= 8"):
        lin(torch.randn(9, 640, device="cuda"))
    assert thor_fp4.verify(lin, x).ok


@gpu
def test_cutlass_named_engine_matches_default():
    import thor_fp4
    a = thor_fp4.Linear(512, 256, bias=False, out_dtype="bf16").cuda()
    b = thor_fp4.Linear(512, 256, bias=False, engine="cutlass").cuda()
    b.load_state_dict(a.state_dict())
    x = torch.randn(33, 512, device="cuda")
    assert rrms(b(x), a(x)) < 8e-3


@gpu
def test_verify_quiet_when_clean_and_flags_injected_faults():
    import thor_fp4
    from thor_fp4 import linear as lin_mod
    lin = thor_fp4.Linear(1024, 512).cuda()
    x = torch.randn(128, 1024, device="cuda")
    rep = thor_fp4.verify(lin, x)
    assert rep.ok and rep.rel_rms < 5e-3, str(rep)
    real_gemm = lin_mod.ops.gemm

    def broken_gemm(*args, **kw):
        real_gemm(*args, **kw)
        args[6].add_(0.25)

    lin_mod.ops.gemm = broken_gemm
    try:
        bad = thor_fp4.verify(lin, x)
    finally:
        lin_mod.ops.gemm = real_gemm
    assert not bad.ok and bad.n_bad > 0 and bad.worst_locations
    real_ops = lin_mod.ops

    class ScrambledOps:
        def __getattr__(self, k):
            return getattr(real_ops, k)

        def quantize_nvfp4(self, *a, **kw):
            p, s = real_ops.quantize_nvfp4(*a, **kw)
            s.copy_(s.roll(97))
            return p, s

    lin_mod.ops = ScrambledOps()
    try:
        bad = thor_fp4.verify(lin, x)
    finally:
        lin_mod.ops = real_ops
    assert not bad.ok
    w = lin._weight_fp4
    saved = w.packed.clone()
    w.packed[:4096] ^= 0xFF          # both paths read the same corrupted codes: still equal
    quiet = thor_fp4.verify(lin, x)
    w.packed.copy_(saved)
    assert quiet.ok
    rep2 = thor_fp4.verify(thor_fp4.Linear(256, 128).cuda(), [torch.randn(8, 256, device="cuda")] * 2)
    assert rep2.n_elements == 2 * 8 * 128 and "ok=" in str(rep2)


class _MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(512, 1024)
        self.fc2 = nn.Linear(1024, 512)
        self.head = nn.Linear(512, 10)

    def forward(self, x):
        return self.head(self.fc2(torch.nn.functional.gelu(self.fc1(x).float())).float()).float()


@gpu
def test_convert_verify_and_capture_module():
    import thor_fp4
    ref_model = _MLP().cuda()
    m = thor_fp4.convert(ref_model, policy={"head": "bf16", "*": "fp4"})
    assert isinstance(m.fc1, thor_fp4.Linear) and isinstance(m.fc2, thor_fp4.Linear)
    assert isinstance(m.head, nn.Linear) and isinstance(ref_model.fc1, nn.Linear)   # deep copy by default
    assert m.thor_fp4_policy == {"fc1": "fp4", "fc2": "fp4", "head": "bf16"}
    x = torch.randn(64, 512, device="cuda")
    rep = thor_fp4.verify(m, x)
    assert rep.ok, str(rep)
    assert set(rep.layers) == {"fc1", "fc2", "<end-to-end>"}
    eager = m(x).clone()
    g = thor_fp4.capture_module(m, x)
    assert torch.equal(g(x), eager)
    x2 = torch.randn(64, 512, device="cuda")
    assert torch.equal(g(x2), m(x2))
    cal = thor_fp4.calibrate(ref_model, [x, x2])
    assert set(cal) == {"fc1", "fc2", "head"} and all(v > 0 for v in cal.values())
    mc = thor_fp4.convert(ref_model, policy="fp4", calibration=cal)
    assert mc.fc1.act_tensor_scale == pytest.approx(cal["fc1"])
    assert thor_fp4.verify(mc, x).ok
    mx = thor_fp4.convert(ref_model, policy="mx8")
    assert mx.fc1.engine_kind == "mx8" and mx.thor_fp4_policy["fc1"].startswith("mx8")


@gpu
def test_plan_cache_is_allocation_free_after_warmup():
    import thor_fp4
    from thor_fp4 import _ext
    lin = thor_fp4.Linear(512, 256, out_dtype="bf16").cuda()
    x = torch.randn(40, 512, device="cuda")
    lin(x)
    h0, m0 = _ext.plan_stats()
    torch.cuda.synchronize()
    mem0 = torch.cuda.memory_allocated()
    for _ in range(5):
        lin(x)
    torch.cuda.synchronize()
    h1, m1 = _ext.plan_stats()
    assert m1 == m0 and h1 == h0 + 5
    assert torch.cuda.memory_allocated() == mem0


@gpu
def test_chunked_sweep_over_row_slices_equals_full_gemm():
    # a resident library swept in 256-row chunks (pointer offsets into codes and scale tiles) gives the
    # same scores as one GEMM over the whole library; the planted neighbour is found in its own chunk
    import thor_fp4
    from thor_fp4 import ops
    g = torch.Generator(device="cuda").manual_seed(11)
    lib = torch.randn(1000, 512, device="cuda", generator=g)
    lib = lib / lib.norm(dim=1, keepdim=True)
    q = torch.randn(4, 512, device="cuda", generator=g)
    q[2] = lib[777] * 3.0
    L = thor_fp4.NVFP4Tensor.from_float(lib.contiguous())
    Q = thor_fp4.NVFP4Tensor.from_float(q.contiguous(), 1.0)
    full = Q.matmul_t(L, "f32")
    parts = torch.empty_like(full)
    for r0, chunk in L.row_chunks(256):
        parts[:, r0:r0 + chunk.shape[0]] = Q.matmul_t(chunk, "f32")
    torch.cuda.synchronize()
    assert torch.equal(parts, full)
    assert int(full[2].argmax()) == 777


@gpu
def test_quantized_checkpoint_restores_the_layer_bit_for_bit(tmp_path):
    import thor_fp4
    torch.manual_seed(2)
    a = thor_fp4.Linear(256, 192, bias=True, out_dtype="bf16", device="cuda", act_tensor_scale=0.5)
    with torch.no_grad():
        a.bias.normal_()
    x = torch.randn(33, 256, device="cuda").bfloat16()
    ya = a(x).clone()
    f = tmp_path / "layer.pt"
    torch.save(a.quantized_state(), f)
    b = thor_fp4.Linear(256, 192, bias=True, out_dtype="bf16", device="cuda")
    b.load_quantized_state(torch.load(f, map_location="cpu", weights_only=True))
    assert torch.equal(b(x), ya)
    assert torch.equal(b._weight_fp4.packed, a._weight_fp4.packed) and torch.equal(b._weight_fp4.sblk, a._weight_fp4.sblk)
    b.refresh_weight()        # the master weight is the dequantized value: re-quantizing it gives the same values
    assert torch.equal(b._weight_fp4.sblk, a._weight_fp4.sblk)     # (codes may differ in the sign nibble of zeros)
    assert torch.equal(b._weight_fp4.dequantize(), a._weight_fp4.dequantize())
    assert torch.equal(b(x), ya)
    assert os.path.getsize(f) < 0.4 * (256 * 192 * 4)
    with pytest.raises(ValueError):
        thor_fp4.Linear(256, 128, device="cuda").load_quantized_state(torch.load(f, map_location="cpu", weights_only=True))


@gpu
@pytest.mark.parametrize("M", [1, 100, 700])
def test_dependent_launch_chain_equals_plain_stream_order(M):
    # quantizer -> GEMM -> split-K reduction chained by programmatic dependent launch (default) must give the
    # bytes of plain stream order, eagerly, back to back on changing inputs, and replayed from a CUDA graph
    import thor_fp4
    from thor_fp4 import _ext
    torch.manual_seed(M)
    lin = thor_fp4.Linear(1024, 768, bias=True, out_dtype="bf16", device="cuda")
    xs = [torch.randn(M, 1024, device="cuda").bfloat16() for _ in range(4)]
    L = _ext.core()
    try:
        L.tfp4_set_dependent_launch(0)
        want = [lin(x).clone() for x in xs]
        L.tfp4_set_dependent_launch(1)
        got = [lin(x).clone() for x in xs]            # each call overwrites the buffers the previous one read
        torch.cuda.synchronize()
        for a, b in zip(want, got):
            assert torch.equal(a, b)
        g = thor_fp4.capture_module(lin, xs[0])
        for i in (1, 2, 3, 0):
            y = g(xs[i])
            assert torch.equal(y, want[i])
    finally:
        L.tfp4_set_dependent_launch(1)


@gpu
def test_two_streams_interleaved_layer_calls_give_serial_results():
    # two layers driven from two streams at once (dependent launches chain only within a stream): every result
    # must equal the one computed alone
    import thor_fp4
    torch.manual_seed(9)
    a = thor_fp4.Linear(2048, 1024, bias=True, out_dtype="bf16", device="cuda")
    b = thor_fp4.Linear(1024, 1536, bias=False, out_dtype="f16", device="cuda")
    xa = [torch.randn(64, 2048, device="cuda").bfloat16() for _ in range(6)]
    xb = [torch.randn(300, 1024, device="cuda").bfloat16() for _ in range(6)]
    want_a = [a(x).clone() for x in xa]
    want_b = [b(x).clone() for x in xb]
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    got_a, got_b = [], []
    for i in range(6):
        with torch.cuda.stream(s1):
            got_a.append(a(xa[i]).clone())
        with torch.cuda.stream(s2):
            got_b.append(b(xb[i]).clone())
    torch.cuda.synchronize()
    for w, g in zip(want_a + want_b, got_a + got_b):
        assert torch.equal(w, g)


@gpu
def test_two_streams_both_split_k_give_serial_results():
    # two small-batch layers (both on the split-K path, each with f32 partial sums) driven from two streams at
    # once: each stream owns its partial-sum block, so every result must equal the one computed alone
    import thor_fp4
    from thor_fp4 import _ext
    torch.manual_seed(10)
    a = thor_fp4.Linear(8192, 1024, bias=True, out_dtype="bf16", device="cuda")
    b = thor_fp4.Linear(4096, 1536, bias=False, out_dtype="f16", device="cuda")
    xa = [torch.randn(64, 8192, device="cuda").bfloat16() for _ in range(8)]
    xb = [torch.randn(100, 4096, device="cuda").bfloat16() for _ in range(8)]
    want_a = [a(x).clone() for x in xa]
    want_b = [b(x).clone() for x in xb]
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    got_a, got_b = [], []
    for i in range(8):
        with torch.cuda.stream(s1):
            got_a.append(a(xa[i]).clone())
        with torch.cuda.stream(s2):
            got_b.append(b(xb[i]).clone())
    torch.cuda.synchronize()
    assert _ext.status() == 0
    for w, g in zip(want_a + want_b, got_a + got_b):
        assert torch.equal(w, g)


@gpu
def test_captured_small_batch_graph_survives_larger_split_k_shapes():
    # a graph captured at a small batch keeps its own partial-sum block: running larger split-K shapes afterwards
    # (which need more workspace) neither frees nor reuses it, so the replay still gives the eager result
    import thor_fp4
    torch.manual_seed(11)
    small = thor_fp4.Linear(4096, 512, bias=True, out_dtype="bf16", device="cuda")
    x16 = torch.randn(16, 4096, device="cuda").bfloat16()
    want = small(x16).clone()
    g = thor_fp4.capture_module(small, x16)
    assert torch.equal(g(x16), want)
    wide = thor_fp4.Linear(5120, 20480, bias=False, out_dtype="bf16", device="cuda")
    for M in (32, 128):
        y = wide(torch.randn(M, 5120, device="cuda").bfloat16())
        assert torch.isfinite(y.float()).all()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        wide(torch.randn(128, 5120, device="cuda").bfloat16())
    torch.cuda.synchronize()
    x2 = torch.randn(16, 4096, device="cuda").bfloat16()
    want2 = small(x2).clone()
    assert torch.equal(g(x2), want2)
    assert torch.equal(g(x16), want)
