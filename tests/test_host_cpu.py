"""CPU tier: the C-ABI library loads and exports every symbol the header declares, the size
helpers match the oracle, and the host-side logic (policies, fake quantizers, sharding,
tensor-parallel reduction over gloo) behaves as the reference's."""
import ctypes
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import oracle as orc

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    from thor_fp4 import _ext
    L = _ext.core()
    header = (ROOT / "include" / "thorfp4_b200.h").read_text()
    declared = set(re.findall(r"\b(tf[pc]4f?_[a-z0-9_]+)\s*\(", header))
    assert {"tfp4_quant", "tfp4_gemm", "tfp4_gemv", "tfp4_quant_mx", "tfc4_gemm"} <= declared
    for name in declared:
        assert hasattr(L, name), f"{name} declared in the header but not exported"
    for name in _ext.SIGNATURES:
        assert name in declared, f"{name} bound by ctypes but not declared in the header"


def test_size_helpers_match_reference_formulas():
    from thor_fp4 import ops
    for R, K in ((1, 64), (5, 128), (128, 1024), (129, 4096), (300, 320)):
        assert ops.pad_rows(R) == orc.pad_rows(R) == (R + 127) // 128 * 128
        assert ops.packed_bytes(R, K) == orc.packed_bytes(R, K)
        assert ops.scale_bytes(R, K) == orc.scale_bytes(R, K)
        assert ops.mx_scale_bytes(R, K) == orc.mx_scale_bytes(R, K)
        for kind in ("mxfp4", "mxfp8"):
            assert ops.mx_packed_bytes(R, K, kind) == orc.mx_packed_bytes(R, K, kind)


def test_variant_registry_keeps_reference_names():
    from thor_fp4 import _ext
    L = _ext.cutlass()
    names = [L.tfc4_variant_name(i).decode() for i in range(L.tfc4_n_variants())]
    assert "nvfp4_128x128x256_c1" in names and "mxfp8xfp4_128x256x128_c2x1" in names
    assert L.tfc4_variant_index(b"nvfp4_128x256x256_c2x1") >= 0 and L.tfc4_variant_index(b"nope") == -1


def test_no_cpu_fallback():
    import thor_fp4
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises((RuntimeError, AssertionError)):
        thor_fp4.quantize_nvfp4(torch.randn(8, 64))
    lin = thor_fp4.Linear(64, 8)
    with pytest.raises((RuntimeError, AssertionError)):
        lin(torch.randn(2, 64))


def test_torch_fake_quantizers_match_oracle(golden):
    import thor_fp4
    for K in (320, 1024):
        x = torch.from_numpy(golden[f"nv_K{K}_x"])
        for mode in ("block", "two"):
            ts = float(golden[f"nv_K{K}_{mode}_ts"])
            assert torch.equal(thor_fp4.nvfp4_fake_quant(x, ts), torch.from_numpy(golden[f"nv_K{K}_{mode}_y"]))
    x = torch.from_numpy(golden["mx_K512_x"])
    for kind in ("mxfp4", "mxfp8"):
        assert torch.equal(thor_fp4.mx_fake_quant(x, kind), torch.from_numpy(golden[f"mx_K512_{kind}_y"]))
    assert thor_fp4.two_level_scale(x) == pytest.approx(orc.two_level_scale(x.numpy()))


def test_auto_decision_and_policies():
    import thor_fp4
    from thor_fp4.convert import _match_policy
    table = {"crossover": {"min_k": 1280, "min_n": 1280},
             "shapes": {"4096x4096": {"4096": {"fp4_ms": 0.1, "bf16_ms": 0.3, "fp4_wins": True}},
                        "512x2048": {"fp4_ms": 0.2, "bf16_ms": 0.1, "fp4_wins": False}}}
    assert thor_fp4.auto_decision(4096, 4096, table).spec == "fp4"
    assert thor_fp4.auto_decision(2048, 512, table).spec == "bf16"
    assert thor_fp4.auto_decision(100, 512, table).spec == "bf16"       # K % 64
    assert thor_fp4.auto_decision(4096, 12, table).spec == "bf16"       # N % 8
    assert thor_fp4.auto_decision(2048, 2048, table).spec == "fp4"      # crossover rule
    assert thor_fp4.auto_decision(512, 2048, table).spec == "bf16"
    assert "crossover" in thor_fp4.load_shape_table()
    lin = nn.Linear(8, 8)
    assert _match_policy({"critic.*": "bf16", "*": "auto"}, "critic.fc", lin) == "bf16"
    assert _match_policy({"critic.*": "bf16"}, "actor.fc", lin) == "auto"
    assert _match_policy(lambda n, m: "fp4", "x", lin) == "fp4"
    with pytest.raises(TypeError):
        _match_policy(3, "x", lin)


def test_convert_on_cpu_model_records_decisions():
    import thor_fp4
    model = nn.Sequential(nn.Linear(2048, 2048), nn.ReLU(), nn.Linear(2048, 100), nn.Linear(100, 10))
    m = thor_fp4.convert(model, policy="auto")
    assert isinstance(m[0], thor_fp4.Linear) and isinstance(m[2], nn.Linear) and isinstance(m[3], nn.Linear)
    assert m.thor_fp4_policy["0"] == "fp4" and m.thor_fp4_policy["2"] == "bf16"
    assert torch.equal(m[0].weight.detach(), model[0].weight.detach())
    allbf = thor_fp4.convert(model, policy="bf16")
    assert all(isinstance(l, nn.Linear) for l in (allbf[0], allbf[2], allbf[3]))
    forced = thor_fp4.convert(model, policy="fp4")
    assert forced.thor_fp4_policy["3"].startswith("bf16 (")        # K=100 refused by the constructor
    cal = thor_fp4.calibrate(model, [torch.randn(4, 2048)])
    assert set(cal) == {"0", "2", "3"}


def test_row_slices_and_checkpoint_of_a_quantized_tensor(tmp_path):
    # a row slice starting on a 128-row boundary is a pointer offset into the code and scale buffers:
    # it must equal the oracle's quantization of those rows alone (same per-tensor scale)
    from thor_fp4.ops import NVFP4Tensor
    rng = np.random.default_rng(5)
    R, K = 700, 320                                      # ragged last tile, scale columns not a multiple of 4 tiles
    x = (rng.standard_normal((R, K)) * np.logspace(-2, 1, K)).astype(np.float32)
    ts = orc.two_level_scale(x)
    p, sc = orc.quantize_nvfp4(x, ts)
    t = NVFP4Tensor(torch.from_numpy(p), torch.from_numpy(sc), ts, (R, K))
    for a, b in ((0, 128), (128, 512), (256, 300), (640, 700), (0, 700)):
        v = t.rows(a, b)
        po, so = orc.quantize_nvfp4(x[a:b], ts)
        n = b - a
        assert v.shape == (n, K) and v.tensor_scale == ts
        assert np.array_equal(v.packed.numpy()[: n * K // 2], po[: n * K // 2])
        want = orc.dequantize_nvfp4(po, so, ts, n, K)
        got = orc.dequantize_nvfp4(v.packed.numpy(), v.sblk.numpy(), ts, n, K)
        assert np.array_equal(got, want)
        assert v.packed.data_ptr() == t.packed.data_ptr() + a * K // 2          # a view, not a copy
    assert [r0 for r0, _ in t.row_chunks(256)] == [0, 256, 512]
    assert [c.shape[0] for _, c in t.row_chunks(256)] == [256, 256, 188]
    with pytest.raises(AssertionError):
        t.rows(64, 128)
    # checkpoint round trip: same bytes, same scale, refuses foreign or truncated files
    f = tmp_path / "w.nvfp4.pt"
    t.save(f)
    u = NVFP4Tensor.load(f)
    assert u.shape == t.shape and u.tensor_scale == t.tensor_scale
    assert torch.equal(u.packed, t.packed) and torch.equal(u.sblk, t.sblk)
    bad = dict(t.state_dict(), format="something else")
    with pytest.raises(ValueError):
        NVFP4Tensor.from_state_dict(bad)
    short = dict(t.state_dict(), packed=t.packed[:-1])
    with pytest.raises(ValueError):
        NVFP4Tensor.from_state_dict(short)


def test_sharding_helpers():
    from thor_fp4.parallel import shard_cols, shard_rows
    w = torch.arange(256 * 128, dtype=torch.float32).reshape(256, 128)
    assert torch.equal(torch.cat([shard_rows(w, 2, r) for r in range(2)], 0), w)
    assert torch.equal(torch.cat([shard_cols(w, 2, r) for r in range(2)], 1), w)
    with pytest.raises(ValueError):
        shard_rows(w, 3, 0)


_WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["TFP4_PKG"])
import torch, torch.distributed as dist, torch.nn as nn
import thor_fp4
from thor_fp4.parallel import TensorParallelGatedMLP, shard_rows, shard_cols

class EmuMLP(nn.Module):
    """CPU stand-in for the rank-local block: the same arithmetic through the torch fake quantizers."""
    def __init__(self, hidden, inter):
        super().__init__()
        self.w_gate = nn.Parameter(torch.zeros(inter, hidden)); self.w_up = nn.Parameter(torch.zeros(inter, hidden))
        self.w_down = nn.Parameter(torch.zeros(hidden, inter)); self.tensor_scales = None; self._q = None
    def forward(self, x):
        q = thor_fp4.nvfp4_fake_quant
        ts_gu, ts_d = self.tensor_scales
        xq = q(x.float())
        g, u = xq @ q(self.w_gate.detach(), ts_gu).t(), xq @ q(self.w_up.detach(), ts_gu).t()
        h = (torch.nn.functional.silu(g.bfloat16().float()) * u.bfloat16().float()).bfloat16().float()
        return q(h) @ q(self.w_down.detach(), ts_d).t()

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
torch.manual_seed(0)
H, I, M = 128, 256, 16
wg, wu, wd = torch.randn(I, H) * 0.1, torch.randn(I, H) * 0.1, torch.randn(H, I) * 0.1
x = torch.randn(M, H)
tp = TensorParallelGatedMLP(H, I, local=EmuMLP(H, I // world)).load_full_weights(wg, wu, wd)
assert tp.local_intermediate == I // world
y = tp(x)
full = EmuMLP(H, I)
full.w_gate.data, full.w_up.data, full.w_down.data = wg, wu, wd
from thor_fp4.parallel import full_tensor_scales
full.tensor_scales = full_tensor_scales(wg, wu, wd)
ref = full(x)
err = ((y - ref).norm() / ref.norm()).item()
assert err < 1e-5, err
# the same block with the partial outputs reduce-scattered by token rows: each rank holds its rows, fully summed
ts = TensorParallelGatedMLP(H, I, local=EmuMLP(H, I // world), exchange="reduce_scatter").load_full_weights(wg, wu, wd)
ys = ts(x)
rows = ts.owned_rows(M, on_device=False)
assert ys.shape == (M // world, H) and rows.numel() == M // world
assert ((ys - ref[rows]).norm() / ref[rows].norm()).item() < 1e-5
assert torch.equal(ts.gather(ys, M), y)
if rank == 0:
    print("TP_OK", err)
dist.destroy_process_group()
'''


def test_tensor_parallel_block_over_gloo(tmp_path):
    """world_size 2 on CPU: column-parallel gate/up + row-parallel down + one all-reduce equals
    the unsharded block (same full-tensor weight scales, per-rank dynamic block scales)."""
    script = tmp_path / "tp_worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, TFP4_PKG=str(ROOT / "thor-fp4_b200"), OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
