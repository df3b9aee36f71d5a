"""Tensor-parallel gated MLP on two GPUs (NCCL): the sharded block with the chunked, overlapped
all-reduce against the unsharded block on one GPU.  Skipped where fewer than two GPUs are visible."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

gpu = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.path.join(sys.argv[1], "thor-fp4_b200"))
    from thor_fp4.fused import NVFP4GatedMLP
    from thor_fp4.parallel import TensorParallelGatedMLP, full_tensor_scales
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    H, I, M = 512, 1024, 1536
    g = torch.Generator().manual_seed(11)
    wg, wu, wd = (torch.randn(I, H, generator=g) * 0.05, torch.randn(I, H, generator=g) * 0.05, torch.randn(H, I, generator=g) * 0.05)
    x = torch.randn(M, H, generator=g).bfloat16().cuda()
    tp = TensorParallelGatedMLP(H, I, device="cuda", reduce_dtype="f32", chunks=3).load_full_weights(wg.cuda(), wu.cuda(), wd.cuda())
    y = tp(x).clone()
    y2 = tp(x).clone()                      # second call: cached buffers, same result
    torch.cuda.synchronize()
    if rank == 0:
        full = NVFP4GatedMLP(H, I, device="cuda", out_dtype="f32")
        with torch.no_grad():
            full.w_gate.copy_(wg); full.w_up.copy_(wu); full.w_down.copy_(wd)
        full.tensor_scales = full_tensor_scales(wg, wu, wd)
        ref = full(x).float()
        err = ((y - ref).norm() / ref.norm()).item()
        print("TP_ERR", err, "REPEAT_EQUAL", bool(torch.equal(y, y2)))
    # the partial outputs reduce-scattered by token rows: each rank's rows equal the all-reduced ones
    ts = TensorParallelGatedMLP(H, I, device="cuda", reduce_dtype="f32", chunks=3, exchange="reduce_scatter")
    ts.load_full_weights(wg.cuda(), wu.cuda(), wd.cuda())
    ys = ts(x).clone()
    rows = ts.owned_rows(M).cuda()
    same = bool(((ys - y[rows]).norm() / y[rows].norm()).item() < 1e-6)
    back = ts.gather(ys, M)
    ok = torch.tensor([int(same and ((back - y).norm() / y.norm()).item() < 1e-6)], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("RS_OK", int(ok.item()))
    # the reduce-scatter with its transfer inside the down projection (TMA stores into the owners' staging buffers)
    tpush = TensorParallelGatedMLP(H, I, device="cuda", reduce_dtype="f32", exchange="push")
    tpush.load_full_weights(wg.cuda(), wu.cuda(), wd.cuda())
    good = True
    for it in range(3):                               # three blocks in a row: both staging sets get reused
        xi = x if it != 1 else (x * 0.5).bfloat16()
        yi = tp(xi).clone()
        yp = tpush(xi).clone()
        rows_p = tpush.owned_rows(M).cuda()
        good = good and yp.shape == (M // 2, H) and ((yp - yi[rows_p]).norm() / yi[rows_p].norm()).item() < 1e-6
        good = good and ((tpush.gather(yp, M) - yi).norm() / yi.norm()).item() < 1e-6
    # ... and with its transfer on the copy engines, chunk by chunk beside the next chunk's GEMMs
    tcopy = TensorParallelGatedMLP(H, I, device="cuda", reduce_dtype="f32", chunks=3, exchange="copy")
    tcopy.load_full_weights(wg.cuda(), wu.cuda(), wd.cuda())
    for it in range(3):
        xi = x if it != 1 else (x * 0.5).bfloat16()
        yi = tp(xi).clone()
        yc = tcopy(xi).clone()
        rows_c = tcopy.owned_rows(M).cuda()
        good = good and yc.shape == (M // 2, H) and ((yc - yi[rows_c]).norm() / yi[rows_c].norm()).item() < 1e-6
        good = good and ((tcopy.gather(yc, M) - yi).norm() / yi.norm()).item() < 1e-6
    torch.cuda.synchronize()
    tcopy.close()
    # bf16 partials through the push epilogue (two 32-column chunks per TMA store): each partial is rounded once to bf16
    # before the sum, so the result tracks the f32 exchange to a few bf16 ulps
    tpb = TensorParallelGatedMLP(H, I, device="cuda", reduce_dtype="bf16", exchange="push")
    tpb.load_full_weights(wg.cuda(), wu.cuda(), wd.cuda())
    for it in range(2):
        yb = tpb(x).float()
        rows_b = tpb.owned_rows(M).cuda()
        good = good and yb.shape == (M // 2, H) and ((yb - y[rows_b]).norm() / y[rows_b].norm()).item() < 8e-3
    # ... and f16 partials: 2^-12 per partial, so the sum stays within 1e-3 of the f32 exchange
    tph = TensorParallelGatedMLP(H, I, device="cuda", reduce_dtype="f16", exchange="push")
    tph.load_full_weights(wg.cuda(), wu.cuda(), wd.cuda())
    for it in range(2):
        yh = tph(x).float()
        good = good and yh.shape == (M // 2, H) and ((yh - y[rows_b]).norm() / y[rows_b].norm()).item() < 1e-3
    torch.cuda.synchronize()
    okp = torch.tensor([int(good)], device="cuda")
    dist.all_reduce(okp, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    tpush.close()
    tpb.close()
    tph.close()
    if rank == 0:
        print("PUSH_OK", int(okp.item()))
    dist.destroy_process_group()
''')


@gpu
def test_tensor_parallel_mlp_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29631", str(script), ROOT],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("TP_ERR")][0].split()
    # the sharded down projection sums two f32 partials instead of one accumulation: same codes, same products
    assert float(line[1]) < 1e-3
    assert line[3] == "True"
    assert "RS_OK 1" in out.stdout
    assert "PUSH_OK 1" in out.stdout
