"""Tensor-parallel NVFP4 SwiGLU block: gate/up column-parallel, down row-parallel, one
all-reduce per block (the reference project is single-GPU; this is the sharding its
linear layers admit: independent output rows, and K slices whose 16-element blocks
never straddle ranks).

One process per GPU over torch.distributed (NCCL on GPUs; the host logic also runs
over gloo).  Every rank quantizes all of x (cheaper than exchanging codes), owns
intermediate/P rows of Wg, Wu and the matching K slice of Wd, and contributes a
partial [M, hidden] sum.  The per-tensor weight scales are those of the FULL
weights, so each rank's codes equal the corresponding slice of the unsharded
quantization.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _ext
from .fused import NVFP4GatedMLP

__all__ = ["TensorParallelGatedMLP", "shard_rows", "shard_cols"]


def _bounds(n: int, world: int, rank: int, align: int) -> tuple[int, int]:
    if n % (world * align) != 0:
        raise ValueError(f"dimension {n} does not split into {world} shards of a multiple of {align}")
    step = n // world
    return rank * step, (rank + 1) * step


def shard_rows(w: torch.Tensor, world: int, rank: int, align: int = 64) -> torch.Tensor:
    """Rows [rank*n/P, (rank+1)*n/P) of a (n, K) weight (column-parallel linear)."""
    a, b = _bounds(w.shape[0], world, rank, align)
    return w[a:b].contiguous()


def shard_cols(w: torch.Tensor, world: int, rank: int, align: int = 64) -> torch.Tensor:
    """Columns (K slice) of a (N, n) weight (row-parallel linear); align keeps whole
    16-element quantization blocks and whole 4-scale tiles on one rank."""
    a, b = _bounds(w.shape[1], world, rank, align)
    return w[:, a:b].contiguous()


def full_tensor_scales(w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> tuple[float, float]:
    """Two-level per-tensor scales of the unsharded [Wg; Wu] and Wd."""
    gu = max(w_gate.abs().amax().item(), w_up.abs().amax().item())
    return (max(gu / (6.0 * 448.0), 1e-30), max(w_down.abs().amax().item() / (6.0 * 448.0), 1e-30))


class _PushStaging:
    """Staging memory of the push exchange on one rank: two sets (used alternately, so that a rank may start pushing
    the next block while a slower rank still sums the previous one) of `world` slots of (rows, hidden) partial
    products - slot s receives rank s's partials for this rank's token rows.  The buffer is exported over CUDA IPC;
    every rank opens every other rank's buffer and keeps, per set and owner, the address of its own slot there."""

    def __init__(self, group, world: int, rank: int, rows: int, hidden: int, dtype: torch.dtype, device):
        L = _ext.device_lib()
        self.L, self.world, self.rank, self.rows, self.hidden = L, world, rank, rows, hidden
        self.esize = 4 if dtype == torch.float32 else 2
        self.set_bytes = world * rows * hidden * self.esize
        base = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        rc = L.tfp4_peer_alloc(2 * self.set_bytes, ctypes.byref(base), handle)
        self.base = base.value if rc == 0 else None
        self.peer_base, self._opened = [], []
        # every rank takes part in every collective below whatever happened locally, and all ranks learn together
        # whether the set-up worked: a rank that raised alone would leave the others waiting in a collective
        mine = torch.tensor(list(handle.raw), dtype=torch.uint8, device=device)
        allh = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine, group=group)
        ok = rc == 0
        for p in range(world):
            if p == rank:
                self.peer_base.append(self.base)
                continue
            ptr = ctypes.c_void_p()
            if ok and L.tfp4_peer_open(bytes(allh[p].cpu().tolist()), ctypes.byref(ptr)) == 0:
                self.peer_base.append(ptr.value)
                self._opened.append(ptr.value)
            else:
                ok = False
                self.peer_base.append(None)
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            self.close()
            raise RuntimeError("push exchange: sharing the staging buffers over CUDA IPC failed on at least one rank "
                               "(tfp4_peer_alloc / tfp4_peer_open; see the library's message on stderr)")
        slot = rank * rows * hidden * self.esize
        self.dest = [(ctypes.c_void_p * world)(*[self.peer_base[o] + k * self.set_bytes + slot for o in range(world)])
                     for k in range(2)]
        self.local_set = [self.base + k * self.set_bytes for k in range(2)]
        self.turn = 0

    def close(self):
        for ptr in self._opened:
            self.L.tfp4_peer_close(ptr)
        self._opened = []
        if self.base:
            self.L.tfp4_peer_free(self.base)
            self.base = None


class TensorParallelGatedMLP(nn.Module):
    """y = sum_p( down_p( nvfp4( silu(x Wg_p^T) * (x Wu_p^T) ) ) ), the sum taken over the ranks.

    `local` computes the rank's partial product; by default it is an NVFP4GatedMLP on
    this rank's GPU (partials in `reduce_dtype`, f32 unless told otherwise: rounding each
    partial to bf16 before the sum costs ~2e-3 relative error; "f16" costs ~3e-4 at half the
    bytes of f32, as long as no partial exceeds the f16 range).
    `group` defaults to the world group.

    exchange:
      "all_reduce"      every rank ends with all M rows of y (what a replicated consumer wants); each rank moves
                        2 (P-1)/P of the partial tensor;
      "reduce_scatter"  every rank ends with M/P rows of y, fully summed - the tokens stay sharded for a consumer
                        that works per token (residual add, norm, the next block's quantizer) and an all-gather is
                        paid only where a replicated tensor is really needed; half the bytes of the all-reduce.
                        forward() then returns the (M/P, hidden) rows `owned_rows(M)` of this rank.
      "push"            the reduce-scatter with its transfer inside the down projection: the GEMM's epilogue stores
                        each 32-row block of this rank's partial product into the staging buffer of the rank that owns
                        those token rows (TMA stores over NVLink into peer memory, issued while the tensor cores work
                        on the next tile), then one small collective orders the ranks and a local kernel sums the
                        staged partials.  No collective kernel competes with the GEMM for SMs.  Rank r ends with rows
                        [r M/P, (r+1) M/P); M must divide by 32 P.
      "copy"            the reduce-scatter with its transfer on the copy engines: the tokens are cut into chunks, each
                        chunk's f32 partial product is written locally by the down projection and then copied, slice by
                        slice (one cudaMemcpyAsync per owner, on a second stream), into the owners' staging buffers over
                        NVLink while the tensor cores work on the next chunk; copy engines use no SM, so the transfer
                        really runs beside the GEMMs and only the last chunk's copies are exposed.  Then the same
                        4-byte collective and local sum as "push".  Row ownership as "reduce_scatter" (rank r owns the
                        r-th 1/P of every chunk).
    The tokens are cut into `chunks` pieces: the exchange of one piece runs on the collective's own stream while
    this rank's GEMMs of the next piece run."""

    def __init__(self, hidden: int, intermediate: int, group=None, device=None,
                 reduce_dtype: str = "f32", weight_std: float | None = 0.02, local: nn.Module | None = None,
                 chunks: int = 4, exchange: str = "all_reduce"):
        super().__init__()
        if exchange not in ("all_reduce", "reduce_scatter", "push", "copy"):
            raise ValueError(f"exchange={exchange!r}: pick 'all_reduce' | 'reduce_scatter' | 'push' | 'copy'")
        self._side = None
        self._push: dict = {}
        self.group = group
        self.exchange = exchange
        self.chunks = max(1, int(chunks))     # token chunks: the exchange of one overlaps the GEMMs of the next
        self._y: dict = {}
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        a, b = _bounds(intermediate, self.world, self.rank, 64)
        self.hidden, self.intermediate, self.local_intermediate = hidden, intermediate, b - a
        self.local = local if local is not None else NVFP4GatedMLP(
            hidden, b - a, device=device, out_dtype=reduce_dtype, weight_std=weight_std)

    @torch.no_grad()
    def load_full_weights(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor):
        """Take this rank's shards of full (unsharded) weights and pin the full-tensor scales."""
        m = self.local
        m.w_gate.copy_(shard_rows(w_gate, self.world, self.rank))
        m.w_up.copy_(shard_rows(w_up, self.world, self.rank))
        m.w_down.copy_(shard_cols(w_down, self.world, self.rank))
        m.tensor_scales = full_tensor_scales(w_gate, w_up, w_down)
        m._q = None
        return self

    def exchange_name(self) -> str:
        if self.exchange == "copy":
            return (f"reduce-scatter by token rows on the copy engines: {self.chunks} token chunks, each chunk's partial rows "
                    "copied into the owners' staging buffers over NVLink (cudaMemcpyAsync on a second stream) beside the next "
                    "chunk's GEMMs, one 4-byte all-reduce as the barrier, local sum")
        if self.exchange == "push":
            return ("reduce-scatter by token rows inside the down projection: TMA stores of the partial tiles into the "
                    "owners' staging buffers over NVLink from the GEMM epilogue, one 4-byte all-reduce as the barrier, local sum")
        kind = "all-reduce" if self.exchange == "all_reduce" else "reduce-scatter by token rows"
        return f"NCCL {kind} of the partial outputs, {self.chunks} token chunks overlapped with the next chunk's GEMMs"

    # ------------------------------------------------------------------ token chunks
    def _chunk_bounds(self, M: int, on_device: bool) -> list[tuple[int, int]]:
        """Token chunks [r0, r1): multiples of 256 rows (whole GEMM tiles) whose sizes divide by the world size."""
        n = self.chunks if (M >= 256 * self.chunks and on_device) else 1
        step = -(-M // n)
        step = -(-step // 256) * 256
        if self.exchange in ("reduce_scatter", "copy") and M % self.world != 0:
            raise ValueError(f"reduce_scatter needs the token count ({M}) to divide by the world size ({self.world})")
        return [(r0, min(M, r0 + step)) for r0 in range(0, M, step)]

    def owned_rows(self, M: int, on_device: bool = True) -> torch.Tensor:
        """Global token indices of the rows forward() returns on this rank under exchange='reduce_scatter'
        (chunk by chunk, this rank's 1/P of each chunk)."""
        if self.exchange == "push":
            n = M // self.world
            return torch.arange(self.rank * n, (self.rank + 1) * n)
        idx = []
        for r0, r1 in self._chunk_bounds(M, on_device):
            n = (r1 - r0) // self.world
            idx.append(torch.arange(r0 + self.rank * n, r0 + (self.rank + 1) * n))
        return torch.cat(idx)

    def gather(self, y_local: torch.Tensor, M: int) -> torch.Tensor:
        """All-gather the reduce-scattered rows back into the replicated (M, hidden) tensor in token order."""
        parts = [torch.empty_like(y_local) for _ in range(self.world)]
        dist.all_gather(parts, y_local.contiguous(), group=self.group)
        if self.exchange == "push":
            return torch.cat(parts, dim=0)
        out = torch.empty(M, y_local.shape[1], dtype=y_local.dtype, device=y_local.device)
        on_device = y_local.is_cuda
        pos = 0
        for r0, r1 in self._chunk_bounds(M, on_device):
            n = (r1 - r0) // self.world
            for p in range(self.world):
                out[r0 + p * n: r0 + (p + 1) * n] = parts[p][pos: pos + n]
            pos += n
        return out

    def _reduce_scatter(self, dst: torch.Tensor, src: torch.Tensor, async_op: bool):
        if dist.get_backend(self.group) == "gloo":      # gloo has no reduce-scatter: same result through an all-reduce
            dist.all_reduce(src, op=dist.ReduceOp.SUM, group=self.group)
            n = src.shape[0] // self.world
            dst.copy_(src[self.rank * n:(self.rank + 1) * n])
            return None
        return dist.reduce_scatter_tensor(dst, src, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)

    def _forward_push(self, x: torch.Tensor) -> torch.Tensor:
        m, L = self.local, _ext.device_lib()
        M, H = x.shape[0], self.hidden
        if M % (32 * self.world) != 0:
            raise ValueError(f"exchange='push' needs the token count ({M}) to divide by 32 x world size ({32 * self.world})")
        rows = M // self.world
        dt = _ext.OUT_TORCH[m.out_dtype]
        if dt not in (torch.float32, torch.float16, torch.bfloat16):
            raise ValueError("exchange='push' stages f32, f16 or bf16 partials")
        st = self._push.get((M, dt))
        if st is None:
            stg = _PushStaging(self.group, self.world, self.rank, rows, H, dt, x.device)
            st = self._push[(M, dt)] = (stg, torch.empty(rows, H, dtype=dt, device=x.device),
                                        torch.zeros(1, dtype=torch.int32, device=x.device))
        stg, ys, flag = st
        hp, hs = m(x, down=False)
        wd = m._q[1]
        k = stg.turn
        stg.turn ^= 1
        rc = L.tfp4_gemm_push(hp.data_ptr(), hs.data_ptr(), 1.0, wd.packed.data_ptr(), wd.sblk.data_ptr(), float(wd.tensor_scale),
                              stg.dest[k], self.world, rows, (self.rank + 1) % self.world, M, H, self.local_intermediate,
                              _ext.OUT_DTYPE[m.out_dtype], _ext.stream())
        assert rc == 0, f"tfp4_gemm_push rc={rc}"
        # every rank's stores have landed once every rank's GEMM has completed: a 4-byte collective in stream order
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        rc = L.tfp4_sum_slots(stg.local_set[k], self.world, rows, H, _ext.IN_DTYPE[dt], ys.data_ptr(),
                              _ext.OUT_DTYPE[m.out_dtype], _ext.stream())
        assert rc == 0, f"tfp4_sum_slots rc={rc}"
        return ys

    def _forward_copy(self, x: torch.Tensor) -> torch.Tensor:
        m, L = self.local, _ext.device_lib()
        M, H = x.shape[0], self.hidden
        bounds = self._chunk_bounds(M, True)
        if any((r1 - r0) % self.world for r0, r1 in bounds):
            raise ValueError(f"exchange='copy' needs every token chunk to divide by the world size ({self.world})")
        rows = M // self.world
        dt = _ext.OUT_TORCH[m.out_dtype]
        if dt not in (torch.float32, torch.float16, torch.bfloat16):
            raise ValueError("exchange='copy' stages f32, f16 or bf16 partials")
        st = self._push.get((M, dt, "copy"))
        if st is None:
            stg = _PushStaging(self.group, self.world, self.rank, rows, H, dt, x.device)
            st = self._push[(M, dt, "copy")] = (stg, torch.empty(rows, H, dtype=dt, device=x.device),
                                                torch.zeros(1, dtype=torch.int32, device=x.device),
                                                torch.empty(M, H, dtype=dt, device=x.device))
        stg, ys, flag, y = st
        if self._side is None:
            self._side = torch.cuda.Stream(device=x.device)
        side, main = self._side, torch.cuda.current_stream()
        k = stg.turn
        stg.turn ^= 1
        row_bytes = H * stg.esize
        pos = 0
        for r0, r1 in bounds:
            m(x[r0:r1], out=y[r0:r1])                                   # this chunk's partial product, local
            ev = torch.cuda.Event()
            ev.record(main)
            side.wait_event(ev)
            n = (r1 - r0) // self.world
            # owner o takes the o-th 1/P of the chunk.  Rank r sends to r+1, r+2, ... in turn: at every step each GPU
            # sends one slice and receives one (all ranks starting with owner 0 would pile three to seven senders onto
            # one receiver's links at a time: measured 400-450 GB/s out per rank instead of the link rate)
            for j in range(1, self.world + 1):
                o = (self.rank + j) % self.world
                dst = stg.dest[k][o] + pos * row_bytes
                src = y.data_ptr() + (r0 + o * n) * row_bytes
                rc = L.tfp4_peer_copy(dst, src, n * row_bytes, side.cuda_stream)
                assert rc == 0, f"tfp4_peer_copy rc={rc}"
            pos += n
        main.wait_stream(side)
        # every rank's copies have landed once every rank has got here: a 4-byte collective in stream order
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        rc = L.tfp4_sum_slots(stg.local_set[k], self.world, rows, H, _ext.IN_DTYPE[dt], ys.data_ptr(),
                              _ext.OUT_DTYPE[m.out_dtype], _ext.stream())
        assert rc == 0, f"tfp4_sum_slots rc={rc}"
        return ys

    def close(self):
        """Release the IPC mappings and staging buffers of the push and copy exchanges (call on every rank before the
        process group goes away; nothing to do for the other exchanges)."""
        for entry in self._push.values():
            entry[0].close()
        self._push = {}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return self.local(x)
        if self.exchange == "push":
            return self._forward_push(x)
        if self.exchange == "copy":
            return self._forward_copy(x)
        M = x.shape[0]
        bounds = self._chunk_bounds(M, x.is_cuda)
        scatter = self.exchange == "reduce_scatter"
        if len(bounds) == 1 and not scatter:
            y = self.local(x)
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            return y
        # The partial outputs are exchanged chunk by chunk: NCCL runs on its own stream, ordered after
        # the chunk's GEMMs, while this stream goes on with the next chunk.
        r0, r1 = bounds[0]
        first = self.local(x[r0:r1])
        key = (M, first.dtype, scatter)
        bufs = self._y.get(key)
        if bufs is None:
            y = torch.empty(M, first.shape[1], dtype=first.dtype, device=first.device)
            ys = torch.empty(M // self.world, first.shape[1], dtype=first.dtype, device=first.device) if scatter else None
            bufs = self._y[key] = (y, ys)
        y, ys = bufs
        works, pos = [], 0
        for i, (r0, r1) in enumerate(bounds):
            if i == 0:
                y[r0:r1].copy_(first)
            else:
                self.local(x[r0:r1], out=y[r0:r1]) if x.is_cuda else y[r0:r1].copy_(self.local(x[r0:r1]))
            if scatter:
                n = (r1 - r0) // self.world
                works.append(self._reduce_scatter(ys[pos:pos + n], y[r0:r1], async_op=True))
                pos += n
            else:
                works.append(dist.all_reduce(y[r0:r1], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        for w in works:
            if w is not None:
                w.wait()
        return ys if scatter else y
