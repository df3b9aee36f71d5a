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

import torch
import torch.distributed as dist
import torch.nn as nn

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


class TensorParallelGatedMLP(nn.Module):
    """y = all_reduce_sum_p( down_p( nvfp4( silu(x Wg_p^T) * (x Wu_p^T) ) ) ).

    `local` computes the rank's partial product; by default it is an NVFP4GatedMLP on
    this rank's GPU (partials in `reduce_dtype`, f32 unless told otherwise, because
    rounding each partial to bf16 before the sum costs ~1.6e-3 relative error).
    `group` defaults to the world group."""

    def __init__(self, hidden: int, intermediate: int, group=None, device=None,
                 reduce_dtype: str = "f32", weight_std: float | None = 0.02, local: nn.Module | None = None,
                 chunks: int = 4):
        super().__init__()
        self.group = group
        self.chunks = max(1, int(chunks))     # token chunks: the all-reduce of one overlaps the GEMMs of the next
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
        return f"NCCL all-reduce of the partial outputs, {self.chunks} token chunks overlapped with the next chunk's GEMMs"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return self.local(x)
        M = x.shape[0]
        n = self.chunks if (M >= 256 * self.chunks and x.is_cuda) else 1
        if n == 1:
            y = self.local(x)
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            return y
        # The partial outputs are summed chunk by chunk: NCCL runs on its own stream, ordered after
        # the chunk's GEMMs, while this stream goes on with the next chunk.
        step = -(-M // n)
        step = -(-step // 256) * 256
        first = self.local(x[:step])
        y = self._y.get((M, first.dtype))
        if y is None:
            y = torch.empty(M, first.shape[1], dtype=first.dtype, device=first.device)
            self._y[(M, first.dtype)] = y
        works = []
        for r0 in range(0, M, step):
            r1 = min(M, r0 + step)
            if r0 == 0:
                y[:r1].copy_(first)
            else:
                self.local(x[r0:r1], out=y[r0:r1])
            works.append(dist.all_reduce(y[r0:r1], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        for w in works:
            w.wait()
        return y
