"""Tensor parallelism for the quantized Linear layers and row sharding for the quantizers (one process per GPU).

The reference distributes models through a fork of torch's DTensor (chop/distributed/launcher.py:57-148) and has no
hand-placed tensor parallelism; for the MX path only two placements matter, so they are written out here:

* column parallel (q/k/v, gate, up): `W[N, K] -> W[N/G, K]`.  MX blocks run along K, so a split along N leaves every
  block, code and scale untouched; the output stays sharded along N and feeds a row-parallel layer.
* row parallel (o, down): `W[N, K] -> W[N, K/G]` with `K/G` a multiple of the block size, so blocks and scales are
  local; each rank produces a float32 partial `[M, N]`, the partials are summed by an all-reduce (NCCL over NVLink) and
  only the sum is rounded to the output dtype.  Summing bf16 partials instead costs ~2e-3 of max, above the parity bar.
* quantizers: every block is independent; shards are contiguous row ranges, no communication.

The collective plumbing is torch.distributed only, so the same code runs under the gloo backend on CPU ranks with an
injected local layer (tests) and under NCCL with the CUDA layers of this package.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor, nn


@dataclass
class TPGroup:
    rank: int
    world: int
    group: object = None  # torch.distributed process group (None = default)

    @staticmethod
    def from_env(group=None) -> "TPGroup":
        if dist.is_available() and dist.is_initialized():
            return TPGroup(dist.get_rank(group), dist.get_world_size(group), group)
        return TPGroup(0, 1, None)


def shard_bounds(n: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Contiguous range [start, stop) of `n` items for `rank`; boundaries are multiples of `multiple`."""
    if n % multiple:
        raise ValueError(f"{n} is not a multiple of {multiple}")
    units = n // multiple
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    stop = start + base + (1 if rank < extra else 0)
    return start * multiple, stop * multiple


def shard_rows_for_quantizer(x: Tensor, block_size: int, tp: TPGroup) -> Tensor:
    """This rank's rows of a 2-D tensor that is quantized in blocks along the last dim (flattened blocks may straddle
    rows, so the split falls on a multiple of lcm(cols, block) elements).  No communication is needed afterwards."""
    rows, cols = x.shape
    per = math.lcm(cols, block_size) // cols
    if rows % per:
        raise ValueError(f"{rows} rows cannot be split on block boundaries of {block_size} with {cols} columns")
    r0, r1 = shard_bounds(rows, tp.world, tp.rank, per)
    return x[r0:r1]


def shard_linear_weight(weight: Tensor, mode: str, tp: TPGroup, block_size: int = 32) -> Tensor:
    """Slice of W[N, K] owned by this rank: rows for mode 'column', columns on block boundaries for mode 'row'."""
    n, k = weight.shape
    if mode == "column":
        a, b = shard_bounds(n, tp.world, tp.rank)
        return weight[a:b]
    if mode == "row":
        if k % (tp.world * block_size):
            raise ValueError(f"in_features {k} must split into {tp.world} shards that are multiples of the block "
                             f"size {block_size} so that blocks and scales stay local")
        a, b = shard_bounds(k, tp.world, tp.rank, block_size)
        return weight[:, a:b]
    raise ValueError(f"unknown mode {mode!r}")


class ColumnParallelLinear(nn.Module):
    """Output features split over the ranks.  `inner` is a quantized Linear of shape [N/G, K] (any module mapping
    [..., K] -> [..., N/G]); the input is replicated, the output stays sharded unless `gather_output`."""

    def __init__(self, inner: nn.Module, tp: TPGroup, gather_output: bool = False):
        super().__init__()
        self.inner, self.tp, self.gather_output = inner, tp, gather_output

    def forward(self, x: Tensor) -> Tensor:
        y = self.inner(x)
        if not self.gather_output or self.tp.world == 1:
            return y
        parts = [torch.empty_like(y) for _ in range(self.tp.world)]
        dist.all_gather(parts, y.contiguous(), group=self.tp.group)
        return torch.cat(parts, dim=-1)


class RowParallelLinear(nn.Module):
    """Input features split over the ranks.  `inner` maps this rank's [..., K/G] slice to a float32 partial
    [..., N] (bias-free); partials are all-reduced, then the bias is added and the sum cast to `out_dtype`.

    With `chunks > 1` the rows are processed in chunks and each chunk's all-reduce is issued asynchronously, so the
    collective of chunk i overlaps the GEMM of chunk i+1."""

    def __init__(self, inner: nn.Module, tp: TPGroup, bias: Tensor | None = None, chunks: int = 1):
        super().__init__()
        self.inner, self.tp, self.chunks = inner, tp, max(1, chunks)
        if hasattr(inner, "output_dtype"):
            inner.output_dtype = torch.float32
        self.bias = None if bias is None else nn.Parameter(bias, requires_grad=False)

    def forward(self, x_shard: Tensor) -> Tensor:
        out_dtype = x_shard.dtype
        lead = x_shard.shape[:-1]
        x2 = x_shard.reshape(-1, x_shard.shape[-1])
        pieces = x2.chunk(self.chunks, dim=0) if self.chunks > 1 and x2.shape[0] >= self.chunks else [x2]
        partials, works = [], []
        for piece in pieces:
            p = self.inner(piece)
            if p.dtype != torch.float32:
                p = p.float()
            if self.tp.world > 1:
                works.append(dist.all_reduce(p, op=dist.ReduceOp.SUM, group=self.tp.group, async_op=True))
            partials.append(p)
        for w in works:
            w.wait()
        y = partials[0] if len(partials) == 1 else torch.cat(partials, dim=0)
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(out_dtype).reshape(*lead, y.shape[-1])


def build_tp_linear(cls, weight: Tensor, bias: Tensor | None, config: dict, mode: str, tp: TPGroup, device=None,
                    dtype=None, **kwargs) -> nn.Module:
    """Shard a full `nn.Linear` state and build the quantized layer `cls` (LinearMXFP / LinearMXInt / LinearBlockFP of
    this package) for this rank, going through `load_state_dict` exactly like the quantize pass does."""
    block = config.get("weight_block_size", 32)
    block = block[-1] if isinstance(block, (list, tuple)) else block
    w = shard_linear_weight(weight, mode, tp, block).contiguous()
    n_local, k_local = w.shape
    device = device if device is not None else weight.device
    dtype = dtype if dtype is not None else weight.dtype
    if mode == "column":
        b = None
        if bias is not None:
            a, e = shard_bounds(weight.shape[0], tp.world, tp.rank)
            b = bias[a:e].contiguous()
        inner = cls(k_local, n_local, bias=b is not None, device=device, dtype=dtype, config=dict(config))
        state = {"weight": w.to(device=device, dtype=dtype)}
        if b is not None:
            state["bias"] = b.to(device=device, dtype=dtype)
        inner.load_state_dict(state, strict=False)
        return ColumnParallelLinear(inner, tp, **kwargs)
    inner = cls(k_local, n_local, bias=False, device=device, dtype=dtype, config=dict(config))
    inner.load_state_dict({"weight": w.to(device=device, dtype=dtype)}, strict=False)
    return RowParallelLinear(inner, tp, None if bias is None else bias.to(device=device, dtype=dtype), **kwargs)


class TPGatedMLP(nn.Module):
    """y = down(silu(gate(x)) * up(x)) with gate/up column parallel and down row parallel: one all-reduce per layer."""

    def __init__(self, gate: nn.Module, up: nn.Module, down: nn.Module):
        super().__init__()
        self.gate, self.up, self.down = gate, up, down

    def forward(self, x: Tensor) -> Tensor:
        return self.down(torch.nn.functional.silu(self.gate(x)) * self.up(x))
