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

reduce="fused" takes the collective library off the data path of the row-parallel layer: the GEMM's epilogue stores
each fp32 tile into the memory of the GPU that owns its rows (symmetric memory, peer stores over NVLink), and one small
kernel per GPU sums its slice in rank order, rounds once and writes the slice into every GPU's output (`PeerReducer`).
"""

from __future__ import annotations

import contextlib
import importlib
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

    def __init__(self, inner: nn.Module, tp: TPGroup, gather_output: bool = False, out_features: int | None = None):
        super().__init__()
        if gather_output and out_features is not None and out_features % tp.world:
            raise ValueError(f"gather_output needs out_features ({out_features}) divisible by the {tp.world} ranks: "
                             "all-gather takes equal shards")
        self.inner, self.tp, self.gather_output = inner, tp, gather_output

    def forward(self, x) -> Tensor:
        # x: a tensor, or the (operand, leading shape) pair a fused row-parallel layer delivers with `emit_packed`
        y = self.inner.forward_quantized(x) if isinstance(x, tuple) else self.inner(x)
        if not self.gather_output or self.tp.world == 1:
            return y
        parts = [torch.empty_like(y) for _ in range(self.tp.world)]
        dist.all_gather(parts, y.contiguous(), group=self.tp.group)
        return torch.cat(parts, dim=-1)


class PeerReducer:
    """Symmetric buffers and launches of the fused row-parallel reduction (mxq_gemm_mxf8_scatter, mxq_peer_barrier,
    mxq_reduce_gather of include/mxq.h) for one tensor-parallel group on one GPU.

    Buffers are allocated once per (rows, columns, output type, tag) through torch's symmetric memory and exchanged
    with the other ranks (a collective call: every rank must ask for the same buffers in the same order).  `tag`
    separates reductions that are in flight at the same time (micro-batches).  The barrier epoch is a plain counter
    that every rank advances in lockstep."""

    _instances: dict = {}

    @classmethod
    def for_group(cls, tp: TPGroup, device) -> "PeerReducer":
        key = (id(tp.group), torch.device(device).index)
        if key not in cls._instances:
            cls._instances[key] = cls(tp, device)
        return cls._instances[key]

    def __init__(self, tp: TPGroup, device):
        import ctypes

        symm_mem = importlib.import_module("torch.distributed._symmetric_memory")
        self.tp, self.device = tp, torch.device(device)
        self._symm = symm_mem
        self._group = tp.group if tp.group is not None else dist.group.WORLD
        self._plans: dict = {}
        self._ctypes = ctypes
        self.epoch = 0
        self.flags, self.flag_ptrs = self._alloc(64, torch.int32)
        self.flags.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=tp.group)  # every rank's flags are zero before anyone publishes an epoch

    @staticmethod
    def available(tp: TPGroup, device) -> bool:
        if tp.world < 2 or tp.world > 8 or torch.device(device).type != "cuda":
            return False
        try:
            importlib.import_module("torch.distributed._symmetric_memory")
        except Exception:
            return False
        return dist.get_backend(tp.group) == "nccl"

    def _alloc(self, numel: int, dtype):
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        hdl = self._symm.rendezvous(t, self._group)
        ptrs = (self._ctypes.c_void_p * self.tp.world)(*[int(p) for p in hdl.buffer_ptrs])
        return t, ptrs

    def plan(self, rows: int, cols: int, out_dtype, tag: int = 0, packed: bool = False) -> dict:
        key = (rows, cols, out_dtype, tag)
        if key not in self._plans:
            slots, slot_ptrs = self._alloc(rows * cols, torch.float32)
            out, out_ptrs = self._alloc(rows * cols, out_dtype)
            self._plans[key] = {"slots": slots, "slot_ptrs": slot_ptrs, "out": out.view(rows, cols), "out_ptrs": out_ptrs}
        plan = self._plans[key]
        if packed and "codes" not in plan:  # operand buffers for a consumer that takes the result as MXFP codes
            from . import _lib

            codes, code_ptrs = self._alloc(rows * cols, torch.uint8)
            scales, scale_ptrs = self._alloc(int(_lib.lib().mxq_mma_scale_bytes(rows, cols)), torch.uint8)
            plan.update({"codes": codes.view(rows, cols), "code_ptrs": code_ptrs, "scales": scales, "scale_ptrs": scale_ptrs})
        return plan

    def barrier(self, status: Tensor, stream) -> None:
        from . import _lib

        self.epoch += 1
        rc = _lib.lib().mxq_peer_barrier(self.flag_ptrs, self.tp.world, self.tp.rank, self.epoch & 0xFFFFFFFF,
                                         status.data_ptr(), 0, stream)
        _lib.check(rc, "mxq_peer_barrier")

    def scatter_gemm(self, a_op, w_op, plan: dict, status: Tensor, options_ptr, stream) -> None:
        """This rank's partial product, stored tile by tile into the owners' slots."""
        from . import _lib

        rc = _lib.lib().mxq_gemm_mxf8_scatter(a_op.codes.data_ptr(), a_op.scales.data_ptr(), w_op.codes.data_ptr(),
                                              w_op.scales.data_ptr(), w_op.format, plan["slot_ptrs"], self.tp.world,
                                              self.tp.rank, a_op.rows, w_op.rows, a_op.k, status.data_ptr(), options_ptr,
                                              stream)
        _lib.check(rc, "mxq_gemm_mxf8_scatter")

    def reduce_gather(self, plan: dict, bias: Tensor | None, max_ctas: int, stream, pack: tuple | None = None) -> None:
        """Sum this rank's slice and write it into every rank's output; with `pack=(E, F)` into every rank's MXFP
        operand buffers instead (the next layer's activation, already quantized)."""
        from . import _lib
        from .quantizers import _DT, _floor_tab_ptr

        rows, cols = plan["out"].shape
        b = None if bias is None else bias.contiguous()
        if pack is not None:
            rc = _lib.lib().mxq_reduce_gather_pack(plan["slots"].data_ptr(), self.tp.world, self.tp.rank,
                                                   rows // self.tp.world, cols, 0 if b is None else b.data_ptr(),
                                                   0 if b is None else _DT[b.dtype], plan["code_ptrs"], plan["scale_ptrs"],
                                                   None, pack[0], pack[1], _floor_tab_ptr(), max_ctas, stream)
            _lib.check(rc, "mxq_reduce_gather_pack")
            return
        rc = _lib.lib().mxq_reduce_gather(plan["slots"].data_ptr(), self.tp.world, self.tp.rank, rows // self.tp.world, cols,
                                          0 if b is None else b.data_ptr(), 0 if b is None else _DT[b.dtype],
                                          plan["out_ptrs"], _DT[plan["out"].dtype], max_ctas, stream)
        _lib.check(rc, "mxq_reduce_gather")


class RowParallelLinear(nn.Module):
    """Input features split over the ranks.  `inner` maps this rank's [..., K/G] slice to a float32 partial
    [..., N] (bias-free); the partials are summed across ranks in float32, then the bias is added and the sum is
    cast to the input dtype.

    reduce="all_reduce": one float32 all-reduce.  reduce="scatter_gather": float32 reduce-scatter over rows, cast,
    all-gather in the output dtype (fewer bytes on the wire; needs rows divisible by the number of ranks and falls
    back to the all-reduce otherwise).  Measured on 8 B200 for [8192, 8192]: 0.72 ms vs 0.62 ms.
    reduce="fused": no collective on the data path (see `PeerReducer`): the inner layer's GEMM stores its fp32 tiles
    into the owning GPUs' memory, then barrier, reduce + all-gather kernel, barrier.  Needs a LinearMXFP inner layer on
    the block-scaled path, rows divisible by 256 x ranks and NCCL ranks on one node; anything else takes the
    scatter_gather route.  The result of a fused call lives in a buffer that the next call with the same shape and
    `tag` overwrites: `forward` returns a copy, `finish(handle, keep=True)` the buffer itself.

    `start(x)` / `finish(handle)` split the call so that a caller can overlap the collective (issued on a side
    stream) with other work; `forward` is `finish(start(x))`."""

    def __init__(self, inner: nn.Module, tp: TPGroup, bias: Tensor | None = None, reduce: str = "all_reduce",
                 reduce_ctas: int = 0):
        super().__init__()
        assert reduce in ("all_reduce", "scatter_gather", "fused")
        self.inner, self.tp, self.reduce = inner, tp, reduce
        self.reduce_ctas = reduce_ctas  # grid cap of the fused reduce + all-gather kernel (0 = whole GPU)
        if hasattr(inner, "output_dtype") and (tp.world > 1 or bias is not None):
            inner.output_dtype = torch.float32  # fp32 until the partial sums and the bias have been added: one rounding
        self.bias = None if bias is None else nn.Parameter(bias, requires_grad=False)
        self._comm_stream = None

    def _side_stream(self, device):
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=device)
        return self._comm_stream

    # ---- fused route ------------------------------------------------------------------------------------------------
    def _fused_applies(self, like: Tensor) -> bool:
        if self.reduce != "fused" or self.tp.world == 1 or not like.is_cuda:
            return False
        inner = self.inner
        rows = like.numel() // like.shape[-1]
        e5m2 = any((inner.config.get(k + "_exponent_width"), inner.config.get(k + "_frac_width")) == (5, 2)
                   for k in ("weight", "data_in")) if hasattr(inner, "config") else False
        return (hasattr(inner, "_uses_packed_path") and inner._uses_packed_path(like) and inner.bias is None and not e5m2
                and rows % (256 * self.tp.world) == 0 and inner.out_features % 8 == 0
                and PeerReducer.available(self.tp, like.device))

    def _start_fused(self, a_op, like: Tensor, tag: int, emit_packed: tuple | None = None):
        from . import gemm

        red = PeerReducer.for_group(self.tp, like.device)
        if emit_packed is not None and (like.dtype != torch.bfloat16 or self.inner.out_features % 128):
            emit_packed = None
        plan = red.plan(a_op.rows, self.inner.out_features, like.dtype, tag, packed=emit_packed is not None)
        status = gemm._status(like.device)
        cur = torch.cuda.current_stream(like.device)
        red.scatter_gemm(a_op, self.inner._packed_weight(), plan, status, gemm._options_ptr(), cur.cuda_stream)
        side = self._side_stream(like.device)
        side.wait_stream(cur)
        red.barrier(status, side.cuda_stream)          # every GPU's tiles have landed
        red.reduce_gather(plan, self.bias, self.reduce_ctas, side.cuda_stream, pack=emit_packed)
        red.barrier(status, side.cuda_stream)          # every GPU's slice has landed
        ev = torch.cuda.Event()
        ev.record(side)
        a_op.codes.record_stream(side)
        if emit_packed is not None:
            op = gemm.MXOperand(plan["codes"], plan["scales"], a_op.rows, self.inner.out_features)
            return (op, ev, like.dtype, like.shape[:-1], "fused_packed")
        return (plan["out"], ev, like.dtype, like.shape[:-1], "fused")

    def start_gated(self, gate: Tensor, up: Tensor, tag: int = 0, emit_packed: tuple | None = None):
        """`start(silu(gate) * up)` for a gated MLP; the product goes straight into the inner layer's quantized
        operand when that layer can take it (`forward_gated`).  `emit_packed=(E, F)` (fused route only): deliver the
        result as the MXFP operand of a consumer that quantizes it with that format, see `finish`."""
        if self._fused_applies(gate):
            from . import gemm

            _, _, x_exp, x_frac = self.inner._input_format()
            k = gate.shape[-1]
            a_op = gemm.pack_gated_operand(gate.reshape(-1, k), up.reshape(-1, k), x_exp, x_frac)
            return self._start_fused(a_op, gate, tag, emit_packed)
        if hasattr(self.inner, "forward_gated"):
            k = gate.shape[-1]
            return self.start(None, partial=self.inner.forward_gated(gate.reshape(-1, k), up.reshape(-1, k)),
                              like=gate)
        return self.start(torch.nn.functional.silu(gate) * up)

    def start(self, x_shard: Tensor | None, partial: Tensor | None = None, like: Tensor | None = None, tag: int = 0):
        """Local GEMM on the current stream, collective on a side stream; returns a handle for `finish`."""
        like = x_shard if like is None else like
        if partial is None and self._fused_applies(like):
            a_op, _ = self.inner.quantize_input(x_shard.reshape(-1, x_shard.shape[-1]))
            return self._start_fused(a_op, like, tag)
        out_dtype = like.dtype
        lead = like.shape[:-1]
        p = partial if partial is not None else self.inner(x_shard.reshape(-1, x_shard.shape[-1]))
        if self.tp.world == 1:  # nothing to add up: the inner layer's result in its own dtype
            return (p, None, out_dtype, lead, None)
        if p.dtype != torch.float32:
            p = p.float()
        rows = p.shape[0]
        use_sg = self.reduce in ("scatter_gather", "fused") and rows % self.tp.world == 0
        if not p.is_cuda:  # CPU ranks (gloo): no streams, plain all-reduce
            dist.all_reduce(p, op=dist.ReduceOp.SUM, group=self.tp.group)
            return (p, None, out_dtype, lead, None)
        side = self._side_stream(p.device)
        side.wait_stream(torch.cuda.current_stream(p.device))
        with torch.cuda.stream(side):
            if use_sg:
                part = torch.empty((rows // self.tp.world, p.shape[1]), dtype=torch.float32, device=p.device)
                dist.reduce_scatter_tensor(part, p, op=dist.ReduceOp.SUM, group=self.tp.group)
                if self.bias is not None:
                    part = part + self.bias.float()
                part = part.to(out_dtype)
                full = torch.empty((rows, p.shape[1]), dtype=out_dtype, device=p.device)
                dist.all_gather_into_tensor(full, part, group=self.tp.group)
                result, done_bias = full, True
            else:
                dist.all_reduce(p, op=dist.ReduceOp.SUM, group=self.tp.group)
                result, done_bias = p, False
            ev = torch.cuda.Event()
            ev.record(side)
        p.record_stream(side)
        return (result, ev, out_dtype, lead, done_bias)

    def finish(self, handle, keep: bool = False) -> Tensor:
        y, ev, out_dtype, lead, done_bias = handle
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        if done_bias == "fused_packed":  # y is an MXOperand in the reducer's buffers: (operand, leading shape)
            return (y, lead)
        if done_bias == "fused":  # y is the reducer's output buffer, already biased and rounded
            y = y if keep else y.clone()
            return y.reshape(*lead, y.shape[-1])
        if not done_bias and self.bias is not None:
            y = (y.float() + self.bias.float())
        return y.to(out_dtype).reshape(*lead, y.shape[-1])

    def forward(self, x_shard: Tensor) -> Tensor:
        return self.finish(self.start(x_shard))


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
        return ColumnParallelLinear(inner, tp, out_features=weight.shape[0], **kwargs)
    inner = cls(k_local, n_local, bias=False, device=device, dtype=dtype, config=dict(config))
    inner.load_state_dict({"weight": w.to(device=device, dtype=dtype)}, strict=False)
    return RowParallelLinear(inner, tp, None if bias is None else bias.to(device=device, dtype=dtype), **kwargs)




class TPGatedMLP(nn.Module):
    """y = down(silu(gate(x)) * up(x)) with gate/up column parallel and down row parallel: one reduction per layer.

    With `gate_up` the two column-parallel projections are one layer whose local weight stacks this rank's gate rows
    on top of its up rows (`[2 * ffn / G, K]`): x is quantized once and one GEMM produces both halves."""

    def __init__(self, gate: nn.Module | None, up: nn.Module | None, down: nn.Module, gate_up: nn.Module | None = None):
        super().__init__()
        assert (gate_up is None) != (gate is None and up is None), "pass gate and up, or gate_up"
        self.gate, self.up, self.down, self.gate_up = gate, up, down, gate_up

    def gate_and_up(self, x: Tensor) -> tuple[Tensor, Tensor]:
        if self.gate_up is None:
            return self.gate(x), self.up(x)
        gu = self.gate_up(x)
        half = gu.shape[-1] // 2
        return gu[..., :half], gu[..., half:]

    def start(self, x, tag: int = 0, emit_packed: tuple | None = None):
        """Both column-parallel GEMMs, SiLU * mul and the row-parallel GEMM on the current stream, the reduction on
        the down layer's side stream; `self.down.finish(handle)` gives the layer's output.  `tag` names the
        micro-batch (reductions in flight at the same time must not share buffers); `emit_packed` asks the down
        layer to deliver its result as the next layer's quantized activation (fused route only)."""
        gate, up = self.gate_and_up(x)
        if hasattr(self.down, "start_gated"):
            return self.down.start_gated(gate, up, tag, emit_packed)
        return self.down.start(torch.nn.functional.silu(gate) * up)

    def packed_input_format(self, like: Tensor) -> tuple | None:
        """(E, F) when this layer's first GEMM takes its input as MXFP tensor-core operands (then a preceding fused
        row-parallel layer can deliver exactly that), else None."""
        if self.gate_up is None:
            return None
        inner = getattr(self.gate_up, "inner", None)
        if inner is None or not hasattr(inner, "_uses_packed_path") or not inner._uses_packed_path(like):
            return None
        _, _, x_exp, x_frac = inner._input_format()
        return (x_exp, x_frac)

    def forward(self, x: Tensor) -> Tensor:
        gate, up = self.gate_and_up(x)
        if hasattr(self.down, "start_gated"):
            return self.down.finish(self.down.start_gated(gate, up))
        return self.down(torch.nn.functional.silu(gate) * up)


def build_tp_gated_mlp(cls, w_gate: Tensor, w_up: Tensor, w_down: Tensor, config: dict, tp: TPGroup, device=None,
                       dtype=None, reduce: str = "all_reduce") -> TPGatedMLP:
    """Shard the three weights of a gated MLP for this rank: gate and up rows are cut the same way and stacked into
    one column-parallel layer, down is row parallel.  MX blocks run along K, so stacking rows changes no block."""
    if w_gate.shape != w_up.shape:
        raise ValueError("gate and up must have the same shape")
    local = torch.cat([shard_linear_weight(w_gate, "column", tp), shard_linear_weight(w_up, "column", tp)], dim=0)
    fused_tp = TPGroup(0, 1, None)  # the stacked weight is already this rank's shard
    gate_up = build_tp_linear(cls, local, None, config, "column", fused_tp, device=device, dtype=dtype)
    del local
    down = build_tp_linear(cls, w_down, None, config, "row", tp, device=device, dtype=dtype, reduce=reduce)
    return TPGatedMLP(None, None, down, gate_up=gate_up)


def run_mlp_stack(layers: list[TPGatedMLP], x: Tensor, micro_batches: int = 1, comm_sms: int = 16) -> Tensor:
    """x -> layer_1 -> ... -> layer_L.  With micro_batches > 1 the rows are split and the cross-GPU reduction of one
    micro-batch (side stream) overlaps the GEMMs of the next one, within and across layers.  The GEMM kernels are
    persistent and fill every SM, so while the pipeline runs they are capped to leave `comm_sms` SMs to the
    reduction's kernels (otherwise those only start when a GEMM ends and nothing overlaps); 0 = no cap."""
    if not hasattr(layers[0].down, "start"):
        for layer in layers:
            x = layer(x)
        return x
    micro_batches = max(1, min(micro_batches, x.shape[0]))
    ctx = contextlib.nullcontext()
    if x.is_cuda and comm_sms > 0 and micro_batches > 1:
        from . import gemm

        sms = torch.cuda.get_device_properties(x.device).multi_processor_count
        ctx = gemm.options(max_ctas=max(1, sms - comm_sms))
    with ctx:
        parts = list(x.chunk(micro_batches, dim=0))
        handles = [None] * len(parts)
        prev_layer = None
        for li, layer in enumerate(layers):
            # a layer whose successor quantizes its input to MXFP anyway delivers that quantized operand directly
            # (fused route): half the all-gather bytes and no pack in the successor
            nxt = layers[li + 1] if li + 1 < len(layers) else None
            emit = nxt.packed_input_format(parts[0]) if nxt is not None and hasattr(nxt, "packed_input_format") else None
            for i in range(len(parts)):
                # a part waits only for its own reduction of the previous layer; the other parts' reductions stay
                # in flight underneath this part's GEMMs.  keep=True: the previous layer's result is consumed here,
                # before anything can overwrite the reducer's buffer it may live in.
                inp = parts[i] if prev_layer is None else prev_layer.down.finish(handles[i], keep=True)
                handles[i] = layer.start(inp, tag=i, emit_packed=emit)
            prev_layer = layer
        outs = [prev_layer.down.finish(h, keep=True) for h in handles]
        return torch.cat(outs, dim=0) if len(outs) > 1 else outs[0].clone()
