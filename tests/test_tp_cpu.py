"""Tensor-parallel plumbing on two CPU ranks (gloo): sharded layers reproduce the unsharded result.

The local layer is injected: here it is the CPU oracle (the CUDA layers need a GPU), so these tests cover the sharding
arithmetic, the float32 partial-sum reduction and the chunked asynchronous all-reduce."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mase_b200 import tp as tpmod
from oracle import mx_oracle as O

CFG = {"weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1,
       "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}


class OracleLinearMXFP(torch.nn.Module):
    """CPU stand-in with the LinearMXFP contract: weight quantized at load, activations per forward, fp32 GEMM."""

    output_dtype = None

    def __init__(self, weight, cfg):
        super().__init__()
        self.cfg = cfg
        self.w_q = O.mxfp_fake(weight, cfg["weight_block_size"], cfg["weight_exponent_width"], cfg["weight_frac_width"], 1)

    def forward(self, x):
        y = O.linear_mxfp(x, self.w_q, None, self.cfg)
        return y.to(self.output_dtype or x.dtype)


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp = tpmod.TPGroup.from_env()
        g = torch.Generator().manual_seed(4)
        h, ffn, m = 128, 256, 24
        x = torch.randn(m, h, generator=g).bfloat16()
        wg = (torch.randn(ffn, h, generator=g) * 0.05).bfloat16()
        wu = (torch.randn(ffn, h, generator=g) * 0.05).bfloat16()
        wd = (torch.randn(h, ffn, generator=g) * 0.05).bfloat16()
        bias = torch.randn(h, generator=g).bfloat16()
        # unsharded reference on every rank
        ref_mlp = tpmod.TPGatedMLP(OracleLinearMXFP(wg, CFG), OracleLinearMXFP(wu, CFG),
                                   tpmod.RowParallelLinear(OracleLinearMXFP(wd, CFG), tpmod.TPGroup(0, 1), bias))
        ref = ref_mlp(x)
        gate = tpmod.ColumnParallelLinear(OracleLinearMXFP(tpmod.shard_linear_weight(wg, "column", tp), CFG), tp)
        up = tpmod.ColumnParallelLinear(OracleLinearMXFP(tpmod.shard_linear_weight(wu, "column", tp), CFG), tp)
        down = tpmod.RowParallelLinear(OracleLinearMXFP(tpmod.shard_linear_weight(wd, "row", tp), CFG), tp, bias)
        mlp = tpmod.TPGatedMLP(gate, up, down)
        y = mlp(x)
        err = float((y.float() - ref.float()).abs().max() / ref.float().abs().max())
        # micro-batched stack runner gives the same rows
        y2 = tpmod.run_mlp_stack([mlp], x, micro_batches=2)
        err = max(err, float((y2.float() - ref.float()).abs().max() / ref.float().abs().max()))
        # column-parallel output gathered back equals the unsharded layer bit for bit
        full = tpmod.ColumnParallelLinear(OracleLinearMXFP(tpmod.shard_linear_weight(wg, "column", tp), CFG), tp,
                                          gather_output=True)(x)
        same = torch.equal(full, OracleLinearMXFP(wg, CFG)(x))
        # quantizer row shards concatenate to the unsharded result
        xs = tpmod.shard_rows_for_quantizer(x, 32, tp)
        parts = [torch.empty_like(xs) for _ in range(world)]
        dist.all_gather(parts, O.mxfp_fake(xs, 32, 4, 3))
        qsame = torch.equal(torch.cat(parts), O.mxfp_fake(x, 32, 4, 3))
        if rank == 0:
            results.put((err, same, qsame))
    finally:
        dist.destroy_process_group()


def test_two_rank_gated_mlp_matches_unsharded():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    err, same, qsame = results.get(timeout=10)
    assert err <= 4e-3, err       # bf16 output rounding; the fp32 partial sums themselves agree to ~1e-7
    assert same and qsame


def test_shard_bounds_and_errors():
    assert tpmod.shard_bounds(10, 3, 0) == (0, 4) and tpmod.shard_bounds(10, 3, 2) == (7, 10)
    assert tpmod.shard_bounds(11008, 8, 3, 32) == (1376 * 3, 1376 * 4)      # 11008 / 8 = 43 blocks of 32
    assert tpmod.shard_bounds(28672, 8, 7, 32) == (3584 * 7, 28672)
    covered = [tpmod.shard_bounds(4096 + 32 * 3, 8, r, 32) for r in range(8)]
    assert covered[0][0] == 0 and covered[-1][1] == 4096 + 96
    assert all(covered[i][1] == covered[i + 1][0] for i in range(7))
    w = torch.zeros(64, 96)
    with pytest.raises(ValueError):
        tpmod.shard_linear_weight(w, "row", tpmod.TPGroup(0, 2), 32)         # 96 / 2 = 48 is not a multiple of 32
    assert tpmod.shard_linear_weight(w, "column", tpmod.TPGroup(1, 2)).shape == (32, 96)
    x = torch.zeros(6, 48)                                                    # blocks of 32 straddle rows: split on 2-row units
    assert tpmod.shard_rows_for_quantizer(x, 32, tpmod.TPGroup(1, 3)).shape == (2, 48)
    with pytest.raises(ValueError):
        tpmod.shard_rows_for_quantizer(torch.zeros(5, 48), 32, tpmod.TPGroup(0, 2))
