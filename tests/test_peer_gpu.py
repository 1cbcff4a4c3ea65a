"""The data path of the fused row-parallel reduction on one GPU: two "ranks" are two calls with their own K shards and
their own buffers in the same device memory (what differs on real peers is only whose memory the addresses reach).
The barrier between the steps is the stream order here; its kernel is exercised with one rank."""

import ctypes

import pytest
import torch

from mase_b200 import _lib, gemm, synthetic
from mase_b200.quantizers import _DT
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ptr_array(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("world,M,K,N,fp4", [(2, 1024, 2048, 512, False), (2, 512, 1024, 1304, True), (4, 2048, 4096, 768, True)])
def test_scatter_gemm_then_reduce_gather_equals_unsharded(world, M, K, N, fp4):
    lib = _lib.lib()
    x, w = synthetic.linear_operands(M, K, N, seed=13)
    g = torch.Generator().manual_seed(13)
    bias = torch.randn(N, generator=g).bfloat16().to(DEV)
    we, wf = (2, 1) if fp4 else (4, 3)
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, we, wf, 1).float().t() + bias.float().cpu()
    rows = M // world
    slots = [torch.full((world, rows, N), float("nan"), dtype=torch.float32, device=DEV) for _ in range(world)]
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    st = gemm._status(torch.device(DEV))
    stream = torch.cuda.current_stream().cuda_stream
    ks = K // world
    for rank in range(world):  # every rank's GEMM over its K shard, tiles stored into the owners' slots
        xs, ws = x[:, rank * ks:(rank + 1) * ks].contiguous(), w[:, rank * ks:(rank + 1) * ks].contiguous()
        a = gemm.pack_mx_operand(xs.to(DEV), 4, 3)
        b = gemm.pack_mx_operand(ws.to(DEV), we, wf, fp4=fp4)
        rc = lib.mxq_gemm_mxf8_scatter(a.codes.data_ptr(), a.scales.data_ptr(), b.codes.data_ptr(), b.scales.data_ptr(),
                                       b.format, ptr_array(slots), world, rank, M, N, ks, st.data_ptr(), None, stream)
        assert rc == 0
    assert lib.mxq_peer_barrier(ptr_array([flags]), 1, 0, 1, st.data_ptr(), 0, stream) == 0
    for rank in range(world):  # every rank reduces its slice and writes it into all outputs
        rc = lib.mxq_reduce_gather(slots[rank].data_ptr(), world, rank, rows, N, bias.data_ptr(), _DT[bias.dtype],
                                   ptr_array(outs), _DT[torch.bfloat16], 0 if rank else 16, stream)
        assert rc == 0
    torch.cuda.synchronize()
    gemm.check_status()
    assert int(flags[0]) == 1
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    assert not torch.isnan(outs[0].float()).any()
    err = float((outs[0].float().cpu() - ref).abs().max() / ref.abs().max())
    assert err <= 4e-3, err
    # the partial sums themselves: slot s of rank r = rows of rank r from the GEMM of shard s (fp32, 1e-3 bar)
    xq, wq = O.mxfp_fake(x, 32, 4, 3).float(), O.mxfp_fake(w, 32, we, wf, 1).float()
    for r in range(world):
        for s in range(world):
            part = xq[r * rows:(r + 1) * rows, s * ks:(s + 1) * ks] @ wq[:, s * ks:(s + 1) * ks].t()
            e = float((slots[r][s].cpu() - part).abs().max() / part.abs().max())
            assert e <= 1e-3, (r, s, e)


def test_reduce_gather_pack_equals_pack_of_the_reduced_output():
    """The reduction that delivers the next layer's activation operand: its E4M3 bytes and scales are those of packing
    the bf16 output of the plain reduction, on every emulated rank's buffers."""
    lib = _lib.lib()
    world, rows, N = 4, 256, 1024
    M = world * rows
    g = torch.Generator().manual_seed(15)
    slots = [(torch.randn(world, rows, N, generator=g) * torch.exp2(torch.randint(-6, 6, (world, rows, 1), generator=g).float())).to(DEV)
             for _ in range(world)]
    bias = torch.randn(N, generator=g).to(DEV)
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    codes = [torch.zeros(M, N, dtype=torch.uint8, device=DEV) for _ in range(world)]
    nsc = int(lib.mxq_mma_scale_bytes(M, N))
    scales = [torch.zeros(nsc, dtype=torch.uint8, device=DEV) for _ in range(world)]
    stream = torch.cuda.current_stream().cuda_stream
    from mase_b200.quantizers import _floor_tab_ptr

    for rank in range(world):
        assert lib.mxq_reduce_gather(slots[rank].data_ptr(), world, rank, rows, N, bias.data_ptr(), _DT[bias.dtype],
                                     ptr_array(outs), _DT[torch.bfloat16], 0, stream) == 0
        assert lib.mxq_reduce_gather_pack(slots[rank].data_ptr(), world, rank, rows, N, bias.data_ptr(), _DT[bias.dtype],
                                          ptr_array(codes), ptr_array(scales), None, 4, 3, _floor_tab_ptr(), 0, stream) == 0
    torch.cuda.synchronize()
    ref = gemm.pack_mx_operand(outs[0], 4, 3)
    for r in range(world):
        assert torch.equal(outs[r], outs[0])
        assert torch.equal(codes[r], ref.codes), f"codes on rank {r}"
        assert torch.equal(scales[r], ref.scales), f"scales on rank {r}"
    # and the bf16 values themselves: fp32 sum in rank order + bias, one rounding
    want = (torch.stack([sum(slots[r][s] for s in range(world)) for r in range(world)])
            .reshape(M, N) + bias).bfloat16()
    assert torch.equal(outs[0], want)


def test_peer_barrier_wait_runs_out_without_a_peer():
    """A rank that never arrives: the wait is bounded, the status word reports it, the stream stays usable."""
    lib = _lib.lib()
    mine = torch.zeros(8, dtype=torch.int32, device=DEV)
    absent = torch.zeros(8, dtype=torch.int32, device=DEV)  # stands in for the flags of a rank that does nothing
    st = gemm._status(torch.device(DEV))
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.mxq_peer_barrier(ptr_array([mine, absent]), 2, 0, 1, st.data_ptr(), 2_000_000, stream) == 0
    with pytest.raises(_lib.MxqError, match="did not arrive"):
        gemm.check_status()
    assert int(absent[0]) == 1 and int(mine[1]) == 0  # this rank published its epoch, the other one never did
    y = torch.ones(4, device=DEV) * 2
    assert float(y.sum()) == 8.0


def test_scatter_arguments_are_checked():
    lib = _lib.lib()
    t = torch.zeros(64, dtype=torch.uint8, device=DEV)
    ptrs = ptr_array([t, t])
    common = (t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 0, ptrs)
    assert lib.mxq_gemm_mxf8_scatter(*common, 2, 0, 300, 256, 128, None, None, None) == -7   # rows per rank not tile-sized
    assert lib.mxq_gemm_mxf8_scatter(*common, 9, 0, 512, 256, 128, None, None, None) == -2   # more ranks than a node has
    assert lib.mxq_gemm_mxf8_scatter(*common[:5], None, 2, 0, 512, 256, 128, None, None, None) == -5
    assert lib.mxq_reduce_gather(t.data_ptr(), 2, 0, 4, 12, None, 0, ptrs, 1, 0, None) == -2    # columns not a multiple of 8
