"""Parity at the benchmark's own sizes: the quantizer sweep up to bf16 [65536, 8192], the MXFP8 Linear at M = 8192 and
the per-GPU shards of the tensor-parallel stack.  The oracle runs on a sample of rows (every 257th), which keeps the CPU
side to seconds while the GPU side runs the full-size launch that the benchmark times."""

import pytest
import torch

import mase_b200 as mb
from mase_b200 import gemm, synthetic
from conftest import assert_bits_equal
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def sampled(rows: int) -> torch.Tensor:
    idx = torch.arange(0, rows, 257)
    return torch.cat([idx, torch.tensor([rows - 1])]) if rows > 1 else idx


@pytest.mark.parametrize("shape", [(4096, 4096), (8192, 8192), (65536, 8192)])
def test_quantizer_sweep_shapes_sampled_rows_vs_oracle(shape):
    """MXFP8 / MXINT8 / block-fp (width 8 tiles of 32, width 7 tiles of 16) fake-quant and the MXFP8 / MXINT8 codes +
    scales of Student-t(3) * 0.02 bf16 tensors: sampled rows bit-exact against the oracle."""
    rows, cols = shape
    x = synthetic.device_student_t3(rows, cols, seed=1, device=DEV)
    idx = sampled(rows)
    xs = x[idx.to(DEV)].cpu()
    take = lambda t: t[idx.to(DEV)].cpu()  # noqa: E731
    y = mb.mxfp_quantizer(x, 32, 4, 3)
    assert_bits_equal(take(y), O.mxfp_fake(xs, 32, 4, 3), "mxfp8 fake")
    del y
    y = mb.mxint_quantizer(x, 32, 8)
    assert_bits_equal(take(y), O.mxint_fake(xs, 32, 8), "mxint8 fake")
    del y
    y = mb.block_fp_quantizer(x, 8, 8, 127, [1, 32], True)
    assert_bits_equal(take(y), O.bfp_fake_rows(xs, 8, 8, 127, 32), "bfp w8 b32")
    del y
    y = mb.block_fp_quantizer(x, 7, 8, 127, [1, 16], True)
    assert_bits_equal(take(y), O.bfp_fake_rows(xs, 7, 8, 127, 16), "bfp w7 b16")
    del y
    bpr = cols // 32  # blocks per row
    sc, co = mb.extract_mxfp_components(x.flatten(), mb.MXFPMeta(32, 8, 4, 3, True, "rn"))
    rs, rc = O.mxfp_extract(xs, 32, 4, 3)
    assert torch.equal(take(co.view(rows, bpr, 32)).reshape(-1, 32), rc), "mxfp8 codes"
    assert torch.equal(take(sc.view(rows, bpr)).reshape(-1, 1), rs), "mxfp8 scales"
    del sc, co
    sc, mant = mb.mxint_codes(x.flatten(), 32, 8)
    rs, rm = O.mxint_extract(xs, 32, 8)
    assert torch.equal(take(mant.view(rows, bpr, 32)).reshape(-1, 32).float(), rm.float().reshape(-1, 32)), "mxint8 mantissas"
    assert torch.equal(take(sc.view(rows, bpr)).reshape(-1).float(), rs.float().reshape(-1)), "mxint8 scales"


def assert_gemm_rows(y, ref, what):
    """fp32-accumulated reference rows: 1e-3 of max for fp32 results; bf16 results additionally within one bf16 ulp of
    the rounded reference wherever the value is not a near-cancellation."""
    y = y.float().cpu()
    err = float((y - ref).abs().max() / ref.abs().max())
    if what.endswith("fp32"):
        assert err <= 1e-3, f"{what}: {err}"
        return
    assert err <= 4e-3, f"{what}: {err}"  # half a bf16 ulp of the largest value
    ulp = (y - ref.bfloat16().float()).abs() / ref.abs().clamp_min(1e-6)
    big = ref.abs() > 1e-3 * ref.abs().max()
    assert float(ulp[big].max()) <= 2.0 ** -7, f"{what}: more than one bf16 ulp from the fp32 reference"


def test_linear_mxfp8_m8192_sampled_rows_vs_oracle():
    """LinearMXFP 4096 -> 4096 at M = 8192: sampled rows against the fp32 GEMM of the oracle-quantized operands, bf16
    and fp32 output."""
    M, K, N = 8192, 4096, 4096
    x, w = synthetic.linear_operands(M, K, N, seed=2)
    cfg = {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    layer = mb.LinearMXFP(K, N, bias=False, device=DEV, dtype=torch.bfloat16, config=cfg)
    layer.load_state_dict({"weight": w.to(DEV)}, strict=False)
    wq = O.mxfp_fake(w, 32, 4, 3, 1)
    assert_bits_equal(layer.weight.data, wq, "weight")
    xd = x.to(DEV)
    y = layer(xd)
    layer.output_dtype = torch.float32
    y32 = layer(xd)
    gemm.check_status()
    idx = sampled(M)
    ref = O.linear_mxfp(x[idx], wq, None, cfg)
    assert_gemm_rows(y[idx.to(DEV)], ref, "M=8192 bf16")
    assert_gemm_rows(y32[idx.to(DEV)], ref, "M=8192 fp32")


@pytest.mark.parametrize("shard", ["column", "row"])
def test_tp_stack_shard_shapes_sampled_rows_vs_oracle(shard):
    """One projection of the 70B-shape stack as an 8-way shard sees it: column 8192 -> 3584 and row 3584 -> 8192,
    MXFP4 (E2M1) weights x MXFP8 (E4M3) activations, M = 8192 tokens."""
    M = 8192
    K, N = (8192, 3584) if shard == "column" else (3584, 8192)
    g = torch.Generator().manual_seed(4)
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    x = torch.randn(M, K, generator=g).bfloat16()
    cfg = dict(synthetic.MXFP4W_MXFP8A_LINEAR)
    layer = mb.LinearMXFP(K, N, bias=False, device=DEV, dtype=torch.bfloat16, config=cfg)
    layer.load_state_dict({"weight": w.to(DEV)}, strict=False)
    wq = O.mxfp_fake(w, 32, 2, 1, 1)
    assert_bits_equal(layer.weight.data, wq, "E2M1 weight")
    assert layer._packed_weight() is not None
    if shard == "row":
        layer.output_dtype = torch.float32  # partial sums stay fp32 until the cross-GPU reduction
    y = layer(x.to(DEV))
    gemm.check_status()
    idx = sampled(M)
    ref = O.linear_mxfp(x[idx], wq, None, cfg)
    assert_gemm_rows(y[idx.to(DEV)], ref, f"{shard} shard " + ("fp32" if shard == "row" else "bf16"))


@pytest.mark.parametrize("shape", [(256, 4096, 512), (1024, 512, 768), (2048, 4096, 4096)])
def test_block_scaled_bf16_output_within_one_ulp_of_fp32_oracle(shape):
    M, K, N = shape
    x, w = synthetic.linear_operands(M, K, N, seed=5)
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, 4, 3, 1).float().t()
    y = gemm.mx_linear(x.to(DEV), gemm.pack_mx_operand(w.to(DEV), 4, 3), None, 4, 3)
    gemm.check_status()
    assert_gemm_rows(y, ref, f"{shape} bf16")


def test_two_threads_two_streams_different_options():
    """Options travel with each call: two host threads issue GEMMs on their own streams with different tile schemes and
    CTA caps at the same time, and each gets the bits of a plain single-threaded call."""
    import threading

    from mase_b200 import _lib

    x, w = synthetic.linear_operands(1024, 2048, 2048, seed=6)
    xp, wp = gemm.pack_mx_operand(x.to(DEV), 4, 3), gemm.pack_mx_operand(w.to(DEV), 4, 3)
    base = gemm.mx_gemm(xp, wp, None, torch.float32)
    torch.cuda.synchronize()
    results, errors = {}, []

    def worker(name, **fields):
        try:
            stream = torch.cuda.Stream(device=DEV)
            with torch.cuda.stream(stream), gemm.options(**fields):
                outs = [gemm.mx_gemm(xp, wp, None, torch.float32) for _ in range(20)]
            stream.synchronize()
            results[name] = outs
        except Exception as exc:  # surfaced below: an exception in a thread would otherwise be lost
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=("single",), kwargs={"tiles": _lib.TILES_SINGLE, "max_ctas": 60}),
               threading.Thread(target=worker, args=("pairs",), kwargs={"tiles": _lib.TILES_PAIRS, "max_ctas": 64})]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors, errors
    gemm.check_status()
    for outs in results.values():
        assert all(torch.equal(o, base) for o in outs)


def test_bounded_wait_runs_out_and_the_next_gemm_is_correct():
    """The error path of the device-side waits, without any fault: a test option makes the loader leave out the last
    operand tile of a one-tile problem and shortens the wait limit, so the MMA issuer's wait runs out, the kernel
    writes a non-zero status and returns, and the next GEMM on the same stream is correct."""
    from mase_b200 import _lib

    x, w = synthetic.linear_operands(128, 512, 64, seed=7)
    xp, wp = gemm.pack_mx_operand(x.to(DEV), 4, 3), gemm.pack_mx_operand(w.to(DEV), 4, 3)
    good = gemm.mx_gemm(xp, wp, None, torch.float32)
    gemm.check_status()
    with gemm.options(test_hook=_lib.TEST_DROP_LAST_LOAD, wait_limit_ns=2_000_000):
        gemm.mx_gemm(xp, wp, None, torch.float32)
    # the MMA issuer waits for the tile that never comes and the epilogue for the accumulator behind it: whichever
    # limit runs out first is the one reported
    with pytest.raises(_lib.MxqError, match="(wait for an operand tile|wait for a finished accumulator) ran out"):
        gemm.check_status()
    again = gemm.mx_gemm(xp, wp, None, torch.float32)
    gemm.check_status()
    assert torch.equal(again, good)
