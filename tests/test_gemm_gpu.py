"""Tensor-core GEMMs (through the C ABI) against fp32 references built from the oracle-quantized operands."""

import pytest
import torch

import mase_b200 as mb
from mase_b200 import _lib, gemm, synthetic
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 1e-3  # max |err| / max |ref|, the bar for fp32 accumulation-order differences


def rel_err(y, ref):
    return float((y.float().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def quantized_operands(M, K, N, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, :: max(1, K // 7)] *= 30
    w = torch.randn(N, K, generator=g) * 0.02
    xq = O.mxfp_fake(x.to(dtype), 32, 4, 3) if K % 32 == 0 else O.mxint_fake(x.to(dtype), 8, 8)
    wq = O.mxfp_fake(w.to(dtype), 32, 4, 3) if K % 32 == 0 else O.mxint_fake(w.to(dtype), 8, 8)
    return xq, wq


@pytest.mark.parametrize("shape", [(128, 64, 256), (128, 256, 256), (256, 512, 512), (1, 128, 256), (77, 192, 384),
                                   (300, 4096, 1000), (128, 72, 256), (2048, 1024, 4096), (256, 512, 4096), (16, 1024, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dense_gemm_matches_fp32_reference(shape, dtype):
    M, K, N = shape
    xq, wq = quantized_operands(M, K, N, seed=M + K + N, dtype=dtype)
    ref = xq.float() @ wq.float().t()
    y = gemm.linear_forward(xq.to(DEV), wq.to(DEV), None, fp32_exact=True)
    gemm.check_status()
    assert y.dtype == dtype and y.shape == (M, N)
    tol = REL_TOL if dtype == torch.float32 else 4e-3  # bf16 output rounding: half an ulp = 2**-9 of the value
    assert rel_err(y, ref) <= tol
    if dtype == torch.bfloat16:  # at most one bf16 ulp from the rounded fp32 reference
        ulp = (y.float().cpu() - ref.bfloat16().float()).abs() / ref.abs().clamp_min(1e-6)
        big = ref.abs() > 1e-3 * ref.abs().max()
        assert float(ulp[big].max()) <= 2.0 ** -7


def test_dense_gemm_bias_and_leading_dims():
    g = torch.Generator().manual_seed(5)
    x = O.mxint_fake(torch.randn(2, 3, 40, 128, generator=g).bfloat16(), 32, 8)
    w = O.mxint_fake((torch.randn(96, 128, generator=g) * 0.05).bfloat16(), 32, 8)
    b = torch.randn(96, generator=g).bfloat16()
    ref = torch.nn.functional.linear(x.float(), w.float(), b.float())
    y = gemm.linear_forward(x.to(DEV), w.to(DEV), b.to(DEV))
    gemm.check_status()
    assert y.shape == (2, 3, 40, 96)
    assert rel_err(y, ref) <= 4e-3
    y32 = gemm.linear_forward(x.float().to(DEV), w.float().to(DEV), b.float().to(DEV), fp32_exact=True)
    assert rel_err(y32, ref) <= REL_TOL


@pytest.mark.parametrize("shape", [(128, 128, 256), (128, 512, 256), (256, 4096, 512), (1, 4096, 4096), (16, 4096, 4096),
                                   (200, 1024, 640), (2048, 4096, 4096), (256, 512, 4096), (128, 4096, 4096)])
def test_mxf8_gemm_matches_oracle(shape):
    """Block-scaled GEMM of MXFP8-quantized activations and weights vs fp32 GEMM of the oracle's fake-quant values."""
    M, K, N = shape
    x, w = synthetic.linear_operands(M, K, N, seed=2)
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, 4, 3, 1).float().t()
    wp = gemm.pack_mx_operand(w.to(DEV), 4, 3)
    y = gemm.mx_linear(x.to(DEV), wp, None, 4, 3)
    gemm.check_status()
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert rel_err(y, ref) <= 4e-3
    xp = gemm.pack_mx_operand(x.to(DEV), 4, 3)
    y32 = gemm.mx_gemm(xp, wp, None, torch.float32)
    gemm.check_status()
    assert rel_err(y32, ref) <= REL_TOL


@pytest.mark.parametrize("shape", [(256, 128, 256), (256, 4096, 256), (512, 1024, 512), (1024, 512, 768), (300, 256, 260),
                                   (129, 512, 129), (2048, 4096, 4096), (1000, 2048, 1304), (4096, 8192, 512)])
def test_mxf8_gemm_cta_pairs_match_single_cta_and_oracle(shape):
    """CTA pairs (cta_group::2, 256 x 256 tiles) give the bits of the single-CTA kernel (same accumulation order),
    with bias, ragged edges and both output types; both match the oracle."""
    M, K, N = shape
    x, w = synthetic.linear_operands(M, K, N, seed=4)
    g = torch.Generator().manual_seed(4)
    b = torch.randn(N, generator=g).to(DEV)
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, 4, 3, 1).float().t() + b.cpu()
    xp = gemm.pack_mx_operand(x.to(DEV), 4, 3)
    wp = gemm.pack_mx_operand(w.to(DEV), 4, 3)
    with gemm.options(tiles=_lib.TILES_SINGLE):
        single = [gemm.mx_gemm(xp, wp, b, dt) for dt in (torch.float32, torch.bfloat16)]
    with gemm.options(tiles=_lib.TILES_PAIRS):
        pair = [gemm.mx_gemm(xp, wp, b, dt) for dt in (torch.float32, torch.bfloat16)]
    gemm.check_status()
    assert torch.equal(single[0], pair[0]) and torch.equal(single[1], pair[1])
    assert rel_err(pair[0], ref) <= REL_TOL
    assert rel_err(pair[1], ref) <= 4e-3


@pytest.mark.parametrize("shape", [(256, 512, 256), (1024, 512, 768), (300, 264, 260), (2048, 4096, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dense_gemm_cta_pairs_match_single_cta(shape, dtype):
    """The dense kinds on CTA pairs give the bits of the single-CTA kernel, with bias and ragged edges."""
    M, K, N = shape
    x, w = quantized_operands(M, K, N, 6, dtype)
    g = torch.Generator().manual_seed(6)
    b = torch.randn(N, generator=g).to(dtype).to(DEV)
    with gemm.options(tiles=_lib.TILES_SINGLE):
        single = gemm.linear_forward(x.to(DEV), w.to(DEV), b, fp32_exact=True)
    with gemm.options(tiles=_lib.TILES_PAIRS):
        pair = gemm.linear_forward(x.to(DEV), w.to(DEV), b, fp32_exact=True)
    gemm.check_status()
    assert torch.equal(single, pair)
    ref = x.float() @ w.float().t() + b.float().cpu()
    assert rel_err(pair, ref) <= (4e-3 if dtype == torch.bfloat16 else REL_TOL)


def test_mxf8_pack_round_trip():
    """Packed codes * scales reproduce the oracle's fake-quant values (up to the documented re-encoding of blocks
    that hold the reference's top E4M3 code)."""
    x, _ = synthetic.linear_operands(300, 1024, 32, seed=2)
    op = gemm.pack_mx_operand(x.to(DEV), 4, 3)
    codes = op.codes.cpu().view(torch.float8_e4m3fn).float()
    sc = op.scales.cpu()
    rows, k = 300, 1024
    r = torch.arange(rows).view(-1, 1)
    kb = torch.arange(k // 32).view(1, -1)
    idx = ((r // 128) * ((k + 127) // 128) + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (kb % 4)
    s = sc[idx.flatten()].view(rows, k // 32).float() - 127
    y = (codes.view(rows, k // 32, 32) * torch.exp2(s).unsqueeze(-1)).view(rows, k)
    ref = O.mxfp_fake(x, 32, 4, 3).float()
    assert not torch.isnan(codes).any()
    blockmax = ref.view(rows, -1, 32).abs().amax(-1, keepdim=True).clamp_min(1e-30)
    err = ((y - ref).view(rows, -1, 32).abs() / blockmax).max()
    assert float(err) <= 2.0 ** -15
    assert float((y != ref).float().mean()) < 1e-3


def test_mxfp4_weight_mxfp8_activation():
    M, K, N = 256, 1024, 512
    x, w = synthetic.linear_operands(M, K, N, seed=4)
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, 2, 1, 1).float().t()
    wp = gemm.pack_mx_operand(w.to(DEV), 2, 1)
    y = gemm.mx_gemm(gemm.pack_mx_operand(x.to(DEV), 4, 3), wp, None, torch.float32)
    gemm.check_status()
    assert rel_err(y, ref) <= REL_TOL


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (16, 4096, 4096), (128, 8192, 2048), (100, 4128, 1000), (7, 8192, 512)])
def test_split_k_over_a_cluster_matches_unsplit(shape):
    """Small problems split K over the two CTAs of a cluster; the sum of the two halves may differ from the unsplit
    accumulation by fp32 rounding only, repeats exactly, and matches the oracle."""
    M, K, N = shape
    x, w = synthetic.linear_operands(M, K, N, seed=8)
    g = torch.Generator().manual_seed(8)
    b = torch.randn(N, generator=g).bfloat16().to(DEV)
    xp, wp = gemm.pack_mx_operand(x.to(DEV), 4, 3), gemm.pack_mx_operand(w.to(DEV), 4, 3)
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, 4, 3, 1).float().t() + b.float().cpu()
    xq, wq = O.mxfp_fake(x, 32, 4, 3).to(DEV), O.mxfp_fake(w, 32, 4, 3, 1).to(DEV)
    with gemm.options(no_split_k=1):
        plain = gemm.mx_gemm(xp, wp, b, torch.float32)
        dense_plain = gemm.linear_forward(xq, wq, b)
    split1 = gemm.mx_gemm(xp, wp, b, torch.float32)
    split2 = gemm.mx_gemm(xp, wp, b, torch.float32)
    split_bf16 = gemm.mx_gemm(xp, wp, b, torch.bfloat16)
    dense_split = gemm.linear_forward(xq, wq, b)
    gemm.check_status()
    assert torch.equal(split1, split2)
    assert rel_err(split1, ref) <= REL_TOL and rel_err(plain, ref) <= REL_TOL
    assert float((split1 - plain).abs().max() / plain.abs().max()) <= 1e-5
    assert rel_err(split_bf16, ref) <= 4e-3
    assert rel_err(dense_split, ref) <= 4e-3 and rel_err(dense_plain, ref) <= 4e-3


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (7, 1024, 1000), (16, 4096, 4096), (17, 160, 96), (32, 8192, 512),
                                   (33, 4128, 1304), (64, 2048, 11008), (100, 512, 768), (128, 4096, 4096)])
def test_transposed_small_m_kernel_vs_oracle_and_regular_tiles(shape):
    """Problems of at most 128 rows run the transposed kernel (weight as the 128-row MMA operand, K split over a
    cluster): against the oracle, against the regular tiles, repeatable, with bias, ragged N and K, both outputs, and
    for the dense kinds on the fake-quantized tensors."""
    M, K, N = shape
    x, w = synthetic.linear_operands(M, K, N, seed=9)
    g = torch.Generator().manual_seed(9)
    b = torch.randn(N, generator=g).bfloat16().to(DEV)
    xq, wq = O.mxfp_fake(x, 32, 4, 3), O.mxfp_fake(w, 32, 4, 3, 1)
    ref = xq.float() @ wq.float().t() + b.float().cpu()
    xp, wp = gemm.pack_mx_operand(x.to(DEV), 4, 3), gemm.pack_mx_operand(w.to(DEV), 4, 3)
    y1 = gemm.mx_gemm(xp, wp, b, torch.float32)
    y2 = gemm.mx_gemm(xp, wp, b, torch.float32)
    y16 = gemm.mx_gemm(xp, wp, b, torch.bfloat16)
    with gemm.options(no_split_k=1):
        y_unsplit = gemm.mx_gemm(xp, wp, b, torch.float32)
    with gemm.options(no_transposed=1):
        y_tiles = gemm.mx_gemm(xp, wp, b, torch.float32)
    d16 = gemm.linear_forward(xq.to(DEV), wq.to(DEV), b)
    d32 = gemm.linear_forward(xq.float().to(DEV), wq.float().to(DEV), b.float(), fp32_exact=True)
    gemm.check_status()
    assert torch.equal(y1, y2)
    assert rel_err(y1, ref) <= REL_TOL and rel_err(y_unsplit, ref) <= REL_TOL and rel_err(y_tiles, ref) <= REL_TOL
    assert float((y1 - y_tiles).abs().max() / y_tiles.abs().max()) <= 1e-5
    assert rel_err(y16, ref) <= 4e-3
    assert rel_err(d16, ref) <= 4e-3 and rel_err(d32, ref) <= REL_TOL


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (16, 1024, 1000), (100, 3968, 768), (128, 512, 512), (300, 1024, 260),
                                   (512, 2048, 1024), (2048, 4096, 4096), (1000, 11008, 1304)])
def test_nibble_packed_mxfp4_weight_matches_e4m3_bytes(shape):
    """MXFP4 weights stored two codes per byte (the copy engine expands them on the way into shared memory) give the
    bits of the same weights stored as E4M3 bytes, on every tile scheme, and match the oracle."""
    M, K, N = shape
    x, w = synthetic.linear_operands(M, K, N, seed=10)
    g = torch.Generator().manual_seed(10)
    b = torch.randn(N, generator=g).bfloat16().to(DEV)
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, 2, 1, 1).float().t() + b.float().cpu()
    xp = gemm.pack_mx_operand(x.to(DEV), 4, 3)
    w8 = gemm.pack_mx_operand(w.to(DEV), 2, 1)
    w4 = gemm.pack_mx_operand(w.to(DEV), 2, 1, fp4=True)
    assert w4.codes.shape == (N, K // 2) and w4.fp4
    # the nibbles are the reference's own codes
    sc, co = O.mxfp_extract(w, 32, 2, 1)
    co = co.view(N, K)
    assert torch.equal(w4.codes.cpu(), co[:, 0::2] | (co[:, 1::2] << 4))
    schemes = [{}] if M <= 128 else [{"tiles": _lib.TILES_SINGLE}, {"tiles": _lib.TILES_PAIRS}]
    if M <= 128:
        schemes.append({"no_transposed": 1})
    for fields in schemes:
        with gemm.options(**fields):
            y8 = gemm.mx_gemm(xp, w8, b, torch.float32)
            y4 = gemm.mx_gemm(xp, w4, b, torch.float32)
            y4_16 = gemm.mx_linear(x.to(DEV), w4, b, 4, 3)
        gemm.check_status()
        assert torch.equal(y8, y4), fields
        assert rel_err(y4, ref) <= REL_TOL and rel_err(y4_16, ref) <= 4e-3, fields


@pytest.mark.parametrize("shape", [(64, 512, 256), (300, 1000, 520), (2048, 1024, 1024)])
def test_unquantized_fp32_operands_keep_fp32_level_products(shape):
    """fp32 operands that are not MX values (bypassed layers, weights that were never quantized): the tf32 tensor cores
    keep 11 significant bits, so the operands are split into a tf32-exact part and a remainder and multiplied as three
    products in one GEMM.  Against a float64 reference the result is within 2e-5 of max (the remainders are themselves truncated to
    tf32), where plain tf32 is more than ten times further off."""
    M, K, N = shape
    g = torch.Generator().manual_seed(14)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) * 0.05
    b = torch.randn(N, generator=g)
    ref = (x.double() @ w.double().t() + b.double()).float()
    y = gemm.linear_forward(x.to(DEV), w.to(DEV), b.to(DEV))
    plain = gemm.linear_forward(x.to(DEV), w.to(DEV), b.to(DEV), fp32_exact=True)  # what tf32 alone would give
    gemm.check_status()
    assert rel_err(y, ref) <= 2e-5
    assert rel_err(plain, ref) > 10 * rel_err(y, ref)
    layer = mb.LinearMXFP(K, N, bias=True, device=DEV, dtype=torch.float32,
                          config={"bypass": True, "weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3})
    layer.load_state_dict({"weight": w.to(DEV), "bias": b.to(DEV)}, strict=False)
    assert rel_err(layer(x.to(DEV)), ref) <= 2e-5


@pytest.mark.parametrize("M", [1, 16, 128, 300])
def test_static_weight_flag_changes_when_the_weight_is_fetched_not_the_result(M):
    """MXQ_GEMM_STATIC_B lets the small-M kernel fetch the weight ahead of the stream dependency; results are the bits
    of the unflagged call, also when calls are issued back to back on one stream (each launch may start under the
    tail of the one before it) and for problems that do not use the small-M kernel at all."""
    x, w = synthetic.linear_operands(M, 1024, 512, seed=M)
    xp, wp = gemm.pack_mx_operand(x.to(DEV), 4, 3), gemm.pack_mx_operand(w.to(DEV), 4, 3)
    torch.cuda.synchronize()  # the weight is complete before anything below is launched: the flag's precondition
    plain = gemm.mx_gemm(xp, wp, None, torch.float32)
    flagged = [gemm.mx_gemm(xp, wp, None, torch.float32, static_b=True) for _ in range(6)]
    with gemm.options(max_ctas=64):  # the flag combines with other per-call options
        flagged.append(gemm.mx_gemm(xp, wp, None, torch.float32, static_b=True))
    gemm.check_status()
    assert all(torch.equal(f, plain) for f in flagged)
    # a weight packed immediately before an unflagged call: nothing is read before the pack has finished
    for _ in range(3):
        wp2 = gemm.pack_mx_operand(w.to(DEV), 4, 3)
        assert torch.equal(gemm.mx_gemm(xp, wp2, None, torch.float32), plain)
    gemm.check_status()
