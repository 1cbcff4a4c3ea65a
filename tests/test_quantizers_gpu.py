"""CUDA quantizers (through the C ABI) against the golden reference vectors and the CPU oracle."""

import pytest
import torch

import mase_b200 as mb
from mase_b200 import synthetic
from conftest import assert_bits_equal
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cases(golden, kind):
    return [c for c in golden.cases if c["kind"] == kind]


# ---- golden vectors produced by the reference itself -------------------------------------------------
def test_mxint_golden(golden):
    for c in _cases(golden, "mxint"):
        x = golden.tensor(c["input"] + "/x").to(DEV)
        meta = mb.MXIntMeta(block_size=c["block"], scale_bits=8, element_bits=c["bits"])
        sc, m = mb.extract_mxint_components(x.flatten(), meta)
        assert_bits_equal(sc, golden.tensor(c["tag"] + "/scale"), c["tag"] + " scale")
        assert_bits_equal(m, golden.tensor(c["tag"] + "/mant"), c["tag"] + " mant")
        assert_bits_equal(mb.mxint_quantizer(x, c["block"], c["bits"]), golden.tensor(c["tag"] + "/fake"), c["tag"] + " fake")
        assert_bits_equal(mb.compose_mxint_tensor(sc, m, meta).reshape(x.shape), golden.tensor(c["tag"] + "/fake"),
                          c["tag"] + " compose")


def test_mxfp_golden(golden):
    for c in _cases(golden, "mxfp"):
        x = golden.tensor(c["input"] + "/x").to(DEV)
        meta = mb.MXFPMeta(block_size=c["block"], scale_exp_bits=8, element_exp_bits=c["E"], element_frac_bits=c["F"],
                           element_is_finite=True, round_mode="rn")
        sc, co = mb.extract_mxfp_components(x.flatten(), meta)
        assert_bits_equal(sc, golden.tensor(c["tag"] + "/scale"), c["tag"] + " scale")
        assert_bits_equal(co, golden.tensor(c["tag"] + "/codes"), c["tag"] + " codes")
        fake = golden.tensor(c["tag"] + "/fake")
        assert_bits_equal(mb.mxfp_quantizer(x, c["block"], c["E"], c["F"]), fake, c["tag"] + " fake")
        assert_bits_equal(mb.compose_mxfp_tensor(sc, co, meta, x.dtype).reshape(x.shape), fake, c["tag"] + " compose")


def test_minifloat_golden(golden):
    for c in _cases(golden, "minifloat"):
        x = golden.tensor(c["input"] + "/x").to(DEV)
        meta = mb.MinifloatMeta(exp_bits=c["E"], frac_bits=c["F"], is_finite=True, round_mode="rn")
        assert_bits_equal(mb.minifloat_quantizer_sim(x, meta), golden.tensor(c["tag"] + "/fake"), c["tag"])


def test_bfp_golden(golden):
    for c in _cases(golden, "bfp"):
        x = golden.tensor(c["input"] + "/x").to(DEV)
        y = mb.block_fp_quantizer(x, c["width"], c["exponent_width"], c["exponent_bias"], c["block_size"], c["skip_first_dim"])
        assert_bits_equal(y, golden.tensor(c["tag"] + "/fake"), c["tag"])


def test_bfp_tiles_golden(golden):
    for c in _cases(golden, "bfp_tiles"):
        x = golden.tensor(f"bfp_tiles/{c['name']}/{c['dtype']}/x").to(DEV)
        for width in c["widths"]:
            ref = golden.tensor(f"bfp_tiles/{c['name']}/{c['dtype']}/w{width}/fake")
            y = mb.block_fp_quantizer(x, width, 8, 127, c["block_size"], c["skip_first_dim"])
            assert_bits_equal(y, ref, f"{c['name']} w{width}", signed_zero=False)


def test_block_dim_golden(golden):
    for c in _cases(golden, "blockdim"):
        dt, bd, blk = c["dtype"], c["block_dim"], c["block"]
        x = golden.tensor(f"blockdim/{dt}/x").to(DEV)
        y = mb.mxint_quantizer(x, blk, 8, bd)
        assert y.shape == x.shape
        assert_bits_equal(y.contiguous(), golden.tensor(f"blockdim/{dt}/mxint_d{bd}/fake"), f"mxint d{bd}")
        assert_bits_equal(mb.mxfp_quantizer(x, blk, 4, 3, bd).contiguous(), golden.tensor(f"blockdim/{dt}/mxfp_d{bd}/fake"),
                          f"mxfp d{bd}")


# ---- CPU oracle on the benchmark configurations' seeded inputs ----------------------------------------
def test_config1_mxint8_fp32_vs_oracle():
    """MXINT8 fake-quant of fp32 [4096,4096] N(0,1) with outliers, seed 0 (a quarter of the rows on the CPU)."""
    x = synthetic.normal_with_outliers(4096, 4096, seed=0)
    y = mb.mxint_quantizer(x.to(DEV), 32, 8)
    rows = slice(0, 1024)
    assert_bits_equal(y[rows], O.mxint_fake(x[rows], 32, 8), "config 1")
    sc, m = mb.mxint_codes(x.to(DEV)[rows].flatten(), 32, 8)
    osc, om = O.mxint_extract(x[rows].flatten(), 32, 8)
    assert_bits_equal(sc.view(-1, 1).float(), osc, "config 1 scales")
    assert_bits_equal(m.float(), om, "config 1 mantissas", signed_zero=False)  # int8 codes have no -0


@pytest.mark.parametrize("shape", [(1, 4096), (16, 4096), (128, 4096), (2048, 4096)])
def test_config2_sweep_vs_oracle(shape):
    """Student-t(3)*0.02 bf16, seed 1: MXFP8-E4M3/32, MXINT8/32, block-fp (8,[1,32]) and (7,[1,16])."""
    x = synthetic.student_t3(*shape, seed=1)
    xd = x.to(DEV)
    assert_bits_equal(mb.mxfp_quantizer(xd, 32, 4, 3), O.mxfp_fake(x, 32, 4, 3), "mxfp8")
    assert_bits_equal(mb.mxfp_quantizer(xd, 32, 2, 1), O.mxfp_fake(x, 32, 2, 1), "mxfp4")
    assert_bits_equal(mb.mxint_quantizer(xd, 32, 8), O.mxint_fake(x, 32, 8), "mxint8")
    assert_bits_equal(mb.block_fp_quantizer(xd, 8, 8, 127, [1, 32], True), O.bfp_fake_rows(x, 8, 8, 127, 32), "bfp8")
    assert_bits_equal(mb.block_fp_quantizer(xd, 7, 8, 127, [1, 16], True), O.bfp_fake_rows(x, 7, 8, 127, 16), "bfp7")
    meta = mb.MXFPMeta(32, 8, 4, 3, True, "rn")
    sc, co = mb.extract_mxfp_components(xd.flatten(), meta)
    osc, oco = O.mxfp_extract(x.flatten(), 32, 4, 3)
    assert_bits_equal(sc, osc, "scales")
    assert_bits_equal(co, oco, "codes")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_wide_dynamic_range_vs_oracle(dtype):
    """Values spread over 2**-140 .. 2**120 including fp32 subnormals, zeros and negative zeros."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(512, 512, generator=g) * torch.exp2(torch.randint(-140, 120, (512, 512), generator=g).float())
    x[::7] = 0
    x[3, :100] = -0.0
    x = x.to(dtype)
    xd = x.to(DEV)
    for E, F in ((4, 3), (2, 1), (5, 2), (3, 2), (2, 3), (1, 2)):
        assert_bits_equal(mb.mxfp_quantizer(xd, 32, E, F), O.mxfp_fake(x, 32, E, F), f"mxfp e{E}m{F}")
        sc, co = mb.extract_mxfp_components(xd.flatten(), mb.MXFPMeta(32, 8, E, F, True, "rn"))
        osc, oco = O.mxfp_extract(x.flatten(), 32, E, F)
        assert_bits_equal(sc, osc, f"scales e{E}m{F}")
        assert_bits_equal(co, oco, f"codes e{E}m{F}")
    for bits in (8, 4, 2):
        assert_bits_equal(mb.mxint_quantizer(xd, 32, bits), O.mxint_fake(x, 32, bits), f"mxint{bits}")
        sc, m = mb.mxint_codes(xd.flatten(), 32, bits)
        osc, om = O.mxint_extract(x.flatten(), 32, bits)
        assert_bits_equal(sc.view(-1, 1).float(), osc.float(), f"mxint{bits} scales")
        assert_bits_equal(m.float(), om.float(), f"mxint{bits} mantissas", signed_zero=False)  # int8 has no -0
    assert_bits_equal(mb.block_fp_quantizer(xd, 8, 8, 127, [1, 32], True), O.bfp_fake_rows(x, 8, 8, 127, 32), "bfp")
    assert_bits_equal(mb.block_fp_quantizer(xd, 12, 8, None, [16], True), O.bfp_fake_rows(x, 12, 8, None, 16), "bfp12")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mxfp_small_codes_exhaustive_vs_oracle(dtype):
    """Every bf16 mantissa (fp32: the same plus ulp neighbours) in the binades around the subnormal code range,
    both signs, odd and even block exponents, next to a block maximum; plus ReLU-sparse data with exact zeros."""
    man = torch.arange(128, dtype=torch.int32) << 16
    vals = []
    for e in range(-34, 2):
        bits = ((127 + e) << 23) + man
        if dtype == torch.float32:
            bits = torch.cat([bits, bits + 1, bits - 1, bits + 0x80, bits + 0xFF, bits + 0x100, bits + 0x7FFF, bits + 0x8000])
        vals.append(bits.view(torch.float32))
    v = torch.cat(vals)
    v = torch.cat([v, -v])
    pad = (-v.numel()) % 31
    v = torch.cat([v, v[:pad]]).view(-1, 31)
    blocks = []
    for top in (1.0, 1.75, 2.0, 3.5):  # block maxima in two adjacent binades: odd and even shared exponents
        blocks.append(torch.cat([torch.full((v.shape[0], 1), top), v], dim=1))
    x = torch.cat(blocks).to(dtype)
    g = torch.Generator().manual_seed(23)
    sparse = torch.randn(256, 1024, generator=g).relu().to(dtype)
    for t in (x, sparse, -sparse):
        td = t.to(DEV)
        for E, F in ((4, 3), (2, 1), (5, 2), (3, 2), (2, 3), (1, 2)):
            assert_bits_equal(mb.mxfp_quantizer(td, 32, E, F), O.mxfp_fake(t, 32, E, F), f"mxfp e{E}m{F}")
            sc, co = mb.extract_mxfp_components(td.flatten(), mb.MXFPMeta(32, 8, E, F, True, "rn"))
            osc, oco = O.mxfp_extract(t.flatten(), 32, E, F)
            assert_bits_equal(sc, osc, f"scales e{E}m{F}")
            assert_bits_equal(co, oco, f"codes e{E}m{F}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_power_of_two_neighbourhoods_vs_oracle(dtype):
    """Block maxima within +-64 ulps of every power of two: exercises the log2 rounding tables."""
    e = torch.arange(-126, 127).float()
    base = torch.exp2(e).view(-1, 1).view(torch.int32)
    step = 1 if dtype == torch.float32 else 1 << 16
    mx = (base + torch.arange(-64, 65, dtype=torch.int32).view(1, -1) * step).view(torch.float32).flatten()
    mx = mx[torch.isfinite(mx) & (mx > 0)]
    g = torch.Generator().manual_seed(11)
    x = torch.rand(mx.numel(), 32, generator=g) * 1.9 - 0.95
    x = x * mx.view(-1, 1)
    x[:, 0] = mx
    x = x.to(dtype)
    xd = x.to(DEV)
    assert_bits_equal(mb.mxint_quantizer(xd, 32, 8), O.mxint_fake(x, 32, 8), "mxint8")
    sc, m = mb.mxint_codes(xd.flatten(), 32, 8)
    osc, om = O.mxint_extract(x.flatten(), 32, 8)
    assert_bits_equal(sc.view(-1, 1).float(), osc.float(), "mxint8 scales")
    assert_bits_equal(m.float(), om.float(), "mxint8 mantissas", signed_zero=False)
    assert_bits_equal(mb.mxfp_quantizer(xd, 32, 4, 3), O.mxfp_fake(x, 32, 4, 3), "mxfp8")
    assert_bits_equal(mb.block_fp_quantizer(xd, 8, 8, 127, [1, 32], True), O.bfp_fake_rows(x, 8, 8, 127, 32), "bfp")


@pytest.mark.parametrize("block", [2, 4, 8, 16, 32, 64, 128, 256, 512, 24, 48])
def test_block_sizes_vs_oracle(block):
    g = torch.Generator().manual_seed(block)
    x = torch.randn(96, 512 * 3, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        xc = x.to(dt)
        xd = xc.to(DEV)
        assert_bits_equal(mb.mxint_quantizer(xd, block, 8), O.mxint_fake(xc, block, 8), f"mxint b{block}")
        assert_bits_equal(mb.mxfp_quantizer(xd, block, 4, 3), O.mxfp_fake(xc, block, 4, 3), f"mxfp b{block}")
        assert_bits_equal(mb.block_fp_quantizer(xd, 8, 8, 127, [1, block], True), O.bfp_fake_rows(xc, 8, 8, 127, block),
                          f"bfp b{block}")


def test_ragged_and_empty_inputs():
    # block-fp pads a ragged last tile with zeros; MX quantizers require divisibility like the reference
    g = torch.Generator().manual_seed(3)
    x = torch.randn(7, 100, generator=g).bfloat16()
    assert_bits_equal(mb.block_fp_quantizer(x.to(DEV), 8, 8, 127, [1, 32], True), O.bfp_fake_rows(x, 8, 8, 127, 32), "ragged")
    b = torch.randn(50, generator=g)
    assert_bits_equal(mb.block_fp_quantizer(b.to(DEV), 7, 8, 127, [16], False), O.bfp_fake_rows(b, 7, 8, 127, 16), "bias")
    x3 = torch.randn(3, 5, 40, generator=g)
    assert_bits_equal(mb.block_fp_quantizer(x3.to(DEV), 8, 8, 127, [1, 16], True), O.bfp_fake_rows(x3, 8, 8, 127, 16), "3d")
    with pytest.raises(AssertionError):
        mb.mxint_quantizer(torch.randn(3, 33, device=DEV), 32, 8)
    with pytest.raises(AssertionError):
        mb.mxfp_quantizer(torch.randn(3, 33, device=DEV), 32, 4, 3)
    e = torch.empty(0, 32, device=DEV)
    assert mb.mxint_quantizer(e, 32, 8).shape == (0, 32)
    assert mb.mxfp_quantizer(e, 32, 4, 3).shape == (0, 32)
    # blocks that straddle rows of the flattened tensor (only numel must divide)
    xs = torch.randn(6, 48, generator=g)
    assert_bits_equal(mb.mxfp_quantizer(xs.to(DEV), 32, 4, 3), O.mxfp_fake(xs, 32, 4, 3), "straddle")
    # non-contiguous input and a misaligned view
    xt = torch.randn(64, 96, generator=g)
    assert_bits_equal(mb.mxint_quantizer(xt.to(DEV).t(), 32, 8).contiguous(), O.mxint_fake(xt.t(), 32, 8).contiguous(), "transposed")
    xo = torch.randn(1 + 32 * 9, generator=g)
    assert_bits_equal(mb.mxint_quantizer(xo.to(DEV)[1:], 32, 8), O.mxint_fake(xo[1:], 32, 8), "offset view")


def test_errors_and_unsupported():
    with pytest.raises(RuntimeError):
        mb.mxint_quantizer(torch.randn(4, 32), 32, 8)  # CPU tensor: no fallback
    with pytest.raises(NotImplementedError):
        mb.mxint_quantizer(torch.randn(4, 32, device=DEV).half(), 32, 8)
    with pytest.raises(NotImplementedError):
        mb.mxfp_quantizer(torch.randn(4, 32, device=DEV), 16, 4, 3, quantile_search=True)  # the search needs blocks of 32
    with pytest.raises(AssertionError):
        mb.mxfp_quantizer(torch.randn(4, 32, device=DEV), 32, 3, 3)
    with pytest.raises(NotImplementedError):
        mb.block_fp_quantizer(torch.randn(2, 8, 64, device=DEV), 8, 8, 127, [16], False)  # 3-D weights: as the reference


def test_output_dtype_and_autograd():
    x = torch.randn(8, 64, device=DEV, requires_grad=True)
    y = mb.mxfp_quantizer(x, 32, 4, 3)
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))  # straight-through estimator
    meta = mb.MXFPMeta(32, 8, 4, 3, True, "rn")
    xb = torch.randn(8, 64).bfloat16()
    y32 = mb.mxfp_quantizer_sim(xb.to(DEV), -1, meta, dtype=torch.float32)
    assert y32.dtype == torch.float32
    assert_bits_equal(y32, O.mxfp_fake(xb, 32, 4, 3, out_dtype=torch.float32), "bf16 -> fp32")
    y16 = mb.mxint_quantizer_sim(xb.float().to(DEV), -1, mb.MXIntMeta(32, 8, 8), dtype=torch.bfloat16)
    assert_bits_equal(y16, O.mxint_fake(xb.float(), 32, 8, out_dtype=torch.bfloat16), "fp32 -> bf16")


# ---- full-size, size-independent properties ---------------------------------------------------------
def test_full_size_properties():
    """bf16 [16384, 8192] (largest-but-one sweep shape): the packed path and the fused fake path agree, a row
    split gives the same result as the whole tensor, MXFP is odd-symmetric, and a sample of rows equals the oracle."""
    rows, cols = 16384, 8192
    x = synthetic.device_student_t3(rows, cols, seed=1, device=DEV)
    meta = mb.MXFPMeta(32, 8, 4, 3, True, "rn")
    y = mb.mxfp_quantizer(x, 32, 4, 3)
    sc, co = mb.extract_mxfp_components(x.flatten(), meta)
    assert torch.equal(mb.compose_mxfp_tensor(sc, co, meta, x.dtype).view(torch.int16), y.flatten().view(torch.int16))
    half = rows // 2
    assert torch.equal(mb.mxfp_quantizer(x[half:], 32, 4, 3).view(torch.int16), y[half:].view(torch.int16))
    assert torch.equal(mb.mxfp_quantizer(-x, 32, 4, 3), -y)
    yi = mb.mxint_quantizer(x, 32, 8)
    sci, mi = mb.mxint_codes(x.flatten(), 32, 8)
    imeta = mb.MXIntMeta(32, 8, 8)
    scf, mf = mb.extract_mxint_components(x.flatten(), imeta)
    assert torch.equal(mf, mi.to(x.dtype)) and torch.equal(scf.flatten(), sci.to(x.dtype))
    assert torch.equal(mb.compose_mxint_tensor(scf, mf, imeta).flatten().view(torch.int16), yi.flatten().view(torch.int16))
    # every dequantized value is a multiple of its block's step and within the block range
    assert bool((mi.to(torch.int16).abs() <= 128).all())
    idx = torch.arange(0, rows, 257, device=DEV)
    xs = x[idx].cpu()
    assert_bits_equal(y[idx], O.mxfp_fake(xs, 32, 4, 3), "sampled rows mxfp8")
    assert_bits_equal(yi[idx], O.mxint_fake(xs, 32, 8), "sampled rows mxint8")
    yb = mb.block_fp_quantizer(x, 8, 8, 127, [1, 32], True)
    assert_bits_equal(yb[idx], O.bfp_fake_rows(xs, 8, 8, 127, 32), "sampled rows bfp")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_fp_two_dimensional_tiles_vs_oracle(dtype):
    """Tiles that span rows: 2-D weights with skip_first_dim=False and 3-D activations (the reference's unfold/fold
    route; signed zeros come out positive there)."""
    g = torch.Generator().manual_seed(21)
    cases = [((64, 96), [16], False, 64, 16), ((64, 96), [16, 16], False, 16, 16), ((70, 100), [16, 32], False, 16, 32),
             ((300, 40), [8], False, 300, 8), ((3, 20, 40), [16], True, 20, 16), ((2, 33, 50), [8, 8], True, 8, 8),
             ((4096, 64), [16], False, 4096, 16)]
    for shape, bs, skip, bh, bw in cases:
        x = torch.randn(*shape, generator=g) * torch.exp2(torch.randint(-12, 6, shape, generator=g).float())
        x.view(-1)[::7] = 0
        x = x.to(dtype)
        for width, ew, eb in ((8, 8, 127), (7, 8, 127), (12, 8, None)):
            y = mb.block_fp_quantizer(x.to(DEV), width, ew, eb, bs, skip)
            assert_bits_equal(y, O.bfp_fake_tiles(x, width, ew, eb, bh, bw), f"{shape} {bs} w{width}", signed_zero=False)


def test_mxint_clipping_search_on_gpu(golden):
    """Calibration-time options of MXINT on the GPU: tensor code whose quantile / norm reductions may round differently
    from the host's, so a few blocks may pick a neighbouring percentile; every block is one of the 11 candidates."""
    for case in (c for c in golden.cases if c["kind"] == "mxint_search"):
        dt, nbits = case["dtype"], case["bits"]
        x = golden.tensor(f"mxint_search/{dt}/x", dt)
        act = golden.tensor(f"mxint_search/{dt}/act", dt)
        meta = mb.MXIntMeta(block_size=32, scale_bits=8, element_bits=nbits)
        for key, kwargs in (("fake", {}), ("fake_act", {"act_tensor": act.to(DEV), "cali_batch_size": 2})):
            y = mb.mxint_quantizer_sim(x.to(DEV), 1, meta, quantile_search=True, **kwargs).cpu()
            ref = golden.tensor(f"mxint_search/{dt}/w{nbits}/{key}", dt)
            same = (y.view(-1, 32) == ref.view(-1, 32)).all(dim=1).float().mean().item()
            assert same >= 0.97, (dt, nbits, key, same)
        y = mb.mxint_quantizer(x.to(DEV), 32, nbits, 1, 8, True).cpu()
        from mase_b200 import quantizers as Q
        cand = Q._mxint_candidates(x.flatten().reshape(-1, 32), meta, torch.tensor(Q._SEARCH_PERCENTILES))
        assert bool((cand.view(11, -1, 32) == y.reshape(1, -1, 32)).all(dim=2).any(dim=0).all())
        sc, mant = mb.extract_mxint_components(x.to(DEV).flatten(), meta, percentile=0.97)
        rs, rm = golden.tensor(f"mxint_search/{dt}/w{nbits}/p97_scale", dt), golden.tensor(f"mxint_search/{dt}/w{nbits}/p97_mant", dt)
        assert (sc.cpu() == rs).float().mean().item() >= 0.97 and (mant.cpu() == rm).all(dim=1).float().mean().item() >= 0.97
    # LinearMXInt with clip_search quantizes its weight through the search
    cfg = {"weight_block_size": 32, "weight_width": 4, "data_in_block_size": 32, "data_in_width": 8, "clip_search": True}
    layer = mb.LinearMXInt(128, 48, bias=False, device=DEV, dtype=torch.bfloat16, config=cfg)
    w = golden.tensor("mxint_search/bf16/x", "bf16")
    layer.load_state_dict({"weight": w.to(DEV)}, strict=False)
    ref = golden.tensor("mxint_search/bf16/w4/fake", "bf16")
    assert (layer.weight.data.cpu().view(-1, 32) == ref.view(-1, 32)).all(dim=1).float().mean().item() >= 0.97
