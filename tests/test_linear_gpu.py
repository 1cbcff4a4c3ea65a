"""Quantized Linear modules on the GPU against the reference's golden outputs and the CPU oracle."""

import copy

import pytest
import torch

import mase_b200 as mb
from mase_b200 import gemm, synthetic
from conftest import assert_bits_equal
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CLASSES = {"LinearMXFP": mb.LinearMXFP, "LinearMXInt": mb.LinearMXInt, "LinearBlockFP": mb.LinearBlockFP}


def rel_err(y, ref):
    return float((y.float().cpu() - ref.float()).abs().max() / ref.float().abs().max())


def test_linear_modules_match_reference_golden(golden):
    """Same constructor + load_state_dict route as the quantize pass; weights bit-exact, outputs within tolerance."""
    for c in [c for c in golden.cases if c["kind"] == "linear"]:
        dt, tag, cfg = c["dtype"], c["tag"], c["config"]
        dtype = torch.float32 if dt == "fp32" else torch.bfloat16
        x = golden.tensor(f"linear/{dt}/x").to(DEV)
        state = {"weight": golden.tensor(f"linear/{dt}/w").to(DEV), "bias": golden.tensor(f"linear/{dt}/b").to(DEV)}
        layer = CLASSES[c["cls"]](c["K"], c["N"], bias=True, device=DEV, dtype=dtype, config=dict(cfg))
        layer.load_state_dict(copy.deepcopy(state), strict=False)
        if c["cls"] != "LinearBlockFP":
            assert_bits_equal(layer.weight.data, golden.tensor(tag + "/w_q"), tag + " w_q")
            assert_bits_equal(layer.bias.data, golden.tensor(tag + "/b_q"), tag + " b_q")
        y = layer(x)
        gemm.check_status()
        y_ref = golden.tensor(tag + "/y")
        assert y.dtype == y_ref.dtype and y.shape == y_ref.shape
        # the reference output went through the CPU library GEMM in x.dtype; compare within accumulation tolerance
        tol = 1e-3 if dt == "fp32" else 8e-3
        assert rel_err(y, y_ref) <= tol, tag


@pytest.mark.parametrize("M", [1, 16, 128, 2048])
def test_config3_linear_mxfp8_vs_oracle(M):
    """MXFP8 Linear 4096 -> 4096, bf16, no bias (seed 2); fp32 GEMM of oracle-quantized operands is the reference."""
    K = N = 4096
    x, w = synthetic.linear_operands(M, K, N, seed=2)
    cfg = {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    layer = mb.LinearMXFP(K, N, bias=False, device=DEV, dtype=torch.bfloat16, config=cfg)
    layer.load_state_dict({"weight": w.to(DEV)}, strict=False)
    wq = O.mxfp_fake(w, 32, 4, 3, 1)
    assert_bits_equal(layer.weight.data, wq, "weight")
    assert layer._packed_weight() is not None  # the block-scaled tensor-core path is the one that runs
    y = layer(x.to(DEV))
    gemm.check_status()
    ref = O.linear_mxfp(x, wq, None, cfg)
    assert rel_err(y, ref) <= 4e-3  # bf16 output: half an ulp is 2**-9 of the value
    # the fake-quantized fallback (dense bf16 MMA) agrees with the block-scaled path
    y2 = gemm.linear_forward(mb.mxfp_quantizer(x.to(DEV), 32, 4, 3), layer.weight, None)
    assert rel_err(y2, ref) <= 4e-3
    assert rel_err(y, y2.cpu()) <= 4e-3


def test_mixed_precision_layer_linears():
    """The Linear children of the Llama-style layer: MXINT8 W+A projections, MXFP4-weight / MXFP8-activation FFN."""
    g = torch.Generator().manual_seed(3)
    h, ffn, tokens = 512, 1376, 96
    x = torch.randn(tokens, h, generator=g).bfloat16()
    int_cfg = {"weight_block_size": 32, "weight_width": 8, "data_in_block_size": 32, "data_in_width": 8}
    ffn_cfg = {"weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1,
               "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    wq = (torch.randn(h, h, generator=g) * 0.02).bfloat16()
    q = mb.LinearMXInt(h, h, bias=False, device=DEV, dtype=torch.bfloat16, config=int_cfg)
    q.load_state_dict({"weight": wq.to(DEV)}, strict=False)
    ref = O.linear_mxint(x, O.mxint_fake(wq, 32, 8, 1), None, int_cfg)
    assert rel_err(q(x.to(DEV)), ref) <= 4e-3
    wu = (torch.randn(ffn, h, generator=g) * 0.02).bfloat16()
    up = mb.LinearMXFP(h, ffn, bias=False, device=DEV, dtype=torch.bfloat16, config=ffn_cfg)
    up.load_state_dict({"weight": wu.to(DEV)}, strict=False)
    assert up._packed_weight() is not None
    ref = O.linear_mxfp(x, O.mxfp_fake(wu, 32, 2, 1, 1), None, ffn_cfg)
    assert rel_err(up(x.to(DEV)), ref) <= 4e-3
    wd = (torch.randn(h, ffn, generator=g) * 0.02).bfloat16()
    down = mb.LinearMXFP(ffn, h, bias=False, device=DEV, dtype=torch.bfloat16, config=ffn_cfg)
    down.load_state_dict({"weight": wd.to(DEV)}, strict=False)
    xa = torch.randn(tokens, ffn, generator=g).bfloat16()
    ref = O.linear_mxfp(xa, O.mxfp_fake(wd, 32, 2, 1, 1), None, ffn_cfg)
    assert rel_err(down(xa.to(DEV)), ref) <= 4e-3
    gemm.check_status()


def test_bypass_and_unloaded_weights():
    cfg = {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    g = torch.Generator().manual_seed(8)
    x = torch.randn(64, 256, generator=g).bfloat16()
    w = (torch.randn(128, 256, generator=g) * 0.05).bfloat16()
    # weights copied without load_state_dict (the FX-pass route): stay unquantized, activations are quantized
    layer = mb.LinearMXFP(256, 128, bias=False, device=DEV, dtype=torch.bfloat16, config=dict(cfg))
    with torch.no_grad():
        layer.weight.copy_(w.to(DEV))
    assert layer._packed_weight() is None
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ w.float().t()
    assert rel_err(layer(x.to(DEV)), ref) <= 4e-3
    by = mb.LinearMXFP(256, 128, bias=False, device=DEV, dtype=torch.bfloat16, config=dict(cfg, bypass=True))
    by.load_state_dict({"weight": w.to(DEV)}, strict=False)
    assert_bits_equal(by.weight.data, w, "bypass keeps the weight")
    assert rel_err(by(x.to(DEV)), x.float() @ w.float().t()) <= 4e-3
    # an in-place update after loading invalidates the packed copy
    layer.load_state_dict({"weight": w.to(DEV)}, strict=False)
    assert layer._packed_weight() is not None
    with torch.no_grad():
        layer.weight.mul_(2.0)
    assert layer._packed_weight() is None
    gemm.check_status()


def test_large_m_with_bias_vs_oracle():
    """Several waves of tiles, a ragged last 128-row panel and a bias."""
    M, K, N = 4736 + 77, 512, 4096
    x, w = synthetic.linear_operands(M, K, N, seed=12)
    g = torch.Generator().manual_seed(12)
    b = torch.randn(N, generator=g).bfloat16()
    cfg = {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    layer = mb.LinearMXFP(K, N, bias=True, device=DEV, dtype=torch.bfloat16, config=cfg)
    layer.load_state_dict({"weight": w.to(DEV), "bias": b.to(DEV)}, strict=False)
    xd = x.to(DEV)
    y1 = layer(xd)
    y2 = layer(xd)
    torch.cuda.synchronize()
    gemm.check_status()
    assert torch.equal(y1, y2)
    ref = O.linear_mxfp(x, O.mxfp_fake(w, 32, 4, 3, 1), b, cfg)
    assert rel_err(y1, ref) <= 4e-3
    # same result as the two-kernel path on one stream
    xp = gemm.pack_mx_operand(xd, 4, 3)
    y3 = gemm.mx_gemm(xp, layer._packed_weight(), layer.bias, torch.bfloat16)
    assert torch.equal(y1, y3)


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (16, 4096, 4096), (128, 2048, 1024), (100, 1024, 1000), (7, 8192, 512),
                                   (5, 96, 72), (13, 160, 8), (16, 4128, 1000), (17, 4096, 256)])
def test_small_m_with_bias_vs_oracle(shape):
    """At most 128 rows (narrow tiles), bias, ragged N, bf16 and fp32 outputs; results are repeatable."""
    M, K, N = shape
    x, w = synthetic.linear_operands(M, K, N, seed=31)
    g = torch.Generator().manual_seed(31)
    b = torch.randn(N, generator=g).bfloat16()
    cfg = {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    layer = mb.LinearMXFP(K, N, bias=True, device=DEV, dtype=torch.bfloat16, config=cfg)
    layer.load_state_dict({"weight": w.to(DEV), "bias": b.to(DEV)}, strict=False)
    y1 = layer(x.to(DEV))
    y2 = layer(x.to(DEV))
    gemm.check_status()
    assert torch.equal(y1, y2)
    ref = O.linear_mxfp(x, O.mxfp_fake(w, 32, 4, 3, 1), b, cfg)
    assert rel_err(y1, ref) <= 4e-3
    layer.output_dtype = torch.float32
    assert rel_err(layer(x.to(DEV)), ref) <= 1e-3


@pytest.mark.parametrize("kind", ["mxfp", "mxint"])
def test_functional_matmul_and_bmm_vs_oracle(kind):
    """matmul_* / bmm_*: both operands fake-quantized along their last dimension, as the reference does."""
    g = torch.Generator().manual_seed(17)
    x = torch.randn(3, 40, 256, generator=g).bfloat16()
    y2 = (torch.randn(256, 96, generator=g) * 0.05).bfloat16()
    y3 = (torch.randn(3, 256, 96, generator=g) * 0.05).bfloat16()
    if kind == "mxfp":
        cfg = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3,
               "weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1}
        q = lambda t, w: O.mxfp_fake(t, 32, *((4, 3) if w == "x" else (2, 1)))
        mm, bmm = mb.matmul_mxfp, mb.bmm_mxfp
    else:
        cfg = {"data_in_block_size": 32, "data_in_width": 8, "weight_block_size": 32, "weight_width": 4}
        q = lambda t, w: O.mxint_fake(t, 32, 8 if w == "x" else 4)
        mm, bmm = mb.matmul_mxint, mb.bmm_mxint
    ref2 = q(x, "x").float() @ q(y2, "y").float()
    ref3 = torch.bmm(q(x, "x").float(), q(y3, "y").float())
    out2 = mm(x.to(DEV), y2.to(DEV), cfg)
    out3 = bmm(x.to(DEV), y3.to(DEV), cfg)
    outb = mm(x.to(DEV), y3.to(DEV), cfg)
    gemm.check_status()
    assert out2.dtype == torch.bfloat16 and out2.shape == (3, 40, 96)
    assert rel_err(out2, ref2) <= 4e-3 and rel_err(out3, ref3) <= 1e-2 and rel_err(outb, ref3) <= 1e-2
    assert torch.equal(mm(x.to(DEV), y2.to(DEV), {"bypass": True}), torch.matmul(x.to(DEV), y2.to(DEV)))


def test_weight_only_storage_round_trip():
    """drop_dense_weight keeps only codes + scales (about half the bytes of the bf16 weight), gives the same outputs,
    and its state_dict loads into a fresh layer."""
    x, w = synthetic.linear_operands(64, 1024, 768, seed=9)
    cfg = {"weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    layer = mb.LinearMXFP(1024, 768, bias=False, device=DEV, dtype=torch.bfloat16, config=dict(cfg))
    layer.load_state_dict({"weight": w.to(DEV)}, strict=False)
    y0 = layer(x.to(DEV))
    dense_bytes = layer.weight.numel() * 2
    layer.drop_dense_weight()
    assert layer.weight.numel() == 0
    packed_bytes = layer.weight_codes.numel() + layer.weight_scales.numel()
    assert layer.weight_codes.shape == (768, 512)  # MXFP4: two codes per byte
    assert packed_bytes <= 0.28 * dense_bytes       # 0.53 bytes per element against 2
    assert torch.equal(layer(x.to(DEV)), y0)
    state = layer.state_dict()
    assert "weight_codes" in state and "weight_scales" in state
    fresh = mb.LinearMXFP(1024, 768, bias=False, device=DEV, dtype=torch.bfloat16, config=dict(cfg))
    fresh.load_state_dict(state)
    assert torch.equal(fresh(x.to(DEV)), y0)
    gemm.check_status()
    with pytest.raises(RuntimeError):
        fresh(x.to(DEV).float())
    # a checkpoint whose packed weight does not fit the layer is refused instead of reaching the GEMM
    other = mb.LinearMXFP(1024, 512, bias=False, device=DEV, dtype=torch.bfloat16, config=dict(cfg))
    with pytest.raises(RuntimeError, match="do not fit"):
        other.load_state_dict(state)
    # MXFP8 weights keep one byte per element
    cfg8 = dict(cfg, weight_exponent_width=4, weight_frac_width=3)
    l8 = mb.LinearMXFP(1024, 768, bias=False, device=DEV, dtype=torch.bfloat16, config=cfg8)
    l8.load_state_dict({"weight": w.to(DEV)}, strict=False)
    y8 = l8(x.to(DEV))
    l8.drop_dense_weight()
    assert l8.weight_codes.shape == (768, 1024) and torch.equal(l8(x.to(DEV)), y8)
    # an update of the dense weight through .data (no version bump) on a moved layer: the packed copy follows .to()
    moved = mb.LinearMXFP(1024, 768, bias=False, device=DEV, dtype=torch.bfloat16, config=dict(cfg))
    moved.load_state_dict({"weight": w.to(DEV)}, strict=False)
    moved.to(DEV)
    assert moved._packed_weight() is not None
    import copy

    twin = copy.deepcopy(moved)
    assert twin._packed_weight() is not None and twin._packed_weight().codes.data_ptr() != moved._packed_weight().codes.data_ptr()
    assert torch.equal(twin(x.to(DEV)), moved(x.to(DEV)))
    with torch.no_grad():
        twin.weight.mul_(1)  # a tracked in-place update invalidates the packed copy (forward then multiplies `weight`)
    assert twin._packed_weight() is None


def test_functional_elementwise_mx_ops_vs_oracle():
    """kv_cache_* / softmax_* / silu_* / rope_*: the quantization is bit-exact, the surrounding torch op is the same."""
    g = torch.Generator().manual_seed(19)
    k = torch.randn(2, 4, 48, 64, generator=g).bfloat16()
    v = torch.randn(2, 4, 48, 64, generator=g).bfloat16()
    cfp = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    cint = {"data_in_block_size": 32, "data_in_width": 8}
    kq, vq = mb.kv_cache_mxfp(k.to(DEV), v.to(DEV), cfp)
    assert_bits_equal(kq, O.mxfp_fake(k, 32, 4, 3), "k")
    assert_bits_equal(vq, O.mxfp_fake(v, 32, 4, 3), "v")
    kq, vq = mb.kv_cache_mxint(k.to(DEV), v.to(DEV), cint)
    assert_bits_equal(kq, O.mxint_fake(k, 32, 8), "k int")
    s = torch.randn(2, 4, 48, 64, generator=g).bfloat16() * 3
    for fn, oq in ((mb.softmax_mxfp, O.mxfp_fake(s, 32, 4, 3)), (mb.softmax_mxint, O.mxint_fake(s, 32, 8))):
        ref = torch.softmax(oq.float(), -1)
        out = fn(s.to(DEV), cfp if fn is mb.softmax_mxfp else cint)
        assert out.dtype == torch.bfloat16 and (out.float().cpu() - ref).abs().max() <= 4e-3
    out = mb.silu_mxfp(s.to(DEV), cfp)
    assert (out.float().cpu() - torch.nn.functional.silu(O.mxfp_fake(s, 32, 4, 3).float())).abs().max() <= 3e-2
    out = mb.silu_mxint(s.to(DEV), cint)
    assert (out.float().cpu() - torch.nn.functional.silu(O.mxint_fake(s, 32, 8).float())).abs().max() <= 3e-2
    ang = torch.rand(2, 48, 64, generator=g) * 6.28
    cos, sin = ang.cos().bfloat16(), ang.sin().bfloat16()
    qe, ke = mb.rope_mxfp(k.to(DEV), v.to(DEV), cos.to(DEV), sin.to(DEV), cfp)
    cq, sq = O.mxfp_fake(cos, 32, 4, 3).float().unsqueeze(1), O.mxfp_fake(sin, 32, 4, 3).float().unsqueeze(1)
    rot = lambda t: torch.cat((-t[..., 32:], t[..., :32]), -1)
    assert (qe.float().cpu() - (k.float() * cq + rot(k.float()) * sq)).abs().max() <= 5e-2
    assert (ke.float().cpu() - (v.float() * cq + rot(v.float()) * sq)).abs().max() <= 5e-2
    qe, ke = mb.rope_mxint(k.to(DEV), v.to(DEV), cos.to(DEV), sin.to(DEV), cint)
    assert qe.shape == k.shape and ke.shape == v.shape


@pytest.mark.parametrize("shape", [(96, 1376, 512), (300, 3584, 256), (2048, 1024, 768)])
def test_gated_pack_and_gated_linear(shape):
    """silu(gate) * up -> MXFP8 operand in one kernel: the codes of packing torch's own bf16 product, the GEMM result
    of the two-step route bit for bit, and the oracle's codes of the CPU product up to the rare element where the
    host's and the device's exp differ in the last fp32 bit before the bf16 rounding."""
    M, F, N = shape
    g = torch.Generator().manual_seed(11)
    gu = (torch.randn(M, 2 * F, generator=g) * 2).bfloat16()
    w = (torch.randn(N, F, generator=g) * 0.02).bfloat16()
    gud = gu.to(DEV)
    gate, up = gud[:, :F], gud[:, F:]          # strided views: the two halves of one GEMM output
    h = torch.nn.functional.silu(gate) * up
    fused = gemm.pack_gated_operand(gate, up, 4, 3)
    plain = gemm.pack_mx_operand(h, 4, 3)
    assert torch.equal(fused.codes, plain.codes)
    wp = gemm.pack_mx_operand(w.to(DEV), 4, 3)
    y_fused = gemm.mx_gated_linear(gate, up, wp, None, 4, 3, torch.float32)
    y_plain = gemm.mx_linear(h, wp, None, 4, 3, torch.float32)
    gemm.check_status()
    assert torch.equal(y_fused, y_plain)
    h_cpu = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    assert float((h_cpu != h.cpu()).float().mean()) < 1e-3
    ref = O.mxfp_fake(h_cpu, 32, 4, 3).float() @ O.mxfp_fake(w, 32, 4, 3, 1).float().t()
    assert rel_err(y_fused, ref) <= 2e-3
    # module level: the down projection of a gated MLP
    cfg = dict(synthetic.MXFP4W_MXFP8A_LINEAR)
    down = mb.LinearMXFP(F, N, bias=False, device=DEV, dtype=torch.bfloat16, config=cfg)
    down.load_state_dict({"weight": w.to(DEV)}, strict=False)
    assert torch.equal(down.forward_gated(gate, up), down(h))


def test_sibling_projections_share_one_activation_quantization():
    from mase_b200.modules import forward_siblings

    g = torch.Generator().manual_seed(12)
    x = torch.randn(3, 50, 512, generator=g).bfloat16().to(DEV)
    for cls, cfg in ((mb.LinearMXInt, synthetic.MXINT8_LINEAR), (mb.LinearMXFP, synthetic.MXFP4W_MXFP8A_LINEAR)):
        layers = []
        for n in (512, 256, 768):
            m = cls(512, n, bias=True, device=DEV, dtype=torch.bfloat16, config=dict(cfg))
            m.load_state_dict({"weight": (torch.randn(n, 512, generator=g) * 0.02).bfloat16().to(DEV),
                               "bias": torch.randn(n, generator=g).bfloat16().to(DEV)}, strict=False)
            layers.append(m)
        shared = forward_siblings(layers, x)
        for m, y in zip(layers, shared):
            assert torch.equal(y, m(x)) and y.shape == (3, 50, m.out_features)
    gemm.check_status()
    # layers that cannot share (different classes) are simply called one by one
    mixed = forward_siblings([layers[0], torch.nn.Linear(512, 64, dtype=torch.bfloat16, device=DEV)], x)
    assert mixed[1].shape == (3, 50, 64)


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (5, 160, 96), (16, 11008, 512), (16, 4096, 4096), (9, 1024, 200)])
@pytest.mark.parametrize("fp4", [False, True])
def test_decode_sized_forward_matches_its_parts(shape, fp4):
    """Up to 16 rows: the fused call (activation pack chained to the GEMM, the weight fetched ahead of the stream
    dependency) must give the bits of packing x and multiplying the packed operands as separate calls, with and
    without bias, bf16 and fp32 output; K not a multiple of 128, K shares that wrap the operand ring, N not a
    multiple of 128."""
    M, K, N = shape
    if fp4 and K % 128:
        pytest.skip("nibble-packed weights need K % 128 == 0")
    x, w = synthetic.linear_operands(M, K, N, seed=M + K)
    x[0, :32] = 0  # an all-zero block
    x[M - 1, 32:64] *= 300  # a block whose top element takes the E4M3 code that the hardware reads as NaN
    xd = x.to(DEV)
    we, wf = (2, 1) if fp4 else (4, 3)
    wp = gemm.pack_mx_operand(w.to(DEV), we, wf, fp4=fp4)
    bias = torch.randn(N, device=DEV).bfloat16()
    for out_dtype in (torch.bfloat16, torch.float32):
        for b in (None, bias):
            fused = gemm.mx_linear(xd, wp, b, 4, 3, out_dtype)
            parts = gemm.mx_gemm(gemm.pack_mx_operand(xd, 4, 3), wp, b, out_dtype)
            gemm.check_status()
            assert torch.equal(fused, parts), (shape, fp4, out_dtype, b is not None)
    ref = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, we, wf, 1).float().t()
    err = float((gemm.mx_linear(xd, wp, None, 4, 3, torch.float32).cpu() - ref).abs().max() / ref.abs().max())
    assert err <= 1e-3, (shape, fp4, err)


@pytest.mark.parametrize("which", ["weight", "activation", "both"])
@pytest.mark.parametrize("shape", [(16, 1024, 512), (256, 512, 384), (1024, 2048, 1024)])
def test_e5m2_operands_on_the_block_scaled_mma(which, shape):
    """MXFP8 with E5M2 elements runs on the block-scaled tensor-core MMA.  The hardware reads exponent code 31 as
    inf / nan, so every block is stored one scale step up with halved values; halving is exact except for elements 30
    binades below their block's maximum, so the result must equal the fp32 product of the oracle-quantized operands to
    1e-5 of the largest output (accumulation order), for the small-M, single-CTA and CTA-pair kernels, through the
    module (fused pack + GEMM) and through separately packed operands."""
    M, K, N = shape
    x, w = synthetic.linear_operands(M, K, N, seed=K)
    x[0, :32] = 0
    x[1, 32:64] *= 1e-3
    x[1, 40] = 90.0  # a block that spans 17 binades
    we, wf = (5, 2) if which in ("weight", "both") else (4, 3)
    xe, xf = (5, 2) if which in ("activation", "both") else (4, 3)
    cfg = {"weight_block_size": 32, "weight_exponent_width": we, "weight_frac_width": wf,
           "data_in_block_size": 32, "data_in_exponent_width": xe, "data_in_frac_width": xf}
    layer = mb.LinearMXFP(K, N, bias=False, device=DEV, dtype=torch.bfloat16, config=cfg)
    layer.load_state_dict({"weight": w.to(DEV)}, strict=False)
    packed = layer._packed_weight()
    assert packed is not None and packed.e5m2 == (we == 5)
    assert_bits_equal(layer.weight.data, O.mxfp_fake(w, 32, we, wf, 1), "weight")
    layer.output_dtype = torch.float32
    y = layer(x.to(DEV))
    xp = gemm.pack_mx_operand(x.to(DEV), xe, xf)
    assert xp.e5m2 == (xe == 5)
    y2 = gemm.mx_gemm(xp, packed, None, torch.float32)
    gemm.check_status()
    ref = O.mxfp_fake(x, 32, xe, xf).float() @ O.mxfp_fake(w, 32, we, wf, 1).float().t()
    for got, what in ((y, "module"), (y2, "parts")):
        err = float((got.cpu() - ref).abs().max() / ref.abs().max())
        assert err <= 1e-5, (which, shape, what, err)


def test_gated_pack_matches_torch_for_every_bf16_gate_value():
    """The fused SiLU*mul pack evaluates silu with a fast exponential and division where that provably rounds like the
    exact expression, and with the exact expression elsewhere: every finite bf16 gate pattern, against five up values,
    must give the codes and scales of packing torch's own `silu(gate) * up`."""
    pat = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    pat = pat[torch.isfinite(pat.float())]
    pad = (-pat.numel()) % 128
    gate_row = torch.cat([pat, torch.zeros(pad, dtype=torch.bfloat16)])
    ups = torch.tensor([1.0, -0.37, 3.0, 1e-3, 117.0], dtype=torch.bfloat16)
    gate = gate_row[None].expand(len(ups), -1).contiguous().to(DEV)
    up = ups[:, None].expand(-1, gate_row.numel()).contiguous().to(DEV)
    fused = gemm.pack_gated_operand(gate, up, 4, 3)
    ref = gemm.pack_mx_operand(torch.nn.functional.silu(gate) * up, 4, 3)
    torch.cuda.synchronize()
    assert torch.equal(fused.codes, ref.codes)
    # scale bytes of the rows that exist (the array is padded to 256-row tiles whose other bytes are never written)
    rows, k = gate.shape
    r = torch.arange(rows)[:, None]
    kb = torch.arange(k // 32)[None]
    off = ((r >> 7) * (k // 128) + (kb >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3)
    assert torch.equal(fused.scales.cpu()[off], ref.scales.cpu()[off])
