"""MX functional ops, Embedding and RMSNorm wrappers on the GPU against the same ops built from the CPU oracle."""

import pytest
import torch

import mase_b200 as mb
from mase_b200 import gemm
from conftest import assert_bits_equal
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FP_CFG = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3,
          "weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3}
INT_CFG = {"data_in_block_size": 32, "data_in_width": 8, "weight_block_size": 32, "weight_width": 8}


def rel_err(y, ref):
    return float((y.float().cpu() - ref.float()).abs().max() / ref.float().abs().max())


@pytest.mark.parametrize("kind", ["mxfp", "mxint"])
def test_batched_products_run_on_the_tensor_core_gemm(kind):
    """bmm_* and matmul_* with a batched second operand: one GEMM launch per batch element, no library GEMM."""
    g = torch.Generator().manual_seed(31)
    x = torch.randn(6, 40, 64, generator=g).bfloat16()
    y = torch.randn(6, 64, 96, generator=g).bfloat16()
    if kind == "mxfp":
        xq, yq = O.mxfp_fake(x, 32, 4, 3), O.mxfp_fake(y, 32, 4, 3)
        fn_b, fn_m, cfg = mb.bmm_mxfp, mb.matmul_mxfp, FP_CFG
    else:
        xq, yq = O.mxint_fake(x, 32, 8), O.mxint_fake(y, 32, 8)
        fn_b, fn_m, cfg = mb.bmm_mxint, mb.matmul_mxint, INT_CFG
    ref = torch.bmm(xq.float(), yq.float())
    out = fn_b(x.to(DEV), y.to(DEV), cfg)
    assert out.shape == ref.shape and out.dtype == torch.bfloat16
    assert rel_err(out, ref) <= 4e-3
    # matmul with broadcast batch dimensions and with a 2-D second operand
    x4 = x.view(2, 3, 40, 64)
    out4 = fn_m(x4.to(DEV), y[:3].to(DEV), cfg)
    ref4 = torch.matmul(xq.view(2, 3, 40, 64).float(), yq[:3].float())
    assert out4.shape == ref4.shape and rel_err(out4, ref4) <= 4e-3
    out2 = fn_m(x.to(DEV), y[0].to(DEV), cfg)
    assert rel_err(out2, torch.matmul(xq.float(), yq[0].float())) <= 4e-3
    gemm.check_status()
    with pytest.raises(RuntimeError):
        fn_b(x[0].to(DEV), y.to(DEV), cfg)


def test_minifloat_functional_wrappers():
    g = torch.Generator().manual_seed(32)
    cfg = {"data_in_exponent_width": 4, "data_in_frac_width": 3}
    x = (torch.randn(4, 8, 16, 32, generator=g) * 3).bfloat16()
    xq = O.minifloat_fake(x, 4, 3)
    assert_bits_equal(mb.silu_minifloat(x.to(DEV), cfg), torch.nn.functional.silu(xq.to(DEV)), "silu_minifloat")
    ref = torch.nn.functional.softmax(xq.to(DEV).float(), dim=-1).to(torch.bfloat16)
    assert_bits_equal(mb.softmax_minifloat(x.to(DEV), cfg), ref, "softmax_minifloat")
    q, k = x[:, :, :, :32], (x * 0.5)
    cos, sin = torch.rand(4, 16, 32, generator=g).bfloat16(), torch.rand(4, 16, 32, generator=g).bfloat16()
    rq, rk = mb.rope_minifloat(q.to(DEV), k.to(DEV), cos.to(DEV), sin.to(DEV), cfg)
    cq, sq = O.minifloat_fake(cos, 4, 3).to(DEV).unsqueeze(1), O.minifloat_fake(sin, 4, 3).to(DEV).unsqueeze(1)
    rot = lambda t: torch.cat((-t[..., 16:], t[..., :16]), dim=-1)  # noqa: E731
    qd = q.to(DEV)
    assert_bits_equal(rq, qd * cq + rot(qd) * sq, "rope_minifloat q")


@pytest.mark.parametrize("cls,cfg,fake", [
    (mb.EmbeddingMXFP, {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3},
     lambda w: O.mxfp_fake(w, 32, 4, 3, 1)),
    (mb.EmbeddingMXInt, {"weight_block_size": 32, "weight_width": 8}, lambda w: O.mxint_fake(w, 32, 8, 1)),
])
def test_embedding_looks_up_then_quantizes(cls, cfg, fake):
    g = torch.Generator().manual_seed(33)
    for dim in (128, 48):  # 48: rows are not whole blocks, the whole table is quantized as in the reference
        emb = cls(1000, dim, config=cfg, padding_idx=0, dtype=torch.bfloat16, device=DEV)
        w = torch.randn(1000, dim, generator=g).bfloat16()
        emb.weight.data.copy_(w)
        idx = torch.randint(0, 1000, (7, 33), generator=g)
        out = emb(idx.to(DEV))
        ref = torch.nn.functional.embedding(idx, fake(w))
        assert_bits_equal(out, ref, f"{cls.__name__} dim {dim}")
    assert cls(10, 32, config={"bypass": True}, device=DEV).bypass


def test_rms_norm_minifloat():
    g = torch.Generator().manual_seed(34)
    qc = {"weight_exponent_width": 4, "weight_frac_width": 3, "data_in_exponent_width": 5, "data_in_frac_width": 2}
    norm = mb.RMSNormMinifloat(256, 1e-6, qc, device=DEV, dtype=torch.bfloat16)
    norm.weight.data.copy_((torch.rand(256, generator=g) + 0.5).bfloat16())
    x = torch.randn(3, 17, 256, generator=g).bfloat16()
    y = norm(x.to(DEV))
    xq = O.minifloat_fake(x, 5, 2).float()
    h = xq * torch.rsqrt(xq.pow(2).mean(-1, keepdim=True) + 1e-6)
    ref = O.minifloat_fake(norm.weight.data.cpu(), 4, 3) * h.to(torch.bfloat16)
    assert y.dtype == torch.bfloat16 and rel_err(y, ref) <= 8e-3  # rsqrt and the mean round differently on the two devices


def test_rope_kernel_equals_the_elementwise_sequence():
    """mxq_rope against torch's own elementwise ops on the same device: bit for bit with tables of the tensor's dtype
    (every product and the sum rounded to it); with fp32 tables and a bf16 tensor both evaluate in fp32 and round once,
    so they agree up to the last fp32 bit before that rounding.  Permuted and batched layouts."""
    from mase_b200 import functional as Fn

    g = torch.Generator().manual_seed(35)
    b, h, s, d = 3, 8, 70, 128
    base = torch.randn(b, s, h, d, generator=g).bfloat16().to(DEV)
    q = base.transpose(1, 2)  # [b, h, s, d] view of [b, s, h, d] memory, as attention code produces it
    cos, sin = torch.rand(b, s, d, generator=g).bfloat16().to(DEV), torch.rand(b, s, d, generator=g).bfloat16().to(DEV)
    rot = lambda t: torch.cat((-t[..., d // 2:], t[..., : d // 2]), dim=-1)  # noqa: E731
    ref = q * cos.unsqueeze(1) + rot(q) * sin.unsqueeze(1)
    out = Fn.rope_apply(q, cos, sin)
    assert out is not None and out.shape == q.shape
    assert_bits_equal(out, ref, "bf16 tables, batched")
    out2 = Fn.rope_apply(q.contiguous(), cos[0], sin[0])
    assert_bits_equal(out2, q * cos[0] + rot(q) * sin[0], "bf16 tables, shared")
    c32, s32 = cos[0].float() * 1.001, sin[0].float() * 0.999
    out3 = Fn.rope_apply(q, c32, s32)
    ref3 = torch.addcmul(q * c32, rot(q), s32).to(torch.bfloat16)
    assert float((out3.float() - ref3.float()).abs().max() / ref3.float().abs().max()) <= 2.0 ** -7
    assert float((out3 != ref3).float().mean()) < 1e-3
    qf = q.float().contiguous()
    outf = Fn.rope_apply(qf, c32, s32)
    assert_bits_equal(outf, qf * c32 + rot(qf) * s32, "fp32")
    # the functional wrappers go through it
    cfg = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    rq, rk = mb.rope_mxfp(q, q * 0.5, cos, sin, cfg)
    cq, sq = mb.mxfp_quantizer(cos, 32, 4, 3), mb.mxfp_quantizer(sin, 32, 4, 3)
    assert_bits_equal(rq, q * cq.unsqueeze(1) + rot(q) * sq.unsqueeze(1), "rope_mxfp q")
    assert Fn.rope_apply(q[..., :24], cos[..., :24], sin[..., :24]) is None  # dim not a multiple of 16: composed ops


def test_softmax_fused_with_its_quantizer():
    """softmax_mxfp / softmax_mxint / softmax_minifloat in one kernel against quantizer + torch softmax on the same
    device: the quantized values are the quantizer's own (bit-exact elsewhere), so the results may differ only by the
    order of the fp32 sum before the one rounding to bf16."""
    g = torch.Generator().manual_seed(36)
    cfp = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    cint = {"data_in_block_size": 32, "data_in_width": 8}
    cmf = {"data_in_exponent_width": 4, "data_in_frac_width": 3}
    for shape in ((2, 4, 48, 64), (3, 1000, 512), (5, 4096), (2, 7, 96)):
        for dtype in (torch.bfloat16, torch.float32):
            x = (torch.randn(*shape, generator=g) * 4).to(dtype).to(DEV)
            for fn, quant in ((mb.softmax_mxfp, lambda t: mb.mxfp_quantizer(t, 32, 4, 3)),
                              (mb.softmax_mxint, lambda t: mb.mxint_quantizer(t, 32, 8)),
                              (mb.softmax_minifloat, lambda t: mb.minifloat_quantizer_sim(t, mb.MinifloatMeta(4, 3, True, "rn")))):
                cfg = cfp if fn is mb.softmax_mxfp else (cint if fn is mb.softmax_mxint else cmf)
                out = fn(x, cfg)
                ref = torch.softmax(quant(x).float(), -1).to(dtype)
                assert out.shape == x.shape and out.dtype == dtype
                tol = 2.0 ** -7 if dtype == torch.bfloat16 else 1e-6
                rel = ((out.float() - ref.float()).abs() / ref.float().clamp_min(1e-30)).max()
                assert float(rel) <= tol, (shape, dtype, fn.__name__, float(rel))
                if dtype == torch.bfloat16:
                    assert float((out != ref).float().mean()) < 5e-3
                assert float((out.float().sum(-1) - 1).abs().max()) < 2e-2
    # a softmax over another dimension, or rows that are not whole blocks, takes the composed route with the same values
    x = torch.randn(4, 64, 48, generator=g).bfloat16().to(DEV)
    ref = torch.softmax(mb.mxfp_quantizer(x, 32, 4, 3).float(), 1).to(torch.bfloat16)
    assert torch.equal(mb.softmax_mxfp(x, cfp, dim=1), ref)
    ref_last = torch.softmax(mb.mxfp_quantizer(x, 32, 4, 3).float(), -1).to(torch.bfloat16)
    assert torch.equal(mb.softmax_mxfp(x, cfp), ref_last)  # 48 columns: blocks straddle rows
