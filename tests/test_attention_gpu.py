"""The quantized attention block and gated MLP against outputs of the reference's own classes
(LlamaAttentionMXFP / LlamaAttentionMXInt / LlamaMLPMXFP run on the CPU when the fixtures were made) and against the
oracle on a larger block.  The projections are plain Linear layers (torch), everything between them runs on this
package's kernels.  Bars: fp32 outputs within 2e-4 of the largest value, bf16 within 2e-2 (a chain of five bf16
roundings whose inputs differ in the last bit between host and device); at least 97 % of the quantized probabilities
identical and none further than a quarter of its block's maximum (4e-3 for blocks of small probabilities)."""

import pytest
import torch

from mase_b200 import attention, gemm
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

FP = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
INT = {"data_in_block_size": 32, "data_in_width": 8}
MINI = {"data_in_exponent_width": 5, "data_in_frac_width": 10}
QCFG = {"mxfp": {"qk_matmul": FP, "av_matmul": FP, "rope": MINI, "softmax": MINI, "kv_cache": FP},
        "mxint": {"qk_matmul": INT, "av_matmul": INT, "rope": MINI, "softmax": MINI, "kv_cache": INT}}
CLS = {"mxfp": attention.AttentionMXFP, "mxint": attention.AttentionMXInt}
WEIGHTS = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight")


class ListCache:
    """The part of a key/value cache the block uses: update() appends along the sequence and returns everything."""

    def __init__(self):
        self.k, self.v = {}, {}

    def update(self, k, v, layer_idx, cache_kwargs=None):
        self.k[layer_idx] = k if layer_idx not in self.k else torch.cat([self.k[layer_idx], k], dim=-2)
        self.v[layer_idx] = v if layer_idx not in self.v else torch.cat([self.v[layer_idx], v], dim=-2)
        return self.k[layer_idx], self.v[layer_idx]


def check(out, probs, ref_out, ref_probs, dt, what, tol=None, elementwise=True):
    tol = tol or (2e-4 if dt == "fp32" else 2e-2)
    diff = out.float().cpu() - ref_out.float()
    err = float(diff.abs().max() / ref_out.float().abs().max())
    assert err <= tol, (what, err)
    rms = float(diff.pow(2).mean().sqrt() / ref_out.float().pow(2).mean().sqrt())
    assert rms <= tol / 4, (what, rms)
    p, r = probs.float().cpu(), ref_probs.float()
    assert float((p == r).float().mean()) >= 0.97, (what, float((p == r).float().mean()))
    # a quarter of the block maximum (two steps of the coarsest grid a block can land on when its maximum sits next to
    # a power of two and the shared exponent differs by one between host and device), or 4e-3 of the row's total where
    # that is larger: a bf16 score of magnitude 30 has a last bit of 0.125, which moves a small probability by 13 %
    step = (r.reshape(-1, 32).abs().amax(dim=1, keepdim=True) / 4).clamp_min(4e-3)
    if elementwise:
        assert bool(((p - r).reshape(-1, 32).abs() <= step + 1e-12).all()), what


def test_attention_matches_reference_vectors(golden):
    cases = [c for c in golden.cases if c["kind"] == "attention"]
    assert len(cases) == 8
    for c in cases:
        dt, fmt, cached = c["dtype"], c["format"], c["cached"]
        t = lambda n: golden.tensor(f"attention/{dt}/{n}", dt).to(DEV)  # noqa: E731
        dtype = torch.float32 if dt == "fp32" else torch.bfloat16
        block = CLS[fmt](None, 0, QCFG[fmt], hidden_size=128, num_heads=4, num_kv_heads=2, device=DEV, dtype=dtype)
        block.load_state_dict({n: t(n) for n in WEIGHTS})
        with torch.no_grad():
            out, probs = block(t("hidden"), (t("cos"), t("sin")), t("mask"), past_key_value=ListCache() if cached else None,
                               cache_position=torch.arange(64, device=DEV))
        gemm.check_status()
        tag = f"attention/{dt}/{fmt}/cache{int(cached)}"
        check(out, probs, golden.tensor(tag + "/out", dt), golden.tensor(tag + "/probs", dt), dt, tag)


def test_qwen3_variant_matches_reference_vectors(golden):
    """The same block with RMS norms over the head dimension of queries and keys (Qwen3AttentionMXFP)."""
    for c in (c for c in golden.cases if c["kind"] == "attention_qwen3"):
        dt = c["dtype"]
        t = lambda n: golden.tensor(f"attention/{dt}/{n}", dt).to(DEV)  # noqa: E731
        dtype = torch.float32 if dt == "fp32" else torch.bfloat16
        block = attention.Qwen3AttentionMXFP(None, 0, QCFG["mxfp"], hidden_size=128, num_heads=4, num_kv_heads=2,
                                             rms_norm_eps=c["eps"], device=DEV, dtype=dtype)
        state = {n: t(n) for n in WEIGHTS}
        state.update({n: t("qwen3/" + n) for n in ("q_norm.weight", "k_norm.weight")})
        block.load_state_dict(state)
        with torch.no_grad():
            out, probs = block(t("hidden"), (t("cos"), t("sin")), t("mask"))
        gemm.check_status()
        check(out, probs, golden.tensor(f"attention/{dt}/qwen3/out", dt), golden.tensor(f"attention/{dt}/qwen3/probs", dt),
              dt, f"qwen3 {dt}")
        again = attention.Qwen3AttentionMXFP.from_attention(block, QCFG["mxfp"])
        assert again.q_norm.variance_epsilon == c["eps"] and torch.equal(again.k_norm.weight, block.k_norm.weight)


def test_gated_mlp_matches_reference_vectors(golden):
    for c in (c for c in golden.cases if c["kind"] == "mlp"):
        dt = c["dtype"]
        dtype = torch.float32 if dt == "fp32" else torch.bfloat16
        mlp = attention.GatedMLPMX(None, 0, MINI, hidden_size=128, intermediate_size=256, device=DEV, dtype=dtype)
        mlp.load_state_dict({n: golden.tensor(f"mlp/{dt}/{n}", dt).to(DEV)
                             for n in ("gate_proj.weight", "up_proj.weight", "down_proj.weight")})
        with torch.no_grad():
            out = mlp(golden.tensor(f"attention/{dt}/hidden", dt).to(DEV))
        ref = golden.tensor(f"mlp/{dt}/out", dt)
        err = float((out.float().cpu() - ref.float()).abs().max() / ref.float().abs().max())
        assert err <= (2e-4 if dt == "fp32" else 2e-2), (dt, err)


def test_larger_block_vs_oracle_and_construction_from_a_config():
    """hidden 512, 8 heads of 64 over 4 key/value heads, 2 x 160 tokens (a key length that is not a multiple of the
    GEMM tile), bf16; built the way the quantize pass builds it (config object, layer index, q_config) and through
    from_attention."""
    class Cfg:
        hidden_size, num_attention_heads, num_key_value_heads, attention_bias, attention_dropout = 512, 8, 4, False, 0.0

    g = torch.Generator().manual_seed(8)
    B, S = 2, 160
    hidden = torch.randn(B, S, 512, generator=g).bfloat16()
    w = {n: (torch.randn(shape, generator=g) * 0.04).bfloat16() for n, shape in
         zip(WEIGHTS, ((512, 512), (256, 512), (256, 512), (512, 512)))}
    pos = torch.arange(S, dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))
    ang = torch.cat([pos[:, None] * inv[None], pos[:, None] * inv[None]], dim=-1)
    cos, sin = ang.cos()[None].expand(B, S, 64).bfloat16(), ang.sin()[None].expand(B, S, 64).bfloat16()
    mask = torch.zeros(B, 1, S, S, dtype=torch.bfloat16).masked_fill(
        torch.ones(S, S, dtype=torch.bool).triu(1)[None, None], torch.finfo(torch.bfloat16).min)
    block = attention.AttentionMXFP(Cfg(), 3, QCFG["mxfp"]).to(device=DEV, dtype=torch.bfloat16)
    assert block.layer_idx == 3 and block.head_dim == 64 and block.num_key_value_groups == 2
    block.load_state_dict(w)
    again = attention.AttentionMXFP.from_attention(block, QCFG["mxfp"])
    with torch.no_grad():
        out, probs = block(hidden.to(DEV), (cos.to(DEV), sin.to(DEV)), mask.to(DEV))
        out2, _ = again(hidden.to(DEV), (cos.to(DEV), sin.to(DEV)), mask.to(DEV))
    gemm.check_status()
    assert torch.equal(out, out2)
    ref_out, ref_probs = O.attention_mx(hidden, w, cos, sin, mask, "mxfp", QCFG["mxfp"], 8, 4, False)
    # 160 keys per row: more probabilities sit on a rounding boundary of their block than in the small fixtures, and
    # one that flips moves an output by a bf16 step or two
    # No element-wise bound here: the reference's element codec drops the carry of a fraction that rounds up out of a
    # binade with an odd exponent code, so a probability a last bit below such a boundary comes out at half the value
    # of one a last bit above it (37 of 409,600 probabilities differ, every one by that factor of two; the device
    # quantizer reproduces the oracle exactly on the device's own unquantized probabilities).
    check(out, probs, ref_out, ref_probs, "bf16", "larger block", tol=4e-2, elementwise=False)
    assert float((probs.float().cpu() == ref_probs.float()).float().mean()) >= 0.999


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(3, 70, 40, 96), (16, 128, 256, 64), (5, 200, 24, 8), (2, 33, 130, 36)])
def test_batched_product_vs_fp64(dtype, shape):
    """The batched GEMM: ragged M, N and K against an fp64 product; matrices at the end of the batch must not leak
    into their neighbours (tiles at a matrix edge)."""
    B, M, N, K = shape
    g = torch.Generator().manual_seed(sum(shape))
    a = torch.randn(B, M, K, generator=g).to(dtype)
    b = torch.randn(B, N, K, generator=g).to(dtype)
    ref = torch.einsum("bmk,bnk->bmn", a.double(), b.double())
    out = gemm.batched_product(a.to(DEV), b.to(DEV), torch.float32, fp32_exact=False)
    gemm.check_status()
    err = float((out.double().cpu() - ref).abs().max() / ref.abs().max())
    assert err <= 2e-5, (shape, dtype, err)
    # the same values as one launch per matrix
    out_same = gemm.batched_product(a.to(DEV), b.to(DEV), dtype, fp32_exact=False)
    loop = torch.stack([gemm.linear_forward(a[i].to(DEV), b[i].to(DEV), None, dtype) for i in range(B)])
    tol = 2e-5 if dtype == torch.float32 else 1e-2  # bf16: the two routes may round an output differently
    assert float((out_same.float() - loop.float()).abs().max()) <= tol * float(ref.abs().max())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("cols", [32, 160, 512, 2048])
def test_fused_attention_softmax_vs_composed_oracle(dtype, cols):
    """mxq_attention_softmax against the separate operations on the CPU: scale, mask, minifloat / MXFP / MXINT / no
    input quantizer, fp32 softmax, MXFP / MXINT / no quantizer of the probabilities.  The exponentials differ in the
    last bit between device and host, so probabilities are compared to 2e-3 of the row maximum before the output
    quantizer and by the share of identical values after it."""
    from mase_b200 import functional as F

    g = torch.Generator().manual_seed(cols)
    B, H, S = 2, 3, 8
    scores = (torch.randn(B, H, S, cols, generator=g) * 6).to(dtype)
    mask = torch.zeros(B, 1, S, cols + 32, dtype=dtype)
    mask[..., cols // 2:] = torch.finfo(dtype).min
    mask[:, :, ::2, : cols // 2 + 7] = 0  # ragged visible lengths
    fp = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    it = {"data_in_block_size": 32, "data_in_width": 8}
    mini = {"data_in_exponent_width": 5, "data_in_frac_width": 10}
    quant = {"mxfp": lambda t: O.mxfp_fake(t, 32, 4, 3, -1), "mxint": lambda t: O.mxint_fake(t, 32, 8, -1),
             "minifloat": lambda t: O.minifloat_fake(t, 5, 10), None: lambda t: t}
    cfgs = {"mxfp": fp, "mxint": it, "minifloat": mini, None: None}
    for in_fmt, out_fmt, scale, use_mask in (("minifloat", "mxfp", 0.125, True), ("minifloat", "mxint", 0.3, True),
                                             (None, None, None, False), ("mxfp", None, 0.5, True),
                                             ("mxint", "mxfp", None, False), ("minifloat", None, 0.125, False)):
        got = F.attention_softmax(scores.to(DEV), scale, mask.to(DEV) if use_mask else None, in_fmt, cfgs[in_fmt],
                                  out_fmt, cfgs[out_fmt])
        assert got is not None, (in_fmt, out_fmt)
        s = scores if scale is None else scores * scale
        if use_mask:
            s = s + mask[:, :, :, :cols]
        p = torch.softmax(quant[in_fmt](s).to(torch.float32), dim=-1).to(dtype)
        if out_fmt is None:
            err = float((got.float().cpu() - p.float()).abs().max())
            assert err <= 2e-3 * float(p.float().max()) + (0.0 if dtype == torch.float32 else 4e-3), (in_fmt, cols, err)
        else:
            ref = quant[out_fmt](p)
            same = float((got.cpu() == ref).float().mean())
            assert same >= 0.97, (in_fmt, out_fmt, cols, same)
    # shapes the kernel does not take are declined, not mangled
    assert F.attention_softmax(scores[..., :20].to(DEV), None, None, None, None, None, None) is None


@pytest.mark.parametrize("fmt", ["mxfp", "mxint"])
def test_decode_step_with_a_cache_matches_the_last_row_of_a_prefill(fmt):
    """One query row against 96 cached keys (the batched products with M = 1, the softmax kernel with one row per
    head): the output must be that of the last token of a 96-token prefill through the same cached path."""
    g = torch.Generator().manual_seed(12)
    B, S, HID = 2, 96, 256
    block = CLS[fmt](None, 0, QCFG[fmt], hidden_size=HID, num_heads=4, num_kv_heads=2, device=DEV, dtype=torch.bfloat16)
    for prm in block.parameters():
        prm.data.copy_((torch.randn(prm.shape, generator=g) * 0.05).to(DEV))
    hidden = torch.randn(B, S, HID, generator=g).bfloat16().to(DEV)
    pos = torch.arange(S, dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))
    ang = torch.cat([pos[:, None] * inv[None], pos[:, None] * inv[None]], dim=-1)
    cos, sin = ang.cos()[None].expand(B, S, 64).bfloat16().to(DEV), ang.sin()[None].expand(B, S, 64).bfloat16().to(DEV)
    causal = torch.zeros(B, 1, S, S, dtype=torch.bfloat16).masked_fill(
        torch.ones(S, S, dtype=torch.bool).triu(1)[None, None], torch.finfo(torch.bfloat16).min).to(DEV)
    with torch.no_grad():
        full, _ = block(hidden, (cos, sin), causal, past_key_value=ListCache())
        # fill the cache with the first 95 tokens through a twin whose probabilities stay unquantized (95 keys are
        # not whole blocks of 32, which the reference's quantizer rejects as well); keys and values are cached alike
        cache = ListCache()
        twin = CLS[fmt](None, 0, dict(QCFG[fmt], av_matmul={"bypass": True}), hidden_size=HID, num_heads=4, num_kv_heads=2,
                        device=DEV, dtype=torch.bfloat16)
        twin.load_state_dict(block.state_dict())
        twin(hidden[:, : S - 1], (cos[:, : S - 1], sin[:, : S - 1]), causal[:, :, : S - 1, : S - 1], past_key_value=cache)
        step, probs = block(hidden[:, S - 1:], (cos[:, S - 1:], sin[:, S - 1:]),
                            torch.zeros(B, 1, 1, S, dtype=torch.bfloat16, device=DEV), past_key_value=cache)
    gemm.check_status()
    assert step.shape == (B, 1, HID) and probs.shape == (B, 4, 1, S)
    ref = full[:, S - 1:].float()
    err = float((step.float() - ref).abs().max() / ref.abs().max())
    assert err <= 2e-2, (fmt, err)
