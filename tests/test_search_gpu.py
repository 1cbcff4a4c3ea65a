"""The calibration-time clipping search kernels against vectors produced by the reference itself and against the
oracle on larger seeded tensors.  Bar: the fake-quantized tensors are bit-identical (NaN blocks included) wherever the
block's winner is not decided by the summation order of an error norm; the share of identical blocks is asserted."""

import pytest
import torch

import mase_b200 as mb
from mase_b200 import quantizers as Q
from conftest import bits_of
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def same_elements(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Bit equality; a NaN equals a NaN (the sign and payload of 0 * inf differ between host and device)."""
    a, b = a.detach().cpu().reshape(-1, 32), b.detach().cpu().reshape(-1, 32)
    assert a.dtype == b.dtype and a.shape == b.shape
    return (bits_of(a) == bits_of(b)) | (torch.isnan(a) & torch.isnan(b))


def same_blocks(a: torch.Tensor, b: torch.Tensor) -> float:
    return float(same_elements(a, b).all(dim=1).float().mean())


def test_mxfp_search_matches_reference_vectors(golden):
    cases = [c for c in golden.cases if c["kind"] == "mxfp_search"]
    assert len(cases) == 6
    for case in cases:
        dt, E, F = case["dtype"], case["E"], case["F"]
        x = golden.tensor(f"mxfp_search/{dt}/x", dt)
        ref = golden.tensor(f"mxfp_search/{dt}/e{E}m{F}/fake", dt)
        meta = mb.MXFPMeta(32, 8, E, F, True, "rn")
        y = mb.mxfp_quantizer_sim(x.to(DEV), 1, meta, quantile_search=True)
        assert same_blocks(y, ref) == 1.0, (dt, E, F, same_blocks(y, ref))
        y2 = mb.mxfp_quantizer(x.to(DEV), 32, E, F, 1, 8, True)  # the autograd wrapper takes the same route
        assert same_blocks(y2, ref) == 1.0


def test_mxint_search_matches_reference_vectors(golden):
    for case in (c for c in golden.cases if c["kind"] == "mxint_search"):
        dt, nbits = case["dtype"], case["bits"]
        x = golden.tensor(f"mxint_search/{dt}/x", dt)
        ref = golden.tensor(f"mxint_search/{dt}/w{nbits}/fake", dt)
        meta = mb.MXIntMeta(block_size=32, scale_bits=8, element_bits=nbits)
        y = mb.mxint_quantizer_sim(x.to(DEV), 1, meta, quantile_search=True)
        assert same_blocks(y, ref) == 1.0, (dt, nbits, same_blocks(y, ref))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_search_kernels_vs_oracle_on_larger_tensors(dtype):
    """[512, 1024] tensors of weight-like values with outliers, zero runs and large magnitudes.  The kernels sum the
    32 squared errors of a block in a butterfly, the host in vector lanes: a block whose two best candidates are
    closer than that rounding may differ, so the bar is 99.9 % identical blocks and every block must be one of the
    eleven candidates of the oracle."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(512, 1024, generator=g) * 0.03
    x[torch.rand(512, 1024, generator=g) < 0.02] *= 25
    x[:64] *= 4000  # scales whose exponent lands in the range where the reference's MXFP measure is non-zero
    x[64:96][torch.rand(32, 1024, generator=g) < 0.7] = 0
    x[100] = 0
    x = x.to(dtype)
    xd = x.to(DEV)
    for nbits in (8, 4):
        meta = mb.MXIntMeta(block_size=32, scale_bits=8, element_bits=nbits)
        y, choice = Q.mxint_clip_search(xd, meta)
        ref, ref_choice = O.mxint_clip_search(x, 32, nbits, 1)
        share = same_blocks(y, ref)
        assert share >= 0.999, ("mxint", nbits, share)
        assert float((choice.cpu().long() == ref_choice).float().mean()) >= 0.999
    for E, F in ((4, 3), (2, 1)):
        meta = mb.MXFPMeta(32, 8, E, F, True, "rn")
        y = mb.mxfp_quantizer_sim(xd, 1, meta, quantile_search=True)
        ref, _ = O.mxfp_clip_search(x, 32, E, F, 1)
        share = same_blocks(y, ref)
        assert share >= 0.999, ("mxfp", E, F, share)
        # a forced candidate is the oracle's extraction at that quantile, exactly
        for i in (0, 3, 10):
            yc, _, metric = Q.mxfp_clip_search(xd.view(-1), meta, candidate=i, want_metric=True)
            sc, co = O.mxfp_extract(x.reshape(-1), 32, E, F, O.SEARCH_PERCENTILES[i])
            assert same_blocks(yc, O.mxfp_compose(sc, co, E, F, dtype)) == 1.0, (E, F, i)
            assert same_blocks(metric, O.mxfp_search_metric(sc, co, F, dtype)) == 1.0, (E, F, i)


def test_search_with_blocks_along_another_dimension_and_with_activations(golden):
    """Forms that run as one launch per candidate plus tensor operations: blocks along dim 0 and the
    activation-weighted error."""
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(64, 96, generator=g) * 300).bfloat16()
    meta = mb.MXFPMeta(32, 8, 4, 3, True, "rn")
    y = mb.mxfp_quantizer_sim(x.to(DEV), 0, meta, quantile_search=True)
    ref, _ = O.mxfp_clip_search(x, 32, 4, 3, 0)
    assert y.shape == x.shape and same_blocks(y.t().contiguous(), ref.t().contiguous()) >= 0.98
    act = torch.randn(4, 6, 32, generator=g).bfloat16()
    xw = (torch.randn(16, 128, generator=g) * 300).bfloat16()
    ya = mb.mxfp_quantizer_sim(xw.to(DEV), 1, meta, act_tensor=act.to(DEV), quantile_search=True, cali_batch_size=2)
    # every block is one of the eleven candidates
    cands = torch.stack([O.mxfp_compose(*O.mxfp_extract(xw.reshape(-1), 32, 4, 3, p), 4, 3, torch.bfloat16).view(-1, 32)
                         for p in O.SEARCH_PERCENTILES])
    got = ya.cpu().reshape(1, -1, 32)
    hit = ((bits_of(cands) == bits_of(got)) | (torch.isnan(cands) & torch.isnan(got))).all(dim=2).any(dim=0)
    assert bool(hit.all())


def test_linear_layers_quantize_their_weight_through_the_search(golden):
    cfg = {"weight_block_size": 32, "weight_width": 4, "data_in_block_size": 32, "data_in_width": 8, "clip_search": True}
    layer = mb.LinearMXInt(128, 48, bias=False, device=DEV, dtype=torch.bfloat16, config=cfg)
    w = golden.tensor("mxint_search/bf16/x", "bf16")
    layer.load_state_dict({"weight": w.to(DEV)}, strict=False)
    assert same_blocks(layer.weight.data, golden.tensor("mxint_search/bf16/w4/fake", "bf16")) == 1.0
