"""Mixed-precision decoder layer (MXINT8 attention projections, MXFP4-weight / MXFP8-activation FFN) against the same
layer built from the oracle's Linear restatements on the CPU."""

import pytest
import torch

import mase_b200 as mb
from mase_b200 import gemm, synthetic
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class OracleLinear(torch.nn.Module):
    """CPU stand-in with the reference's semantics: weight quantized at load, activations per call, fp32 GEMM."""

    def __init__(self, k, n, kind, cfg):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.empty(n, k, dtype=torch.bfloat16), requires_grad=False)
        self.kind, self.cfg = kind, cfg

    def load_state_dict(self, state, strict=True):
        w = state["weight"]
        if self.kind == "mxint":
            w = O.mxint_fake(w, self.cfg["weight_block_size"], self.cfg["weight_width"], 1)
        else:
            w = O.mxfp_fake(w, self.cfg["weight_block_size"], self.cfg["weight_exponent_width"],
                            self.cfg["weight_frac_width"], 1)
        self.weight.data.copy_(w)

    def forward(self, x):
        fn = O.linear_mxint if self.kind == "mxint" else O.linear_mxfp
        return fn(x, self.weight.data, None, self.cfg).to(x.dtype)


@pytest.mark.parametrize("shape", [(512, 4, 1376, 2, 64), (1024, 8, 2752, 1, 96)])
def test_decoder_layer_matches_oracle_layer(shape):
    hidden, heads, ffn, batch, seq = shape
    g = torch.Generator().manual_seed(33)
    x = torch.randn(batch, seq, hidden, generator=g).bfloat16()

    ours = synthetic.quantize_decoder_layer(
        synthetic.DecoderLayer(hidden, heads, ffn).to(DEV),
        lambda k, n: mb.LinearMXInt(k, n, bias=False, device=DEV, dtype=torch.bfloat16, config=dict(synthetic.MXINT8_LINEAR)),
        lambda k, n: mb.LinearMXFP(k, n, bias=False, device=DEV, dtype=torch.bfloat16,
                                   config=dict(synthetic.MXFP4W_MXFP8A_LINEAR)))
    ref = synthetic.quantize_decoder_layer(
        synthetic.DecoderLayer(hidden, heads, ffn),
        lambda k, n: OracleLinear(k, n, "mxint", synthetic.MXINT8_LINEAR),
        lambda k, n: OracleLinear(k, n, "mxfp", synthetic.MXFP4W_MXFP8A_LINEAR))
    assert isinstance(ours.q_proj, mb.LinearMXInt) and isinstance(ours.down_proj, mb.LinearMXFP)
    # weights quantized at load are bit-identical
    for name in synthetic.DecoderLayer.ATTENTION + synthetic.DecoderLayer.FFN:
        assert torch.equal(getattr(ours, name).weight.data.cpu(), getattr(ref, name).weight.data), name
    with torch.no_grad():
        y = ours(x.to(DEV))
        gemm.check_status()
        y_ref = ref(x)
    assert y.shape == x.shape and y.dtype == torch.bfloat16
    err = (y.float().cpu() - y_ref.float()).abs().max() / y_ref.float().abs().max()
    # bf16 activations between the unquantized stages (attention, SiLU) differ in rounding between the two devices
    assert err <= 2e-2, err
