"""The CPU oracle against vectors produced by the MASE reference itself (tests/golden/make_golden.py)."""

import pytest
import torch

from conftest import assert_bits_equal, mase_chop_dir
from oracle import mx_oracle as O


def _cases(golden, kind):
    return [c for c in golden.cases if c["kind"] == kind]


def test_fixture_inventory(golden):
    kinds = {c["kind"] for c in golden.cases}
    assert kinds == {"mxint", "mxfp", "minifloat", "bfp", "bfp_tiles", "blockdim", "linear", "mxint_search",
                     "mxfp_search", "gptq", "attention", "mlp",
                     "attention_qwen3"}
    assert len(golden.cases) >= 200


def test_mxint_oracle_matches_reference(golden):
    for c in _cases(golden, "mxint"):
        x = golden.tensor(c["input"] + "/x")
        sc, m = O.mxint_extract(x.flatten(), c["block"], c["bits"])
        assert_bits_equal(sc, golden.tensor(c["tag"] + "/scale"), c["tag"] + " scale")
        assert_bits_equal(m, golden.tensor(c["tag"] + "/mant"), c["tag"] + " mant")
        assert_bits_equal(O.mxint_fake(x, c["block"], c["bits"]), golden.tensor(c["tag"] + "/fake"), c["tag"] + " fake")


def test_mxfp_oracle_matches_reference(golden):
    for c in _cases(golden, "mxfp"):
        x = golden.tensor(c["input"] + "/x")
        sc, co = O.mxfp_extract(x.flatten(), c["block"], c["E"], c["F"])
        assert_bits_equal(sc, golden.tensor(c["tag"] + "/scale"), c["tag"] + " scale")
        assert_bits_equal(co, golden.tensor(c["tag"] + "/codes"), c["tag"] + " codes")
        assert_bits_equal(O.mxfp_fake(x, c["block"], c["E"], c["F"]), golden.tensor(c["tag"] + "/fake"), c["tag"] + " fake")


def test_minifloat_oracle_matches_reference(golden):
    for c in _cases(golden, "minifloat"):
        x = golden.tensor(c["input"] + "/x")
        assert_bits_equal(O.minifloat_fake(x, c["E"], c["F"]), golden.tensor(c["tag"] + "/fake"), c["tag"])


def test_bfp_oracle_matches_reference(golden):
    for c in _cases(golden, "bfp"):
        x = golden.tensor(c["input"] + "/x")
        y = O.bfp_fake_rows(x, c["width"], c["exponent_width"], c["exponent_bias"], c["block_size"][-1])
        assert_bits_equal(y, golden.tensor(c["tag"] + "/fake"), c["tag"])


def test_bfp_tiles_oracle_matches_reference(golden):
    from mase_b200.quantizers import _bfp_tile

    for c in _cases(golden, "bfp_tiles"):
        x = golden.tensor(f"bfp_tiles/{c['name']}/{c['dtype']}/x")
        bh, bw = _bfp_tile(tuple(c["shape"]), c["block_size"], c["skip_first_dim"])
        for width in c["widths"]:
            ref = golden.tensor(f"bfp_tiles/{c['name']}/{c['dtype']}/w{width}/fake")
            assert_bits_equal(O.bfp_fake_tiles(x, width, 8, 127, bh, bw), ref, f"{c['name']} w{width}", signed_zero=False)


def test_block_dim_oracle_matches_reference(golden):
    for c in _cases(golden, "blockdim"):
        dt, bd, blk = c["dtype"], c["block_dim"], c["block"]
        x = golden.tensor(f"blockdim/{dt}/x")
        assert_bits_equal(O.mxint_fake(x, blk, 8, bd).contiguous(), golden.tensor(f"blockdim/{dt}/mxint_d{bd}/fake"), f"mxint d{bd}")
        assert_bits_equal(O.mxfp_fake(x, blk, 4, 3, bd).contiguous(), golden.tensor(f"blockdim/{dt}/mxfp_d{bd}/fake"), f"mxfp d{bd}")


def test_known_answers_e4m3():
    """The encoder quirks, as values at block scale 2**0 (block maximum 256 -> shared exponent 0)."""
    x = torch.zeros(32)
    vals = [256.0, 1.97, 3.97, 7.9, 480.0, 500.0, 2.0**-7, 1.5 * 2.0**-7]
    x[: len(vals)] = torch.tensor(vals)
    sc, co = O.mxfp_extract(x, 32, 4, 3)
    assert int(sc) == 127
    assert co[0, : len(vals)].tolist() == [0x78, 0x38, 0x48, 0x48, 0x7F, 0x78, 0x00, 0x06]
    y = O.mxfp_fake(x, 32, 4, 3)
    assert y[: len(vals)].tolist() == [256.0, 1.0, 4.0, 4.0, 480.0, 256.0, 0.0, 1.5 * 2.0**-7]


def test_known_answers_mxint_saturation():
    x = torch.zeros(32)
    x[:3] = torch.tensor([1.0, -1.0, 0.5])
    sc, m = O.mxint_extract(x, 32, 8)
    assert int(sc) == 127 and m[0, :3].tolist() == [127.0, -128.0, 64.0]
    xb = torch.zeros(32, dtype=torch.bfloat16)
    xb[0] = 16.125  # log2(16.125) = 4.011 rounds to 4.0 in bf16: the exponent stays 4 and the maximum clips
    sc, m = O.mxint_extract(xb, 32, 8)
    assert int(sc) == 131 and float(m[0, 0]) == 127.0
    sc, m = O.mxint_extract(xb.float(), 32, 8)  # in fp32 the logarithm is not an integer: exponent 5
    assert int(sc) == 132 and float(m[0, 0]) == 64.0


def test_linear_oracle_matches_reference(golden):
    """Weights quantized like load_state_dict does; forward vs the reference's own output."""
    for c in _cases(golden, "linear"):
        dt, tag, cfg = c["dtype"], c["tag"], c["config"]
        x = golden.tensor(f"linear/{dt}/x")
        w = golden.tensor(f"linear/{dt}/w")
        b = golden.tensor(f"linear/{dt}/b")
        w_ref, b_ref, y_ref = golden.tensor(tag + "/w_q"), golden.tensor(tag + "/b_q"), golden.tensor(tag + "/y")
        if c["cls"] == "LinearMXFP":
            wq = O.mxfp_fake(w, cfg["weight_block_size"], cfg["weight_exponent_width"], cfg["weight_frac_width"], 1)
            bq = b
            if "bias_block_size" in cfg:
                bq = O.mxfp_fake(b, cfg["bias_block_size"], cfg["bias_exponent_width"], cfg["bias_frac_width"], 0)
            y = O.linear_mxfp(x, wq, bq, cfg)
        elif c["cls"] == "LinearMXInt":
            wq, bq = O.mxint_fake(w, cfg["weight_block_size"], cfg["weight_width"], 1), b
            y = O.linear_mxint(x, wq, bq, cfg)
        else:
            wq, bq = w, b
            y = O.linear_block_fp(x, w, b, cfg)
        if c["cls"] != "LinearBlockFP":
            assert_bits_equal(wq.contiguous(), w_ref, tag + " w_q")
            assert_bits_equal(bq.contiguous(), b_ref, tag + " b_q")
        # the reference output is in x.dtype from the library GEMM; the oracle accumulates in fp32
        err = (y - y_ref.float()).abs().max() / y_ref.float().abs().max()
        tol = 1e-5 if dt == "fp32" else 8e-3  # bf16 output rounding: half an ulp = 2**-9 relative
        assert float(err) <= tol, f"{tag}: {float(err)}"


@pytest.mark.skipif(mase_chop_dir() is None, reason="no MASE checkout")
def test_oracle_vs_live_reference_random():
    """Where a MASE checkout is present, compare on fresh random data as well (larger than the fixtures)."""
    import sys, os
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_golden

    make_golden.import_reference(mase_chop_dir())
    import chop.nn.quantizers as q

    g = torch.Generator().manual_seed(2024)
    x = torch.randn(256, 512, generator=g) * torch.exp2(torch.randint(-20, 20, (256, 1), generator=g).float())
    for dt in (torch.float32, torch.bfloat16):
        xd = x.to(dt)
        assert_bits_equal(O.mxint_fake(xd, 32, 8), q.mxint_quantizer(xd, 32, 8), "mxint")
        assert_bits_equal(O.mxfp_fake(xd, 32, 4, 3), q.mxfp_quantizer(xd, 32, 4, 3), "mxfp e4m3")
        assert_bits_equal(O.mxfp_fake(xd, 32, 2, 1), q.mxfp_quantizer(xd, 32, 2, 1), "mxfp e2m1")
        assert_bits_equal(O.bfp_fake_rows(xd, 8, 8, 127, 32), q.block_fp_quantizer(xd, 8, 8, 127, [1, 32], True), "bfp")


def test_clip_search_oracles_match_reference(golden):
    """The clipping searches of both formats, bit for bit (NaN blocks of zero-quantile candidates included)."""
    for c in _cases(golden, "mxfp_search"):
        dt, E, F = c["dtype"], c["E"], c["F"]
        x = golden.tensor(f"mxfp_search/{dt}/x", dt)
        y, chosen = O.mxfp_clip_search(x, 32, E, F, 1)
        assert_bits_equal(y.contiguous(), golden.tensor(f"mxfp_search/{dt}/e{E}m{F}/fake", dt), f"mxfp search {dt} E{E}M{F}")
        assert int(chosen.max()) > 0  # the large-magnitude rows do leave the first candidate
    for c in _cases(golden, "mxint_search"):
        dt, nbits = c["dtype"], c["bits"]
        x = golden.tensor(f"mxint_search/{dt}/x", dt)
        y, _ = O.mxint_clip_search(x, 32, nbits, 1)
        assert_bits_equal(y.contiguous(), golden.tensor(f"mxint_search/{dt}/w{nbits}/fake", dt), f"mxint search {dt} w{nbits}")


def test_gptq_oracle_matches_reference(golden):
    """Hessian accumulation and the block-wise GPTQ sweep with MXFP4 / MXINT4 inner quantizers, with and without
    the clipping search, against the reference's own output on one 128 -> 48 layer."""
    w, acts = golden.tensor("gptq/w"), golden.tensor("gptq/acts")
    H = O.gptq_hessian([acts[i : i + 1] for i in range(acts.shape[0])])
    inner = {
        ("mxfp", False): lambda W1: O.mxfp_fake(W1, 32, 2, 1, 1),
        ("mxfp", True): lambda W1: O.mxfp_clip_search(W1, 32, 2, 1, 1)[0],
        ("mxint", False): lambda W1: O.mxint_fake(W1, 32, 4, 1),
        ("mxint", True): lambda W1: O.mxint_clip_search(W1, 32, 4, 1)[0],
    }
    for c in _cases(golden, "gptq"):
        tag = f"gptq/{c['format']}/search{int(c['search'])}"
        assert_bits_equal(H, golden.tensor(tag + "/hessian"), tag + " hessian")
        Q = O.gptq_quantize(w, H, inner[(c["format"], c["search"])], 32)
        assert_bits_equal(Q, golden.tensor(tag + "/q"), tag + " q")


def test_attention_and_mlp_oracles_match_reference(golden):
    """The attention block (MXFP and MXINT operands, minifloat rotary tables and softmax input, with and without a
    key/value cache) and the gated MLP with a minifloat SiLU input against the reference's own classes, bit for bit."""
    fp = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    it = {"data_in_block_size": 32, "data_in_width": 8}
    mini = {"data_in_exponent_width": 5, "data_in_frac_width": 10}
    qc = {"mxfp": {"qk_matmul": fp, "av_matmul": fp, "rope": mini, "softmax": mini, "kv_cache": fp},
          "mxint": {"qk_matmul": it, "av_matmul": it, "rope": mini, "softmax": mini, "kv_cache": it}}
    for c in _cases(golden, "attention"):
        dt, fmt = c["dtype"], c["format"]
        t = lambda n: golden.tensor(f"attention/{dt}/{n}", dt)  # noqa: E731
        w = {n: t(n) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight")}
        out, probs = O.attention_mx(t("hidden"), w, t("cos"), t("sin"), t("mask"), fmt, qc[fmt], 4, 2, c["cached"])
        tag = f"attention/{dt}/{fmt}/cache{int(c['cached'])}"
        assert_bits_equal(out, golden.tensor(tag + "/out", dt), tag + " out")
        assert_bits_equal(probs, golden.tensor(tag + "/probs", dt), tag + " probs")
    for c in _cases(golden, "attention_qwen3"):
        dt = c["dtype"]
        t = lambda n: golden.tensor(f"attention/{dt}/{n}", dt)  # noqa: E731
        w = {n: t(n) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight")}
        w.update({n: t("qwen3/" + n) for n in ("q_norm.weight", "k_norm.weight")})
        out, probs = O.attention_mx(t("hidden"), w, t("cos"), t("sin"), t("mask"), "mxfp", qc["mxfp"], 4, 2, False, c["eps"])
        assert_bits_equal(out, t("qwen3/out"), f"qwen3 {dt} out")
        assert_bits_equal(probs, t("qwen3/probs"), f"qwen3 {dt} probs")
    for c in _cases(golden, "mlp"):
        dt = c["dtype"]
        t = lambda n: golden.tensor(f"mlp/{dt}/{n}", dt)  # noqa: E731
        out = O.gated_mlp_minifloat(golden.tensor(f"attention/{dt}/hidden", dt), t("gate_proj.weight"), t("up_proj.weight"),
                                    t("down_proj.weight"), mini)
        assert_bits_equal(out, t("out"), f"mlp {dt}")
