"""`mase_b200.patch` against a real MASE checkout (skipped where none is mounted): the map entries that the quantize
pass reads are replaced, and the pass then builds this package's classes."""

import os
import sys

import pytest
import torch

import mase_b200 as mb
from conftest import mase_chop_dir

CHOP = mase_chop_dir()
pytestmark = pytest.mark.skipif(CHOP is None, reason="no MASE checkout")


@pytest.fixture(scope="module")
def chop_modules():
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_golden

    make_golden.import_reference(CHOP)
    import chop.nn.quantizers as q
    import chop.nn.quantized.modules as qm
    from chop.passes.module.transforms.quantize.quantize import quantize_module_transform_pass

    saved = (dict(q.quantizer_map), dict(qm.quantized_module_map))
    yield q, qm, quantize_module_transform_pass
    q.quantizer_map.update(saved[0])
    qm.quantized_module_map.update(saved[1])


def test_patch_replaces_the_entries_the_pass_reads(chop_modules):
    q, qm, run_pass = chop_modules
    done = mb.patch()
    assert q.quantizer_map["mxfp"] is mb.mxfp_quantizer
    assert q.quantizer_map["mxint"] is mb.mxint_quantizer
    assert q.quantizer_map["block_fp"] is mb.block_fp_quantizer
    assert qm.quantized_module_map["linear_mxfp"] is mb.LinearMXFP
    assert qm.quantized_module_map["linear_mxint"] is mb.LinearMXInt
    assert qm.quantized_module_map["linear_block_fp"] is mb.LinearBlockFP
    assert any("quantized_module_map" in d for d in done)

    # the unmodified pass now instantiates this package's class and calls its load_state_dict, which refuses CPU
    # tensors (there is no CPU fallback); with bypass the swap completes on the CPU
    model = torch.nn.Sequential(torch.nn.Linear(64, 32), torch.nn.ReLU(), torch.nn.Linear(32, 8))
    cfg = {"name": "mxfp", "weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
           "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    with pytest.raises(RuntimeError, match="CUDA"):
        run_pass(model, {"by": "type", "linear": {"config": dict(cfg)}})
    model = torch.nn.Sequential(torch.nn.Linear(64, 32), torch.nn.ReLU(), torch.nn.Linear(32, 8))
    out, _ = run_pass(model, {"by": "type", "linear": {"config": dict(cfg, bypass=True)}})
    assert isinstance(out[0], mb.LinearMXFP) and isinstance(out[2], mb.LinearMXFP)
    assert out[0].config["weight_exponent_width"] == 4


def test_patch_registers_the_llama_wrappers_and_the_gptq_entry(chop_modules):
    """The family wrappers are looked up as quantized_module_map[f"{prefix}_{name}"] and built with
    (config, layer_idx, q_config): the entries are this package's classes and accept that call."""
    from mase_b200 import attention, gptq

    _, qm, _ = chop_modules
    mb.patch()
    assert qm.quantized_module_map["llama_self_attention_mxfp"] is attention.AttentionMXFP
    assert qm.quantized_module_map["llama_self_attention_mxint"] is attention.AttentionMXInt
    assert qm.quantized_module_map["llama_mlp_mxfp"] is attention.GatedMLPMX
    assert qm.quantized_module_map["llama_rms_norm_minifloat"] is mb.RMSNormMinifloat
    assert qm.quantized_module_map["qwen3_self_attention_mxfp"] is attention.Qwen3AttentionMXFP
    assert qm.quantized_module_map["qwen3_mlp_mxint"] is attention.GatedMLPMX

    class Cfg:
        hidden_size, intermediate_size, num_attention_heads, num_key_value_heads = 64, 128, 4, 2
        attention_bias, mlp_bias, attention_dropout, rms_norm_eps = False, False, 0.0, 1e-5

    attn = qm.quantized_module_map["llama_self_attention_mxfp"](config=Cfg(), layer_idx=2, q_config={"rope": {"bypass": True}})
    assert attn.layer_idx == 2 and attn.rope_bypass and not attn.qk_bypass
    assert attn.k_proj.out_features == 32 and attn.num_key_value_groups == 2
    assert set(attn.state_dict()) == {"q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight"}
    mlp = qm.quantized_module_map["llama_mlp_mxint"](config=Cfg(), layer_idx=2, q_config={"bypass": True})
    assert mlp.bypass and mlp.down_proj.in_features == 128
    norm = qm.quantized_module_map["llama_rms_norm_minifloat"](config=Cfg(), layer_idx=2, q_config={"bypass": True})
    assert norm.variance_epsilon == 1e-5 and norm.weight.shape == (64,)
    qwen = qm.quantized_module_map["qwen3_self_attention_mxint"](config=Cfg(), layer_idx=0, q_config={})
    assert set(qwen.state_dict()) == {"q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "q_norm.weight",
                                      "k_norm.weight"}
    assert qwen.q_norm.variance_epsilon == 1e-5 and qwen.q_norm.weight.shape == (16,)
    gp = sys.modules.get("chop.passes.module.transforms.gptq")
    if gp is not None:
        assert gp.run_gptq is gptq.run_gptq
