"""Regenerates the golden fixtures in this directory by running the MASE reference itself on the CPU.

Usage (only where a MASE checkout is available; the fixtures are committed, so tests never need it):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/mase/src/chop

The reference package cannot be imported whole in a minimal environment (its top-level `__init__`
pulls plotting and training dependencies), so the script registers empty parent packages that point at
the checkout and imports only the quantizer and quantized-module files.

Every fixture stores the *bit patterns* of inputs and outputs (float tensors as integer views) so that
comparisons are exact, including signed zeros and NaN payload-free NaNs.
"""

from __future__ import annotations

import importlib
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(root: str):
    for name, path in [
        ("chop", root),
        ("chop.nn", root + "/nn"),
        ("chop.passes", root + "/passes"),
        ("chop.passes.module", root + "/passes/module"),
        ("chop.passes.module.transforms", root + "/passes/module/transforms"),
    ]:
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m
    # names that newer `transformers` releases dropped but the reference still imports
    importlib.import_module("transformers.models.roberta.modeling_roberta")
    importlib.import_module("transformers.models.bert.modeling_bert")
    for modname, attr in [
        ("transformers.models.roberta.modeling_roberta", "RobertaSdpaSelfAttention"),
        ("transformers.models.bert.modeling_bert", "BertSdpaSelfAttention"),
        ("transformers", "TFPreTrainedModel"),
    ]:
        mod = sys.modules[modname]
        try:
            getattr(mod, attr)
        except Exception:
            mod.__dict__[attr] = type(attr, (), {})


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.numpy()


def sample_inputs() -> dict[str, torch.Tensor]:
    """fp32 [rows, 128] inputs covering the distributions of the benchmark configs plus edge cases."""
    g = torch.Generator().manual_seed(1234)
    R, C = 48, 128
    out = {}
    x = torch.randn(R, C, generator=g)
    m = torch.rand(R, C, generator=g) < 1e-2
    out["normal_outliers"] = torch.where(m, torch.randn(R, C, generator=g) * 100, x)
    # Student-t(3) * 0.02 from a ratio of seeded normals
    z = torch.randn(R, C, generator=g)
    chi = (torch.randn(3, R, C, generator=g) ** 2).sum(0) / 3
    out["student_t"] = z / chi.sqrt() * 0.02
    out["wide_range"] = x * torch.exp2(torch.randint(-60, 60, (R, C), generator=g).float())
    zz = x.clone()
    zz[::3] = 0
    zz[1, :40] = -0.0
    zz[2, 5] = 1e-9
    zz[2, 6] = -1e-9
    zz[2, 7] = 1e-8
    zz[4] = x[4] * 1e-39  # fp32 subnormals
    zz[5] = x[5] * 1e-37
    zz[7] = x[7] * 3e37
    out["zeros_tiny_huge"] = zz
    # exact powers of two and their neighbours as block maxima
    e = torch.arange(-30, 31).float()
    pw = torch.exp2(e)
    nb = []
    for d in (-2, -1, 0, 1, 2, 3):
        nb.append((pw.view(torch.int32) + d).view(torch.float32))
    mx = torch.cat(nb)[: R * 4]  # one value per 32-block
    blk = torch.randn(R * 4, 32, generator=g).clamp(-0.95, 0.95) * mx.view(-1, 1)
    blk[:, 0] = mx
    out["pow2_block_max"] = blk.reshape(R, C)
    # the E4M3 carry / underflow cases at block scale 2**0 (block max 256 -> shared exponent 0)
    kat = torch.zeros(4, 32)
    kat[0, :12] = torch.tensor([256.0, 1.97, 3.97, 7.9, 480.0, 500.0, 2.0**-7, 1.5 * 2.0**-7, 2.0**-6, 2.0**-9, -1.97, -(2.0**-9)])
    kat[1, :8] = torch.tensor([4.0, 0.49, 0.26, 0.74, 1.49, 2.9, 3.6, 5.9])  # E2M1 binades (block max 4)
    kat[2, :4] = torch.tensor([1.0, 0.99609375, -1.0, 0.5])  # MXINT: +1.0 saturates to 127/128, -1.0 kept
    kat[3, :4] = torch.tensor([1.0078125, 1.0, 0.75, -0.3])  # bf16 value just above a power of two
    out["kat"] = torch.cat([kat.reshape(1, 128), torch.zeros(R - 1, C)])
    return out


def main(root: str) -> None:
    import_reference(root)
    import chop.nn.quantizers as q
    from chop.nn.quantizers.mxint.fake import extract_mxint_components
    from chop.nn.quantizers.mxint.meta import MXIntMeta
    from chop.nn.quantizers.mxfp.fake import extract_mxfp_components
    from chop.nn.quantizers.mxfp.meta import MXFPMeta
    from chop.nn.quantizers._minifloat_mx import MinifloatMeta, minifloat_quantizer_sim
    from chop.nn.quantized.modules.linear import LinearBlockFP, LinearMXFP, LinearMXInt

    inputs = sample_inputs()
    arrays: dict[str, np.ndarray] = {}
    index: list[dict] = []
    for name, x32 in inputs.items():
        for dt_name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
            x = x32.to(dt)
            key = f"{name}/{dt_name}"
            arrays[f"{key}/x"] = bits(x)
            for block, nbits in ((32, 8), (16, 4)):
                meta = MXIntMeta(block_size=block, scale_bits=8, element_bits=nbits)
                sc, mant = extract_mxint_components(x.flatten(), meta)
                y = q.mxint_quantizer(x, block, nbits)
                tag = f"{key}/mxint_b{block}_w{nbits}"
                arrays[f"{tag}/scale"] = bits(sc)
                arrays[f"{tag}/mant"] = bits(mant)
                arrays[f"{tag}/fake"] = bits(y)
                index.append({"kind": "mxint", "input": key, "tag": tag, "block": block, "bits": nbits})
            for E, F in ((4, 3), (2, 1), (5, 2), (3, 2), (2, 3), (1, 2)):
                for block in (32, 16):
                    if block == 16 and (E, F) not in ((4, 3), (2, 1)):
                        continue
                    meta = MXFPMeta(block_size=block, scale_exp_bits=8, element_exp_bits=E, element_frac_bits=F,
                                    element_is_finite=True, round_mode="rn")
                    sc, co = extract_mxfp_components(x.flatten(), meta)
                    y = q.mxfp_quantizer(x, block, E, F)
                    tag = f"{key}/mxfp_b{block}_e{E}m{F}"
                    arrays[f"{tag}/scale"] = bits(sc)
                    arrays[f"{tag}/codes"] = bits(co)
                    arrays[f"{tag}/fake"] = bits(y)
                    index.append({"kind": "mxfp", "input": key, "tag": tag, "block": block, "E": E, "F": F})
            for E, F in ((4, 3), (2, 1), (5, 10), (8, 7), (3, 12)):  # 8-bit, fp16-like, bf16-like, a long fraction
                y = minifloat_quantizer_sim(x, MinifloatMeta(exp_bits=E, frac_bits=F, is_finite=True, round_mode="rn"))
                tag = f"{key}/minifloat_e{E}m{F}"
                arrays[f"{tag}/fake"] = bits(y)
                index.append({"kind": "minifloat", "input": key, "tag": tag, "E": E, "F": F})
            for width, ew, eb, bs, skip in ((8, 8, 127, [1, 32], True), (7, 8, 127, [1, 16], True),
                                            (12, 8, None, [16], True), (8, 4, None, [1, 48], True)):
                y = q.block_fp_quantizer(x, width, ew, eb, bs, skip)
                tag = f"{key}/bfp_w{width}_e{ew}_b{bs[-1]}"
                arrays[f"{tag}/fake"] = bits(y)
                index.append({"kind": "bfp", "input": key, "tag": tag, "width": width, "exponent_width": ew,
                              "exponent_bias": eb, "block_size": bs, "skip_first_dim": skip})

    # block floating point with tiles that span rows (2-D weights, 3-D activations: the unfold / fold route)
    g = torch.Generator().manual_seed(55)
    for tname, shape, bs, skip in (("w64x96_b16", (64, 96), [16], False), ("w70x100_b16x32", (70, 100), [16, 32], False),
                                   ("a3x20x40_b16", (3, 20, 40), [16], True), ("a2x33x50_b8x8", (2, 33, 50), [8, 8], True)):
        xt = torch.randn(*shape, generator=g) * torch.exp2(torch.randint(-12, 6, shape, generator=g).float())
        xt.view(-1)[::7] = 0
        for dt_name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
            x = xt.to(dt)
            arrays[f"bfp_tiles/{tname}/{dt_name}/x"] = bits(x)
            for width in (8, 12):
                arrays[f"bfp_tiles/{tname}/{dt_name}/w{width}/fake"] = bits(q.block_fp_quantizer(x, width, 8, 127, bs, skip))
            index.append({"kind": "bfp_tiles", "name": tname, "dtype": dt_name, "shape": list(shape), "block_size": bs,
                          "skip_first_dim": skip, "widths": [8, 12]})

    # block_dim other than the last, on a 3-D tensor
    g = torch.Generator().manual_seed(99)
    x3 = torch.randn(6, 64, 10, generator=g)
    for dt_name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        x = x3.to(dt)
        arrays[f"blockdim/{dt_name}/x"] = bits(x)
        for bd in (1, -2, 2, 0):
            block = 32 if x.shape[bd] % 32 == 0 else 2
            arrays[f"blockdim/{dt_name}/mxint_d{bd}/fake"] = bits(q.mxint_quantizer(x, block, 8, bd))
            arrays[f"blockdim/{dt_name}/mxfp_d{bd}/fake"] = bits(q.mxfp_quantizer(x, block, 4, 3, bd))
            index.append({"kind": "blockdim", "dtype": dt_name, "block_dim": bd, "block": block})

    # quantized Linear forward: small layers, weights quantized through load_state_dict like the pass does
    g = torch.Generator().manual_seed(7)
    M, K, N = 24, 256, 96
    for dt_name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        base = torch.nn.Linear(K, N, bias=True)
        with torch.no_grad():
            base.weight.copy_(torch.randn(N, K, generator=g) * 0.02)
            base.bias.copy_(torch.randn(N, generator=g) * 0.1)
        base = base.to(dt)
        x = torch.randn(M, K, generator=g)
        x[:, ::37] *= 50
        x = x.to(dt)
        arrays[f"linear/{dt_name}/x"] = bits(x)
        arrays[f"linear/{dt_name}/w"] = bits(base.weight.data)
        arrays[f"linear/{dt_name}/b"] = bits(base.bias.data)
        cfgs = {
            "mxfp_e4m3": (LinearMXFP, {"weight_block_size": 32, "weight_exponent_width": 4, "weight_frac_width": 3,
                                       "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}),
            "mxfp_w4a8": (LinearMXFP, {"weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1,
                                       "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3,
                                       "bias_block_size": 32, "bias_exponent_width": 4, "bias_frac_width": 3}),
            "mxint8": (LinearMXInt, {"weight_block_size": 32, "weight_width": 8,
                                     "data_in_block_size": 32, "data_in_width": 8}),
            "block_fp": (LinearBlockFP, {"weight_block_size": [1, 16], "weight_width": 7, "weight_exponent_width": 8,
                                         "weight_exponent_bias": 127, "data_in_block_size": [1, 16],
                                         "data_in_width": 7, "data_in_exponent_width": 8, "data_in_exponent_bias": 127,
                                         "bias_block_size": [16], "bias_width": 7, "bias_exponent_width": 8,
                                         "bias_exponent_bias": 127}),
        }
        for cname, (cls, cfg) in cfgs.items():
            layer = cls(K, N, bias=True, dtype=dt, config=dict(cfg))
            layer.load_state_dict(base.state_dict(), strict=False)
            y = layer(x)
            tag = f"linear/{dt_name}/{cname}"
            arrays[f"{tag}/w_q"] = bits(layer.weight.data)
            arrays[f"{tag}/b_q"] = bits(layer.bias.data)
            arrays[f"{tag}/y"] = bits(y.detach())
            index.append({"kind": "linear", "dtype": dt_name, "tag": tag, "cls": cls.__name__, "config": cfg,
                          "M": M, "K": K, "N": N})

    # MXINT clipping search (calibration-time option): weight-like tensors with outliers, with and without activations
    from chop.nn.quantizers.mxint.mxint import mxint_quantizer_sim

    g = torch.Generator().manual_seed(123)
    w32 = torch.randn(48, 128, generator=g) * 0.02
    w32[torch.rand(48, 128, generator=g) < 0.02] *= 30
    act32 = torch.randn(5, 7, 32, generator=g)  # the reference only accepts activations whose last dim is the block
    for dt_name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        w, act = w32.to(dt), act32.to(dt)
        arrays[f"mxint_search/{dt_name}/x"] = bits(w)
        arrays[f"mxint_search/{dt_name}/act"] = bits(act)
        for nbits in (8, 4):
            meta = MXIntMeta(block_size=32, scale_bits=8, element_bits=nbits)
            arrays[f"mxint_search/{dt_name}/w{nbits}/fake"] = bits(
                mxint_quantizer_sim(w, 1, meta, quantile_search=True))
            arrays[f"mxint_search/{dt_name}/w{nbits}/fake_act"] = bits(
                mxint_quantizer_sim(w, 1, meta, act_tensor=act, quantile_search=True, cali_batch_size=2))
            sc, mant = extract_mxint_components(w.flatten(), meta, percentile=0.97)
            arrays[f"mxint_search/{dt_name}/w{nbits}/p97_scale"] = bits(sc)
            arrays[f"mxint_search/{dt_name}/w{nbits}/p97_mant"] = bits(mant)
            index.append({"kind": "mxint_search", "dtype": dt_name, "bits": nbits, "block": 32})

    # MXFP clipping search: ordinary weights (the search returns the plain result), large magnitudes (the reference's
    # error on raw code bytes is non-zero there) and sparse rows (zero quantiles)
    from chop.nn.quantizers.mxfp.mxfp import mxfp_quantizer_sim
    from chop.nn.quantizers.mxfp.meta import MXFPMeta

    g = torch.Generator().manual_seed(321)
    parts = []
    for magnitude in (0.02, 1.0, 40.0, 300.0, 3000.0):
        w = torch.randn(16, 128, generator=g) * magnitude
        w[torch.rand(16, 128, generator=g) < 0.03] *= 20
        parts.append(w)
    sparse = torch.randn(16, 128, generator=g) * 200
    sparse[torch.rand(16, 128, generator=g) < 0.6] = 0
    sparse[3] = 0
    parts.append(sparse)
    w32 = torch.cat(parts)
    for dt_name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        w = w32.to(dt)
        arrays[f"mxfp_search/{dt_name}/x"] = bits(w)
        for E, F in ((4, 3), (2, 1), (3, 2)):
            meta = MXFPMeta(block_size=32, scale_exp_bits=8, element_exp_bits=E, element_frac_bits=F,
                            element_is_finite=True, round_mode="rn")
            arrays[f"mxfp_search/{dt_name}/e{E}m{F}/fake"] = bits(mxfp_quantizer_sim(w, 1, meta, quantile_search=True))
            index.append({"kind": "mxfp_search", "dtype": dt_name, "E": E, "F": F, "block": 32})

    # GPTQ (passes/module/transforms/gptq/gptq.py): one small Linear, Hessian from seeded activations, MXFP4 / MXINT4
    # inner quantizer with and without the clipping search
    pkg = types.ModuleType("chop.passes.module.transforms.gptq")
    pkg.__path__ = [root + "/passes/module/transforms/gptq"]
    sys.modules["chop.passes.module.transforms.gptq"] = pkg
    from chop.passes.module.transforms.gptq.gptq import GPTQ

    g = torch.Generator().manual_seed(77)
    lin = torch.nn.Linear(128, 48, bias=False)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(48, 128, generator=g) * 0.05)
    acts = torch.randn(6, 40, 128, generator=g) * (1 + 3 * torch.rand(128, generator=g))
    arrays["gptq/w"] = bits(lin.weight.data)
    arrays["gptq/acts"] = bits(acts)
    for fmt, cfg in (("mxfp", {"weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1}),
                     ("mxint", {"weight_block_size": 32, "weight_width": 4})):
        for search in (False, True):
            solver = GPTQ(lin)
            for i in range(acts.shape[0]):
                solver.add_batch(acts[i : i + 1], None)
            arrays[f"gptq/{fmt}/search{int(search)}/hessian"] = bits(solver.H.clone())
            arrays[f"gptq/{fmt}/search{int(search)}/q"] = bits(
                solver.fasterquant(None, fmt, cfg, percdamp=0.01, quant_search=search))
            index.append({"kind": "gptq", "format": fmt, "search": search})

    # Quantized Llama attention and MLP wrappers (nn/quantized/modules/llama/{attention,mlp}.py): one small block in
    # bf16 and fp32 with a causal mask, with and without a key/value cache
    for name in ("chop.nn.quantized", "chop.nn.quantized.modules", "chop.nn.quantized.modules.llama"):
        if name not in sys.modules or not hasattr(sys.modules[name], "__path__"):
            m = types.ModuleType(name)
            m.__path__ = [root + name[len("chop"):].replace(".", "/")]
            sys.modules[name] = m
    from chop.nn.quantized.modules.llama.attention import LlamaAttentionMXFP, LlamaAttentionMXInt
    from chop.nn.quantized.modules.llama.mlp import LlamaMLPMXFP
    from transformers import LlamaConfig
    from transformers.cache_utils import DynamicCache
    from transformers.models.llama.modeling_llama import LlamaRotaryEmbedding

    hf = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=1, num_attention_heads=4,
                     num_key_value_heads=2, vocab_size=64, max_position_embeddings=128)
    hf._attn_implementation = "eager"
    fp_cfg = {"data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}
    int_cfg = {"data_in_block_size": 32, "data_in_width": 8}
    mini = {"data_in_exponent_width": 5, "data_in_frac_width": 10}
    q_fp = {"qk_matmul": fp_cfg, "av_matmul": fp_cfg, "rope": mini, "softmax": mini, "kv_cache": fp_cfg}
    q_int = {"qk_matmul": int_cfg, "av_matmul": int_cfg, "rope": mini, "softmax": mini, "kv_cache": int_cfg}
    g = torch.Generator().manual_seed(2024)
    B, S = 2, 64
    hidden32 = torch.randn(B, S, 128, generator=g)
    weights32 = {n: torch.randn(shape, generator=g) * 0.06 for n, shape in
                 (("q_proj.weight", (128, 128)), ("k_proj.weight", (64, 128)), ("v_proj.weight", (64, 128)),
                  ("o_proj.weight", (128, 128)))}
    causal = torch.ones(S, S, dtype=torch.bool).triu(1)[None, None].expand(B, 1, S, S)
    pos = torch.arange(S)[None].expand(B, S)
    for dt_name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        hidden = hidden32.to(dt)
        cos, sin = LlamaRotaryEmbedding(hf)(hidden, pos)
        arrays[f"attention/{dt_name}/hidden"] = bits(hidden)
        arrays[f"attention/{dt_name}/cos"] = bits(cos)
        arrays[f"attention/{dt_name}/sin"] = bits(sin)
        # additive mask the way the model builds it: the most negative finite value of the dtype (an infinite score is
        # outside the minifloat quantizer's domain)
        mask = torch.zeros(B, 1, S, S, dtype=dt).masked_fill(causal, torch.finfo(dt).min)
        arrays[f"attention/{dt_name}/mask"] = bits(mask)
        for wname, w in weights32.items():
            arrays[f"attention/{dt_name}/{wname}"] = bits(w.to(dt))
        for fmt, cls, qc in (("mxfp", LlamaAttentionMXFP, q_fp), ("mxint", LlamaAttentionMXInt, q_int)):
            for cached in (False, True):
                attn = cls(hf, 0, qc).to(dt).eval()
                attn.load_state_dict({n: w.to(dt) for n, w in weights32.items()})
                with torch.no_grad():
                    out, probs = attn(hidden, (cos, sin), mask, past_key_value=DynamicCache() if cached else None,
                                      cache_position=torch.arange(S))
                arrays[f"attention/{dt_name}/{fmt}/cache{int(cached)}/out"] = bits(out)
                arrays[f"attention/{dt_name}/{fmt}/cache{int(cached)}/probs"] = bits(probs)
                index.append({"kind": "attention", "dtype": dt_name, "format": fmt, "cached": cached})
        # the Qwen3 variant: RMS norms over the head dimension of queries and keys before the rotary embedding
        # (nn/quantized/modules/qwen3/attention.py:20-120)
        if "chop.nn.quantized.modules.qwen3" not in sys.modules:
            m = types.ModuleType("chop.nn.quantized.modules.qwen3")
            m.__path__ = [root + "/nn/quantized/modules/qwen3"]
            sys.modules["chop.nn.quantized.modules.qwen3"] = m
        from chop.nn.quantized.modules.qwen3.attention import Qwen3AttentionMXFP
        from transformers import Qwen3Config

        qw = Qwen3Config(hidden_size=128, intermediate_size=256, num_hidden_layers=1, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, vocab_size=64, max_position_embeddings=128)
        qw._attn_implementation = "eager"
        attn = Qwen3AttentionMXFP(qw, 0, q_fp).to(dt).eval()
        state = {n: w.to(dt) for n, w in weights32.items()}
        state["q_norm.weight"] = (1 + 0.2 * torch.randn(32, generator=g)).to(dt)
        state["k_norm.weight"] = (1 + 0.2 * torch.randn(32, generator=g)).to(dt)
        attn.load_state_dict(state)
        with torch.no_grad():
            out, probs = attn(hidden, (cos, sin), mask)
        arrays[f"attention/{dt_name}/qwen3/q_norm.weight"] = bits(state["q_norm.weight"])
        arrays[f"attention/{dt_name}/qwen3/k_norm.weight"] = bits(state["k_norm.weight"])
        arrays[f"attention/{dt_name}/qwen3/out"] = bits(out)
        arrays[f"attention/{dt_name}/qwen3/probs"] = bits(probs)
        index.append({"kind": "attention_qwen3", "dtype": dt_name, "eps": qw.rms_norm_eps})
        mlp = LlamaMLPMXFP(hf, 0, mini).to(dt).eval()
        with torch.no_grad():
            for n, prm in mlp.named_parameters():
                prm.copy_((torch.randn(prm.shape, generator=g) * 0.06).to(dt))
                arrays[f"mlp/{dt_name}/{n}"] = bits(prm.data)
            arrays[f"mlp/{dt_name}/out"] = bits(mlp(hidden))
        index.append({"kind": "mlp", "dtype": dt_name})

    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **arrays)
    with open(os.path.join(HERE, "reference_vectors.json"), "w") as fh:
        json.dump({"torch": torch.__version__, "cases": index}, fh, indent=1)
    print(f"wrote {len(arrays)} arrays, {len(index)} cases")


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("MASE_CHOP_DIR"):
        raise SystemExit("usage: python make_golden.py <path to src/chop of a MASE checkout>  (or set MASE_CHOP_DIR)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["MASE_CHOP_DIR"])
