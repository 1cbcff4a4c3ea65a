"""Registers the B200 implementations inside an imported MASE (`chop`) package.

    import chop, mase_b200
    mase_b200.patch(chop)

After this, `quantize_module_transform_pass` (chop/passes/module/transforms/quantize/quantize.py:95-151) and the
FX quantize pass build the classes of this package for `"mxfp"`, `"mxint"` and `"block_fp"` configs, because
they look classes up in `quantized_module_map[f"linear_{name}"]`
(chop/passes/module/module_modify_helper.py:149-176) at call time.
"""

from __future__ import annotations

import importlib
import sys

from . import functional, modules, quantizers

_QUANTIZER_NAMES = {
    "mxfp_quantizer": quantizers.mxfp_quantizer,
    "mxint_quantizer": quantizers.mxint_quantizer,
    "block_fp_quantizer": quantizers.block_fp_quantizer,
}


def _maybe(name: str):
    try:
        return sys.modules.get(name) or importlib.import_module(name)
    except Exception:
        return None


def patch(chop=None) -> list[str]:
    """Overwrite the map entries and module-level names of `chop`; returns what was patched."""
    done = []
    q = _maybe("chop.nn.quantizers")
    if q is not None:
        for key, fn in quantizers.quantizer_map.items():
            q.quantizer_map[key] = fn
            done.append(f"chop.nn.quantizers.quantizer_map[{key!r}]")
        for name, fn in _QUANTIZER_NAMES.items():
            setattr(q, name, fn)
    mm = _maybe("chop.nn.quantized.modules")
    if mm is not None and hasattr(mm, "quantized_module_map"):
        for key, cls in modules.quantized_module_map.items():
            mm.quantized_module_map[key] = cls
            done.append(f"chop.nn.quantized.modules.quantized_module_map[{key!r}]")
        for cls in modules.quantized_module_map.values():
            setattr(mm, cls.__name__, cls)
        for cls in (modules.EmbeddingMXFP, modules.EmbeddingMXInt):  # exported by the package, not in its map
            setattr(mm, cls.__name__, cls)
            done.append(f"chop.nn.quantized.modules.{cls.__name__}")
    me = _maybe("chop.nn.quantized.modules.embedding")
    if me is not None:
        me.EmbeddingMXFP, me.EmbeddingMXInt = modules.EmbeddingMXFP, modules.EmbeddingMXInt
        done.append("chop.nn.quantized.modules.embedding")
    ml = _maybe("chop.nn.quantized.modules.linear")
    if ml is not None:
        for cls in modules.quantized_module_map.values():
            setattr(ml, cls.__name__, cls)
        for name, fn in _QUANTIZER_NAMES.items():
            if hasattr(ml, name):
                setattr(ml, name, fn)
        done.append("chop.nn.quantized.modules.linear")
    fm = _maybe("chop.nn.quantized.functional")
    if fm is not None and hasattr(fm, "quantized_func_map"):
        fm.quantized_func_map["linear_block_fp"] = modules.linearBlockFP
        done.append("chop.nn.quantized.functional.quantized_func_map['linear_block_fp']")
        for key, fn in functional.quantized_func_map.items():
            fm.quantized_func_map[key] = fn
            if hasattr(fm, key):
                setattr(fm, key, fn)
            done.append(f"chop.nn.quantized.functional.quantized_func_map[{key!r}]")
    fl = _maybe("chop.nn.quantized.functional.linear")
    if fl is not None:
        fl.linearBlockFP = modules.linearBlockFP
        fl.block_fp_quantizer = quantizers.block_fp_quantizer
        done.append("chop.nn.quantized.functional.linear")
    # attention / MLP wrappers of the Llama family: looked up as quantized_module_map[f"{prefix}_{name}"] and built with
    # (config, layer_idx, q_config) (chop/passes/module/module_modify_helper.py:265-275)
    if mm is not None and hasattr(mm, "quantized_module_map"):
        from . import attention

        for key, cls in (("llama_self_attention_mxfp", attention.AttentionMXFP),
                         ("llama_self_attention_mxint", attention.AttentionMXInt),
                         ("llama_mlp_mxfp", attention.GatedMLPMX), ("llama_mlp_mxint", attention.GatedMLPMX),
                         ("llama_rms_norm_minifloat", modules.RMSNormMinifloat),
                         ("qwen3_self_attention_mxfp", attention.Qwen3AttentionMXFP),
                         ("qwen3_self_attention_mxint", attention.Qwen3AttentionMXInt),
                         ("qwen3_mlp_mxfp", attention.GatedMLPMX), ("qwen3_mlp_mxint", attention.GatedMLPMX),
                         ("qwen3_rms_norm_minifloat", modules.RMSNormMinifloat)):
            if key in mm.quantized_module_map:
                mm.quantized_module_map[key] = cls
                done.append(f"chop.nn.quantized.modules.quantized_module_map[{key!r}]")
    # the GPTQ pre-pass is looked up as `..gptq.run_gptq` when the quantize pass runs
    # (chop/passes/module/transforms/quantize/quantize.py:134-138); its package only imports where the reference's
    # dataset loaders do
    gp = _maybe("chop.passes.module.transforms.gptq")
    if gp is not None:
        from . import gptq

        gp.run_gptq = gptq.run_gptq
        for name in ("chop.passes.module.transforms.gptq.gptq", "chop.passes.module.transforms.gptq.quantize_dispatch"):
            sub = _maybe(name)
            if sub is not None:
                if hasattr(sub, "GPTQ"):
                    sub.GPTQ = gptq.GPTQ
                sub.quantize_tensor = gptq.quantize_tensor
        done.append("chop.passes.module.transforms.gptq.run_gptq")
    return done
