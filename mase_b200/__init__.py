"""mase_b200 -- sm_100a (B200) implementation of MASE's MX / block-floating-point quantized-inference path.

Public surface (same names as in `chop.nn.quantizers` / `chop.nn.quantized`):
  quantizers: mxint_quantizer, mxfp_quantizer, block_fp_quantizer, *_quantizer_sim, extract_* / compose_*
  modules:    LinearMXFP, LinearMXInt, LinearBlockFP, linearBlockFP, EmbeddingMXFP / MXInt, RMSNormMinifloat,
              AttentionMXFP / MXInt (+ the Qwen3 variants), GatedMLPMX            (mase_b200.attention)
  functional: matmul / bmm / kv_cache / softmax / silu / rope for mxfp, mxint, minifloat
  calibration: the clipping search inside *_quantizer_sim(quantile_search=True); GPTQ (mase_b200.gptq)
  patch(chop) registers them in an imported MASE so that its quantize passes pick them up.

All compute goes through libmxq.so (C ABI in include/mxq.h); there is no CPU or eager fallback.
"""

from .quantizers import (  # noqa: F401
    MinifloatMeta,
    MXFPMeta,
    MXIntMeta,
    block_fp_quantizer,
    compose_mxfp_tensor,
    compose_mxint_tensor,
    extract_mxfp_components,
    extract_mxint_components,
    minifloat_quantizer_sim,
    mxfp_quantizer,
    mxfp_quantizer_sim,
    mxint_codes,
    mxint_quantizer,
    mxint_quantizer_sim,
    quantizer_map,
)
from .modules import (  # noqa: F401
    EmbeddingMXFP,
    EmbeddingMXInt,
    RMSNormMinifloat,
    LinearBlockFP,
    LinearMXFP,
    LinearMXInt,
    linearBlockFP,
    quantized_func_map,
    quantized_module_map,
)
from .functional import (  # noqa: F401
    bmm_mxfp, bmm_mxint, kv_cache_mxfp, kv_cache_mxint, matmul_mxfp, matmul_mxint, rope_minifloat, rope_mxfp, rope_mxint,
    silu_minifloat, silu_mxfp, silu_mxint, softmax_minifloat, softmax_mxfp, softmax_mxint,
)
from .attention import (  # noqa: F401
    AttentionMXFP, AttentionMXInt, GatedMLPMX, Qwen3AttentionMXFP, Qwen3AttentionMXInt,
)
from .patch import patch  # noqa: F401

__all__ = [n for n in dir() if not n.startswith("_")]
