"""MX matrix products of `chop.nn.quantized.functional` on the GPU kernels of this package.

    matmul_mxfp / matmul_mxint / bmm_mxfp / bmm_mxint   chop/nn/quantized/functional/matmul.py:437-512
    kv_cache_mxfp / kv_cache_mxint                      chop/nn/quantized/functional/kvcache.py:8-43
    softmax_mxfp / softmax_mxint                        chop/nn/quantized/functional/softmax.py:10-39
    silu_mxfp / silu_mxint                              chop/nn/quantized/functional/silu.py:10-40
    rope_mxfp / rope_mxint                              chop/nn/quantized/functional/rope.py:30-77

Both operands are fake-quantized along their last dimension (x[..., M, K] along K, y[..., K, N] along N, as the
reference does) and multiplied.  A two-dimensional y goes through this package's tensor-core GEMM (exact products of
the quantized values, fp32 accumulation); a batched y is multiplied by torch.matmul / torch.bmm per the reference.
"""

from __future__ import annotations

import torch
from torch import Tensor

from .gemm import linear_forward
from .quantizers import mxfp_quantizer, mxint_quantizer


def _product(x: Tensor, y: Tensor, style: str) -> Tensor:
    if style == "matmul" and y.dim() == 2 and x.dim() >= 2 and x.shape[-1] % 8 == 0:
        return linear_forward(x, y.t().contiguous(), None, x.dtype)
    return torch.bmm(x, y) if style == "bmm" else torch.matmul(x, y)


def _generic_matmul_mxfp(x: Tensor, y: Tensor, config: dict, style: str) -> Tensor:
    if config.get("bypass", False):
        return torch.bmm(x, y) if style == "bmm" else torch.matmul(x, y)
    x = mxfp_quantizer(x, block_size=config["data_in_block_size"], element_exp_bits=config["data_in_exponent_width"],
                       element_frac_bits=config["data_in_frac_width"], block_dim=-1)
    y = mxfp_quantizer(y, block_size=config["weight_block_size"], element_exp_bits=config["weight_exponent_width"],
                       element_frac_bits=config["weight_frac_width"], block_dim=-1)
    return _product(x, y, style)


def _generic_matmul_mxint(x: Tensor, y: Tensor, config: dict, style: str) -> Tensor:
    if config.get("bypass", False):
        return torch.bmm(x, y) if style == "bmm" else torch.matmul(x, y)
    x = mxint_quantizer(x, block_size=config["data_in_block_size"], element_bits=config["data_in_width"], block_dim=-1)
    y = mxint_quantizer(y, block_size=config["weight_block_size"], element_bits=config["weight_width"], block_dim=-1)
    return _product(x, y, style)


def matmul_mxfp(x: Tensor, y: Tensor, config: dict) -> Tensor:
    return _generic_matmul_mxfp(x, y, config, "matmul")


def matmul_mxint(x: Tensor, y: Tensor, config: dict) -> Tensor:
    return _generic_matmul_mxint(x, y, config, "matmul")


def bmm_mxfp(x: Tensor, y: Tensor, config: dict) -> Tensor:
    return _generic_matmul_mxfp(x, y, config, "bmm")


def bmm_mxint(x: Tensor, y: Tensor, config: dict) -> Tensor:
    return _generic_matmul_mxint(x, y, config, "bmm")


def _x_mxfp(config: dict):
    return lambda t: mxfp_quantizer(t, block_size=config["data_in_block_size"],
                                    element_exp_bits=config["data_in_exponent_width"],
                                    element_frac_bits=config["data_in_frac_width"], block_dim=-1)


def _x_mxint(config: dict):
    return lambda t: mxint_quantizer(t, block_size=config["data_in_block_size"], element_bits=config["data_in_width"],
                                     block_dim=-1)


def kv_cache_mxfp(key_states: Tensor, value_states: Tensor, config: dict = None) -> tuple[Tensor, Tensor]:
    q = _x_mxfp(config)
    return q(key_states), q(value_states)


def kv_cache_mxint(key_states: Tensor, value_states: Tensor, config: dict = None) -> tuple[Tensor, Tensor]:
    q = _x_mxint(config)
    return q(key_states), q(value_states)


def softmax_mxfp(x: Tensor, config: dict = None, dim: int = -1) -> Tensor:
    x = _x_mxfp(config)(x)
    return torch.nn.functional.softmax(x.to(torch.float32), dim=dim).to(x.dtype)


def softmax_mxint(x: Tensor, config: dict = None, dim: int = -1) -> Tensor:
    x = _x_mxint(config)(x)
    return torch.nn.functional.softmax(x.to(torch.float32), dim=dim).to(x.dtype)


def silu_mxfp(x: Tensor, config: dict = None) -> Tensor:
    return torch.nn.functional.silu(_x_mxfp(config)(x))


def silu_mxint(x: Tensor, config: dict = None) -> Tensor:
    return torch.nn.functional.silu(_x_mxint(config)(x))


def _rotate_half(x: Tensor) -> Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def _apply_rope(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, unsqueeze_dim: int):
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    seq_len = q.size(-2)
    cos, sin = cos[..., :seq_len, :], sin[..., :seq_len, :]
    return (q * cos) + (_rotate_half(q) * sin), (k * cos) + (_rotate_half(k) * sin)


def rope_mxfp(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, config: dict = None, unsqueeze_dim: int = 1):
    """Rotary embedding with MXFP-quantized cos / sin tables."""
    quant = _x_mxfp(config)
    return _apply_rope(q, k, quant(cos), quant(sin), unsqueeze_dim)


def rope_mxint(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, config: dict = None, unsqueeze_dim: int = 1):
    quant = _x_mxint(config)
    return _apply_rope(q, k, quant(cos), quant(sin), unsqueeze_dim)


quantized_func_map = {
    "kv_cache_mxfp": kv_cache_mxfp,
    "kv_cache_mxint": kv_cache_mxint,
    "softmax_mxfp": softmax_mxfp,
    "softmax_mxint": softmax_mxint,
    "silu_mxfp": silu_mxfp,
    "silu_mxint": silu_mxint,
    "rope_mxfp": rope_mxfp,
    "rope_mxint": rope_mxint,
    "matmul_mxfp": matmul_mxfp,
    "matmul_mxint": matmul_mxint,
    "bmm_mxfp": bmm_mxfp,
    "bmm_mxint": bmm_mxint,
}
