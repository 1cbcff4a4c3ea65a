"""MX matrix products of `chop.nn.quantized.functional` on the GPU kernels of this package.

    matmul_mxfp / matmul_mxint / bmm_mxfp / bmm_mxint   chop/nn/quantized/functional/matmul.py:437-512

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


quantized_func_map = {
    "matmul_mxfp": matmul_mxfp,
    "matmul_mxint": matmul_mxint,
    "bmm_mxfp": bmm_mxfp,
    "bmm_mxint": bmm_mxint,
}
