"""y = x @ W^T (+ bias) for operands that already hold quantized values.

The operands of the quantized Linear modules are fake-quantized tensors: every value is a minifloat /
integer mantissa times a power of two and is exactly representable in bf16 (and fp32), so products are
exact and only the fp32 accumulation order differs from the reference's `F.linear`
(chop/nn/quantized/modules/linear.py:895, :972).
"""

from __future__ import annotations

import torch
from torch import Tensor


def linear_forward(x: Tensor, weight: Tensor, bias: Tensor | None) -> Tensor:
    if not x.is_cuda:
        raise RuntimeError("mase_b200 runs on CUDA devices only (no CPU fallback)")
    return torch.nn.functional.linear(x, weight, bias)
