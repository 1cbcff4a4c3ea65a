"""Per-exponent correction tables for the shared-exponent selection.

MASE picks a block's shared exponent with `torch.log2` on the host: `ceil(log2(amax))` evaluated in the
tensor's dtype for MXINT (chop/nn/quantizers/mxint/fake.py:45) and block floating point
(chop/nn/quantizers/block_fp.py:58), `floor(log2(amax))` in fp32 for MXFP (chop/nn/quantizers/mxfp/fake.py:58).
Next to a power of two the rounded logarithm is an exact integer although the true one is not, so the
selected exponent differs from the exact integer ceil/floor for a few mantissa values per binade
(thousands of bf16 values in total).  The kernels compute the exact integer from the bits of amax and
apply these tables, which are built here from this host's own `torch.log2`, i.e. they reproduce what the
reference would select when run on this host.
"""

from __future__ import annotations

import functools

import numpy as np
import torch

_WINDOW = 255  # mantissas scanned on each side of a power of two (observed counts are <= 44)


def _prefix_len(hit: torch.Tensor) -> torch.Tensor:
    """Length of the leading run of True along dim 1; the hits must form exactly that run."""
    run = hit.to(torch.int64).cumprod(dim=1).sum(dim=1)
    if int(hit.sum()) != int(run.sum()):
        raise RuntimeError("log2 rounding pattern on this host is not a contiguous run; tables cannot represent it")
    if int(run.max()) >= _WINDOW:
        raise RuntimeError("log2 rounding run reaches the scan window")
    return run


@functools.lru_cache(maxsize=None)
def ceil_table(dtype: torch.dtype) -> np.ndarray:
    """t[ex]: mantissas 1..t[ex] (in units of the dtype's mantissa lsb) have ceil(log2(x)) == ex-127."""
    ex = torch.arange(1, 255, dtype=torch.int32).view(-1, 1)
    if dtype == torch.float32:
        m = torch.arange(1, _WINDOW + 1, dtype=torch.int32).view(1, -1)
        x = ((ex << 23) | m).view(torch.float32)
    elif dtype == torch.bfloat16:
        m = torch.arange(1, 128, dtype=torch.int32).view(1, -1)
        x = ((ex << 7) | m).to(torch.int16).view(torch.bfloat16)
    else:
        raise NotImplementedError(f"no log2 table for {dtype}")
    hit = torch.log2(x).ceil().to(torch.int32) == (ex - 127)
    t = np.zeros(256, dtype=np.uint8)
    run = _prefix_len(hit) if dtype == torch.float32 else hit.to(torch.int64).cumprod(dim=1).sum(dim=1)
    if dtype == torch.bfloat16 and int(hit.sum()) != int(run.sum()):
        raise RuntimeError("bf16 log2 rounding pattern on this host is not a contiguous run")
    t[1:255] = run.numpy().astype(np.uint8)
    return t


@functools.lru_cache(maxsize=None)
def floor_table() -> np.ndarray:
    """t[ex]: the top t[ex] fp32 mantissas of binade ex have floor(log2(x)) == ex-126."""
    ex = torch.arange(1, 255, dtype=torch.int32).view(-1, 1)
    j = torch.arange(0, _WINDOW, dtype=torch.int32).view(1, -1)
    x = ((ex << 23) | (0x7FFFFF - j)).view(torch.float32)
    hit = torch.log2(x).floor().to(torch.int32) == (ex - 126)
    t = np.zeros(256, dtype=np.uint8)
    t[1:255] = _prefix_len(hit).numpy().astype(np.uint8)
    return t
