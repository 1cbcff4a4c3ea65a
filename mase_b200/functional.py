"""MX matrix products of `chop.nn.quantized.functional` on the GPU kernels of this package.

    matmul_mxfp / matmul_mxint / bmm_mxfp / bmm_mxint   chop/nn/quantized/functional/matmul.py:437-512
    kv_cache_mxfp / kv_cache_mxint                      chop/nn/quantized/functional/kvcache.py:8-43
    softmax_mxfp / softmax_mxint                        chop/nn/quantized/functional/softmax.py:10-39
    silu_mxfp / silu_mxint                              chop/nn/quantized/functional/silu.py:10-40
    rope_mxfp / rope_mxint                              chop/nn/quantized/functional/rope.py:30-77

    softmax_minifloat / silu_minifloat / rope_minifloat chop/nn/quantized/functional/softmax.py:42-57, silu.py:43-58,
                                                        rope.py:78-101

Both operands are fake-quantized along their last dimension (x[..., M, K] along K, y[..., K, N] along N, as the
reference does) and multiplied on this package's tensor-core GEMM (exact products of the quantized values, fp32
accumulation): a two-dimensional y in one launch over all rows of x, a batched y in one launch over the whole batch
(`mxq_gemm_dense_batched`).
Only `bypass` configurations, which the reference leaves unquantized, go to torch.matmul / torch.bmm.
"""

from __future__ import annotations

import torch
from torch import Tensor

from .gemm import batched_product, linear_forward
from .quantizers import MinifloatMeta, minifloat_quantizer_sim, mxfp_quantizer, mxint_quantizer


def _product(x: Tensor, y: Tensor, style: str) -> Tensor:
    """x @ y for already-quantized operands.  y[..., K, N] is brought to the K-major [N, K] form the GEMM reads."""
    if style == "bmm" and (x.dim() != 3 or y.dim() != 3):
        raise RuntimeError(f"batch1 and batch2 must be 3D tensors, got {x.dim()}D and {y.dim()}D")
    if x.dim() < 2 or y.dim() < 2:  # vector operands: as torch.matmul defines them
        xv, yv = (x.unsqueeze(0) if x.dim() == 1 else x), (y.unsqueeze(-1) if y.dim() == 1 else y)
        out = _product(xv, yv, "matmul")
        if x.dim() == 1:
            out = out.squeeze(-2)
        return out.squeeze(-1) if y.dim() == 1 else out
    if y.dim() == 2:
        return linear_forward(x, y.t().contiguous(), None, x.dtype, fp32_exact=True)
    # batched y: broadcast the batch dimensions, then one batched GEMM launch
    batch = torch.broadcast_shapes(x.shape[:-2], y.shape[:-2])
    xb = x.expand(*batch, *x.shape[-2:]).reshape(-1, *x.shape[-2:])
    yt = y.expand(*batch, *y.shape[-2:]).reshape(-1, *y.shape[-2:]).transpose(-1, -2).contiguous()  # [B, N, K]
    out = batched_product(xb, yt, x.dtype)  # one launch for the whole batch
    return out.reshape(*batch, x.shape[-2], y.shape[-1])


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


def _x_minifloat(config: dict):
    meta = MinifloatMeta(exp_bits=config["data_in_exponent_width"], frac_bits=config["data_in_frac_width"],
                         is_finite=config.get("data_in_is_finite", True), round_mode=config.get("data_in_round_mode", "rn"))
    return lambda t: minifloat_quantizer_sim(t, minifloat_meta=meta)


def _x_mxint(config: dict):
    return lambda t: mxint_quantizer(t, block_size=config["data_in_block_size"], element_bits=config["data_in_width"],
                                     block_dim=-1)


def kv_cache_mxfp(key_states: Tensor, value_states: Tensor, config: dict = None) -> tuple[Tensor, Tensor]:
    q = _x_mxfp(config)
    return q(key_states), q(value_states)


def kv_cache_mxint(key_states: Tensor, value_states: Tensor, config: dict = None) -> tuple[Tensor, Tensor]:
    q = _x_mxint(config)
    return q(key_states), q(value_states)


def _fused_softmax(x: Tensor, dim: int, quantizer: int, block: int, p0: int, p1: int) -> Tensor | None:
    """Quantize along the last dimension + softmax over it in one kernel (mxq_softmax_quant); None when the kernel does
    not take the case (softmax over another dimension, rows that are not whole blocks or too long for shared memory,
    autograd), and the caller composes quantizer and softmax instead."""
    from . import _lib
    from .quantizers import _DT, _ceil_tab_ptr, _floor_tab_ptr, _on_device, _stream

    if not x.is_cuda or x.dtype not in _DT or x.dim() < 1 or dim not in (-1, x.dim() - 1):
        return None
    if x.requires_grad and torch.is_grad_enabled():
        return None
    cols = x.shape[-1]
    if cols == 0 or cols > 12288 or (quantizer != 2 and cols % block):
        return None
    xc = x.contiguous()
    y = torch.empty_like(xc)
    tab = 0 if quantizer == 2 else (_floor_tab_ptr() if quantizer == 0 else _ceil_tab_ptr(x.dtype))
    with _on_device(xc):
        rc = _lib.lib().mxq_softmax_quant(xc.data_ptr(), y.data_ptr(), _DT[x.dtype], xc.numel() // cols, cols, quantizer,
                                          block, p0, p1, tab, _stream(xc))
    if rc == -7:
        return None
    _lib.check(rc, "mxq_softmax_quant")
    return y


def _quantizer_code(fmt: str | None, cfg: dict | None, dtype: torch.dtype):
    """(kind, block, p0, p1, table address) of a quantizer for the fused softmax kernel; kind 3 = none."""
    from .quantizers import _ceil_tab_ptr, _floor_tab_ptr

    if fmt is None or cfg is None or cfg.get("bypass", False):
        return 3, 0, 0, 0, 0
    if fmt == "mxfp":
        return 0, cfg["data_in_block_size"], cfg["data_in_exponent_width"], cfg["data_in_frac_width"], _floor_tab_ptr()
    if fmt == "mxint":
        return 1, cfg["data_in_block_size"], cfg["data_in_width"], 0, _ceil_tab_ptr(dtype)
    if fmt == "minifloat":
        if not cfg.get("data_in_is_finite", True) or cfg.get("data_in_round_mode", "rn") != "rn":
            return None
        return 2, 1, cfg["data_in_exponent_width"], cfg["data_in_frac_width"], 0
    raise ValueError(f"unknown quantizer {fmt!r}")


def attention_softmax(scores: Tensor, scale: float | None, mask: Tensor | None, in_fmt: str | None, in_cfg: dict | None,
                      out_fmt: str | None, out_cfg: dict | None) -> Tensor | None:
    """softmax over the last dimension of scores[batch, heads, q_len, k_len] together with what surrounds it in an
    attention block -- `scores * scale`, `+ mask[:, :, :, :k_len]`, the input quantizer of the softmax
    (`in_fmt` "mxfp" / "mxint" / "minifloat" / None with its config), and the quantizer of the probabilities
    (`out_fmt` "mxfp" / "mxint" / None) -- in one kernel (mxq_attention_softmax), with the roundings of the separate
    tensor operations.  Returns None when the kernel does not take the case (the caller composes the operations)."""
    from . import _lib
    from .quantizers import _DT, _on_device, _stream

    if not scores.is_cuda or scores.dtype not in _DT or scores.dim() != 4:
        return None
    if scores.requires_grad and torch.is_grad_enabled():
        return None
    b, h, sq, sk = scores.shape
    if sk % 32 or sk > 2048 or scores.numel() == 0:
        return None
    qi, qo = _quantizer_code(in_fmt, in_cfg, scores.dtype), _quantizer_code(out_fmt, out_cfg, scores.dtype)
    if qi is None or qo is None or (qi[0] in (0, 1) and qi[1] != 32) or (qo[0] in (0, 1) and qo[1] != 32) or qo[0] == 2:
        return None
    mask_ptr, mask_ld = 0, 0
    if mask is not None:
        mask = mask[:, :, :, :sk]
        if (mask.dtype != scores.dtype or mask.dim() != 4 or mask.shape[0] != b or mask.shape[1] != 1 or mask.shape[2] != sq
                or mask.stride(3) != 1 or (b > 1 and mask.stride(0) != sq * mask.stride(2))):
            return None
        mask_ptr, mask_ld = mask.data_ptr(), mask.stride(2)
    x = scores.contiguous()
    y = torch.empty_like(x)
    with _on_device(x):
        rc = _lib.lib().mxq_attention_softmax(x.data_ptr(), y.data_ptr(), _DT[x.dtype], b * h * sq, sk,
                                              0 if scale is None else 1, 1.0 if scale is None else float(scale), mask_ptr,
                                              mask_ld, sq, h, qi[0], qi[1], qi[2], qi[3], qi[4], qo[0], qo[1], qo[2], qo[3],
                                              qo[4], _stream(x))
    if rc == -7:
        return None
    _lib.check(rc, "mxq_attention_softmax")
    return y


def softmax_mxfp(x: Tensor, config: dict = None, dim: int = -1) -> Tensor:
    out = _fused_softmax(x, dim, 0, config["data_in_block_size"], config["data_in_exponent_width"],
                         config["data_in_frac_width"])
    if out is not None:
        return out
    x = _x_mxfp(config)(x)
    return torch.nn.functional.softmax(x.to(torch.float32), dim=dim).to(x.dtype)


def softmax_mxint(x: Tensor, config: dict = None, dim: int = -1) -> Tensor:
    out = _fused_softmax(x, dim, 1, config["data_in_block_size"], config["data_in_width"], 0)
    if out is not None:
        return out
    x = _x_mxint(config)(x)
    return torch.nn.functional.softmax(x.to(torch.float32), dim=dim).to(x.dtype)


def softmax_minifloat(x: Tensor, config: dict = None, dim: int = -1) -> Tensor:
    if config.get("data_in_is_finite", True) and config.get("data_in_round_mode", "rn") == "rn":
        out = _fused_softmax(x, dim, 2, 1, config["data_in_exponent_width"], config["data_in_frac_width"])
        if out is not None:
            return out
    x = _x_minifloat(config)(x)
    return torch.nn.functional.softmax(x.to(torch.float32), dim=dim).to(x.dtype)


def silu_minifloat(x: Tensor, config: dict = None) -> Tensor:
    return torch.nn.functional.silu(_x_minifloat(config)(x))


def silu_mxfp(x: Tensor, config: dict = None) -> Tensor:
    return torch.nn.functional.silu(_x_mxfp(config)(x))


def silu_mxint(x: Tensor, config: dict = None) -> Tensor:
    return torch.nn.functional.silu(_x_mxint(config)(x))


def _rotate_half(x: Tensor) -> Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def rope_apply(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor | None:
    """x * cos + rotate_half(x) * sin in one kernel (mxq_rope) for x[batch, heads, seq, dim] on a CUDA device with
    tables [seq, dim] or [batch, seq, dim]; x may be a strided view (transposed projection output), the result is
    contiguous.  Returns None for layouts the kernel does
    not take (the caller then composes the elementwise ops)."""
    from . import _lib
    from .quantizers import _DT, _on_device, _stream

    if not (x.is_cuda and x.dim() == 4 and x.dtype in _DT and cos.dtype in _DT and cos.dtype == sin.dtype
            and cos.shape == sin.shape and cos.dim() in (2, 3)):
        return None
    if x.dtype == torch.float32 and cos.dtype != torch.float32:
        return None
    b, h, s, d = x.shape
    if d % 16 or x.stride(3) != 1 or cos.shape[-1] != d or cos.shape[-2] < s:
        return None
    if cos.dim() == 3 and cos.shape[0] not in (1, b):
        return None
    cos, sin = cos.contiguous(), sin.contiguous()
    tb = cos.stride(0) if cos.dim() == 3 and cos.shape[0] == b and b > 1 else 0
    ts = cos.stride(-2)
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)  # contiguous [b, h, s, d] whatever x's strides are
    with _on_device(x):
        rc = _lib.lib().mxq_rope(x.data_ptr(), y.data_ptr(), cos.data_ptr(), sin.data_ptr(), _DT[x.dtype], _DT[cos.dtype],
                                 b, h, s, d, x.stride(0), x.stride(1), x.stride(2), tb, ts, _stream(x))
    if rc in (-2, -4):  # strides or alignment the kernel does not take
        return None
    _lib.check(rc, "mxq_rope")
    return y


def _apply_rope(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, unsqueeze_dim: int):
    if unsqueeze_dim == 1 and cos.dtype == q.dtype == k.dtype:
        rq = rope_apply(q, cos, sin)
        rk = rope_apply(k, cos, sin) if rq is not None else None
        if rk is not None:
            return rq, rk
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


def rope_minifloat(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, config: dict = None, unsqueeze_dim: int = 1):
    quant = _x_minifloat(config)
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
    "softmax_minifloat": softmax_minifloat,
    "silu_minifloat": silu_minifloat,
    "rope_minifloat": rope_minifloat,
    "matmul_mxfp": matmul_mxfp,
    "matmul_mxint": matmul_mxint,
    "bmm_mxfp": bmm_mxfp,
    "bmm_mxint": bmm_mxint,
}
