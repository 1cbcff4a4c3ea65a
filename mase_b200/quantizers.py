"""MX / block-floating-point quantizers with MASE's function signatures, running on libmxq (sm_100a).

Drop-in counterparts of (paths inside the MASE repository, `src/chop/nn/quantizers/`):

  mxint/mxint.py:211   mxint_quantizer            mxint/mxint.py:14   mxint_quantizer_sim
  mxint/fake.py:11     extract_mxint_components   mxint/fake.py:59    compose_mxint_tensor
  mxfp/mxfp.py:187     mxfp_quantizer             mxfp/mxfp.py:14     mxfp_quantizer_sim
  mxfp/fake.py:12      extract_mxfp_components    mxfp/fake.py:75     compose_mxfp_tensor
  _minifloat_mx/minifloat.py:12  minifloat_quantizer_sim
  _minifloat_mx/fake.py:11,96    extract_minifloat_component / compose_minifloat_component
  block_fp.py:111      block_fp_quantizer

Same names, parameter names, defaults, return types and error behaviour.  Tensors must live on a CUDA
device: there is no CPU path.  fp32 and bf16 inputs are supported; other dtypes raise
NotImplementedError rather than silently computing something else.  The calibration-time clipping search
(`quantile_search=True`) runs as one kernel per tensor for blocks of 32 along a contiguous last dimension without
activations (what the quantized Linear layers and GPTQ ask for); its other forms (`act_tensor`, other block sizes or
dimensions, MXINT `percentile != 1.0`) run as tensor operations on the tensor's device around the kernels.  The MXFP
search keeps the reference's own error measure: raw code bytes scaled by a power of two evaluated in uint8
arithmetic, so for tensors of ordinary magnitude it returns the plain quantization.
"""

from __future__ import annotations

import functools
from dataclasses import dataclass
from typing import Literal

import torch
from torch import Tensor

from . import _lib
from .log2_tables import ceil_table, floor_table

_DT = {torch.float32: 0, torch.bfloat16: 1}


# ---------------------------------------------------------------------------------------------------
# metadata classes (same fields and checks as the reference's dataclasses)
# ---------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class MinifloatMeta:
    """_minifloat_mx/meta.py:11-35"""

    exp_bits: int
    frac_bits: int
    is_finite: bool
    round_mode: Literal["rn", "rd", "ru", "rz"]

    def __post_init__(self):
        assert self.exp_bits > 0
        assert self.frac_bits > 0
        assert self.exp_bits + self.frac_bits < 16

    @functools.cached_property
    def n_bits(self) -> int:
        return self.exp_bits + self.frac_bits + 1


@dataclass
class MinifloatTensorMeta:
    device: str
    dtype: str
    shape: tuple[int, ...]
    meta: MinifloatMeta


@dataclass(frozen=True)
class MXFPMeta:
    """mxfp/meta.py:12-59"""

    block_size: int
    scale_exp_bits: int
    element_exp_bits: int
    element_frac_bits: int
    element_is_finite: bool
    round_mode: Literal["rn", "ru", "rd", "rz"]

    def __post_init__(self):
        legal_scale_exp_bits = (8,)
        assert self.scale_exp_bits in legal_scale_exp_bits, (
            f"Invalid scale exponent bits: {self.scale_exp_bits}. Legal values are: {legal_scale_exp_bits}."
        )
        legal = ((4, 3), (5, 2), (2, 3), (3, 2), (2, 1), (1, 2))
        ef = (self.element_exp_bits, self.element_frac_bits)
        assert ef in legal, f"Invalid element exp/frac bits: {ef}. Legal values are: {legal}."

    @functools.cached_property
    def element_meta(self) -> MinifloatMeta:
        return MinifloatMeta(
            exp_bits=self.element_exp_bits,
            frac_bits=self.element_frac_bits,
            is_finite=self.element_is_finite,
            round_mode=self.round_mode,
        )


@dataclass(frozen=True)
class MXFPTensorMeta:
    device: str
    dtype: str
    shape: tuple[int, ...]
    block_dim: int
    meta: MXFPMeta


@dataclass
class MXIntMeta:
    """mxint/meta.py:8-23"""

    block_size: int
    scale_bits: int
    element_bits: int


@dataclass
class MXIntTensorMeta:
    device: str
    dtype: str
    shape: tuple[int, ...]
    block_dim: int
    meta: MXIntMeta


# ---------------------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------------------
def _require_cuda(t: Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what}: tensor is on '{t.device}'; mase_b200 runs on CUDA devices only (no CPU fallback)")


def _dtype_code(dt: torch.dtype, what: str) -> int:
    if dt not in _DT:
        raise NotImplementedError(f"{what}: dtype {dt} is not supported (float32 and bfloat16 are)")
    return _DT[dt]


_BINDING = None


def _binding():
    """The compiled torch binding when it is built and has the quantizer entry (see mase_b200.gemm._ext), else False."""
    global _BINDING
    if _BINDING is None:
        from . import gemm

        ext = gemm._ext()
        _BINDING = ext if ext and hasattr(ext, "mx_fake") else False
    return _BINDING


def _stream(t: Tensor) -> int:
    return torch._C._cuda_getCurrentRawStream(t.device.index)


class _on_device:
    """Makes the tensor's device current for the launch; a no-op when it already is (the common case)."""

    __slots__ = ("idx", "prev")

    def __init__(self, t: Tensor):
        self.idx = t.device.index

    def __enter__(self):
        self.prev = torch.cuda.current_device()
        if self.prev != self.idx:
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev != self.idx:
            torch.cuda.set_device(self.prev)
        return False


def _is_last_dim_contiguous(t: Tensor, block_dim: int) -> bool:
    return (block_dim % t.dim()) == t.dim() - 1 and t.is_contiguous()


_TAB_PTRS: dict = {}


def _ceil_tab_ptr(dtype: torch.dtype) -> int:
    """Host address of the ceil(log2) table for tensors of `dtype` (the arrays are cached for the process)."""
    p = _TAB_PTRS.get(dtype)
    if p is None:
        p = _TAB_PTRS[dtype] = ceil_table(dtype).ctypes.data
    return p


def _floor_tab_ptr() -> int:
    p = _TAB_PTRS.get("floor")
    if p is None:
        p = _TAB_PTRS["floor"] = floor_table().ctypes.data
    return p


@functools.lru_cache(maxsize=None)
def _mxfp_meta(block_size, scale_exp_bits, element_exp_bits, element_frac_bits):
    return MXFPMeta(block_size=block_size, scale_exp_bits=scale_exp_bits, element_exp_bits=element_exp_bits,
                    element_frac_bits=element_frac_bits, element_is_finite=True, round_mode="rn")


def flatten_for_quantize(tensor: Tensor, block_dim: int) -> Tensor:
    """Move `block_dim` last and flatten (mxfp/helpers.py:8-29)."""
    nd = tensor.dim()
    d = block_dim % nd
    order = list(range(nd))
    order.append(order.pop(d))
    return tensor.permute(order).flatten()


def permute_for_dequantize(flatten_tensor: Tensor, ori_shape: tuple[int, ...], block_dim: int) -> Tensor:
    """Undo `flatten_for_quantize`; the result is a permuted view (mxfp/helpers.py:32-63)."""
    nd = len(ori_shape)
    d = block_dim % nd
    moved = list(ori_shape)
    moved.append(moved.pop(d))
    inv = list(range(nd))
    inv.insert(d, inv.pop(-1))
    return flatten_tensor.reshape(moved).permute(inv)


def _flat_contiguous(x: Tensor) -> Tensor:
    if x.dim() != 1:
        x = x.flatten()
    if not x.is_contiguous() or x.data_ptr() % 16:
        x = x.contiguous()
        if x.data_ptr() % 16:
            x = x.clone(memory_format=torch.contiguous_format)
    return x


# ---------------------------------------------------------------------------------------------------
# MXINT
# ---------------------------------------------------------------------------------------------------
def _mxint_fake_flat(flat: Tensor, meta: MXIntMeta, out_dtype: torch.dtype) -> Tensor:
    B = meta.block_size
    assert flat.numel() % B == 0, f"Input tensor size {flat.numel()} is not divisible by block size {B}."
    if meta.scale_bits != 8:
        raise NotImplementedError("mxint: only scale_bits=8 is supported")
    if not 2 <= meta.element_bits <= 8:
        raise NotImplementedError("mxint: element_bits must be between 2 and 8")
    di = _dtype_code(flat.dtype, "mxint")
    do = _dtype_code(out_dtype, "mxint")
    flat = _flat_contiguous(flat)
    ext = _binding()
    if ext:
        return ext.mx_fake(flat, 1, B, meta.element_bits, 0, out_dtype, _ceil_tab_ptr(flat.dtype))
    y = torch.empty(flat.shape, dtype=out_dtype, device=flat.device)
    with _on_device(flat):
        rc = _lib.lib().mxq_mxint_fake(flat.data_ptr(), y.data_ptr(), di, do, flat.numel() // B, B, meta.element_bits,
                                       _ceil_tab_ptr(flat.dtype), _stream(flat))
    _lib.check(rc, "mxq_mxint_fake")
    return y


def mxint_codes(x: Tensor, block_size: int, element_bits: int) -> tuple[Tensor, Tensor]:
    """Packed MXINT codes of an already-flattened tensor: (scales uint8 [n_blocks], mantissas int8 [n_blocks, B])."""
    _require_cuda(x, "mxint_codes")
    B = block_size
    assert x.numel() % B == 0, f"Input tensor size {x.numel()} is not divisible by block size {B}."
    if not 2 <= element_bits <= 8:
        raise NotImplementedError("mxint: element_bits must be between 2 and 8")
    di = _dtype_code(x.dtype, "mxint")
    flat = _flat_contiguous(x)
    n = flat.numel() // B
    mant = torch.empty((n, B), dtype=torch.int8, device=x.device)
    scales = torch.empty((n,), dtype=torch.uint8, device=x.device)
    with _on_device(x):
        rc = _lib.lib().mxq_mxint_extract(flat.data_ptr(), mant.data_ptr(), scales.data_ptr(), di, n, B, element_bits,
                                          _ceil_tab_ptr(x.dtype), _stream(x))
    _lib.check(rc, "mxq_mxint_extract")
    return scales, mant


def extract_mxint_components(x: Tensor, mxint_meta: MXIntMeta, percentile: float = 1.0) -> tuple[Tensor, Tensor]:
    """(scale [n_blocks,1], mantissa [n_blocks,B]), both integer-valued tensors of x.dtype (mxint/fake.py:11-56)."""
    _require_cuda(x, "extract_mxint_components")
    if percentile != 1.0:  # calibration-time clipping: tensor operations, see _mxint_candidates
        B = mxint_meta.block_size
        assert x.numel() % B == 0, f"Input tensor size {x.numel()} is not divisible by block size {B}."
        _dtype_code(x.dtype, "mxint")
        blocks = x.flatten().reshape(-1, B)
        x_max = blocks.abs().to(torch.float32).quantile(percentile, dim=1, keepdim=True).to(x.dtype)
        x_max = x_max.clamp(min=torch.finfo(x.dtype).tiny)
        scale = _ceil_log2_like_host(x_max)
        scale_bias = 2 ** (mxint_meta.scale_bits - 1) - 1
        mant = blocks / 2**scale * 2 ** (mxint_meta.element_bits - 1)
        scale = (scale + scale_bias).clamp(min=0, max=2**mxint_meta.scale_bits - 1)
        mant = mant.round().clamp(min=-(2 ** (mxint_meta.element_bits - 1)), max=2 ** (mxint_meta.element_bits - 1) - 1)
        return scale, mant
    if mxint_meta.scale_bits != 8:
        raise NotImplementedError("mxint: only scale_bits=8 is supported")
    scales, mant = mxint_codes(x, mxint_meta.block_size, mxint_meta.element_bits)
    # the reference keeps mantissas as floats, where a small negative value rounds to -0.0
    mant_f = torch.copysign(mant.to(x.dtype), x.reshape(mant.shape))
    return scales.view(-1, 1).to(x.dtype), mant_f


def compose_mxint_tensor(shared_scales: Tensor, elements: Tensor, mxint_meta: MXIntMeta) -> Tensor:
    """elements / 2**(bits-1) * 2**(scale-127), shape [n_blocks, B], dtype of `elements` (mxint/fake.py:59-80)."""
    _require_cuda(elements, "compose_mxint_tensor")
    do = _dtype_code(elements.dtype, "mxint")
    B = mxint_meta.block_size
    mant = elements.to(torch.int8).contiguous()
    sc = shared_scales.to(torch.uint8).contiguous()
    y = torch.empty(elements.shape, dtype=elements.dtype, device=elements.device)
    with _on_device(elements):
        rc = _lib.lib().mxq_mxint_compose(mant.data_ptr(), sc.data_ptr(), y.data_ptr(), do, mant.numel() // B, B,
                                          mxint_meta.element_bits, _stream(elements))
    _lib.check(rc, "mxq_mxint_compose")
    return torch.copysign(y, elements)  # int8 codes cannot carry the sign of a -0.0 mantissa


def mxint_quantizer_sim(
    tensor: Tensor,
    block_dim: int,
    mxint_meta: MXIntMeta,
    act_tensor: Tensor | None = None,
    dtype: torch.dtype | None = None,
    quantile_search: bool = False,
    cali_batch_size: int = 32,
) -> Tensor:
    """Quantize-dequantize along `block_dim` (mxint/mxint.py:14-171, non-search branch)."""
    _require_cuda(tensor, "mxint_quantizer_sim")
    if quantile_search:
        if act_tensor is None and mxint_meta.block_size == 32 and _is_last_dim_contiguous(tensor, block_dim):
            return mxint_clip_search(tensor, mxint_meta)[0]
        out = _mxint_clip_search(tensor, block_dim, mxint_meta, act_tensor, cali_batch_size)
        return out.to(tensor.dtype)
    ori_shape = tuple(tensor.shape)
    ndim = len(ori_shape)
    assert block_dim < ndim and block_dim >= -ndim
    if _is_last_dim_contiguous(tensor, block_dim):  # no permutation needed: the tensor already is a run of blocks
        return _mxint_fake_flat(tensor.view(-1), mxint_meta, dtype or tensor.dtype).view(ori_shape)
    flat = flatten_for_quantize(tensor, block_dim)
    y = _mxint_fake_flat(flat, mxint_meta, dtype or tensor.dtype)
    return permute_for_dequantize(y, ori_shape, block_dim)


def mxint_clip_search(tensor: Tensor, mxint_meta: MXIntMeta) -> tuple[Tensor, Tensor]:
    """The clipping search of mxint_quantizer_sim(quantile_search=True) without activations (mxint/mxint.py:40-136)
    for blocks of 32 along a contiguous last dimension, in one kernel.  Returns (fake-quantized tensor, uint8 index
    of the winning quantile per block)."""
    _require_cuda(tensor, "mxint_clip_search")
    dt = _dtype_code(tensor.dtype, "mxint")
    if mxint_meta.scale_bits != 8:
        raise NotImplementedError("mxint: only scale_bits=8 is supported")
    assert mxint_meta.block_size == 32 and tensor.numel() % 32 == 0
    flat = _flat_contiguous(tensor)
    n = flat.numel() // 32
    y = torch.empty_like(flat)
    choice = torch.empty((n,), dtype=torch.uint8, device=tensor.device)
    with _on_device(tensor):
        rc = _lib.lib().mxq_mxint_clip_search(flat.data_ptr(), y.data_ptr(), choice.data_ptr(), dt, n, 32,
                                              mxint_meta.element_bits, _ceil_tab_ptr(tensor.dtype), _stream(tensor))
    _lib.check(rc, "mxq_mxint_clip_search")
    return y.view(tensor.shape), choice


# The other forms of the calibration-time clipping search (mxint/mxint.py:40-136: with activations, block sizes other
# than 32, blocks along another dimension) are not on the inference path and run as the reference's own sequence of
# tensor operations on the tensor's device.  The one exception is the shared exponent, which uses the same
# host-derived table as the kernels instead of the device's log2.
_SEARCH_PERCENTILES = (1.0, 0.995, 0.99, 0.97, 0.95, 0.93, 0.90, 0.80, 0.70, 0.60, 0.50)


def _ceil_log2_like_host(x: Tensor) -> Tensor:
    """ceil(log2(x)) evaluated in x.dtype as torch computes it on this host; x > 0 and normal.  Result in x.dtype."""
    bits = x.float().contiguous().view(torch.int32)
    ex = bits >> 23
    man = ((bits >> 16) & 0x7F) if x.dtype == torch.bfloat16 else (bits & 0x7FFFFF)
    tab = torch.from_numpy(ceil_table(x.dtype).astype("int32")).to(x.device)
    return (ex - 127 + (man > tab[ex.long()]).to(torch.int32)).to(x.dtype)


def _mxint_candidates(blocks: Tensor, meta: MXIntMeta, percentiles: Tensor) -> Tensor:
    """Fake-quantized blocks for every clipping percentile: [len(percentiles), n_blocks, B] in blocks.dtype."""
    dt = blocks.dtype
    x_max = blocks.abs().to(torch.float32).quantile(percentiles, dim=1, keepdim=True).to(dt)
    x_max = x_max.clamp(min=torch.finfo(dt).tiny)
    scale = _ceil_log2_like_host(x_max)
    scale_bias = 2 ** (meta.scale_bits - 1) - 1
    x = blocks / 2**scale
    mant = x * 2 ** (meta.element_bits - 1)
    scale = (scale + scale_bias).clamp(min=0, max=2**meta.scale_bits - 1)
    mant = mant.round().clamp(min=-(2 ** (meta.element_bits - 1)), max=2 ** (meta.element_bits - 1) - 1)
    return mant / 2 ** (meta.element_bits - 1) * 2 ** (scale - scale_bias)


def _mxint_clip_search(tensor: Tensor, block_dim: int, meta: MXIntMeta, act_tensor: Tensor | None,
                       cali_batch_size: int) -> Tensor:
    _dtype_code(tensor.dtype, "mxint")
    B = meta.block_size
    ori_shape = tuple(tensor.shape)
    ndim = len(ori_shape)
    assert block_dim < ndim and block_dim >= -ndim
    target = tensor.flatten().reshape(-1, B)  # the error is taken against the tensor in its original order
    blocks = flatten_for_quantize(tensor, block_dim).flatten().reshape(-1, B)
    n_blocks = blocks.shape[0]
    percentiles = torch.tensor(_SEARCH_PERCENTILES, device=tensor.device, dtype=torch.float32)
    cand = _mxint_candidates(blocks, meta, percentiles).reshape(len(_SEARCH_PERCENTILES), n_blocks, B)
    if act_tensor is None:
        err = torch.norm(cand - target, p=2, dim=-1)
        best = torch.argmin(err, dim=0).reshape(-1)
    else:
        last = act_tensor.shape[-1]
        if last != B:
            assert last % B == 0
            act_tensor = act_tensor.view(*act_tensor.shape[:-1], last // B, B)
        err = torch.zeros([len(_SEARCH_PERCENTILES), n_blocks], device=tensor.device, dtype=tensor.dtype)
        with torch.no_grad():
            for b in range(0, act_tensor.shape[0], cali_batch_size):
                act_b = act_tensor[b : b + cali_batch_size]
                out_orig = torch.matmul(act_b, target.T)
                out_q = torch.einsum("asb,phb->pash", act_b, cand.to(act_tensor.dtype))
                err += torch.norm(out_q - out_orig, p=2, dim=(1, 2))
        best = torch.argmin(err, dim=0)
    chosen = cand[best, torch.arange(n_blocks, device=tensor.device)]
    return permute_for_dequantize(chosen, ori_shape, block_dim)


class MXIntQuantize(torch.autograd.Function):
    """Straight-through estimator around the quantizer (mxint/mxint.py:179-208)."""

    @staticmethod
    def forward(ctx, x, block_size, element_bits, block_dim, scale_bits, quantile_search):
        meta = MXIntMeta(block_size=block_size, scale_bits=scale_bits, element_bits=element_bits)
        return mxint_quantizer_sim(tensor=x, block_dim=block_dim, mxint_meta=meta, quantile_search=quantile_search)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output.clone(), None, None, None, None, None


def mxint_quantizer(
    x: Tensor,
    block_size: int,
    element_bits: int,
    block_dim: int = -1,
    scale_bits: int = 8,
    quantile_search: bool = False,
) -> Tensor:
    """MXINT fake quantization, same interface as chop.nn.quantizers.mxint_quantizer (mxint/mxint.py:211-251)."""
    if not (x.requires_grad and torch.is_grad_enabled()):  # nothing to differentiate: skip the autograd wrapper
        meta = MXIntMeta(block_size=block_size, scale_bits=scale_bits, element_bits=element_bits)
        return mxint_quantizer_sim(tensor=x, block_dim=block_dim, mxint_meta=meta, quantile_search=quantile_search)
    return MXIntQuantize.apply(x, block_size, element_bits, block_dim, scale_bits, quantile_search)


# ---------------------------------------------------------------------------------------------------
# MXFP
# ---------------------------------------------------------------------------------------------------
def _check_mxfp_meta(meta: MXFPMeta) -> None:
    if not meta.element_is_finite or meta.round_mode != "rn":
        raise NotImplementedError("mxfp: only element_is_finite=True with round_mode='rn' is provided "
                                  "(what chop's mxfp_quantizer hard-codes)")


def extract_mxfp_components(tensor: Tensor, mxfp_meta: MXFPMeta, percentile: float = 1.0) -> tuple[Tensor, Tensor]:
    """(scales uint8 [n_blocks,1], elements uint8 [n_blocks,B]) (mxfp/fake.py:12-72)."""
    _require_cuda(tensor, "extract_mxfp_components")
    if percentile != 1.0:
        raise NotImplementedError("extract_mxfp_components: percentile clipping returns no codes here; "
                                  "mxfp_clip_search(flat, meta, candidate=i) gives the dequantized blocks of the "
                                  "reference's clipping quantiles")
    _check_mxfp_meta(mxfp_meta)
    B = mxfp_meta.block_size
    assert tensor.numel() % B == 0
    di = _dtype_code(tensor.dtype, "mxfp")
    flat = _flat_contiguous(tensor)
    n = flat.numel() // B
    codes = torch.empty((n, B), dtype=torch.uint8, device=tensor.device)
    scales = torch.empty((n, 1), dtype=torch.uint8, device=tensor.device)
    with _on_device(tensor):
        rc = _lib.lib().mxq_mxfp_extract(flat.data_ptr(), codes.data_ptr(), scales.data_ptr(), di, n, B,
                                         mxfp_meta.element_exp_bits, mxfp_meta.element_frac_bits,
                                         _floor_tab_ptr(), _stream(tensor))
    _lib.check(rc, "mxq_mxfp_extract")
    return scales, codes


def compose_mxfp_tensor(scales: Tensor, elements: Tensor, mxfp_meta: MXFPMeta, output_dtype: torch.dtype) -> Tensor:
    """Flat dequantized tensor of `output_dtype` (mxfp/fake.py:75-104)."""
    assert scales.dtype == torch.uint8
    assert elements.dtype == torch.uint8
    _require_cuda(elements, "compose_mxfp_tensor")
    do = _dtype_code(output_dtype, "mxfp")
    B = mxfp_meta.block_size
    elements = elements.contiguous()
    scales = scales.contiguous()
    y = torch.empty((elements.numel(),), dtype=output_dtype, device=elements.device)
    with _on_device(elements):
        rc = _lib.lib().mxq_mxfp_compose(elements.data_ptr(), scales.data_ptr(), y.data_ptr(), do,
                                         elements.numel() // B, B, mxfp_meta.element_exp_bits,
                                         mxfp_meta.element_frac_bits, _stream(elements))
    _lib.check(rc, "mxq_mxfp_compose")
    return y


def _mxfp_fake_flat(flat: Tensor, meta: MXFPMeta, out_dtype: torch.dtype) -> Tensor:
    _check_mxfp_meta(meta)
    B = meta.block_size
    assert flat.numel() % B == 0
    di = _dtype_code(flat.dtype, "mxfp")
    do = _dtype_code(out_dtype, "mxfp")
    flat = _flat_contiguous(flat)
    ext = _binding()
    if ext:
        return ext.mx_fake(flat, 0, B, meta.element_exp_bits, meta.element_frac_bits, out_dtype, _floor_tab_ptr())
    y = torch.empty(flat.shape, dtype=out_dtype, device=flat.device)
    with _on_device(flat):
        rc = _lib.lib().mxq_mxfp_fake(flat.data_ptr(), y.data_ptr(), di, do, flat.numel() // B, B,
                                      meta.element_exp_bits, meta.element_frac_bits, _floor_tab_ptr(),
                                      _stream(flat))
    _lib.check(rc, "mxq_mxfp_fake")
    return y


def mxfp_quantizer_sim(
    tensor: Tensor,
    block_dim: int,
    mxfp_meta: MXFPMeta,
    act_tensor: Tensor | None = None,
    dtype: torch.dtype | None = None,
    quantile_search: bool = False,
    cali_batch_size: int = 32,
) -> Tensor:
    """Quantize-dequantize along `block_dim` (mxfp/mxfp.py:14-115, non-search branch)."""
    _require_cuda(tensor, "mxfp_quantizer_sim")
    if quantile_search:
        return _mxfp_clip_search(tensor, block_dim, mxfp_meta, act_tensor, dtype, cali_batch_size)
    ori_shape = tuple(tensor.shape)
    ndim = len(ori_shape)
    assert block_dim < ndim and block_dim >= -ndim
    if _is_last_dim_contiguous(tensor, block_dim):  # no permutation needed: the tensor already is a run of blocks
        return _mxfp_fake_flat(tensor.view(-1), mxfp_meta, dtype or tensor.dtype).view(ori_shape)
    flat = flatten_for_quantize(tensor, block_dim)
    y = _mxfp_fake_flat(flat, mxfp_meta, dtype or tensor.dtype)
    return permute_for_dequantize(y, ori_shape, block_dim)


def mxfp_clip_search(flat: Tensor, mxfp_meta: MXFPMeta, out_dtype: torch.dtype | None = None, candidate: int = -1,
                     want_metric: bool = False):
    """One launch of the MXFP search kernel on a flat run of blocks of 32.  candidate < 0: the search of
    mxfp_quantizer_sim(quantile_search=True) without activations (mxfp/mxfp.py:40-104); 0..10: only that clipping
    quantile.  Returns (dequantized flat tensor, uint8 winner per block, metric or None); `metric` holds what the
    reference's error compares with the tensor (raw code bytes scaled in uint8 arithmetic)."""
    _require_cuda(flat, "mxfp_clip_search")
    _check_mxfp_meta(mxfp_meta)
    if mxfp_meta.block_size != 32 or mxfp_meta.scale_exp_bits != 8:
        raise NotImplementedError("mxfp: the clipping search is provided for blocks of 32 with 8-bit scales")
    di = _dtype_code(flat.dtype, "mxfp")
    do = _dtype_code(out_dtype or flat.dtype, "mxfp")
    flat = _flat_contiguous(flat)
    assert flat.numel() % 32 == 0
    n = flat.numel() // 32
    y = torch.empty(flat.shape, dtype=out_dtype or flat.dtype, device=flat.device)
    choice = torch.empty((n,), dtype=torch.uint8, device=flat.device)
    metric = torch.empty_like(flat) if want_metric else None
    with _on_device(flat):
        rc = _lib.lib().mxq_mxfp_clip_search(flat.data_ptr(), y.data_ptr(), metric.data_ptr() if want_metric else None,
                                             choice.data_ptr(), di, do, n, 32, mxfp_meta.element_exp_bits,
                                             mxfp_meta.element_frac_bits, candidate, _floor_tab_ptr(), _stream(flat))
    _lib.check(rc, "mxq_mxfp_clip_search")
    return y, choice, metric


def _mxfp_clip_search(tensor: Tensor, block_dim: int, meta: MXFPMeta, act_tensor: Tensor | None,
                      dtype: torch.dtype | None, cali_batch_size: int) -> Tensor:
    ori_shape = tuple(tensor.shape)
    ndim = len(ori_shape)
    assert block_dim < ndim and block_dim >= -ndim
    in_order = _is_last_dim_contiguous(tensor, block_dim)
    flat = tensor.reshape(-1) if in_order else flatten_for_quantize(tensor, block_dim)
    restore = (lambda y: y.view(ori_shape)) if in_order else (lambda y: permute_for_dequantize(y, ori_shape, block_dim))
    if act_tensor is None and in_order:
        return restore(mxfp_clip_search(flat, meta, dtype)[0])
    # with activations, or with blocks along another dimension (the reference then compares against the tensor in
    # its original element order): one launch per candidate, errors and the running best as tensor operations
    B = meta.block_size
    target = tensor.flatten().reshape(-1, B)
    n_blocks = target.shape[0]
    best = torch.full([n_blocks], float("inf"), device=tensor.device, dtype=tensor.dtype)
    best_y = None
    if act_tensor is not None and act_tensor.shape[-1] != B:
        assert act_tensor.shape[-1] % B == 0
        act_tensor = act_tensor.view(*act_tensor.shape[:-1], act_tensor.shape[-1] // B, B)
    for i in range(len(_SEARCH_PERCENTILES)):
        y, _, metric = mxfp_clip_search(flat, meta, dtype, candidate=i, want_metric=True)
        y, q = y.view(n_blocks, B), metric.view(n_blocks, B)
        if best_y is None:
            best_y = y.clone()
        if act_tensor is not None:
            err = torch.zeros(n_blocks, device=tensor.device, dtype=tensor.dtype)
            for b in range(0, act_tensor.shape[0], cali_batch_size):
                act_b = act_tensor[b : b + cali_batch_size]
                diff = _act_product(act_b, q) - _act_product(act_b, target)
                err += torch.norm(diff, p=2, dim=tuple(range(diff.dim() - 1)))
        else:
            d = (q - target).abs_()
            err = torch.sum(d * d, 1)
        better = err < best
        best = torch.where(better, err, best)
        best_y[better] = y[better]
    return restore(best_y.reshape(-1))


def _act_product(act: Tensor, blocks: Tensor) -> Tensor:
    """act [..., B] @ blocks[n, B]^T on the package's own GEMM (the reduction is one block long)."""
    from .gemm import linear_forward

    lead = act.shape[:-1]
    a2 = act.reshape(-1, act.shape[-1]).to(blocks.dtype).contiguous()
    return linear_forward(a2, blocks.contiguous(), None, blocks.dtype).reshape(*lead, blocks.shape[0])


class MXFPQuantize(torch.autograd.Function):
    """Straight-through estimator around the quantizer (mxfp/mxfp.py:151-184)."""

    @staticmethod
    def forward(ctx, x, block_size, element_exp_bits, element_frac_bits, block_dim, scale_exp_bits, quantile_search):
        meta = MXFPMeta(
            block_size=block_size,
            scale_exp_bits=scale_exp_bits,
            element_exp_bits=element_exp_bits,
            element_frac_bits=element_frac_bits,
            element_is_finite=True,
            round_mode="rn",
        )
        return mxfp_quantizer_sim(tensor=x, block_dim=block_dim, mxfp_meta=meta, quantile_search=quantile_search)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output.clone(), None, None, None, None, None, None


def mxfp_quantizer(
    x: Tensor,
    block_size: int,
    element_exp_bits: int,
    element_frac_bits: int,
    block_dim: int = -1,
    scale_exp_bits: int = 8,
    quantile_search: bool = False,
) -> Tensor:
    """MXFP fake quantization, same interface as chop.nn.quantizers.mxfp_quantizer (mxfp/mxfp.py:187-230)."""
    if not (x.requires_grad and torch.is_grad_enabled()):  # nothing to differentiate: skip the autograd wrapper
        meta = _mxfp_meta(block_size, scale_exp_bits, element_exp_bits, element_frac_bits)
        return mxfp_quantizer_sim(tensor=x, block_dim=block_dim, mxfp_meta=meta, quantile_search=quantile_search)
    return MXFPQuantize.apply(x, block_size, element_exp_bits, element_frac_bits, block_dim, scale_exp_bits,
                              quantile_search)


# ---------------------------------------------------------------------------------------------------
# element-wise minifloat
# ---------------------------------------------------------------------------------------------------
def minifloat_quantizer_sim(tensor: Tensor, minifloat_meta: MinifloatMeta, output_dtype: torch.dtype | None = None) -> Tensor:
    """Element-wise quantize-dequantize (_minifloat_mx/minifloat.py:12-33)."""
    _require_cuda(tensor, "minifloat_quantizer_sim")
    if not minifloat_meta.is_finite or minifloat_meta.round_mode != "rn":
        raise NotImplementedError("minifloat: only is_finite=True with round_mode='rn' is provided")
    out_dtype = output_dtype or tensor.dtype
    di = _dtype_code(tensor.dtype, "minifloat")
    do = _dtype_code(out_dtype, "minifloat")
    x = tensor.contiguous()
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    with _on_device(x):
        rc = _lib.lib().mxq_minifloat_fake(x.data_ptr(), y.data_ptr(), di, do, x.numel(), minifloat_meta.exp_bits,
                                           minifloat_meta.frac_bits, _stream(x))
    _lib.check(rc, "mxq_minifloat_fake")
    return y


# ---------------------------------------------------------------------------------------------------
# block floating point
# ---------------------------------------------------------------------------------------------------
def _infer_block_shape(x_shape: list[int], block_shape: list[int]) -> list[int]:
    """Right-align block_shape with x_shape, -1 / oversize entries take the whole dim (utils.py:_infer_block_shape)."""
    nd = len(x_shape)
    if len(block_shape) >= nd:
        inferred = list(block_shape[-nd:])
    else:
        inferred = [-1] * (nd - len(block_shape)) + list(block_shape)
    return [x_shape[i] if inferred[i] == -1 or inferred[i] > x_shape[i] else inferred[i] for i in range(nd)]


def _bfp_tile(shape: tuple[int, ...], block_size: list[int], skip_first_dim: bool) -> tuple[int, int]:
    """(tile rows, tile columns) over the last two dims, following the reference's `block` dispatch
    (chop/nn/quantizers/utils.py:486-514): 1-D bias, 2-D activation (first dim never blocked), 2-D weight,
    3-D activation.  Tile rows == 1 means tiles of consecutive elements of the last dimension."""
    nd = len(shape)
    if nd == 1:
        assert skip_first_dim is False, "skip_first_dim must be False for bias to be blocked"
        return 1, _infer_block_shape(list(shape), block_size)[0]
    if nd == 2:
        ref_shape = [1, shape[1]] if skip_first_dim else list(shape)
        tile = _infer_block_shape(ref_shape, block_size)
        return tile[0], tile[1]
    if nd == 3:
        if not skip_first_dim:
            raise NotImplementedError("block 3d weight is not supported.")
        tile = _infer_block_shape([1, *shape[1:]], block_size)
        return tile[1], tile[2]
    raise RuntimeError(f"Unsupported x.ndim = {nd}")


def _block_fp_quantize(x: Tensor, width=12, exponent_width=8, exponent_bias=None, block_size=[16], skip_first_dim=True):
    _require_cuda(x, "block_fp_quantizer")
    if isinstance(block_size, int):
        block_size = [block_size]
    dt = _dtype_code(x.dtype, "block_fp")
    if exponent_bias in (None, "none", "None"):
        exponent_bias = 2 ** (exponent_width - 1) - 1
    bh, bw = _bfp_tile(tuple(x.shape), list(block_size), skip_first_dim)
    if x.numel() == 0:
        return x.clone()
    xc = x.contiguous()
    cols = xc.shape[-1]
    y = torch.empty_like(xc)
    lib = _lib.lib()
    with _on_device(x):
        if bh == 1 or x.dim() == 1 or xc.shape[-2] == 1:
            # tiles of consecutive elements of the last dimension
            rc = lib.mxq_bfp_fake(xc.data_ptr(), y.data_ptr(), dt, xc.numel() // cols, cols, bw, width, exponent_width,
                                  int(exponent_bias), _ceil_tab_ptr(x.dtype), _stream(x))
            what = "mxq_bfp_fake"
        else:
            rows = xc.shape[-2]
            rc = lib.mxq_bfp_fake_tiles(xc.data_ptr(), y.data_ptr(), dt, xc.numel() // (rows * cols), rows, cols, bh, bw,
                                        width, exponent_width, int(exponent_bias), _ceil_tab_ptr(x.dtype), _stream(x))
            what = "mxq_bfp_fake_tiles"
    _lib.check(rc, what)
    return y


class BlockFPQuantize(torch.autograd.Function):
    """Straight-through estimator (block_fp.py:85-108)."""

    @staticmethod
    def forward(ctx, x, width=12, exponent_width=8, exponent_bias=None, block_size=[16], skip_first_dim=True):
        return _block_fp_quantize(x, width, exponent_width, exponent_bias, block_size, skip_first_dim)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output.clone(), None, None, None, None, None


def block_fp_quantizer(
    x: Tensor,
    width: int = 12,
    exponent_width: int = 8,
    exponent_bias: int = None,
    block_size: list[int] = [16],
    skip_first_dim: bool = True,
):
    """Block floating point (MSFP) fake quantization, interface of chop.nn.quantizers.block_fp_quantizer
    (block_fp.py:111-142): one shared exponent per tile, sign-magnitude mantissas of `width-1` bits."""
    if not (x.requires_grad and torch.is_grad_enabled()):
        return _block_fp_quantize(x, width, exponent_width, exponent_bias, block_size, skip_first_dim)
    return BlockFPQuantize.apply(x, width, exponent_width, exponent_bias, block_size, skip_first_dim)


# entries of chop.nn.quantizers.quantizer_map (nn/quantizers/__init__.py:14-28) provided here
quantizer_map = {
    "mxfp": mxfp_quantizer,
    "mxint": mxint_quantizer,
    "block_fp": block_fp_quantizer,
}
