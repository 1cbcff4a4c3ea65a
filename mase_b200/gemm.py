"""Forward GEMM of the quantized Linear modules on the tcgen05 tensor cores (libmxq, include/mxq.h).

`linear_forward(x, weight, bias)` replaces the `F.linear` at the end of LinearMXFP / LinearMXInt / linearBlockFP
(chop/nn/quantized/modules/linear.py:895, :972; chop/nn/quantized/functional/linear.py:278).  Its operands already
hold quantized values: every value is a small-significand number times a power of two, exactly representable in
bf16 (and in tf32 for fp32 tensors), so products are exact and only the fp32 accumulation order differs from the
reference.

`MXOperand` / `mx_linear` are the block-scaled path: the operands stay as E4M3 codes with one E8M0 scale per 32
elements of K and are multiplied by `tcgen05.mma.kind::mxf8f6f4.block_scale`.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
import threading
from dataclasses import dataclass

import torch
from torch import Tensor

from . import _lib
from .quantizers import _DT, _floor_tab_ptr, _on_device, _require_cuda, _stream

_STATUS: dict[int, Tensor] = {}
_CHECK_EVERY_CALL = os.environ.get("MXQ_CHECK_STATUS", "0") == "1"

_STATUS_TEXT = {
    1: "TMA producer: wait for a free shared-memory slot ran out",
    2: "MMA issuer: wait for an operand tile ran out",
    3: "MMA issuer: wait for a free accumulator ran out",
    4: "epilogue: wait for a finished accumulator ran out",
    5: "CTA pair: the two CTAs got different tensor-memory addresses",
    7: "peer barrier: a GPU of the tensor-parallel group did not arrive within the wait limit",
}


_TLS = threading.local()
_EXT = None


def _ext():
    """The compiled torch binding (mase_b200/lib/_mxq_torch*.so, `python -m mase_b200.build`) or False when it has not
    been built: it issues the same C calls as the ctypes path below with a fraction of the per-call host cost."""
    global _EXT
    if _EXT is None:
        _EXT = False
        if os.environ.get("MXQ_NO_TORCH_BINDING", "0") != "1":
            from . import build

            path = build.ext_path()
            if os.path.exists(path):
                import importlib.util

                _lib.lib()  # libmxq.so first: the binding links against it
                spec = importlib.util.spec_from_file_location(build.EXT_NAME, path)
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                _EXT = mod
    return _EXT


@contextlib.contextmanager
def options(**fields):
    """Per-call GEMM options (`mxq_gemm_options` of include/mxq.h) for every GEMM this thread issues inside the
    `with` block: `max_ctas` (leave SMs to a concurrent kernel), `tiles` (_lib.TILES_AUTO / TILES_SINGLE /
    TILES_PAIRS), `no_split_k`, `no_transposed`, `wait_limit_ns`, `test_hook`, `flags` (_lib.GEMM_STATIC_B).  The options travel with each call into
    the library, which keeps no settings of its own; other threads are not affected.  Blocks nest: inner fields
    override outer ones."""
    prev = getattr(_TLS, "opts", None)
    merged = dict(prev[1]) if prev else {}
    merged.update(fields)
    _TLS.opts = (_lib.GemmOptions(**merged), merged)
    try:
        yield
    finally:
        _TLS.opts = prev


_FLAG_ONLY: dict[int, "_lib.GemmOptions"] = {}


def _options_ptr(static_b: bool = False, a_e5m2: bool = False):
    """Address of the options struct of this thread's `options(...)` block (None outside one), with the flags a call
    adds itself: MXQ_GEMM_STATIC_B (operand B is a weight packed long ago, which the small-M kernel may fetch ahead of
    the stream dependency) and MXQ_GEMM_A_E5M2 (operand A holds E5M2 bytes)."""
    extra = (_lib.GEMM_STATIC_B if static_b else 0) | (_lib.GEMM_A_E5M2 if a_e5m2 else 0)
    cur = getattr(_TLS, "opts", None)
    if not extra:
        return None if cur is None else ctypes.addressof(cur[0])
    if cur is None:
        opt = _FLAG_ONLY.get(extra)
        if opt is None:
            opt = _FLAG_ONLY[extra] = _lib.GemmOptions(flags=extra)
        return ctypes.addressof(opt)
    cache = cur[2] if len(cur) > 2 else {}
    if extra not in cache:
        fields = dict(cur[1])
        fields["flags"] = fields.get("flags", 0) | extra
        cache[extra] = _lib.GemmOptions(**fields)
        cur = _TLS.opts = (cur[0], cur[1], cache)
    return ctypes.addressof(cache[extra])


def _status(device: torch.device) -> Tensor:
    t = _STATUS.get(device.index)
    if t is None:
        t = _STATUS[device.index] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def check_status(device=None) -> None:
    """Synchronise and raise if a GEMM kernel on `device` reported that one of its bounded waits ran out."""
    devices = list(_STATUS) if device is None else [torch.device(device).index or 0]
    for idx in devices:
        t = _STATUS.get(idx)
        if t is None:
            continue
        code = int(t.item())
        if code:
            t.zero_()
            raise _lib.MxqError(f"GEMM kernel on cuda:{idx} gave up: {_STATUS_TEXT.get(code, code)}")


def _bias_args(bias: Tensor | None):
    if bias is None:
        return None, 0
    if bias.dtype not in _DT:
        raise NotImplementedError(f"bias dtype {bias.dtype} is not supported")
    return bias.contiguous(), _DT[bias.dtype]


def _tf32_split(t: Tensor) -> tuple[Tensor, Tensor]:
    """t = hi + lo with hi holding the top 11 significant bits (exact in tf32) and lo the rest (exact in fp32)."""
    hi = (t.view(torch.int32) & -8192).view(torch.float32)  # clear the low 13 mantissa bits
    return hi, t - hi


def linear_forward(x: Tensor, weight: Tensor, bias: Tensor | None, out_dtype: torch.dtype | None = None,
                   fp32_exact: bool = False) -> Tensor:
    """x[..., K] @ weight[N, K]^T + bias, output in x.dtype (or `out_dtype`); bf16 operands use kind::f16 (exact
    products), fp32 operands kind::tf32.  tf32 keeps 11 significant bits: callers whose fp32 operands are known to fit
    (MX / block-fp values of at most 11 significant bits) pass `fp32_exact=True`; any other fp32 operands (bypassed
    layers, weights that were never quantized) are split into a tf32-exact high part and a remainder and multiplied as
    hi*hi + hi*lo + lo*hi in one GEMM over 3K, which recovers fp32-level products (error ~2**-21 per product)."""
    _require_cuda(x, "linear_forward")
    if x.dtype != weight.dtype:
        raise RuntimeError(f"expected input and weight to have the same dtype, got {x.dtype} and {weight.dtype}")
    if x.dtype not in _DT:
        raise NotImplementedError(f"linear_forward: dtype {x.dtype} is not supported (float32 and bfloat16 are)")
    N, K = weight.shape
    if x.shape[-1] != K:
        raise RuntimeError(f"mat1 and mat2 shapes cannot be multiplied ({tuple(x.shape)} and {K}x{N})")
    ext = _ext()
    if ext and (x.dtype == torch.bfloat16 or fp32_exact) and K % (8 if x.dtype == torch.bfloat16 else 4) == 0:
        if bias is not None and bias.dtype not in _DT:
            raise NotImplementedError(f"bias dtype {bias.dtype} is not supported")
        out = ext.dense_linear(x, weight, bias, out_dtype, _status(x.device), _options_ptr() or 0)
        if _CHECK_EVERY_CALL:
            check_status(x.device)
        return out
    lead = x.shape[:-1]
    a = x.reshape(-1, K)
    if not a.is_contiguous() or a.data_ptr() % 16:
        a = a.contiguous().clone() if a.data_ptr() % 16 else a.contiguous()
    w = weight if weight.is_contiguous() else weight.contiguous()
    M = a.shape[0]
    if x.dtype == torch.float32 and not fp32_exact:
        a_hi, a_lo = _tf32_split(a)
        w_hi, w_lo = _tf32_split(w)
        a, w = torch.cat([a_hi, a_hi, a_lo], dim=1), torch.cat([w_hi, w_lo, w_hi], dim=1)
        K = 3 * K
    need = 8 if x.dtype == torch.bfloat16 else 4
    if K % need:
        # rows must be multiples of 16 bytes for the tensor maps: pad K with zeros (contributes nothing)
        pad = need - K % need
        a = torch.nn.functional.pad(a, (0, pad))
        w = torch.nn.functional.pad(w, (0, pad))
        K += pad
    out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    b, bdt = _bias_args(bias)
    st = _status(x.device)
    with _on_device(x):
        rc = _lib.lib().mxq_gemm_dense(a.data_ptr(), w.data_ptr(), out.data_ptr(), 0 if b is None else b.data_ptr(),
                                       _DT[x.dtype], _DT[out.dtype], bdt, M, N, K, st.data_ptr(), _options_ptr(),
                                       _stream(x))
    _lib.check(rc, "mxq_gemm_dense")
    if _CHECK_EVERY_CALL:
        check_status(x.device)
    return out.reshape(*lead, N)


def batched_product(a: Tensor, b: Tensor, out_dtype: torch.dtype | None = None, fp32_exact: bool = True) -> Tensor:
    """out[i] = a[i] @ b[i]^T for a[B, M, K] and b[B, N, K] in one launch: the GEMM's tensor maps carry the batch index
    as a third coordinate.  bf16 products are exact; fp32 operands run as tf32, which is exact for MX / block-fp values
    (`fp32_exact=True`); other fp32 operands are split into tf32-exact parts first, as in `linear_forward`."""
    _require_cuda(a, "batched_product")
    if a.dtype != b.dtype or a.dtype not in _DT:
        raise NotImplementedError(f"batched_product: dtypes {a.dtype} / {b.dtype} are not supported")
    assert a.dim() == 3 and b.dim() == 3 and a.shape[0] == b.shape[0] and a.shape[2] == b.shape[2]
    B, M, K = a.shape
    N = b.shape[1]
    if a.dtype == torch.float32 and not fp32_exact:
        a_hi, a_lo = _tf32_split(a)
        b_hi, b_lo = _tf32_split(b)
        a, b, K = torch.cat([a_hi, a_hi, a_lo], dim=2), torch.cat([b_hi, b_lo, b_hi], dim=2), 3 * K
    need = 8 if a.dtype == torch.bfloat16 else 4
    if K % need:  # rows must be multiples of 16 bytes for the tensor maps: pad K with zeros (contributes nothing)
        pad = need - K % need
        a, b, K = torch.nn.functional.pad(a, (0, pad)), torch.nn.functional.pad(b, (0, pad)), K + pad
    a = a if a.is_contiguous() and a.data_ptr() % 16 == 0 else a.contiguous().clone()
    b = b if b.is_contiguous() and b.data_ptr() % 16 == 0 else b.contiguous().clone()
    out = torch.empty((B, M, N), dtype=out_dtype or a.dtype, device=a.device)
    if B == 0 or M == 0 or N == 0:
        return out
    sa, sb = M * K, N * K  # multiples of 16 bytes because K is
    st = _status(a.device)
    with _on_device(a):
        rc = _lib.lib().mxq_gemm_dense_batched(a.data_ptr(), b.data_ptr(), out.data_ptr(), _DT[a.dtype], _DT[out.dtype], B, M,
                                               N, K, sa, sb, M * N, st.data_ptr(), _options_ptr(), _stream(a))
    _lib.check(rc, "mxq_gemm_dense_batched")
    if _CHECK_EVERY_CALL:
        check_status(a.device)
    return out


@dataclass
class MXOperand:
    """A [rows, K] matrix as tensor-core operands: hardware FP8 bytes and E8M0 scales in the MMA chunk layout."""

    codes: Tensor   # uint8 [rows, K] (E4M3 bytes, or E5M2 bytes with `e5m2`) or [rows, K / 2] (two E2M1 nibbles per byte, `fp4`)
    scales: Tensor  # uint8 [mxq_mma_scale_bytes(rows, K)]
    rows: int
    k: int
    fp4: bool = False  # weights only: MXFP4 codes nibble-packed; the copy engine expands them on the way to the MMA
    e5m2: bool = False  # MXFP8 with E5M2 elements: hardware E5M2 bytes, every block one scale step up (values halved)

    @property
    def format(self) -> int:
        return _lib.CODES_E2M1X2 if self.fp4 else (_lib.CODES_E5M2 if self.e5m2 else _lib.CODES_E4M3)


def mma_supported(exp_bits: int, frac_bits: int, block_size: int, k: int) -> bool:
    """Formats the block-scaled GEMM can take, blocks of 32 along K: elements that are E4M3 numbers (E <= 4, F <= 3),
    or E5M2."""
    return block_size == 32 and k % 32 == 0 and ((exp_bits <= 4 and frac_bits <= 3) or (exp_bits, frac_bits) == (5, 2))


def fp4_supported(exp_bits: int, frac_bits: int, k: int) -> bool:
    """Weights that can be kept as nibble-packed MXFP4: E2M1 elements and rows of whole 128-element chunks."""
    return exp_bits == 2 and frac_bits == 1 and k % 128 == 0


def pack_mx_operand(x: Tensor, exp_bits: int, frac_bits: int, fp4: bool = False) -> MXOperand:
    """MXFP(exp_bits, frac_bits), block 32 along the last dim, of a 2-D tensor, stored for the tensor cores.
    `fp4=True` (E2M1 weights): two codes per byte instead of one E4M3 byte per element."""
    _require_cuda(x, "pack_mx_operand")
    if x.dtype not in _DT:
        raise NotImplementedError(f"pack_mx_operand: dtype {x.dtype} is not supported")
    assert x.dim() == 2
    rows, k = x.shape
    if not mma_supported(exp_bits, frac_bits, 32, k):
        raise NotImplementedError("block-scaled operands need E <= 4 and F <= 3, or E5M2, and K divisible by 32")
    xc = x.contiguous()
    if xc.data_ptr() % 16:
        xc = xc.clone()
    lib = _lib.lib()
    scales = torch.empty((int(lib.mxq_mma_scale_bytes(rows, k)),), dtype=torch.uint8, device=x.device)
    if fp4:
        if not fp4_supported(exp_bits, frac_bits, k):
            raise NotImplementedError("nibble-packed operands need E2M1 elements and K divisible by 128")
        codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
        with _on_device(x):
            rc = lib.mxq_mxfp4_pack_mma(xc.data_ptr(), codes.data_ptr(), scales.data_ptr(), _DT[x.dtype], rows, k,
                                        _floor_tab_ptr(), _stream(x))
        _lib.check(rc, "mxq_mxfp4_pack_mma")
        return MXOperand(codes, scales, rows, k, True)
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    with _on_device(x):
        rc = lib.mxq_mxfp_pack_mma(xc.data_ptr(), codes.data_ptr(), scales.data_ptr(), _DT[x.dtype], rows, k, exp_bits,
                                   frac_bits, _floor_tab_ptr(), _stream(x))
    _lib.check(rc, "mxq_mxfp_pack_mma")
    return MXOperand(codes, scales, rows, k, False, (exp_bits, frac_bits) == (5, 2))


def pack_gated_operand(gate: Tensor, up: Tensor, exp_bits: int, frac_bits: int) -> MXOperand:
    """MXFP(exp_bits, frac_bits) tensor-core operand of silu(gate) * up in one pass over gate and up (bf16 [rows, k]
    views with the same row stride, e.g. the two halves of a [rows, 2k] GEMM output).  The product is rounded exactly
    as `torch.nn.functional.silu(gate) * up` rounds it in bf16, so codes and scales equal those of packing that
    tensor."""
    _require_cuda(gate, "pack_gated_operand")
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16:
        raise NotImplementedError("pack_gated_operand: gate and up must be bfloat16")
    assert gate.dim() == 2 and gate.shape == up.shape
    rows, k = gate.shape
    if not mma_supported(exp_bits, frac_bits, 32, k) or exp_bits > 4:
        raise NotImplementedError("the fused SiLU*mul pack needs E <= 4, F <= 3 and K divisible by 32")
    ok = lambda t: t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0  # noqa: E731
    if not (ok(gate) and ok(up) and gate.stride(0) == up.stride(0)):
        gate, up = gate.contiguous(), up.contiguous()
    lib = _lib.lib()
    codes = torch.empty((rows, k), dtype=torch.uint8, device=gate.device)
    scales = torch.empty((int(lib.mxq_mma_scale_bytes(rows, k)),), dtype=torch.uint8, device=gate.device)
    with _on_device(gate):
        rc = lib.mxq_silu_mul_pack_mma(gate.data_ptr(), up.data_ptr(), gate.stride(0), codes.data_ptr(), scales.data_ptr(),
                                       rows, k, exp_bits, frac_bits, _floor_tab_ptr(), _stream(gate))
    _lib.check(rc, "mxq_silu_mul_pack_mma")
    return MXOperand(codes, scales, rows, k)


def mx_gated_linear(gate: Tensor, up: Tensor, weight: MXOperand, bias: Tensor | None, exp_bits: int, frac_bits: int,
                    out_dtype: torch.dtype | None = None) -> Tensor:
    """(silu(gate) * up) quantized to MXFP(exp_bits, frac_bits) along K and multiplied with a packed weight, in one
    C call: the second half of a gated MLP without materialising the hidden state."""
    _require_cuda(gate, "mx_gated_linear")
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16:
        raise NotImplementedError("mx_gated_linear: gate and up must be bfloat16")
    K = gate.shape[-1]
    assert K == weight.k and gate.shape == up.shape
    lead = gate.shape[:-1]
    g2, u2 = gate.reshape(-1, K), up.reshape(-1, K)
    ok = lambda t: t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0  # noqa: E731
    if not (ok(g2) and ok(u2) and g2.stride(0) == u2.stride(0)):
        g2, u2 = g2.contiguous(), u2.contiguous()
    M, N = g2.shape[0], weight.rows
    lib = _lib.lib()
    ws_bytes = int(lib.mxq_mx_linear_workspace_bytes(M, K))
    ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=gate.device)
    out = torch.empty((M, N), dtype=out_dtype or gate.dtype, device=gate.device)
    bb, bdt = _bias_args(bias)
    st = _status(gate.device)
    with _on_device(gate):
        rc = lib.mxq_mx_gated_linear(g2.data_ptr(), u2.data_ptr(), g2.stride(0), weight.codes.data_ptr(),
                                     weight.scales.data_ptr(), weight.format, out.data_ptr(),
                                     0 if bb is None else bb.data_ptr(),
                                     _DT[out.dtype], bdt, M, N, K, exp_bits, frac_bits, _floor_tab_ptr(), ws.data_ptr(),
                                     ws_bytes, st.data_ptr(), _options_ptr(), _stream(gate))
    _lib.check(rc, "mxq_mx_gated_linear")
    if _CHECK_EVERY_CALL:
        check_status(gate.device)
    return out.reshape(*lead, N)


def mx_gemm(a: MXOperand, b: MXOperand, bias: Tensor | None, out_dtype: torch.dtype, static_b: bool = False) -> Tensor:
    """[a.rows, b.rows] = a @ b^T (+ bias) with block-scaled MXFP8 tensor-core MMAs, fp32 accumulation.
    static_b: b was packed before any kernel that may still be running on the stream was launched (a layer's weight);
    never set it for an operand that the stream is still producing."""
    assert a.k == b.k and not a.fp4, "the first operand holds one byte per element"
    out = torch.empty((a.rows, b.rows), dtype=out_dtype, device=a.codes.device)
    bb, bdt = _bias_args(bias)
    st = _status(a.codes.device)
    with _on_device(a.codes):
        rc = _lib.lib().mxq_gemm_mxf8(a.codes.data_ptr(), a.scales.data_ptr(), b.codes.data_ptr(), b.scales.data_ptr(),
                                      b.format, out.data_ptr(), 0 if bb is None else bb.data_ptr(), _DT[out_dtype], bdt, a.rows,
                                      b.rows, a.k, st.data_ptr(), _options_ptr(static_b, a.e5m2), _stream(a.codes))
    _lib.check(rc, "mxq_gemm_mxf8")
    if _CHECK_EVERY_CALL:
        check_status(a.codes.device)
    return out


def mx_linear(x: Tensor, weight: MXOperand, bias: Tensor | None, exp_bits: int, frac_bits: int,
              out_dtype: torch.dtype | None = None) -> Tensor:
    """Quantize x[..., K] to MXFP(exp_bits, frac_bits) along K and multiply with a packed weight (one C call;
    the packed activations live in a scratch tensor allocated here)."""
    _require_cuda(x, "mx_linear")
    if x.dtype not in _DT:
        raise NotImplementedError(f"mx_linear: dtype {x.dtype} is not supported")
    K = x.shape[-1]
    assert K == weight.k
    ext = _ext()
    if ext:
        if bias is not None and bias.dtype not in _DT:
            raise NotImplementedError(f"bias dtype {bias.dtype} is not supported")
        out = ext.mx_linear(x, weight.codes, weight.scales, weight.format, weight.rows, bias, exp_bits, frac_bits, out_dtype,
                            _floor_tab_ptr(), _status(x.device), _options_ptr() or 0)
        if _CHECK_EVERY_CALL:
            check_status(x.device)
        return out
    lead = x.shape[:-1]
    a = x.reshape(-1, K)
    if not a.is_contiguous() or a.data_ptr() % 16:
        a = a.contiguous().clone() if a.data_ptr() % 16 else a.contiguous()
    M, N = a.shape[0], weight.rows
    lib = _lib.lib()
    ws_bytes = int(lib.mxq_mx_linear_workspace_bytes(M, K))
    ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=x.device)
    out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    bb, bdt = _bias_args(bias)
    st = _status(x.device)
    with _on_device(x):
        rc = lib.mxq_mx_linear(a.data_ptr(), _DT[x.dtype], weight.codes.data_ptr(), weight.scales.data_ptr(),
                               weight.format, out.data_ptr(), 0 if bb is None else bb.data_ptr(), _DT[out.dtype], bdt, M, N, K, exp_bits,
                               frac_bits, _floor_tab_ptr(), ws.data_ptr(), ws_bytes, st.data_ptr(), _options_ptr(),
                               _stream(x))
    _lib.check(rc, "mxq_mx_linear")
    if _CHECK_EVERY_CALL:
        check_status(x.device)
    return out.reshape(*lead, N)
