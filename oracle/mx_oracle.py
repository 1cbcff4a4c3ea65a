"""CPU oracle for the MX / block-floating-point quantizers and the quantized Linear forward.

TEST INFRASTRUCTURE ONLY.  This file restates, on the CPU, the arithmetic of MASE's
`chop.nn.quantizers.{mxint,mxfp,_minifloat_mx,block_fp}` and of the `LinearMX*` forward.  It is the
checker that the CUDA path is compared against; nothing in the shipped package may import it.
Only the test-suite, the smoke entry point and the benchmark's CPU-baseline leg use it.

The restatement is written on the *integer fields* of the IEEE encodings (sign / biased exponent /
mantissa) rather than as the reference's chain of floating tensor ops, so that it documents what the
chain computes.  The one floating operation whose rounding is observable, `log2` of a block maximum,
is evaluated with `torch.log2` on the CPU in the same dtype the reference evaluates it in; the result
therefore follows the host's libm exactly as the reference would on this host.

Parity is pinned: `tests/golden/*.npz` were produced by importing the reference implementation itself
(`tests/golden/make_golden.py`) and every function here is checked against them bit-for-bit.

Reference locations (paths inside the MASE repository, `src/chop/...`):
  nn/quantizers/mxint/fake.py:11-80          extract_mxint_components / compose_mxint_tensor
  nn/quantizers/mxfp/fake.py:12-104          extract_mxfp_components / compose_mxfp_tensor
  nn/quantizers/_minifloat_mx/fake.py:11-149 extract/compose_minifloat_component
  nn/quantizers/mxfp/helpers.py:8-63         flatten_for_quantize / permute_for_dequantize
  nn/quantizers/block_fp.py:7-82             _block_fp_quantize
  nn/quantized/modules/linear.py:817-972     LinearMXFP / LinearMXInt
  nn/quantized/functional/linear.py:220-278  linearBlockFP
  nn/quantizers/mxint/mxint.py:40-136        MXINT clipping search
  nn/quantizers/mxfp/mxfp.py:40-104          MXFP clipping search
  passes/module/transforms/gptq/gptq.py      GPTQ with an MX inner quantizer
  nn/quantized/modules/llama/attention.py:130-457   quantized attention (MXFP / MXINT operands, minifloat rope and softmax)
  nn/quantized/modules/llama/mlp.py:48-77    gated MLP with a minifloat SiLU input
"""

from __future__ import annotations

import torch
from torch import Tensor

_I32 = torch.int32


# --------------------------------------------------------------------------------------------------
# layout helpers (mxfp/helpers.py:8-63)
# --------------------------------------------------------------------------------------------------
def flatten_blocks(x: Tensor, block_dim: int) -> Tensor:
    """Move `block_dim` last and flatten; blocks are then consecutive runs of the flat tensor."""
    nd = x.dim()
    d = block_dim % nd
    order = [i for i in range(nd) if i != d] + [d]
    return x.permute(order).reshape(-1)


def unflatten_blocks(flat: Tensor, shape: tuple[int, ...], block_dim: int) -> Tensor:
    """Inverse of `flatten_blocks`; returns a permuted view like the reference does."""
    nd = len(shape)
    d = block_dim % nd
    moved = [shape[i] for i in range(nd) if i != d] + [shape[d]]
    inv = list(range(nd - 1))
    inv.insert(d, nd - 1)
    return flat.reshape(moved).permute(inv)


def _pow2(k: Tensor) -> Tensor:
    """Exact 2**k as float64 for an integer tensor k (|k| well inside the double range)."""
    k = k.to(_I32)
    return torch.ldexp(torch.ones(k.shape, dtype=torch.float64), k)


# --------------------------------------------------------------------------------------------------
# MXINT (mxint/fake.py:11-80)
# --------------------------------------------------------------------------------------------------
def mxint_scale_exponent(x_blocks: Tensor) -> Tensor:
    """ceil(log2(block max)) evaluated in the input dtype, as int32 [n_blocks, 1].

    The block maximum is clamped from below by the smallest normal number of the dtype
    (mxint/fake.py:44) and `log2` is rounded to the input dtype before `ceil` (mxint/fake.py:45):
    for bf16 inputs this differs from the exact ceil(log2) for mantissas just above a power of two.
    """
    dt = x_blocks.dtype
    amax = x_blocks.abs().amax(dim=1, keepdim=True)
    amax = amax.clamp(min=torch.finfo(dt).tiny)
    return torch.log2(amax).ceil().to(_I32)


def _mxint_codes_for_exponent(xb: Tensor, s: Tensor, bits: int, scale_bits: int = 8) -> tuple[Tensor, Tensor]:
    """(scale [n,1], mantissa [n,block]) of blocks xb for shared exponents s (int32 [n,1])."""
    dt = xb.dtype
    half = 1 << (bits - 1)
    xd = xb.to(torch.float64)
    # x / 2**s * 2**(bits-1): exact power-of-two scalings (results below the dtype's normal range only
    # occur for values that round to zero anyway).  2**128 overflows to +inf in fp32 and bf16, so a
    # block whose exponent is 128 divides by infinity and every mantissa becomes (signed) zero.
    inf_blk = s >= 128
    v = xd * _pow2(half.bit_length() - 1 - s.clamp(max=127))
    v = torch.where(inf_blk, torch.copysign(torch.zeros_like(v), xd), v)
    m = torch.round(v).clamp(-half, half - 1)
    bias = (1 << (scale_bits - 1)) - 1
    sc = (s + bias).clamp(0, (1 << scale_bits) - 1)
    return sc.to(dt), m.to(dt)


def mxint_extract(x: Tensor, block: int, bits: int, scale_bits: int = 8) -> tuple[Tensor, Tensor]:
    """Returns (scale [n,1], mantissa [n,block]) in x.dtype, integer valued (mxint/fake.py:45-56)."""
    assert x.numel() % block == 0, "numel must be divisible by the block size"
    xb = x.reshape(-1, block)
    return _mxint_codes_for_exponent(xb, mxint_scale_exponent(xb), bits, scale_bits)


def mxint_compose(scale: Tensor, mant: Tensor, bits: int, scale_bits: int = 8) -> Tensor:
    """mant / 2**(bits-1) * 2**(scale-bias) in mant.dtype (mxint/fake.py:75-80)."""
    dt = mant.dtype
    bias = (1 << (scale_bits - 1)) - 1
    k = scale.to(_I32) - bias
    md = mant.to(torch.float64) / float(1 << (bits - 1))
    y = md * _pow2(k.clamp(max=127))
    # 2**128 is +inf in the working dtype: 0 * inf = nan, m * inf = +-inf
    big = k >= 128
    y = torch.where(big, md * float("inf"), y)
    return y.to(torch.float32).to(dt)


def mxint_fake(x: Tensor, block: int, bits: int, block_dim: int = -1, out_dtype=None) -> Tensor:
    """Quantize-dequantize (mxint/mxint.py:145-171)."""
    flat = flatten_blocks(x, block_dim)
    sc, m = mxint_extract(flat, block, bits)
    y = mxint_compose(sc, m, bits).reshape(-1)
    return unflatten_blocks(y, tuple(x.shape), block_dim).to(out_dtype or x.dtype)


# --------------------------------------------------------------------------------------------------
# minifloat element codec (_minifloat_mx/fake.py:11-149), is_finite=True, round "rn"
# --------------------------------------------------------------------------------------------------
def minifloat_encode(v: Tensor, E: int, F: int) -> Tensor:
    """fp32 tensor -> int32 codes (sign | exponent | fraction), reproducing the reference encoder.

    Quirks kept on purpose: the low 8 mantissa bits are dropped before rounding; a fraction that
    rounds up to 2**F is OR-ed into the exponent field, so the carry is lost when the exponent code
    is odd; the value 1.0 * 2**emin encodes as zero; there is a single, truncating subnormal binade.
    """
    v = v.to(torch.float32)
    bits = v.contiguous().view(_I32)
    neg = v < 0  # -0.0 is not negative
    a = bits & 0x7FFFFFFF
    ex = a >> 23
    flushed = ex == 0
    bias = (1 << (E - 1)) - 1
    top = (1 << E) - 1
    e = ex - 127
    m15 = (a & 0x7FFFFF) >> 8
    sh = 15 - F
    q = m15 >> sh
    rem = m15 & ((1 << sh) - 1)
    half = 1 << (sh - 1)
    f = q + ((rem > half) | ((rem == half) & ((q & 1) == 1))).to(_I32)
    ye = e + bias
    sub = (ye == 0) & (f != 0)
    f = torch.where(sub, (f | (1 << F)) >> 1, f)
    under = e < -bias
    over = e > top - bias
    f = torch.where(under, 0, f)
    ye = torch.where(under, 0, ye)
    f = torch.where(over, (1 << F) - 1, f)
    ye = torch.where(over, top, ye)
    f = torch.where(flushed, 0, f)
    ye = torch.where(flushed, 0, ye)
    code = (ye << F) | f
    return code + neg.to(_I32) * (1 << (E + F))


def minifloat_decode(code: Tensor, E: int, F: int) -> Tensor:
    """int codes -> fp32 values (_minifloat_mx/fake.py:96-149, is_finite=True)."""
    c = code.to(_I32)
    neg = (c >> (E + F)) & 1
    ye = (c >> F) & ((1 << E) - 1)
    f = c & ((1 << F) - 1)
    bias = (1 << (E - 1)) - 1
    fd = f.to(torch.float64) / float(1 << F)
    normal = _pow2(ye - bias) * (1.0 + fd)
    subn = float(2.0 ** (1 - bias)) * fd
    y = torch.where(ye == 0, subn, normal)
    y = torch.where(neg == 1, -y, y)
    return y.to(torch.float32)


def minifloat_fake(x: Tensor, E: int, F: int, out_dtype=None) -> Tensor:
    """Element-wise quantize-dequantize (_minifloat_mx/minifloat.py:12-33)."""
    return minifloat_decode(minifloat_encode(x, E, F), E, F).to(out_dtype or x.dtype)


# --------------------------------------------------------------------------------------------------
# MXFP (mxfp/fake.py:12-104)
# --------------------------------------------------------------------------------------------------
def mxfp_extract(x: Tensor, block: int, E: int, F: int, percentile: float = 1.0) -> tuple[Tensor, Tensor]:
    """Returns (scales uint8 [n,1], codes uint8 [n,block]).  `percentile` < 1 takes that quantile of |x| per block
    (linear interpolation between order statistics, `torch.quantile`) in place of the block maximum
    (mxfp/fake.py:57)."""
    assert x.numel() % block == 0
    xf = x.to(torch.float32).reshape(-1, block).contiguous()
    bits = xf.view(_I32)
    flushed = (bits & 0x7F800000) == 0
    xf = torch.where(flushed, torch.zeros_like(xf), xf)
    if percentile == 1.0:
        amax = xf.abs().amax(dim=1, keepdim=True)
    else:
        amax = xf.abs().quantile(percentile, dim=1, keepdim=True)
    all_zero = flushed.all(dim=1, keepdim=True)
    zero_q = amax == 0
    bias = (1 << (E - 1)) - 1
    emax_b = ((1 << E) - 1) - bias
    # floor(log2(amax)) in fp32
    lf = torch.log2(torch.where(zero_q, torch.ones_like(amax), amax)).floor().to(_I32)
    sh = (lf - emax_b).clamp(-127, 128)
    # amax == 0: log2(0) = -inf converts to the lowest int32, the subtraction of emax wraps around and the clamp
    # returns the top, 128.  The block is then divided by exp2(128) = inf and every element becomes +0.
    sh = torch.where(zero_q, torch.full_like(sh, 128), sh)
    scale = torch.where(all_zero, torch.zeros_like(sh), sh + 127).to(torch.uint8)
    # the reference divides in fp32 by exp2(sh) (a subnormal divisor for sh = -127)
    v = xf / torch.exp2(sh.to(torch.float32))
    v = torch.where(flushed, torch.zeros_like(v), v)
    codes = minifloat_encode(v, E, F).to(torch.uint8)
    return scale, codes


def mxfp_compose(scales: Tensor, codes: Tensor, E: int, F: int, out_dtype) -> Tensor:
    """decode(codes) * 2**(scale-127) in fp32, then cast (mxfp/fake.py:93-104)."""
    k = scales.to(_I32) - 127
    sf = torch.exp2(k.to(torch.float32))
    y = minifloat_decode(codes, E, F) * sf
    return y.reshape(-1).to(out_dtype)


def mxfp_fake(x: Tensor, block: int, E: int, F: int, block_dim: int = -1, out_dtype=None) -> Tensor:
    """Quantize-dequantize (mxfp/mxfp.py:106-115)."""
    flat = flatten_blocks(x, block_dim)
    sc, co = mxfp_extract(flat, block, E, F)
    y = mxfp_compose(sc, co, E, F, out_dtype or x.dtype)
    return unflatten_blocks(y, tuple(x.shape), block_dim)


# --------------------------------------------------------------------------------------------------
# calibration-time clipping search (mxint/mxint.py:40-136, mxfp/mxfp.py:40-104)
# --------------------------------------------------------------------------------------------------
SEARCH_PERCENTILES = (1.0, 0.995, 0.99, 0.97, 0.95, 0.93, 0.90, 0.80, 0.70, 0.60, 0.50)


def mxint_clip_search(x: Tensor, block: int, bits: int, block_dim: int = -1) -> tuple[Tensor, Tensor]:
    """Per block, the candidate among eleven clipping quantiles with the smallest 2-norm error
    (mxint/mxint.py:40-136 without activations).  Returns (fake-quantized tensor, index of the chosen candidate
    per block).  Intermediates live in x.dtype as in the reference; the error is taken against the tensor in its
    original element order."""
    dt = x.dtype
    target = x.reshape(-1, block)
    xb = flatten_blocks(x, block_dim).reshape(-1, block)
    errs, cands = [], []
    for p in SEARCH_PERCENTILES:
        q = torch.tensor([p], dtype=torch.float32)
        x_max = xb.abs().to(torch.float32).quantile(q, dim=1, keepdim=True)[0].to(dt).clamp(min=torch.finfo(dt).tiny)
        s = torch.log2(x_max).ceil().to(_I32)
        sc, m = _mxint_codes_for_exponent(xb, s, bits)
        cand = mxint_compose(sc, m, bits).reshape(-1, block)
        cands.append(cand)
        errs.append(torch.norm(cand - target, p=2, dim=-1))
    best = torch.argmin(torch.stack(errs), dim=0)
    chosen = torch.stack(cands)[best, torch.arange(xb.shape[0])]
    return unflatten_blocks(chosen.reshape(-1), tuple(x.shape), block_dim).to(dt), best


def mxfp_search_metric(scales: Tensor, codes: Tensor, F: int, dt) -> Tensor:
    """The per-element values the reference's MXFP search compares with the tensor (mxfp/mxfp.py:57-63): the raw
    code bytes divided by 2**(F-1), times 2**(scale - 127) evaluated in uint8 arithmetic, i.e. 2**k for
    k = (scale - 127) mod 256 below 8 and 0 otherwise."""
    k = (scales.to(_I32) - 127) & 255
    pw = torch.where(k < 8, torch.ones_like(k) << k.clamp(max=7), torch.zeros_like(k))
    return (codes.to(torch.float32) / 2 ** (F - 1) * pw.to(torch.float32)).to(dt)


def mxfp_clip_search(x: Tensor, block: int, E: int, F: int, block_dim: int = -1, out_dtype=None) -> tuple[Tensor, Tensor]:
    """mxfp_quantizer_sim(quantile_search=True) without activations (mxfp/mxfp.py:40-104): candidates in the order of
    SEARCH_PERCENTILES, each accepted only if its error is strictly below the best before it; the first candidate is
    the initial answer.  Returns (fake-quantized tensor, chosen candidate per block)."""
    dt = x.dtype
    target = x.flatten().reshape(-1, block)
    flat = flatten_blocks(x, block_dim)
    best_err = torch.full([target.shape[0]], float("inf"), dtype=dt)
    best_sc, best_co = mxfp_extract(flat, block, E, F, 1.0)
    best_sc, best_co = best_sc.clone(), best_co.clone()
    chosen = torch.zeros(target.shape[0], dtype=torch.int64)
    for i, p in enumerate(SEARCH_PERCENTILES):
        sc, co = mxfp_extract(flat, block, E, F, p)
        d = mxfp_search_metric(sc, co, F, dt)
        d = (d - target).abs()
        err = (d * d).sum(1)
        better = err < best_err
        best_err = torch.where(better, err, best_err)
        best_sc[better], best_co[better], chosen[better] = sc[better], co[better], i
    y = mxfp_compose(best_sc, best_co, E, F, out_dtype or dt)
    return unflatten_blocks(y, tuple(x.shape), block_dim), chosen


# --------------------------------------------------------------------------------------------------
# GPTQ with an MX inner quantizer (passes/module/transforms/gptq/gptq.py:17-123)
# --------------------------------------------------------------------------------------------------
def gptq_hessian(batches) -> Tensor:
    """Running average of 2/n * X^T X over calibration batches [b, s, in] (gptq.py:28-38)."""
    H, n = None, 0
    for x in batches:
        x = x.unsqueeze(0) if x.dim() == 2 else x
        b = x.shape[0]
        x2 = x.reshape(-1, x.shape[-1]).t()
        if H is None:
            H = torch.zeros(x2.shape[0], x2.shape[0])
        H *= n / (n + b)
        n += b
        x2 = (2 / n) ** 0.5 * x2.float()
        H += x2.matmul(x2.t())
    return H


def gptq_quantize(w: Tensor, hessian: Tensor, quantize_block, block: int, percdamp: float = 0.01) -> Tensor:
    """Column blocks of `block` weights are quantized left to right; the error of each block, weighted by the
    inverse Hessian's Cholesky factor, is fed forward into the columns not yet quantized (gptq.py:40-118).
    `quantize_block(W1)` is the inner fake-quantizer of a [rows, block] slice."""
    W = w.clone()
    H = hessian.clone()
    cols = W.shape[1]
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W[:, dead] = 0
    idx = torch.arange(cols)
    H[idx, idx] += percdamp * torch.mean(torch.diag(H))
    H = torch.linalg.cholesky(H)
    H = torch.cholesky_inverse(H)
    Hinv = torch.linalg.cholesky(H, upper=True)
    Q = torch.zeros_like(W)
    for c0 in range(0, cols, block):
        c1 = min(c0 + block, cols)
        W1 = W[:, c0:c1].clone()
        Q1 = quantize_block(W1)
        err = (W1 - Q1) / torch.diag(Hinv[c0:c1, c0:c1]).unsqueeze(0)
        Q[:, c0:c1] = Q1
        W[:, c1:] -= err.matmul(Hinv[c0:c1, c1:])
    return Q


# --------------------------------------------------------------------------------------------------
# block floating point, tiles of `bs` consecutive elements of the last dim (block_fp.py:7-82)
# --------------------------------------------------------------------------------------------------
def bfp_fake_rows(x: Tensor, width: int, exponent_width: int, exponent_bias, bs: int) -> Tensor:
    """Row-tile block floating point.

    Covers the tilings of the reference in which a tile is `bs` consecutive elements of the last
    dimension: 1-D biases, 2-D activations (`skip_first_dim=True`, any block_size), 2-D weights and
    3-D activations with block_size `[1, bs]`.  A ragged last tile is padded with zeros
    (utils.py:_infer_padding_shape).  Every step that the reference evaluates in x.dtype is rounded
    to x.dtype here as well.
    """
    dt = x.dtype
    shape = x.shape
    C = shape[-1]
    bs = min(bs, C)
    x2 = x.reshape(-1, C)
    R = x2.shape[0]
    pad = (-C) % bs
    xp = torch.nn.functional.pad(x2, (0, pad)) if pad else x2
    xb = xp.reshape(R, -1, bs)
    amax = xb.abs().amax(dim=2, keepdim=True)
    # tiles that are entirely zero take a substitute maximum (block_fp.py:40-44); every element of
    # such a tile is returned unquantized below, so the substitute never reaches the output
    amax = torch.where(amax == 0, torch.ones_like(amax), amax)
    if exponent_bias in (None, "none", "None"):
        exponent_bias = 2 ** (exponent_width - 1) - 1
    e_max = 2**exponent_width - 1 - exponent_bias
    e_min = -exponent_bias
    mb = width - 1
    e = torch.log2(amax).ceil().clamp(e_min, e_max).to(_I32)
    val = (xb.abs() + 1e-9).to(dt)  # rounded to x.dtype
    sgn = torch.sign((xb + 1e-9).to(dt)).to(torch.float64)
    vd = val.to(torch.float64)
    scaled = vd * _pow2((mb - e).clamp(min=-1000, max=1000))
    scaled = torch.where(e >= 128, torch.zeros_like(scaled), scaled)  # division by 2**128 = inf
    # the clamp bound is converted to x.dtype by torch.clamp: 2**mb - 1 is not a bf16 number for mb > 8
    hi = float(torch.tensor(float(2**mb - 1)).to(dt))
    mi = torch.round(scaled).clamp(0, hi)
    y = sgn * _pow2(e.clamp(max=127)) * (mi / float(2**mb))
    y = torch.where((e >= 128) & (mi == 0), torch.full_like(y, float("nan")), y)
    y = y.to(torch.float32).to(dt).reshape(R, -1)[:, :C]
    close = x2.to(torch.float64).abs() <= float(torch.tensor(1e-8).to(dt))
    # (~close) * y + close * x, evaluated literally so that signed zeros follow the reference
    out = (~close).to(dt) * y + close.to(dt) * x2
    return out.reshape(shape)


def bfp_fake_tiles(x: Tensor, width: int, exponent_width: int, exponent_bias, bh: int, bw: int) -> Tensor:
    """Block floating point with tiles of bh x bw over the last two dimensions (2-D weights with
    `skip_first_dim=False`, 3-D activations: utils.py:_block_2d_weight / _block_3d_activation).  Ragged edges
    are padded with zeros at the end of each dimension.  The reference reassembles the tiles with F.fold, which
    adds them into a zero tensor, so a -0.0 result becomes +0.0 on this route."""
    shape = x.shape
    R, C = shape[-2], shape[-1]
    bh, bw = min(bh, R), min(bw, C)
    x3 = x.reshape(-1, R, C)
    B = x3.shape[0]
    pr, pc = (-R) % bh, (-C) % bw
    xp = torch.nn.functional.pad(x3, (0, pc, 0, pr))
    Rp, Cp = R + pr, C + pc
    tiles = xp.reshape(B, Rp // bh, bh, Cp // bw, bw).permute(0, 1, 3, 2, 4).reshape(-1, bh * bw)
    yt = bfp_fake_rows(tiles, width, exponent_width, exponent_bias, bh * bw)
    y = yt.reshape(B, Rp // bh, Cp // bw, bh, bw).permute(0, 1, 3, 2, 4).reshape(B, Rp, Cp)[:, :R, :C]
    return (y + torch.zeros_like(y)).reshape(shape)  # -0.0 + 0.0 = +0.0, as after F.fold


# --------------------------------------------------------------------------------------------------
# quantized Linear forward (quantized/modules/linear.py:877-895, 956-972; functional/linear.py:220-278)
# --------------------------------------------------------------------------------------------------
def linear_mxfp(x: Tensor, w_q: Tensor, bias, cfg: dict) -> Tensor:
    """Forward of LinearMXFP with an already-quantized weight: quantize x along K, then GEMM in fp32.

    The fp32 GEMM of the quantized operands is the value the CUDA path is compared with; the
    reference's own bf16 `F.linear` differs from it only by the library's accumulation/rounding.
    """
    if cfg.get("data_in_block_size") is not None and cfg.get("data_in_exponent_width") is not None:
        x = mxfp_fake(x, cfg["data_in_block_size"], cfg["data_in_exponent_width"], cfg["data_in_frac_width"])
    y = torch.nn.functional.linear(x.float(), w_q.float(), None if bias is None else bias.float())
    return y


def linear_mxint(x: Tensor, w_q: Tensor, bias, cfg: dict) -> Tensor:
    if cfg.get("data_in_block_size") is not None and cfg.get("data_in_width") is not None:
        x = mxint_fake(x, cfg["data_in_block_size"], cfg["data_in_width"])
    return torch.nn.functional.linear(x.float(), w_q.float(), None if bias is None else bias.float())


def linear_block_fp(x: Tensor, w: Tensor, bias, cfg: dict) -> Tensor:
    xq = bfp_fake_rows(x, cfg["data_in_width"], cfg["data_in_exponent_width"], cfg["data_in_exponent_bias"],
                       cfg["data_in_block_size"][-1])
    wq = bfp_fake_rows(w, cfg["weight_width"], cfg["weight_exponent_width"], cfg["weight_exponent_bias"],
                       cfg["weight_block_size"][-1])
    bq = None
    if bias is not None:
        bq = bfp_fake_rows(bias, cfg["bias_width"], cfg["bias_exponent_width"], cfg["bias_exponent_bias"],
                           cfg["bias_block_size"][-1]).float()
    return torch.nn.functional.linear(xq.float(), wq.float(), bq)


# --------------------------------------------------------------------------------------------------
# quantized attention and gated MLP (nn/quantized/modules/llama/attention.py:130-457, mlp.py:48-77)
# --------------------------------------------------------------------------------------------------
def _operand_quantizer(fmt: str, cfg: dict):
    if fmt == "mxfp":
        return lambda t: mxfp_fake(t, cfg["data_in_block_size"], cfg["data_in_exponent_width"], cfg["data_in_frac_width"], -1)
    return lambda t: mxint_fake(t, cfg["data_in_block_size"], cfg["data_in_width"], -1)


def _minifloat(t: Tensor, cfg: dict) -> Tensor:
    return minifloat_fake(t, cfg["data_in_exponent_width"], cfg["data_in_frac_width"])


def _rotate_half(t: Tensor) -> Tensor:
    half = t.shape[-1] // 2
    return torch.cat((-t[..., half:], t[..., :half]), dim=-1)


def _head_rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    xf = x.to(torch.float32)
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * xf.to(x.dtype)


def attention_mx(hidden: Tensor, weights: dict, cos: Tensor, sin: Tensor, mask, fmt: str, q_config: dict, heads: int,
                 kv_heads: int, cached: bool, qk_norm_eps: float | None = None) -> tuple[Tensor, Tensor]:
    """Forward of the reference's MX attention block with plain Linear projections: minifloat cos / sin in the rotary
    embedding, MX key / value states when a cache is attached, MX queries into Q K^T, scaling, mask, minifloat input
    of an fp32 softmax, MX probabilities into P V (attention.py:148-214, 334-394).  `qk_norm_eps` adds the Qwen3
    variant's RMS norms of queries and keys over the head dimension.  Returns (output, probabilities)."""
    B, S, _ = hidden.shape
    lin = torch.nn.functional.linear
    q = lin(hidden, weights["q_proj.weight"]).view(B, S, heads, -1)
    k = lin(hidden, weights["k_proj.weight"]).view(B, S, kv_heads, -1)
    if qk_norm_eps is not None:  # the Qwen3 variant (qwen3/attention.py:47-53)
        q = _head_rms_norm(q, weights["q_norm.weight"], qk_norm_eps)
        k = _head_rms_norm(k, weights["k_norm.weight"], qk_norm_eps)
    q, k = q.transpose(1, 2), k.transpose(1, 2)
    v = lin(hidden, weights["v_proj.weight"]).view(B, S, kv_heads, -1).transpose(1, 2)
    c, s_ = _minifloat(cos, q_config["rope"]).unsqueeze(1), _minifloat(sin, q_config["rope"]).unsqueeze(1)
    q, k = q * c + _rotate_half(q) * s_, k * c + _rotate_half(k) * s_
    if cached:
        kv_q = _operand_quantizer(fmt, q_config["kv_cache"])
        k, v = kv_q(k), kv_q(v)
    rep = heads // kv_heads
    k = k[:, :, None].expand(B, kv_heads, rep, S, k.shape[-1]).reshape(B, heads, S, -1)
    v = v[:, :, None].expand(B, kv_heads, rep, S, v.shape[-1]).reshape(B, heads, S, -1)
    q = _operand_quantizer(fmt, q_config["qk_matmul"])(q)
    scores = torch.matmul(q, k.transpose(2, 3)) * (q.shape[-1] ** -0.5)
    if mask is not None:
        scores = scores + mask[:, :, :, :S]
    probs = torch.softmax(_minifloat(scores, q_config["softmax"]).to(torch.float32), dim=-1).to(scores.dtype)
    probs = _operand_quantizer(fmt, q_config["av_matmul"])(probs)
    out = torch.matmul(probs, v).transpose(1, 2).contiguous().reshape(B, S, -1)
    return lin(out, weights["o_proj.weight"]), probs


def gated_mlp_minifloat(x: Tensor, gate_w: Tensor, up_w: Tensor, down_w: Tensor, cfg: dict) -> Tensor:
    """down(silu(minifloat(gate(x))) * up(x)) (mlp.py:56-61 with functional/silu.py:43-58)."""
    lin = torch.nn.functional.linear
    return lin(torch.nn.functional.silu(_minifloat(lin(x, gate_w), cfg)) * lin(x, up_w), down_w)
