// Packing of MXFP operands for the block-scaled tensor-core GEMM: per-lane routines of the pack kernels in
// mxq_quant.cu (hardware E4M3 bytes plus E8M0 scale bytes in the tensor-core chunk layout).
#pragma once

#include <cuda_fp8.h>

#include "mxq_common.cuh"

namespace mxq {

template <typename T>
__device__ __forceinline__ T group_max(T v, int group) {
  for (int o = 1; o < group; o <<= 1) {
    T w = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = v > w ? v : w;
  }
  return v;
}

// Fast path of the MXFP element codec.
//
// With K = (biased exponent of the block maximum) - (2**E - 1), an element whose biased fp32 exponent is ex has
// the minifloat exponent code ye = ex - K.  When K >= 1 and every element of the vector has ye >= 1 (no
// subnormal code, no underflow, no flushed input), quantize-dequantize reduces to rounding |x| to F fraction
// bits (half to even, after dropping the low 8 fp32 mantissa bits) with the block scale cancelling out, except
// that a fraction carry is lost when ye is odd (the reference ORs the carry into the exponent field): then the
// result is 2**e instead of 2**(e+1).  That is a handful of integer operations on the bit patterns; for bf16
// tensors two elements are processed per 32-bit register.  Everything else takes the general element codec.
template <int F>
__device__ __forceinline__ uint32_t mxfp_round_pair(uint32_t a2, uint32_t kodd2) {
  constexpr uint32_t kHalf2 = ((1u << (6 - F)) - 1u) * 0x00010001u;
  constexpr uint32_t kMask2 = ((0xFFFFu << (7 - F)) & 0xFFFFu) * 0x00010001u;
  const uint32_t lsb2 = (a2 >> (7 - F)) & 0x00010001u;
  uint32_t y2 = (a2 + kHalf2 + lsb2) & kMask2;                   // no carry crosses bit 15: a2 < 0x7F80 per half
  y2 -= (y2 ^ a2) & (a2 ^ kodd2) & 0x00800080u;                  // exponent lsb flipped (carry) and ye odd
  return y2;
}
// The same on vectors that also hold elements with ye <= 0 (subnormal codes and underflow), still with K >= 1 and no
// inf / nan.  With lo = the pattern of 2**(K - 127):
//   ye == 0 : the F-bit rounded fraction f is stored as (f | 2**F) >> 1, or as 0 when f == 0: the output keeps the
//             element's exponent and the rounded fraction with its last bit cleared; a carry out of the binade gives
//             lo itself (the OR loses it), and f == 0 <=> |x| <= lo + half an F-bit step gives zero;
//   ye <  0 : zero.
// The sign survives unless the input is flushed (biased exponent 0, -0.0 included) or x / 2**sh rounds to zero in
// fp32, i.e. for |x| patterns from `tmin` up.  The three thresholds become per-element masks with one packed bf16
// comparison each.
struct SubThresholds2 {
  __nv_bfloat162 t1, thr, tmin;  // first normal pattern, first pattern that does not round to zero, sign threshold
};
template <int E, int F>
__device__ __forceinline__ SubThresholds2 sub_thresholds2(int K) {
  constexpr int kBias = (1 << (E - 1)) - 1;
  const uint32_t lo = (uint32_t)K << 7;
  const uint32_t t1 = (lo + 0x80u) * 0x00010001u;
  const uint32_t thr = (lo + (1u << (6 - F)) + 1u) * 0x00010001u;
  const uint32_t tmin = (uint32_t)max(0x80, ((K + kBias - 150) << 7) + 1) * 0x00010001u;
  SubThresholds2 t;
  t.t1 = *reinterpret_cast<const __nv_bfloat162 *>(&t1);
  t.thr = *reinterpret_cast<const __nv_bfloat162 *>(&thr);
  t.tmin = *reinterpret_cast<const __nv_bfloat162 *>(&tmin);
  return t;
}
// r2 = two raw bf16 elements; returns the two quantize-dequantized elements, signs included
template <int F>
__device__ __forceinline__ uint32_t mxfp_round_pair_sub(uint32_t r2, uint32_t kodd2, const SubThresholds2 &t) {
  constexpr uint32_t kHalf2 = ((1u << (6 - F)) - 1u) * 0x00010001u;
  constexpr uint32_t kMask2 = ((0xFFFFu << (7 - F)) & 0xFFFFu) * 0x00010001u;
  constexpr uint32_t kLsb2 = (1u << (7 - F)) * 0x00010001u;
  const uint32_t a2 = r2 & 0x7FFF7FFFu;
  const __nv_bfloat162 av = *reinterpret_cast<const __nv_bfloat162 *>(&a2);
  const uint32_t normal = __hge2_mask(av, t.t1);
  const uint32_t nonzero = __hge2_mask(av, t.thr);
  const uint32_t signed_ = __hge2_mask(av, t.tmin);
  const uint32_t lsb2 = (a2 >> (7 - F)) & 0x00010001u;
  uint32_t y2 = (a2 + kHalf2 + lsb2) & kMask2;
  y2 -= (y2 ^ a2) & 0x00800080u & ((a2 ^ kodd2) | ~normal);  // carry lost: ye odd, or ye == 0
  y2 &= ~(kLsb2 & ~normal);
  return (y2 & nonzero) | (r2 & signed_ & 0x80008000u);
}
// fp32 version; `b` = raw bits, K as above
template <int E, int F>
__device__ __forceinline__ uint32_t mxfp_round_one_sub(uint32_t b, int K) {
  constexpr int kBias = (1 << (E - 1)) - 1;
  constexpr uint32_t kHalf = (1u << (22 - F)) - 1u;
  constexpr uint32_t kMask = ~((1u << (23 - F)) - 1u);
  const uint32_t a = b & 0x7FFFFFFFu, at = a & 0x7FFFFF00u;
  const uint32_t lo = (uint32_t)K << 23;
  const bool normal = a >= lo + 0x00800000u;
  const uint32_t lsb = (at >> (23 - F)) & 1u;
  uint32_t y = (at + kHalf + lsb) & kMask;
  y -= (y ^ at) & 0x00800000u & (normal ? (at ^ ((uint32_t)K << 23)) : 0xFFFFFFFFu);
  if (!normal) y &= ~(1u << (23 - F));
  if (a < lo + (1u << (22 - F)) + 0x100u) y = 0;
  if (a >= (uint32_t)max(0x00800000, ((K + kBias - 150) << 23) + 1)) y |= b & 0x80000000u;
  return y;
}
template <int F>
__device__ __forceinline__ uint32_t mxfp_round_one(uint32_t at, uint32_t kodd) {
  constexpr uint32_t kHalf = (1u << (22 - F)) - 1u;
  constexpr uint32_t kMask = ~((1u << (23 - F)) - 1u);
  const uint32_t lsb = (at >> (23 - F)) & 1u;
  uint32_t y = (at + kHalf + lsb) & kMask;
  y -= (y ^ at) & (at ^ kodd) & 0x00800000u;
  return y;
}

// Operands for the block-scaled tensor-core GEMM: blocks of 32 along K of a [rows, K] matrix.
//   codes  : one hardware E4M3 byte per element, row-major [rows, K];
//   scales : E8M0 bytes in chunks of 512 bytes per (128 rows x 128 columns of K), chunk (r/128, k/128) at
//            ((r/128) * ceil(K/128) + k/128) * 512, byte (r%32)*16 + ((r%128)/32)*4 + (k%128)/32 inside a chunk --
//            the arrangement tcgen05.cp (32x128b.warpx4) moves into tensor memory unchanged.
// Every element keeps the exact value of the reference's (E, F) code times its scale: minifloat formats with
// E <= 4 and F <= 3 are subsets of E4M3.  One exception: the reference's E4M3 uses the top code (480) as a
// number, which is NaN to the hardware.  A block that contains it is stored one binade lower with its scale
// raised by one; only elements of the two lowest binades of such a block can round (by at most 2**-16 of the
// block maximum).
//
// pack_f32 handles one 16-byte vector of 4 fp32 elements; a block of 32 is shared by 8 neighbouring lanes, so it must
// be called by all 32 lanes of a warp together (lanes without data pass zeros).  It returns the vector's four E4M3
// bytes and the block's E8M0 scale.
template <int E, int F>
__device__ __forceinline__ uint32_t pack_f32(const uint4 &raw, const Log2Tab &tab, int &scale_out) {
  constexpr int kGroup = 8;
  constexpr int kTop = (1 << E) - 1;
  constexpr int kBias = (1 << (E - 1)) - 1;
  constexpr int kEmax = kTop - kBias;
  const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t a[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) a[k] = r[k] & 0x7FFFFFFFu;
  const uint32_t m = group_max(max(max(a[0], a[1]), max(a[2], a[3])), kGroup);
  const uint32_t amax = (m >> 23) ? m : 0u;
  const int exm = (int)(amax >> 23);
  int up = 0;
  const uint32_t man = amax & 0x7FFFFFu;
  if (man >= 0x7FFF00u) up = (0x7FFFFFu - man) < tab.t[exm] ? 1 : 0;
  const int K = exm + up - kTop;
  const uint32_t kodd = (K & 1) ? 0x00800000u : 0u;
  // `fast`: the block's scale is not clamped, elements with exponent code >= 2 are handled on bit patterns.
  // `clean`: every element of this vector is such an element; the others are patched one by one afterwards.
  const bool fast = K >= 1;
  const uint32_t t1 = (uint32_t)(K + 2) << 23;  // smallest |x| pattern with exponent code >= 2
  bool clean = true;
#pragma unroll
  for (int k = 0; k < 4; ++k) clean = clean && a[k] >= t1;
  int sh, scale;
  if (fast) {
    sh = exm + up - 127 - kEmax, scale = sh + 127;
  } else {
    const MxfpBlock p = mxfp_block(amax, E, tab);
    sh = p.sh, scale = p.scale;
  }
  // pass 1: the reference's rounding.  Nothing rounds above the top code (a carry out of the top binade is lost),
  // so a block holds the top E4M3 code (exponent code 15, fraction 7 -- any element of the top binade can land
  // on it, not only the maximum) iff the largest rounded pattern of the block equals it.
  uint32_t yq[4];  // fast path: rounded |x| patterns
  uint32_t cw[4];  // general path: reference codes
  int top = 0;
  if (fast) {
#pragma unroll
    for (int k = 0; k < 4; ++k) yq[k] = mxfp_round_one<F>(a[k] & 0x7FFFFF00u, kodd);
    if constexpr (E == 4 && F == 3)
      top = max(max(yq[0], yq[1]), max(yq[2], yq[3])) == (((uint32_t)exm << 23) | (7u << 20)) ? 1 : 0;
    if (up) top = 0;  // the maximum was assigned exponent code 14: nothing reaches code 15
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t b = (a[k] >> 23) == 0 ? 0u : r[k];
      cw[k] = mxfp_encode(b, sh, E, F);
      if constexpr (E == 4 && F == 3) top |= (cw[k] & 0x7Fu) == 0x7Fu ? 1 : 0;
    }
  }
  if constexpr (E == 4 && F == 3) {
    for (int o = 1; o < kGroup; o <<= 1) top |= __shfl_xor_sync(0xFFFFFFFFu, top, o);
  }
  // pass 2: hardware E4M3 bytes.  With exponent codes >= 2 everywhere the byte is sign | (exponent code, fraction)
  // re-biased to E4M3 -- read straight off the rounded pattern -- and raising the scale by one just lowers the
  // exponent code by one.  The general path goes through the value and the hardware conversion.
  const float half = top ? 0.5f : 1.f;
  uint32_t bytes[4];
  if (fast) {
    const uint32_t kh = (uint32_t)(K + kBias - 7 + top) << 3;  // pattern exponent -> E4M3 exponent code
#pragma unroll
    for (int k = 0; k < 4; ++k) bytes[k] = (((yq[k] >> 20) - kh) & 0x7Fu) | ((r[k] >> 24) & 0x80u);
    if (!clean) {
      // elements below exponent code 2 (subnormal codes, underflow, zeros): the reference's element codec, then
      // the exact value (halved if the scale was raised) through the hardware conversion
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (a[k] < t1) {
          const uint32_t bb = (a[k] >> 23) == 0 ? 0u : r[k];
          const float v = mxfp_decode(mxfp_encode(bb, sh, E, F), E, F) * half;
          bytes[k] = __nv_cvt_float2_to_fp8x2(make_float2(v, 0.f), __NV_SATFINITE, __NV_E4M3) & 0xFFu;
        }
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; k += 2) {
      const uint32_t two = __nv_cvt_float2_to_fp8x2(
          make_float2(mxfp_decode(cw[k], E, F) * half, mxfp_decode(cw[k + 1], E, F) * half), __NV_SATFINITE, __NV_E4M3);
      bytes[k] = two & 0xFFu, bytes[k + 1] = (two >> 8) & 0xFFu;
    }
  }
  scale_out = scale + top;
  return bytes[0] | (bytes[1] << 8) | (bytes[2] << 16) | (bytes[3] << 24);
}

// Rare paths of pack_bf16, kept out of line so that the common path stays small.
//
// patch_small_bf16: elements below exponent code 2 (subnormal codes, underflow, zeros) of a block on the fast path:
// the reference's element codec, then the exact value (halved if the scale was raised) through the hardware
// conversion.  r = the 8 input words, bytes = two E4M3 bytes per word in bytes 1 and 3.
struct Words8 {
  uint32_t w[8];
};
template <int E, int F>
__device__ __noinline__ Words8 patch_small_bf16(Words8 rr, Words8 out, int K, int sh, int top) {
  const uint32_t(&r)[8] = rr.w;
  uint32_t(&bytes)[8] = out.w;
  const float half = top ? 0.5f : 1.f;
  const uint32_t t1 = (uint32_t)(K + 2) << 23;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t b = h ? (r[k] & 0xFFFF0000u) : (r[k] << 16);
      if ((b & 0x7FFFFFFFu) < t1) {
        const uint32_t bb = ((b & 0x7FFFFFFFu) >> 23) == 0 ? 0u : b;
        const float val = mxfp_decode(mxfp_encode(bb, sh, E, F), E, F) * half;
        const uint32_t byte = __nv_cvt_float2_to_fp8x2(make_float2(val, 0.f), __NV_SATFINITE, __NV_E4M3) & 0xFFu;
        bytes[k] = h ? ((bytes[k] & 0x00FFFFFFu) | (byte << 24)) : ((bytes[k] & 0xFFFF00FFu) | (byte << 8));
      }
    }
  }
  return out;
}
// pack_general_bf16: blocks with a clamped scale, inf / nan or only zeros; called by both lanes of a block (one
// shuffle inside).  Returns the bytes and, in *scale_out, the E8M0 scale.
template <int E, int F>
__device__ __noinline__ Words8 pack_general_bf16(Words8 rr, uint32_t amax, const Log2Tab &tab, int *scale_out) {
  const uint32_t(&r)[8] = rr.w;
  Words8 out;
  uint32_t(&bytes)[8] = out.w;
  const MxfpBlock p = mxfp_block(amax, E, tab);
  uint32_t cw[16];
  int top = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t b = h ? (r[k] & 0xFFFF0000u) : (r[k] << 16);
      cw[2 * k + h] = mxfp_encode(((b & 0x7FFFFFFFu) >> 23) == 0 ? 0u : b, p.sh, E, F);
      if constexpr (E == 4 && F == 3) top |= (cw[2 * k + h] & 0x7Fu) == 0x7Fu ? 1 : 0;
    }
  }
  if constexpr (E == 4 && F == 3) top |= __shfl_xor_sync(0xFFFFFFFFu, top, 1);
  const float half = top ? 0.5f : 1.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t two = __nv_cvt_float2_to_fp8x2(
        make_float2(mxfp_decode(cw[2 * k], E, F) * half, mxfp_decode(cw[2 * k + 1], E, F) * half), __NV_SATFINITE,
        __NV_E4M3);
    bytes[k] = ((two & 0xFFu) << 8) | ((two & 0xFF00u) << 16);
  }
  *scale_out = p.scale + top;
  return out;
}

// pack_bf16 handles 16 consecutive bf16 elements (two 16-byte vectors, half a block of 32) per lane; the two lanes
// of a block exchange their maxima, so all 32 lanes of a warp call it together (lanes without data pass zeros).
// It returns the 16 E4M3 bytes and the block's E8M0 scale.
//
// Integer issue slots are the scarce resource here, so the work that can run on the floating-point pipes does:
//   * rounding |x| to F fraction bits, half to even: with p = the element's own power of two (sign and exponent
//     bits of x), t = fma(p, 2**(7-F), x) has its last bit at the F-th fraction bit of x and the fma rounds there;
//     fma(p, -2**(7-F), t) then subtracts the offset exactly.  The sign rides along.  (Checked against the integer
//     formula for every bf16 pattern.)
//   * the block maximum, the "every element has an exponent code >= 2" test and the search for the top code use
//     packed bf16 max / compare instructions with |x| operands.
template <int E, int F>
__device__ __forceinline__ uint4 pack_bf16(const uint4 &raw0, const uint4 &raw1, const Log2Tab &tab, int &scale_out) {
  constexpr int kTop = (1 << E) - 1;
  constexpr int kBias = (1 << (E - 1)) - 1;
  constexpr int kEmax = kTop - kBias;
  const Words8 rr = {{raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w}};
  const uint32_t(&r)[8] = rr.w;
  __nv_bfloat162 v[8], av[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    v[k] = *reinterpret_cast<const __nv_bfloat162 *>(&r[k]);
    av[k] = __hmax2(v[k], __hneg2(v[k]));  // |x| on the floating-point pipe
  }
  const __nv_bfloat162 m2 = __hmax2(__hmax2(__hmax2(av[0], av[1]), __hmax2(av[2], av[3])),
                                    __hmax2(__hmax2(av[4], av[5]), __hmax2(av[6], av[7])));
  const uint32_t mb = *reinterpret_cast<const uint32_t *>(&m2);
  uint32_t m = max(mb & 0xFFFFu, mb >> 16);
  m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
  const int exm = (int)(m >> 7);                      // 0: every element is zero or flushed
  const uint32_t amax = exm ? (m << 16) : 0u;
  const int K = exm - kTop;
  // `fast`: the scale is not clamped, no inf / nan, and the rounding offset 2**(e + 7 - F) stays finite
  const bool fast = K >= 1 && exm <= 240;
  const uint32_t t1 = (uint32_t)((K + 2) << 7) * 0x00010001u;  // smallest |x| pattern with exponent code >= 2
  const __nv_bfloat162 t1v = *reinterpret_cast<const __nv_bfloat162 *>(&t1);
  Words8 out;
  uint32_t(&bytes)[8] = out.w;  // two E4M3 bytes per word, in bytes 1 and 3
  int top = 0;
  if (fast) {
    bool clean = true;
#pragma unroll
    for (int k = 0; k < 8; ++k) clean = clean && __hbge2(av[k], t1v);
    const uint32_t kodd2 = (K & 1) ? 0x00800080u : 0u;
    constexpr uint32_t kOff = (uint32_t)((127 + 7 - F) << 7) * 0x00010001u;  // 2**(7-F), both halves
    const __nv_bfloat162 off = *reinterpret_cast<const __nv_bfloat162 *>(&kOff);
    const __nv_bfloat162 noff = __hneg2(off);
    uint32_t yq[8];  // rounded patterns, signs included
    bool none_top = true;
    const uint32_t topw = (((uint32_t)exm << 7) | (7u << 4)) * 0x00010001u;
    const __nv_bfloat162 topv = *reinterpret_cast<const __nv_bfloat162 *>(&topw);
    const __nv_bfloat162 ntopv = __hneg2(topv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t pw = r[k] & 0xFF80FF80u;
      const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162 *>(&pw);
      const __nv_bfloat162 y = __hfma2(p, noff, __hfma2(p, off, v[k]));
      yq[k] = *reinterpret_cast<const uint32_t *>(&y);
      yq[k] -= (yq[k] ^ r[k]) & (r[k] ^ kodd2) & 0x00800080u;  // exponent lsb flipped (carry) and code exponent odd
      // a carry out of the top binade is lost, so nothing rounds above the top code: the block holds it iff some
      // rounded pattern equals it (any element of the top binade can land there, not only the maximum)
      if constexpr (E == 4 && F == 3) {
        const __nv_bfloat162 yv = *reinterpret_cast<const __nv_bfloat162 *>(&yq[k]);
        none_top = none_top && __hbne2(yv, topv) && __hbne2(yv, ntopv);
      }
    }
    if constexpr (E == 4 && F == 3) {
      top = none_top ? 0 : 1;
      top |= __shfl_xor_sync(0xFFFFFFFFu, top, 1);
    }
    // sign | (exponent code, fraction) re-biased to E4M3, read off the rounded pattern; a raised scale (top code
    // present) lowers every exponent code by one.  One multiply-add per pair of elements: the pattern times 16 puts
    // (low four exponent bits, top three fraction bits) of the two elements into bits 8..14 and 24..30, the addend
    // subtracts the exponent offset from both fields at once.  Bit 23 of the addend is a guard: an element too small
    // for this path (patched below) makes its field borrow, and the guard absorbs the borrow of the low element
    // before it reaches the high one.  Bits 15 and 31 are still the signs of the input.
    const uint32_t koff = (uint32_t)(K + kBias - 7 + top);
    const uint32_t addend = (1u << 23) - (koff << 11) - (koff << 27);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t e = yq[k] * 16u + addend;
      bytes[k] = (e & 0x7F007F00u) | (r[k] & ~0x7F007F00u);  // bytes 1 and 3
    }
    if (!clean) out = patch_small_bf16<E, F>(rr, out, K, exm - 127 - kEmax, top);
    scale_out = exm - kEmax + top;
  } else {
    out = pack_general_bf16<E, F>(rr, amax, tab, &scale_out);
  }
  return make_uint4(__byte_perm(bytes[0], bytes[1], 0x7531), __byte_perm(bytes[2], bytes[3], 0x7531),
                    __byte_perm(bytes[4], bytes[5], 0x7531), __byte_perm(bytes[6], bytes[7], 0x7531));
}


// ---- reference codes (sign | exponent code | fraction) for 16 consecutive bf16 elements ----------------------------
// Same structure as pack_bf16, for the code-emitting mode of the quantizer (blocks of 32): elements with a normal code
// (ye >= 1) are read off the rounded pattern with one multiply-add per pair, the others (subnormal codes, underflow,
// zeros) go through the element codec out of line, and so do blocks with clamped scales, inf / nan or only zeros.
template <int E, int F>
__device__ __noinline__ Words8 codes_patch_bf16(Words8 rr, Words8 out, int K, int sh) {
  const uint32_t(&r)[8] = rr.w;
  uint32_t(&bytes)[8] = out.w;
  const uint32_t t1 = (uint32_t)(K + 1) << 23;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t b = h ? (r[k] & 0xFFFF0000u) : (r[k] << 16);
      if ((b & 0x7FFFFFFFu) < t1) {
        const uint32_t byte = mxfp_encode(((b & 0x7FFFFFFFu) >> 23) == 0 ? 0u : b, sh, E, F) & 0xFFu;
        bytes[k] = h ? ((bytes[k] & 0x00FFFFFFu) | (byte << 24)) : ((bytes[k] & 0xFFFF00FFu) | (byte << 8));
      }
    }
  }
  return out;
}
template <int E, int F>
__device__ __noinline__ Words8 codes_general_bf16(Words8 rr, uint32_t amax, const Log2Tab &tab, int *scale_out) {
  const uint32_t(&r)[8] = rr.w;
  Words8 out;
  const MxfpBlock p = mxfp_block(amax, E, tab);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    uint32_t c[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t b = h ? (r[k] & 0xFFFF0000u) : (r[k] << 16);
      c[h] = mxfp_encode(((b & 0x7FFFFFFFu) >> 23) == 0 ? 0u : b, p.sh, E, F) & 0xFFu;
    }
    out.w[k] = (c[0] << 8) | (c[1] << 24);
  }
  *scale_out = p.scale;
  return out;
}
template <int E, int F>
__device__ __forceinline__ uint4 codes_bf16(const uint4 &raw0, const uint4 &raw1, const Log2Tab &tab, int &scale_out) {
  constexpr int kTop = (1 << E) - 1;
  constexpr int kBias = (1 << (E - 1)) - 1;
  constexpr int kEmax = kTop - kBias;
  const Words8 rr = {{raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w}};
  const uint32_t(&r)[8] = rr.w;
  __nv_bfloat162 v[8], av[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    v[k] = *reinterpret_cast<const __nv_bfloat162 *>(&r[k]);
    av[k] = __hmax2(v[k], __hneg2(v[k]));
  }
  const __nv_bfloat162 m2 = __hmax2(__hmax2(__hmax2(av[0], av[1]), __hmax2(av[2], av[3])),
                                    __hmax2(__hmax2(av[4], av[5]), __hmax2(av[6], av[7])));
  const uint32_t mb = *reinterpret_cast<const uint32_t *>(&m2);
  uint32_t m = max(mb & 0xFFFFu, mb >> 16);
  m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
  const int exm = (int)(m >> 7);
  const uint32_t amax = exm ? (m << 16) : 0u;
  const int K = exm - kTop;
  Words8 out;
  uint32_t(&bytes)[8] = out.w;  // two codes per word, in bytes 1 and 3
  if (K >= 1 && exm <= 240) {
    const uint32_t t1 = (uint32_t)((K + 1) << 7) * 0x00010001u;  // smallest |x| pattern with a normal code
    const __nv_bfloat162 t1v = *reinterpret_cast<const __nv_bfloat162 *>(&t1);
    bool clean = true;
#pragma unroll
    for (int k = 0; k < 8; ++k) clean = clean && __hbge2(av[k], t1v);
    const uint32_t kodd2 = (K & 1) ? 0x00800080u : 0u;
    constexpr uint32_t kOff = (uint32_t)((127 + 7 - F) << 7) * 0x00010001u;  // 2**(7-F), both halves
    const __nv_bfloat162 off = *reinterpret_cast<const __nv_bfloat162 *>(&kOff);
    const __nv_bfloat162 noff = __hneg2(off);
    // pattern * 2**(F+1) puts (exponent, fraction) of the two elements at bit 8 and bit 24; the addend subtracts K
    // from both exponents; bit 23 guards the high element against a borrow of the low one
    const uint32_t addend = (1u << 23) - ((uint32_t)K << (8 + F)) - ((uint32_t)K << (24 + F));
    constexpr uint32_t kField = ((1u << (E + F)) - 1u) * 0x01000100u;  // exponent code and fraction, bytes 1 and 3
    constexpr uint32_t kSign = (1u << (E + F)) * 0x01000100u;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t pw = r[k] & 0xFF80FF80u;
      const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162 *>(&pw);
      const __nv_bfloat162 y = __hfma2(p, noff, __hfma2(p, off, v[k]));  // |x| rounded to F fraction bits
      uint32_t yq = *reinterpret_cast<const uint32_t *>(&y);
      yq -= (yq ^ r[k]) & (r[k] ^ kodd2) & 0x00800080u;  // carry lost when the exponent code is odd
      const uint32_t e = yq * (1u << (F + 1)) + addend;
      if constexpr (E + F == 7)
        bytes[k] = (e & kField) | (r[k] & ~kField);                      // the sign is already at bit 7 of the byte
      else
        bytes[k] = (e & kField) | ((r[k] >> (7 - E - F)) & kSign);
    }
    if (!clean) out = codes_patch_bf16<E, F>(rr, out, K, exm - 127 - kEmax);
    scale_out = exm - kEmax;
  } else {
    out = codes_general_bf16<E, F>(rr, amax, tab, &scale_out);
  }
  return make_uint4(__byte_perm(bytes[0], bytes[1], 0x7531), __byte_perm(bytes[2], bytes[3], 0x7531),
                    __byte_perm(bytes[4], bytes[5], 0x7531), __byte_perm(bytes[6], bytes[7], 0x7531));
}


// ---- MXINT mantissas (int8) and shared exponents for 16 consecutive bf16 elements (half a block of 32) ----------------
// mant = clamp(rint(x / 2**s * 2**(bits-1))) with s = ceil(log2(amax)) as the host evaluates it in bf16.  The scalings
// are exact in fp32; rint is the add of 1.5 * 2**23 inside an fma (round half to even in the last integer bit), after
// which the integer sits in the low bits of the pattern and is clamped with integer min / max.
__device__ __forceinline__ uint4 mxint_codes_bf16(const uint4 &raw0, const uint4 &raw1, const Log2Tab &tab, int bits,
                                                  int &scale_out) {
  const uint32_t r[8] = {raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w};
  __nv_bfloat162 av[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162 *>(&r[k]);
    av[k] = __hmax2(v, __hneg2(v));
  }
  const __nv_bfloat162 m2 = __hmax2(__hmax2(__hmax2(av[0], av[1]), __hmax2(av[2], av[3])),
                                    __hmax2(__hmax2(av[4], av[5]), __hmax2(av[6], av[7])));
  const uint32_t mb = *reinterpret_cast<const uint32_t *>(&m2);
  uint32_t m = max(mb & 0xFFFFu, mb >> 16);
  m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
  m = max(m, 0x0080u);  // finfo.tiny: the same pattern for bf16 and fp32 exponents
  const int ex = (int)(m >> 7);
  const int s = ex - 127 + ((m & 0x7Fu) > tab.t[ex] ? 1 : 0);
  scale_out = min(max(s + 127, 0), 255);
  uint32_t out[4];
  if (s >= 128) {  // the reference divides by 2**128 = inf: every mantissa is a (signed) zero
    out[0] = out[1] = out[2] = out[3] = 0u;
  } else {
    const float c1a = pow2f(-s), c1b = (float)(1 << (bits - 1));
    const int hi = 0x4B400000 + (1 << (bits - 1)) - 1, lo = 0x4B400000 - (1 << (bits - 1));
    uint32_t q[16];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float x = __uint_as_float(h ? (r[k] & 0xFFFF0000u) : (r[k] << 16));
        const float t = __fmaf_rn(x * c1a, c1b, 12582912.f);  // 1.5 * 2**23
        q[2 * k + h] = (uint32_t)min(max(__float_as_int(t), lo), hi);
      }
    }
#pragma unroll
    for (int w = 0; w < 4; ++w)  // low bytes of four integers
      out[w] = __byte_perm(__byte_perm(q[4 * w], q[4 * w + 1], 0x0040), __byte_perm(q[4 * w + 2], q[4 * w + 3], 0x0040), 0x5410);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

}  // namespace mxq
