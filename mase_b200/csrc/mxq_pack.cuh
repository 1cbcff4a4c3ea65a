// Packing of MXFP operands for the block-scaled tensor-core GEMM (shared by the stand-alone pack kernel and by the
// quantizer warps of the fused Linear kernel).
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
// pack_vector handles one 16-byte vector (8 bf16 or 4 fp32 elements); a block of 32 is shared by 32 / N neighbouring
// lanes, so it must be called by all 32 lanes of a warp together (lanes without data pass zeros).  It returns the
// vector's E4M3 bytes (two per word of c2, low 16 bits) and the block's E8M0 scale.
template <typename Tin, int E, int F>
__device__ __forceinline__ void pack_vector(const uint4 &raw, const Log2Tab &tab, uint32_t (&c2)[Elem<Tin>::kVec / 2],
                                            int &scale_out) {
  constexpr int N = Elem<Tin>::kVec;
  constexpr bool kBf16In = Elem<Tin>::kBf16;
  constexpr int kGroup = 32 / N;
  constexpr int kTop = (1 << E) - 1;
  constexpr int kBias = (1 << (E - 1)) - 1;
  constexpr int kEmax = kTop - kBias;
  const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t a[4], amax;
  if constexpr (kBf16In) {
    __nv_bfloat162 m2 = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&(a[0] = r[0] & 0x7FFF7FFFu)),
                                *reinterpret_cast<const __nv_bfloat162 *>(&(a[1] = r[1] & 0x7FFF7FFFu)));
    m2 = __hmax2(m2, __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&(a[2] = r[2] & 0x7FFF7FFFu)),
                             *reinterpret_cast<const __nv_bfloat162 *>(&(a[3] = r[3] & 0x7FFF7FFFu))));
    const uint32_t mb = *reinterpret_cast<uint32_t *>(&m2);
    const uint32_t m = group_max(max(mb & 0xFFFFu, mb >> 16), kGroup);
    amax = (m >> 7) ? (m << 16) : 0u;
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) a[k] = r[k] & 0x7FFFFFFFu;
    const uint32_t m = group_max(max(max(a[0], a[1]), max(a[2], a[3])), kGroup);
    amax = (m >> 23) ? m : 0u;
  }
  const int exm = (int)(amax >> 23);
  int up = 0;
  if constexpr (!kBf16In) {
    const uint32_t man = amax & 0x7FFFFFu;
    if (man >= 0x7FFF00u) up = (0x7FFFFFu - man) < tab.t[exm] ? 1 : 0;
  }
  const int K = exm + up - kTop;
  const uint32_t kodd = (K & 1) ? 0x00800000u : 0u;
  // `fast`: the block's scale is not clamped, elements with exponent code >= 2 are handled on bit patterns.
  // `clean`: every element of this vector is such an element; the others are patched one by one afterwards.
  const bool fast = K >= 1;
  const uint32_t t1_32 = (uint32_t)(K + 2) << 23;  // smallest |x| pattern with exponent code >= 2
  bool clean = true;
  if constexpr (kBf16In) {
    const uint32_t t1 = (uint32_t)((K + 2) << 7) * 0x00010001u;
    const __nv_bfloat162 t1v = *reinterpret_cast<const __nv_bfloat162 *>(&t1);
#pragma unroll
    for (int k = 0; k < 4; ++k) clean = clean && __hbge2(*reinterpret_cast<const __nv_bfloat162 *>(&a[k]), t1v);
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) clean = clean && a[k] >= t1_32;
  }
  int sh, scale;
  if (K >= 1) {
    sh = exm + up - 127 - kEmax, scale = sh + 127;
  } else {
    const MxfpBlock p = mxfp_block(amax, E, tab);
    sh = p.sh, scale = p.scale;
  }
  // pass 1: the reference's rounding.  Nothing rounds above the top code (a carry out of the top binade is lost),
  // so a block holds the top E4M3 code (exponent code 15, fraction 7 -- any element of the top binade can land
  // on it, not only the maximum) iff the largest rounded pattern of the block equals it.
  uint32_t yq[4];     // fast path: rounded |x| patterns (bf16: two per word)
  uint32_t cw[N];     // general path: reference codes
  uint32_t ymax = 0;  // largest rounded pattern (fast) or largest code magnitude moved to the same scale (general)
  if (fast) {
    if constexpr (kBf16In) {
      const uint32_t kodd2 = kodd ? 0x00800080u : 0u;
#pragma unroll
      for (int k = 0; k < 4; ++k) yq[k] = mxfp_round_pair<F>(a[k], kodd2);
      if constexpr (E == 4 && F == 3) {
        __nv_bfloat162 mx = __hmax2(__hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&yq[0]),
                                            *reinterpret_cast<const __nv_bfloat162 *>(&yq[1])),
                                    __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&yq[2]),
                                            *reinterpret_cast<const __nv_bfloat162 *>(&yq[3])));
        const uint32_t mxb = *reinterpret_cast<uint32_t *>(&mx);
        ymax = max(mxb & 0xFFFFu, mxb >> 16) == (((uint32_t)exm << 7) | (7u << 4)) ? 1u : 0u;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) yq[k] = mxfp_round_one<F>(a[k] & 0x7FFFFF00u, kodd);
      if constexpr (E == 4 && F == 3)
        ymax = max(max(yq[0], yq[1]), max(yq[2], yq[3])) == (((uint32_t)exm << 23) | (7u << 20)) ? 1u : 0u;
    }
    if (up) ymax = 0;  // the maximum was assigned exponent code 14: nothing reaches code 15
  } else {
    uint32_t b[N];
    unpack(raw, b);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      if (((b[k] & 0x7FFFFFFFu) >> 23) == 0) b[k] = 0;
      cw[k] = mxfp_encode(b[k], sh, E, F);
      if constexpr (E == 4 && F == 3) ymax |= (cw[k] & 0x7Fu) == 0x7Fu ? 1u : 0u;
    }
  }
  int top = (int)ymax;
  if constexpr (E == 4 && F == 3) {
    for (int o = 1; o < kGroup; o <<= 1) top |= __shfl_xor_sync(0xFFFFFFFFu, top, o);
  }
  // pass 2: hardware E4M3 bytes.  With exponent codes >= 2 everywhere the byte is sign | (exponent code, fraction)
  // re-biased to E4M3 -- read straight off the rounded pattern -- and raising the scale by one just lowers the
  // exponent code by one.  The general path goes through the value and the hardware conversion.
  if (fast) {
    const uint32_t kh = (uint32_t)(K + kBias - 7 + top) << 3;  // pattern exponent -> E4M3 exponent code
    if constexpr (kBf16In) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // bit 15 of each half absorbs the borrow of an element that is too small for this path (patched below)
        const uint32_t m2 = ((((yq[k] >> 4) | 0x80008000u) - kh * 0x00010001u) & 0x007F007Fu) | ((r[k] >> 8) & 0x00800080u);
        c2[k] = __byte_perm(m2, 0, 0x4420);  // bytes 0 and 2 -> low 16 bits
      }
    } else {
      uint32_t m[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) m[k] = (((yq[k] >> 20) - kh) & 0x7Fu) | ((r[k] >> 24) & 0x80u);
      c2[0] = m[0] | (m[1] << 8), c2[1] = m[2] | (m[3] << 8);
    }
    if (!clean) {
      // elements below exponent code 2 (subnormal codes, underflow, zeros): the reference's element codec, then
      // the exact value (halved if the scale was raised) through the hardware conversion
      uint32_t b[N];
      unpack(raw, b);
      const float half = top ? 0.5f : 1.f;
#pragma unroll
      for (int k = 0; k < N; ++k) {
        if ((b[k] & 0x7FFFFFFFu) < t1_32) {
          const uint32_t bb = ((b[k] & 0x7FFFFFFFu) >> 23) == 0 ? 0u : b[k];
          const float v = mxfp_decode(mxfp_encode(bb, sh, E, F), E, F) * half;
          const uint32_t byte = __nv_cvt_float2_to_fp8x2(make_float2(v, 0.f), __NV_SATFINITE, __NV_E4M3) & 0xFFu;
          c2[k / 2] = (k & 1) ? ((c2[k / 2] & 0x00FFu) | (byte << 8)) : ((c2[k / 2] & 0xFF00u) | byte);
        }
      }
    }
  } else {
    const float half = top ? 0.5f : 1.f;
#pragma unroll
    for (int k = 0; k < N; k += 2)
      c2[k / 2] = __nv_cvt_float2_to_fp8x2(
          make_float2(mxfp_decode(cw[k], E, F) * half, mxfp_decode(cw[k + 1], E, F) * half), __NV_SATFINITE, __NV_E4M3);
  }
  scale_out = scale + top;
}

}  // namespace mxq
