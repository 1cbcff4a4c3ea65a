// Shared device helpers for the block quantizer kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mxq.h"

namespace mxq {

// 256 thresholds indexed by the biased fp32 exponent of a block maximum; passed to kernels by value.
struct Log2Tab {
  uint8_t t[256];
};

// Exact 2**k as fp32 for k in [-149, 127]; +inf above, 0 below.
__device__ __forceinline__ float pow2f(int k) {
  if (k > 127) return __int_as_float(0x7F800000);
  if (k >= -126) return __int_as_float((k + 127) << 23);
  if (k >= -149) return __int_as_float(1 << (k + 149));
  return 0.f;
}

// ---- 16-byte vectors of the two supported element types, handled as fp32 bit patterns -------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kVec = 4;  // elements per 16-byte vector
  static constexpr bool kBf16 = false;
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static constexpr bool kBf16 = true;
};

__device__ __forceinline__ uint4 ld_stream(const uint4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4 *p, uint4 v) { __stcs(p, v); }

// raw 16 bytes -> fp32 bit patterns
__device__ __forceinline__ void unpack(const uint4 &r, uint32_t (&b)[4]) {
  b[0] = r.x, b[1] = r.y, b[2] = r.z, b[3] = r.w;
}
__device__ __forceinline__ void unpack(const uint4 &r, uint32_t (&b)[8]) {
  b[0] = r.x << 16, b[1] = r.x & 0xFFFF0000u;
  b[2] = r.y << 16, b[3] = r.y & 0xFFFF0000u;
  b[4] = r.z << 16, b[5] = r.z & 0xFFFF0000u;
  b[6] = r.w << 16, b[7] = r.w & 0xFFFF0000u;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), round-to-nearest-even
  return *reinterpret_cast<uint32_t *>(&v);
}

// store N consecutive fp32 values as Tout starting at element index `e` (e is a multiple of N)
template <int N>
__device__ __forceinline__ void store_vals(float *y, int64_t e, const float (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N; i += 4)
    st_stream(reinterpret_cast<uint4 *>(y + e + i),
              make_uint4(__float_as_uint(v[i]), __float_as_uint(v[i + 1]), __float_as_uint(v[i + 2]),
                         __float_as_uint(v[i + 3])));
}
__device__ __forceinline__ void store_vals(__nv_bfloat16 *y, int64_t e, const float (&v)[8]) {
  st_stream(reinterpret_cast<uint4 *>(y + e), make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                           pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7])));
}
__device__ __forceinline__ void store_vals(__nv_bfloat16 *y, int64_t e, const float (&v)[4]) {
  __stcs(reinterpret_cast<uint2 *>(y + e), make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3])));
}
// N one-byte codes
__device__ __forceinline__ void store_bytes(uint8_t *c, int64_t e, const uint32_t (&v)[4]) {
  __stcs(reinterpret_cast<uint32_t *>(c + e), v[0] | (v[1] << 8) | (v[2] << 16) | (v[3] << 24));
}
__device__ __forceinline__ void store_bytes(uint8_t *c, int64_t e, const uint32_t (&v)[8]) {
  __stcs(reinterpret_cast<uint2 *>(c + e), make_uint2(v[0] | (v[1] << 8) | (v[2] << 16) | (v[3] << 24),
                                                        v[4] | (v[5] << 8) | (v[6] << 16) | (v[7] << 24)));
}

__device__ __forceinline__ float load_scalar(const float *p) { return *p; }
__device__ __forceinline__ float load_scalar(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
__device__ __forceinline__ void store_scalar(float *p, float v) { *p = v; }
__device__ __forceinline__ void store_scalar(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// round an fp32 value to the element type and back (identity for fp32)
template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// ---- shared exponent selection --------------------------------------------------------------------
// ceil(log2(amax)) as the reference's host log2 gives it; amax is a positive normal fp32 value.
template <bool kBf16>
__device__ __forceinline__ int ceil_log2_ref(float amax, const Log2Tab &tab) {
  const uint32_t b = __float_as_uint(amax);
  const uint32_t ex = b >> 23;
  const uint32_t man = kBf16 ? ((b >> 16) & 0x7Fu) : (b & 0x7FFFFFu);
  return (int)ex - 127 + (man > tab.t[ex] ? 1 : 0);
}
// floor(log2(amax)) in fp32 as the reference's host log2 gives it; bits of a positive normal fp32 value.
__device__ __forceinline__ int floor_log2_ref(uint32_t amax_bits, const Log2Tab &tab) {
  const uint32_t ex = amax_bits >> 23;
  const uint32_t below = 0x7FFFFFu - (amax_bits & 0x7FFFFFu);  // distance to the next power of two, minus one ulp
  return (int)ex - 127 + (below < tab.t[ex] ? 1 : 0);
}

// ---- MXINT element math -----------------------------------------------------------------------------
struct MxintBlock {
  float c1a, c1b;  // v * c1a * c1b = x / 2**s * 2**(bits-1)
  float c2;        // dequant factor 2**(s - (bits-1))
  float lo, hi;
  int scale;       // clamp(s + 127, 0, 255)
  bool inf_block;  // s == 128: the reference divides by 2**128 = inf
};
template <bool kBf16>
__device__ __forceinline__ MxintBlock mxint_block(float amax, int bits, const Log2Tab &tab) {
  amax = fmaxf(amax, __int_as_float(0x00800000));  // finfo.tiny, the same for fp32 and bf16
  const int s = ceil_log2_ref<kBf16>(amax, tab);
  MxintBlock p;
  p.inf_block = s >= 128;
  p.c1a = pow2f(-s);
  p.c1b = (float)(1 << (bits - 1));
  p.c2 = pow2f(s - (bits - 1));
  p.lo = -(float)(1 << (bits - 1));
  p.hi = (float)((1 << (bits - 1)) - 1);
  p.scale = min(max(s + 127, 0), 255);
  return p;
}
__device__ __forceinline__ float mxint_mant(float x, const MxintBlock &p) {
  if (p.inf_block) return copysignf(0.f, x);
  return fminf(fmaxf(rintf(x * p.c1a * p.c1b), p.lo), p.hi);
}
__device__ __forceinline__ float mxint_dequant(float m, const MxintBlock &p) {
  if (p.inf_block) return m * __int_as_float(0x7F800000);  // 0 * inf = nan, as in the reference
  return m * p.c2;
}

// ---- MXFP element math ------------------------------------------------------------------------------
struct MxfpBlock {
  int sh;         // shared exponent (unbiased), clamp(floor(log2 amax) - emax, -127, 128)
  int scale;      // E8M0 code
  float scale_f;  // 2**sh
};
__device__ __forceinline__ MxfpBlock mxfp_block(uint32_t amax_bits, int E, const Log2Tab &tab) {
  MxfpBlock p;
  if (amax_bits == 0) {  // every element is zero or an fp32 subnormal
    p.sh = -127, p.scale = 0;
  } else {
    const int bias = (1 << (E - 1)) - 1;
    const int emax = ((1 << E) - 1) - bias;
    p.sh = min(max(floor_log2_ref(amax_bits, tab) - emax, -127), 128);
    p.scale = p.sh + 127;
  }
  p.scale_f = pow2f(p.sh);
  return p;
}
// `b` = fp32 bits of the element (sign included).  Returns the 1+E+F bit code.
__device__ __forceinline__ uint32_t mxfp_encode(uint32_t b, int sh, int E, int F) {
  const uint32_t a = b & 0x7FFFFFFFu;
  const int ex = (int)(a >> 23);
  const int bias = (1 << (E - 1)) - 1;
  const int top = (1 << E) - 1;
  int ye = ex - (127 + sh - bias);
  const uint32_t m15 = (a >> 8) & 0x7FFFu;  // the low 8 mantissa bits are dropped before rounding
  const int shf = 15 - F;
  uint32_t f = (m15 + ((1u << (shf - 1)) - 1u) + ((m15 >> shf) & 1u)) >> shf;  // round half to even, 0..2**F
  if (ye == 0 && f != 0) f = (f | (1u << F)) >> 1;                               // one truncating subnormal binade
  if (ye < 0) ye = 0, f = 0;
  if (ye > top) ye = top, f = (1u << F) - 1u;
  if (ex == 0) ye = 0, f = 0;  // zero / flushed input
  uint32_t code = ((uint32_t)ye << F) | f;  // OR, not add: a fraction carry is lost when ye is odd
  // sign: the reference tests (x / 2**sh) < 0 in fp32, false when the quotient rounds to zero
  const int ev = ex - 127 - sh;
  const bool to_zero = ev < -150 || (ev == -150 && (a & 0x7FFFFFu) == 0);
  if ((b >> 31) && ex != 0 && !to_zero) code |= 1u << (E + F);
  return code;
}
// value of a code in units of the block scale
__device__ __forceinline__ float mxfp_decode(uint32_t code, int E, int F) {
  const int bias = (1 << (E - 1)) - 1;
  const uint32_t ye = (code >> F) & ((1u << E) - 1u);
  const uint32_t f = code & ((1u << F) - 1u);
  float v = ye == 0 ? (float)f * pow2f(1 - bias - F) : __uint_as_float(((ye + 127u - bias) << 23) | (f << (23 - F)));
  return (code >> (E + F)) & 1u ? -v : v;
}

// ---- block floating point element math ---------------------------------------------------------------
struct BfpBlock {
  float ka, kb;  // val * ka * kb = val / 2**e * 2**mb
  float pe;      // 2**e (inf for e = 128)
  float inv;     // 2**-mb
  float hi;      // clamp bound rounded to the element type
  float thr;     // 1e-8 rounded to the element type
};
template <typename T>
__device__ __forceinline__ BfpBlock bfp_block(float amax, int width, int exp_width, int exp_bias, const Log2Tab &tab) {
  const int mb = width - 1;
  int e;
  const uint32_t ab = __float_as_uint(amax);
  if ((ab >> 23) == 0) {
    e = -127;  // zero or subnormal maximum: every element of the tile is returned unquantized
  } else {
    e = ceil_log2_ref<Elem<T>::kBf16>(amax, tab);
  }
  e = min(max(e, -exp_bias), (1 << exp_width) - 1 - exp_bias);
  BfpBlock p;
  const int k = mb - e;
  const int k1 = k / 2;
  p.ka = pow2f(k1), p.kb = pow2f(k - k1);
  if (e >= 128) p.ka = 0.f;  // division by 2**128 = inf
  p.pe = pow2f(e);
  p.inv = pow2f(-mb);
  p.hi = round_to<T>((float)((1 << mb) - 1));
  p.thr = round_to<T>(1e-8f);
  return p;
}
template <typename T>
__device__ __forceinline__ float bfp_elem(float x, const BfpBlock &p) {
  const float val = round_to<T>(fabsf(x) + 1e-9f);
  const float xs = round_to<T>(x + 1e-9f);
  const float sgn = xs > 0.f ? 1.f : (xs < 0.f ? -1.f : 0.f);
  const float mi = fminf(fmaxf(rintf(val * p.ka * p.kb), 0.f), p.hi);
  const float y = round_to<T>((sgn * p.pe) * (mi * p.inv));
  const bool close = fabsf(x) <= p.thr;
  // (~close) * y + close * x, evaluated literally (0 * nan = nan, signed zeros)
  const float a = close ? 0.f : 1.f, c = close ? 1.f : 0.f;
  return __fadd_rn(__fmul_rn(a, y), __fmul_rn(c, x));
}

}  // namespace mxq
