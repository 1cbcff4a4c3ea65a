// Softmax over the last dimension of a tensor whose rows are MX-quantized first, in one kernel:
// softmax_mxfp / softmax_mxint / softmax_minifloat (chop/nn/quantized/functional/softmax.py:10-57) quantize x along
// its last dimension, take the softmax in fp32 and cast back.  Here one CTA reads a row once, quantizes it block by
// block with the element codecs of the quantizer kernels (the fake-quantized values, rounded to the tensor's dtype
// as the quantizer would return them, stay in shared memory), reduces maximum and sum, and writes
// exp(q - max) / sum rounded to the tensor's dtype.  One pass over HBM instead of four (quantize, cast, softmax, cast).

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mxq.h"
#include "mxq_common.cuh"
#include "mxq_internal.h"

namespace mxq {
namespace softmax {

constexpr int kThreads = 256;
enum Quantizer { kMxfp = 0, kMxint = 1, kMinifloat = 2 };

__device__ __forceinline__ float block_reduce(float v, float *scratch, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];  // fixed order
  return r;
}

// p0, p1: (E, F) for kMxfp / kMinifloat, (bits, unused) for kMxint.  cols % block == 0.
template <typename T, int kQ>
__global__ void __launch_bounds__(kThreads)
softmax_quant_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int cols, int block, int p0, int p1,
                     const __grid_constant__ Log2Tab tab) {
  extern __shared__ float q[];  // the quantized row, then its exponentials
  __shared__ float scratch[kThreads / 32];
  const int n_blocks = cols / block;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *xr = x + row * cols;
    float tmax = -INFINITY;
    for (int b = threadIdx.x; b < n_blocks; b += kThreads) {
      const T *xb = xr + b * block;
      float *qb = q + b * block;
      if constexpr (kQ == kMxfp) {
        uint32_t amax = 0;
        for (int k = 0; k < block; ++k) {
          const uint32_t a = __float_as_uint(load_scalar(xb + k)) & 0x7FFFFFFFu;
          amax = max(amax, (a >> 23) == 0 ? 0u : a);
        }
        const MxfpBlock p = mxfp_block(amax, p0, tab);
        for (int k = 0; k < block; ++k) {
          uint32_t bits = __float_as_uint(load_scalar(xb + k));
          if (((bits & 0x7FFFFFFFu) >> 23) == 0) bits = 0;
          const float v = round_to<T>(mxfp_decode(mxfp_encode(bits, p.sh, p0, p1), p0, p1) * p.scale_f);
          qb[k] = v, tmax = fmaxf(tmax, v);
        }
      } else if constexpr (kQ == kMxint) {
        float amax = 0.f;
        for (int k = 0; k < block; ++k) amax = fmaxf(amax, fabsf(load_scalar(xb + k)));
        const MxintBlock p = mxint_block<Elem<T>::kBf16>(amax, p0, tab);
        for (int k = 0; k < block; ++k) {
          const float v = round_to<T>(mxint_dequant(mxint_mant(load_scalar(xb + k), p), p));
          qb[k] = v, tmax = fmaxf(tmax, v);
        }
      } else {
        for (int k = 0; k < block; ++k) {
          const uint32_t bits = __float_as_uint(load_scalar(xb + k));
          uint32_t c = mxfp_encode(bits & 0x7FFFFFFFu, 0, p0, p1);
          if ((bits >> 31) && (bits & 0x7FFFFFFFu) != 0) c |= 1u << (p0 + p1);
          const float v = round_to<T>(mxfp_decode(c, p0, p1));
          qb[k] = v, tmax = fmaxf(tmax, v);
        }
      }
    }
    const float mx = block_reduce(tmax, scratch, true);  // (also publishes q to the whole CTA)
    float sum = 0.f;
    for (int i = threadIdx.x; i < cols; i += kThreads) {
      const float e = expf(q[i] - mx);
      q[i] = e, sum += e;
    }
    const float total = block_reduce(sum, scratch, false);
    T *yr = y + row * cols;
    for (int i = threadIdx.x; i < cols; i += kThreads) store_scalar(yr + i, q[i] / total);
    __syncthreads();  // q is reused by the next row
  }
}

// ---- rows of up to 2048 elements: one warp per row ---------------------------------------------------------------
// Lane l holds elements l, l + 32, l + 64, ... of the row in registers, so a block of 32 consecutive elements is one
// element per lane: block maxima, the row maximum and the row sum are xor-shuffles, loads and stores are coalesced,
// and nothing goes through shared memory.  The same kernel can do what surrounds the softmax in an attention block
// (chop/nn/quantized/modules/llama/attention.py:352-388) with the roundings of the separate tensor operations:
//   s = round_T(x * scale); s = round_T(s + mask)      (mask[b, 0, i, :] broadcast over heads)
//   q = quantizer_in(s)                                (MXFP / MXINT blocks of 32, element-wise minifloat, or none)
//   p = round_T(softmax_fp32(q))
//   y = quantizer_out(p)                               (MXFP / MXINT blocks of 32, or none)
constexpr int kNone = 3;
struct Fuse {
  float scale;
  int use_scale;
  const void *mask;      // T [batch, 1, mask_rows, >= cols] with row stride mask_ld, or nullptr
  long long mask_ld;
  int mask_rows, heads;  // row r of x belongs to batch r / (heads * mask_rows), query r % mask_rows
  int out_q, out_p0, out_p1;
  Log2Tab out_tab;
};

// The element codecs with (E, F) known at compile time fold to a fraction of the generic ones; the formats attention
// configurations use get their own instance, the rest take the generic one (cE = 0).
template <typename T, int cE, int cF>
__device__ __forceinline__ float minifloat_q(float v, int p0, int p1) {
  const int E = cE ? cE : p0, F = cE ? cF : p1;
  const uint32_t bits = __float_as_uint(v);
  const int bias = (1 << (E - 1)) - 1, top = (1 << E) - 1;
  const int ye = (int)((bits >> 23) & 0xFFu) - 127 + bias;  // exponent code of the element
  if (ye > top) return copysignf(mxfp_decode(((uint32_t)top << F) | ((1u << F) - 1u), E, F), v);  // saturates
  // a bf16 value has 7 fraction bits: with F >= 7 nothing is rounded away, so normal codes return the value itself
  if (Elem<T>::kBf16 && F >= 7 && ye >= 1) return v;
  uint32_t c = mxfp_encode(bits & 0x7FFFFFFFu, 0, E, F);
  if ((bits >> 31) && (bits & 0x7FFFFFFFu) != 0) c |= 1u << (E + F);
  return round_to<T>(mxfp_decode(c, E, F));
}
template <typename T, int cE, int cF>
__device__ __forceinline__ float mxfp_q(float v, int p0, int p1, const Log2Tab &tab) {
  const int E = cE ? cE : p0, F = cE ? cF : p1;
  uint32_t bits = __float_as_uint(v);
  if (((bits & 0x7FFFFFFFu) >> 23) == 0) bits = 0;
  uint32_t amax = bits & 0x7FFFFFFFu;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  const MxfpBlock p = mxfp_block(amax, E, tab);
  return round_to<T>(mxfp_decode(mxfp_encode(bits, p.sh, E, F), E, F) * p.scale_f);
}

template <typename T>
__device__ __forceinline__ float warp_block_quant(float v, int kind, int p0, int p1, const Log2Tab &tab) {
  if (kind == kMxfp) {
    if (p0 == 4 && p1 == 3) return mxfp_q<T, 4, 3>(v, p0, p1, tab);
    if (p0 == 2 && p1 == 1) return mxfp_q<T, 2, 1>(v, p0, p1, tab);
    return mxfp_q<T, 0, 0>(v, p0, p1, tab);
  }
  if (kind == kMxint) {
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const MxintBlock p = mxint_block<Elem<T>::kBf16>(amax, p0, tab);
    return round_to<T>(mxint_dequant(mxint_mant(v, p), p));
  }
  if (kind == kMinifloat) {
    if (p0 == 5 && p1 == 10) return minifloat_q<T, 5, 10>(v, p0, p1);
    if (p0 == 8 && p1 == 7) return minifloat_q<T, 8, 7>(v, p0, p1);
    if (p0 == 4 && p1 == 3) return minifloat_q<T, 4, 3>(v, p0, p1);
    return minifloat_q<T, 0, 0>(v, p0, p1);
  }
  return v;
}

template <typename T, int kJ>
__global__ void __launch_bounds__(kThreads)
softmax_quant_warp_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int cols, int kind, int p0, int p1,
                          const __grid_constant__ Log2Tab tab, const __grid_constant__ Fuse f) {
  const int lane = threadIdx.x & 31;
  const int nj = cols >> 5;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const T *xr = x + row * cols + lane;
    float q[kJ];
#pragma unroll
    for (int j = 0; j < kJ; ++j) q[j] = j < nj ? load_scalar(xr + 32 * j) : 0.f;
    if (f.use_scale) {
#pragma unroll
      for (int j = 0; j < kJ; ++j) q[j] = round_to<T>(q[j] * f.scale);
    }
    if (f.mask != nullptr) {
      const int64_t per_batch = (int64_t)f.heads * f.mask_rows;
      const int64_t mrow = (row / per_batch) * f.mask_rows + row % f.mask_rows;
      const T *mr = static_cast<const T *>(f.mask) + mrow * f.mask_ld + lane;
#pragma unroll
      for (int j = 0; j < kJ; ++j)
        if (j < nj) q[j] = round_to<T>(q[j] + load_scalar(mr + 32 * j));
    }
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      if (j < nj) {  // uniform across the warp: the shuffles inside are safe
        q[j] = warp_block_quant<T>(q[j], kind, p0, p1, tab);
        mx = fmaxf(mx, q[j]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      // e**d rounds to zero in fp32 below d = -104 (masked positions sit ~1e5 below the row maximum)
      if (j < nj) q[j] = q[j] - mx < -110.f ? 0.f : expf(q[j] - mx), sum += q[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    T *yr = y + row * cols + lane;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      if (j < nj) {
        float p = 0.f;
        if (!__all_sync(0xFFFFFFFFu, q[j] == 0.f)) {  // a block of zero probabilities stays zero under every quantizer
          p = round_to<T>(q[j] / sum);
          p = warp_block_quant<T>(p, f.out_q, f.out_p0, f.out_p1, f.out_tab);
        }
        store_scalar(yr + 32 * j, p);
      }
    }
  }
}

template <typename T>
static int launch_warp(const void *x, void *y, int64_t rows, int cols, int kind, int p0, int p1, const Log2Tab &tab,
                       const Fuse &f, cudaStream_t st) {
  const int64_t per_cta = kThreads / 32;
  int64_t grid = (rows + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)mxq::gemm::sm_count() * 16;
  if (grid > cap) grid = cap;
  const int nj = cols / 32;
#define MXQ_SW(kj)   softmax_quant_warp_kernel<T, kj><<<(int)grid, kThreads, 0, st>>>((const T *)x, (T *)y, rows, cols, kind, p0, p1, tab, f)
  if (nj <= 8)
    MXQ_SW(8);
  else if (nj <= 16)
    MXQ_SW(16);
  else if (nj <= 32)
    MXQ_SW(32);
  else
    MXQ_SW(64);
#undef MXQ_SW
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

template <typename T>
static int launch(const void *x, void *y, int64_t rows, int cols, int kind, int block, int p0, int p1, const Log2Tab &tab,
                  cudaStream_t st) {
  const size_t smem = (size_t)cols * sizeof(float);
  int64_t grid = rows;
  const int64_t cap = (int64_t)mxq::gemm::sm_count() * 8;
  if (grid > cap) grid = cap;
#define MXQ_SM(kq)                                                                                                  \
  softmax_quant_kernel<T, kq><<<(int)grid, kThreads, smem, st>>>((const T *)x, (T *)y, rows, cols, block, p0, p1, tab)
  if (kind == kMxfp)
    MXQ_SM(kMxfp);
  else if (kind == kMxint)
    MXQ_SM(kMxint);
  else
    MXQ_SM(kMinifloat);
#undef MXQ_SM
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

}  // namespace softmax
}  // namespace mxq

static bool legal_quantizer(int q, int p0, int p1, bool allow_none) {
  using namespace mxq::softmax;
  if (q == kNone) return allow_none;
  if (q == kMxint) return p0 >= 2 && p0 <= 8;
  if (q == kMxfp) return p0 >= 1 && p1 >= 1 && p0 + p1 <= 7;
  if (q == kMinifloat) return p0 >= 1 && p1 >= 1 && p0 + p1 <= 15;
  return false;
}

extern "C" int mxq_attention_softmax(const void *x, void *y, int dtype, int64_t rows, int64_t cols, int use_scale, float scale,
                                     const void *mask, int64_t mask_ld, int64_t mask_rows, int64_t heads, int quantizer,
                                     int block, int p0, int p1, const uint8_t *tab_host, int out_quantizer, int out_block,
                                     int out_p0, int out_p1, const uint8_t *out_tab_host, void *stream) {
  using namespace mxq::softmax;
  if (rows == 0 || cols == 0) return MXQ_OK;
  if (!x || !y) return MXQ_ERR_NULL;
  if (rows < 0 || cols < 0) return MXQ_ERR_SHAPE;
  if (!legal_quantizer(quantizer, p0, p1, true) || !legal_quantizer(out_quantizer, out_p0, out_p1, true) ||
      out_quantizer == kMinifloat)
    return MXQ_ERR_FORMAT;
  if (cols % 32 || cols > 2048) return MXQ_ERR_UNSUPPORTED;  // one warp per row, whole blocks of 32 per iteration
  if ((quantizer == kMxfp || quantizer == kMxint) && (block != 32 || !tab_host)) return MXQ_ERR_UNSUPPORTED;
  if ((out_quantizer == kMxfp || out_quantizer == kMxint) && (out_block != 32 || !out_tab_host)) return MXQ_ERR_UNSUPPORTED;
  if (mask && (mask_ld < cols || mask_rows < 1 || heads < 1 || rows % (heads * mask_rows))) return MXQ_ERR_SHAPE;
  mxq::Log2Tab tab;
  Fuse f;
  for (int i = 0; i < 256; ++i) tab.t[i] = tab_host ? tab_host[i] : 0, f.out_tab.t[i] = out_tab_host ? out_tab_host[i] : 0;
  f.scale = scale, f.use_scale = use_scale != 0, f.mask = mask, f.mask_ld = mask_ld;
  f.mask_rows = (int)(mask ? mask_rows : 1), f.heads = (int)(mask ? heads : 1);
  f.out_q = out_quantizer, f.out_p0 = out_p0, f.out_p1 = out_p1;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == MXQ_F32) return launch_warp<float>(x, y, rows, (int)cols, quantizer, p0, p1, tab, f, st);
  if (dtype == MXQ_BF16) return launch_warp<__nv_bfloat16>(x, y, rows, (int)cols, quantizer, p0, p1, tab, f, st);
  return MXQ_ERR_DTYPE;
}

extern "C" int mxq_softmax_quant(const void *x, void *y, int dtype, int64_t rows, int64_t cols, int quantizer, int block,
                                 int p0, int p1, const uint8_t *tab_host, void *stream) {
  using namespace mxq::softmax;
  // short rows in whole blocks of 32: one warp per row
  if (rows > 0 && cols > 0 && cols % 32 == 0 && cols <= 2048 && quantizer >= kMxfp && quantizer <= kMinifloat &&
      (quantizer == kMinifloat || block == 32))
    return mxq_attention_softmax(x, y, dtype, rows, cols, 0, 1.f, nullptr, 0, 0, 0, quantizer, block, p0, p1, tab_host, kNone,
                                 0, 0, 0, nullptr, stream);
  if (rows == 0 || cols == 0) return MXQ_OK;
  if (!x || !y) return MXQ_ERR_NULL;
  if (rows < 0 || cols < 0) return MXQ_ERR_SHAPE;
  if (quantizer < kMxfp || quantizer > kMinifloat) return MXQ_ERR_FORMAT;
  if (quantizer != kMinifloat && (!tab_host || block < 1 || cols % block)) return MXQ_ERR_SHAPE;
  if (quantizer == kMxint ? (p0 < 2 || p0 > 8) : (p0 < 1 || p1 < 1 || p0 + p1 > (quantizer == kMinifloat ? 15 : 7))) return MXQ_ERR_FORMAT;
  if (cols * (int64_t)sizeof(float) > 48 * 1024) return MXQ_ERR_UNSUPPORTED;  // the row lives in shared memory
  mxq::Log2Tab tab;
  for (int i = 0; i < 256; ++i) tab.t[i] = tab_host ? tab_host[i] : 0;
  if (quantizer == kMinifloat) block = 1;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == MXQ_F32) return launch<float>(x, y, rows, (int)cols, quantizer, block, p0, p1, tab, st);
  if (dtype == MXQ_BF16) return launch<__nv_bfloat16>(x, y, rows, (int)cols, quantizer, block, p0, p1, tab, st);
  return MXQ_ERR_DTYPE;
}
