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

extern "C" int mxq_softmax_quant(const void *x, void *y, int dtype, int64_t rows, int64_t cols, int quantizer, int block,
                                 int p0, int p1, const uint8_t *tab_host, void *stream) {
  using namespace mxq::softmax;
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
