// Calibration-time clipping search of the MX quantizers (chop/nn/quantizers/mxint/mxint.py:40-136,
// chop/nn/quantizers/mxfp/mxfp.py:40-104) as one kernel per tensor.
//
// For every block of 32 elements the reference derives eleven candidate shared exponents from eleven quantiles of |x|
// (1.0, 0.995, ... 0.50; linear interpolation between order statistics), quantizes the block with each, measures an
// error against the unquantized block and keeps the candidate with the smallest error.  Here one warp owns one block:
// the lanes sort |x| with a bitonic network of shuffles, every candidate is evaluated in registers, errors are summed
// with xor-shuffles, and only the winner is stored.  The tensor is read once and written once.
//
// Arithmetic follows the reference step by step, including the working dtype of every intermediate (T = the tensor's
// dtype) and the host's log2 (threshold tables, as in the other quantizer kernels).  The MXFP error is the reference's
// own: it compares x with raw_code / 2**(F-1) * (2**((scale - 127) mod 256) mod 256), the value its uint8 arithmetic
// produces, and accepts a candidate only when strictly better than the ones before it.

#include "mxq_common.cuh"
#include "mxq_internal.h"

namespace mxq {

constexpr int kSearchThreads = 256;
constexpr int kCandidates = 11;
__constant__ float kPercentiles[kCandidates] = {1.0f, 0.995f, 0.99f, 0.97f, 0.95f, 0.93f, 0.90f, 0.80f, 0.70f, 0.60f, 0.50f};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// ascending sort of one value per lane
__device__ __forceinline__ float warp_sort(float v, int lane) {
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const float o = __shfl_xor_sync(0xFFFFFFFFu, v, j);
      const bool up = (lane & k) == 0, low = (lane & j) == 0;
      v = (up == low) ? fminf(v, o) : fmaxf(v, o);
    }
  }
  return v;
}

// the q-quantile of 32 sorted values (one per lane), linear interpolation, as a vectorised fp32 lerp evaluates it
__device__ __forceinline__ float warp_quantile(float sorted, float q) {
  const float rank = __fmul_rn(q, 31.0f);
  const float below = floorf(rank);
  const float w = __fsub_rn(rank, below);
  const float lo = __shfl_sync(0xFFFFFFFFu, sorted, (int)below);
  const float hi = __shfl_sync(0xFFFFFFFFu, sorted, (int)ceilf(rank));
  const bool small = fabsf(w) < 0.5f;
  return fmaf(small ? w : __fsub_rn(w, 1.0f), __fsub_rn(hi, lo), small ? lo : hi);
}

template <typename T>
__global__ void __launch_bounds__(kSearchThreads)
mxint_clip_search_kernel(const T *__restrict__ x, T *__restrict__ y, uint8_t *__restrict__ choice, int64_t n_blocks,
                         int bits, const __grid_constant__ Log2Tab tab) {
  constexpr bool kBf16 = Elem<T>::kBf16;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kSearchThreads / 32);
  for (int64_t blk = (int64_t)blockIdx.x * (kSearchThreads / 32) + (threadIdx.x >> 5); blk < n_blocks; blk += warps) {
    const float xf = load_scalar(x + blk * 32 + lane);
    const float sorted = warp_sort(fabsf(xf), lane);
    float best_err = 0.f, best_val = 0.f;
    int best = -1;
#pragma unroll 1
    for (int c = 0; c < kCandidates; ++c) {
      const float x_max = round_to<T>(warp_quantile(sorted, kPercentiles[c]));
      const MxintBlock p = mxint_block<kBf16>(x_max, bits, tab);
      const float v = round_to<T>(mxint_dequant(mxint_mant(xf, p), p));
      const float d = round_to<T>(v - xf);
      const float err = round_to<T>(sqrtf(warp_sum(d * d)));
      // argmin over the candidates: the first smallest, a NaN counting as smallest
      const bool better = best < 0 || err < best_err || (err != err && best_err == best_err);
      if (better) best = c, best_err = err, best_val = v;
    }
    store_scalar(y + blk * 32 + lane, best_val);
    if (choice && lane == 0) choice[blk] = (uint8_t)best;
  }
}

// `forced` >= 0 evaluates only that candidate (y = its dequantized block; metric, when given, = the values the
// reference's error compares with x, in T).
template <typename T, typename Tout>
__global__ void __launch_bounds__(kSearchThreads)
mxfp_clip_search_kernel(const T *__restrict__ x, Tout *__restrict__ y, T *__restrict__ metric,
                        uint8_t *__restrict__ choice, int64_t n_blocks, int E, int F, int forced,
                        const __grid_constant__ Log2Tab tab) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kSearchThreads / 32);
  const int bias = (1 << (E - 1)) - 1;
  const int emax = ((1 << E) - 1) - bias;
  const float inv_f = pow2f(-(F - 1));
  for (int64_t blk = (int64_t)blockIdx.x * (kSearchThreads / 32) + (threadIdx.x >> 5); blk < n_blocks; blk += warps) {
    const float xf = load_scalar(x + blk * 32 + lane);
    uint32_t b = __float_as_uint(xf);
    if (((b & 0x7FFFFFFFu) >> 23) == 0) b = 0;  // zero and fp32-subnormal inputs are flushed
    const bool all_flushed = __all_sync(0xFFFFFFFFu, b == 0);
    const float sorted = warp_sort(__uint_as_float(b & 0x7FFFFFFFu), lane);
    float best_err = __int_as_float(0x7F800000), best_val = 0.f, best_metric = 0.f;
    int best = 0;
    const int c0 = forced >= 0 ? forced : 0, c1 = forced >= 0 ? forced + 1 : kCandidates;
#pragma unroll 1
    for (int c = c0; c < c1; ++c) {
      const uint32_t qb = __float_as_uint(warp_quantile(sorted, kPercentiles[c]));
      // floor(log2(q)) - emax as int32 arithmetic on the host: log2(0) = -inf converts to INT_MIN and the subtraction
      // wraps, which the clamp turns into the largest exponent
      int sh;
      if (qb == 0)
        sh = 128;
      else if ((qb >> 23) == 0)
        sh = -127;  // a subnormal quantile (interpolated next to zero): below every exponent the clamp allows
      else
        sh = min(max(floor_log2_ref(qb, tab) - emax, -127), 128);
      const int scale = all_flushed ? 0 : sh + 127;
      // a zero quantile divides the block by exp2(128) = inf: every element becomes +0
      const uint32_t code = qb == 0 ? 0u : mxfp_encode(b, sh, E, F);
      // exp2(scale - 127) of the dequantization: inf for scale 255, so that block decodes to 0 * inf = NaN
      const float v = mxfp_decode(code, E, F) * pow2f(scale - 127);
      const int k = (scale - 127) & 255;
      const float m = round_to<T>((float)code * inv_f * (k < 8 ? (float)(1 << k) : 0.f));
      float d = round_to<T>(m - xf);
      d = round_to<T>(fabsf(d) * fabsf(d));
      const float err = round_to<T>(warp_sum(d));
      // accepted when strictly better than everything before; the first candidate is also the initial answer
      if (c == c0 || err < best_err) best = c, best_val = v, best_metric = m;
      if (err < best_err) best_err = err;
    }
    store_scalar(y + blk * 32 + lane, best_val);
    if (metric) store_scalar(metric + blk * 32 + lane, best_metric);
    if (choice && lane == 0) choice[blk] = (uint8_t)best;
  }
}

static Log2Tab search_tab(const uint8_t *host) {
  Log2Tab t;
  for (int i = 0; i < 256; ++i) t.t[i] = host[i];
  return t;
}
static int search_grid(int64_t n_blocks) {
  const int64_t per_cta = kSearchThreads / 32;
  const int64_t cap = (int64_t)gemm::sm_count() * 16;
  const int64_t g = (n_blocks + per_cta - 1) / per_cta;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace mxq

extern "C" {

int mxq_mxint_clip_search(const void *x, void *y, uint8_t *choice, int dtype, int64_t n_blocks, int block, int bits,
                          const uint8_t *ceil_tab_host, void *stream) {
  using namespace mxq;
  if (n_blocks == 0) return MXQ_OK;
  if (!x || !y || !ceil_tab_host) return MXQ_ERR_NULL;
  if (n_blocks < 0) return MXQ_ERR_SHAPE;
  if (block != 32) return MXQ_ERR_UNSUPPORTED;
  if (bits < 2 || bits > 8) return MXQ_ERR_FORMAT;
  const Log2Tab tab = search_tab(ceil_tab_host);
  const int grid = search_grid(n_blocks);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == MXQ_F32)
    mxint_clip_search_kernel<float><<<grid, kSearchThreads, 0, st>>>((const float *)x, (float *)y, choice, n_blocks, bits, tab);
  else if (dtype == MXQ_BF16)
    mxint_clip_search_kernel<__nv_bfloat16>
        <<<grid, kSearchThreads, 0, st>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, choice, n_blocks, bits, tab);
  else
    return MXQ_ERR_DTYPE;
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

int mxq_mxfp_clip_search(const void *x, void *y, void *metric, uint8_t *choice, int in_dtype, int out_dtype,
                         int64_t n_blocks, int block, int E, int F, int candidate, const uint8_t *floor_tab_host,
                         void *stream) {
  using namespace mxq;
  if (n_blocks == 0) return MXQ_OK;
  if (!x || !y || !floor_tab_host) return MXQ_ERR_NULL;
  if (n_blocks < 0) return MXQ_ERR_SHAPE;
  if (block != 32) return MXQ_ERR_UNSUPPORTED;
  if (E < 1 || F < 1 || E + F > 7 || E > 5) return MXQ_ERR_FORMAT;
  if (candidate >= kCandidates) return MXQ_ERR_SHAPE;
  const Log2Tab tab = search_tab(floor_tab_host);
  const int grid = search_grid(n_blocks);
  cudaStream_t st = (cudaStream_t)stream;
#define MXQ_SEARCH(TI, TO)                                                                                        \
  mxfp_clip_search_kernel<TI, TO><<<grid, kSearchThreads, 0, st>>>((const TI *)x, (TO *)y, (TI *)metric, choice, \
                                                                   n_blocks, E, F, candidate, tab)
  if (in_dtype == MXQ_F32 && out_dtype == MXQ_F32)
    MXQ_SEARCH(float, float);
  else if (in_dtype == MXQ_F32 && out_dtype == MXQ_BF16)
    MXQ_SEARCH(float, __nv_bfloat16);
  else if (in_dtype == MXQ_BF16 && out_dtype == MXQ_F32)
    MXQ_SEARCH(__nv_bfloat16, float);
  else if (in_dtype == MXQ_BF16 && out_dtype == MXQ_BF16)
    MXQ_SEARCH(__nv_bfloat16, __nv_bfloat16);
  else
    return MXQ_ERR_DTYPE;
#undef MXQ_SEARCH
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

}  // extern "C"
