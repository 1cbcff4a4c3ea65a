// Rotary position embedding in one pass: y = x * cos + rotate_half(x) * sin over the last dimension of a
// [batch, heads, seq, dim] tensor (any strides with a contiguous last dimension), 16 bytes per thread and side.
//
// The elementwise sequence it replaces (chop/nn/quantized/functional/rope.py:17-28) makes five passes over q and k
// and, with fp32 tables, writes fp32 intermediates; here q or k is read once and written once.  Roundings follow the
// framework's: with bf16 / fp32 tables of the tensor's own dtype each product and the sum are rounded to that dtype;
// with fp32 tables for a bf16 tensor everything is evaluated in fp32 and rounded once.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mxq.h"
#include "mxq_internal.h"

namespace mxq {
namespace rope {

struct Shape {
  int64_t heads, seq, half;        // half = dim / 2
  int64_t xs_b, xs_h, xs_s;        // element strides of x; y is contiguous [batch, heads, seq, dim]
  int64_t ts_b, ts_s;              // element strides of the tables: [batch or 1, seq, dim]
  int64_t total;                   // batch * heads * seq * half / 8 groups of 8 element pairs
};

__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8]) {
  const uint4 r = *reinterpret_cast<const uint4 *>(p);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) v[2 * i] = __uint_as_float(w[i] << 16), v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
}
__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16 *p, const float (&v)[8]) {
  uint4 r;
  __nv_bfloat162 h;
  h = __floats2bfloat162_rn(v[0], v[1]), r.x = *reinterpret_cast<uint32_t *>(&h);
  h = __floats2bfloat162_rn(v[2], v[3]), r.y = *reinterpret_cast<uint32_t *>(&h);
  h = __floats2bfloat162_rn(v[4], v[5]), r.z = *reinterpret_cast<uint32_t *>(&h);
  h = __floats2bfloat162_rn(v[6], v[7]), r.w = *reinterpret_cast<uint32_t *>(&h);
  *reinterpret_cast<uint4 *>(p) = r;
}
__device__ __forceinline__ void store8(float *p, const float (&v)[8]) {
  *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <typename T>
__device__ __forceinline__ float round_as(float v) {
  if constexpr (sizeof(T) == 2) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}

// T: element type of x / y; TT: element type of the tables.  kStepwise: round each product and the sum to T (what the
// framework does when the tables have the tensor's dtype); otherwise evaluate in fp32 and round once.
template <typename T, typename TT, bool kStepwise>
__global__ void __launch_bounds__(256)
rope_kernel(const T *__restrict__ x, T *__restrict__ y, const TT *__restrict__ cos, const TT *__restrict__ sin,
            const Shape s) {
  const int64_t per_row = s.half / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < s.total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / per_row, d = (i - row * per_row) * 8;
    const int64_t bh = row / s.seq, pos = row - bh * s.seq;
    const int64_t b = bh / s.heads, h = bh - b * s.heads;
    const int64_t xo = b * s.xs_b + h * s.xs_h + pos * s.xs_s + d;
    const int64_t to = b * s.ts_b + pos * s.ts_s + d;
    float lo[8], hi[8], c_lo[8], c_hi[8], s_lo[8], s_hi[8], o_lo[8], o_hi[8];
    load8(x + xo, lo), load8(x + xo + s.half, hi);
    load8(cos + to, c_lo), load8(cos + to + s.half, c_hi);
    load8(sin + to, s_lo), load8(sin + to + s.half, s_hi);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // rotate_half(x) = (-x_hi, x_lo)
      if constexpr (kStepwise) {
        // separate roundings (no contraction into a fused multiply-add): product, product, sum
        o_lo[j] = __fadd_rn(round_as<T>(__fmul_rn(lo[j], c_lo[j])), round_as<T>(__fmul_rn(-hi[j], s_lo[j])));
        o_hi[j] = __fadd_rn(round_as<T>(__fmul_rn(hi[j], c_hi[j])), round_as<T>(__fmul_rn(lo[j], s_hi[j])));
      } else {
        o_lo[j] = fmaf(-hi[j], s_lo[j], lo[j] * c_lo[j]);
        o_hi[j] = fmaf(lo[j], s_hi[j], hi[j] * c_hi[j]);
      }
    }
    const int64_t yo = row * (2 * s.half) + d;
    store8(y + yo, o_lo), store8(y + yo + s.half, o_hi);
  }
}

}  // namespace rope
}  // namespace mxq

using namespace mxq::rope;

extern "C" int mxq_rope(const void *x, void *y, const void *cos, const void *sin, int dtype, int table_dtype,
                        int64_t batch, int64_t heads, int64_t seq, int64_t dim, int64_t x_stride_b, int64_t x_stride_h,
                        int64_t x_stride_s, int64_t table_stride_b, int64_t table_stride_s, void *stream) {
  if (batch == 0 || heads == 0 || seq == 0 || dim == 0) return MXQ_OK;
  if (!x || !y || !cos || !sin) return MXQ_ERR_NULL;
  if (batch < 0 || heads < 0 || seq < 0 || dim < 0 || dim % 16) return MXQ_ERR_SHAPE;
  if ((dtype != MXQ_F32 && dtype != MXQ_BF16) || (table_dtype != MXQ_F32 && table_dtype != MXQ_BF16)) return MXQ_ERR_DTYPE;
  if (dtype == MXQ_F32 && table_dtype == MXQ_BF16) return MXQ_ERR_DTYPE;
  const int64_t align = dtype == MXQ_BF16 ? 8 : 4;  // elements per 16 bytes
  if ((x_stride_b | x_stride_h | x_stride_s) % align || (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u)
    return MXQ_ERR_ALIGN;
  const int64_t talign = table_dtype == MXQ_BF16 ? 8 : 4;
  if ((table_stride_b | table_stride_s) % talign ||
      (reinterpret_cast<uintptr_t>(cos) | reinterpret_cast<uintptr_t>(sin)) & 15u)
    return MXQ_ERR_ALIGN;
  Shape s;
  s.heads = heads, s.seq = seq, s.half = dim / 2;
  s.xs_b = x_stride_b, s.xs_h = x_stride_h, s.xs_s = x_stride_s, s.ts_b = table_stride_b, s.ts_s = table_stride_s;
  s.total = batch * heads * seq * (dim / 16);
  int64_t grid = (s.total + 255) / 256;
  const int64_t cap = (int64_t)mxq::gemm::sm_count() * 32;
  if (grid > cap) grid = cap;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == MXQ_BF16 && table_dtype == MXQ_BF16)
    rope_kernel<__nv_bfloat16, __nv_bfloat16, true><<<(int)grid, 256, 0, st>>>(
        (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, (const __nv_bfloat16 *)cos, (const __nv_bfloat16 *)sin, s);
  else if (dtype == MXQ_BF16)
    rope_kernel<__nv_bfloat16, float, false><<<(int)grid, 256, 0, st>>>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y,
                                                                       (const float *)cos, (const float *)sin, s);
  else
    rope_kernel<float, float, true><<<(int)grid, 256, 0, st>>>((const float *)x, (float *)y, (const float *)cos,
                                                               (const float *)sin, s);
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}
