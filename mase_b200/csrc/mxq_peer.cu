// Row-parallel Linear across the GPUs of one node without a collective library on the data path.
//
//   1. mxq_gemm_mxf8_scatter   the block-scaled GEMM whose epilogue stores each fp32 tile straight into the memory of
//                              the GPU that owns the tile's rows (bulk tensor stores through peer mappings over
//                              NVLink): the reduce-scatter's traffic moves tile by tile while the MMAs run.
//   2. mxq_peer_barrier        every GPU tells every other that its stores are done and waits (bounded) for theirs.
//   3. mxq_reduce_gather       each GPU adds the G partial sums of its row slice in rank order (repeatable), adds the
//                              bias, rounds once to the output type and writes the slice into every GPU's copy of the
//                              output (plain peer stores): the all-gather.
//   4. mxq_peer_barrier        the output is complete everywhere.
//
// All buffers are the caller's (symmetric allocations whose peer addresses it passes in); nothing is kept between calls.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mxq.h"
#include "mxq_internal.h"
#include "mxq_pack.cuh"

namespace mxq {
namespace peer {

constexpr int kMaxPeers = 8;
constexpr int kErrPeerBarrier = 7;  // status code: a GPU of the group did not arrive within the wait limit

struct PeerPtrs {
  void *p[kMaxPeers];
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// One warp.  Lane r < world: publish `epoch` in GPU r's flag word for this rank, then wait until GPU r's epoch has
// arrived in this GPU's flag word for rank r.  Epochs only grow, so no flag is ever reset.
__global__ void peer_barrier_kernel(PeerPtrs flags, int world, int rank, uint32_t epoch, int *status,
                                    unsigned long long wait_ns) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();  // everything this GPU wrote before the barrier (earlier kernels of the stream included)
  uint32_t *theirs = reinterpret_cast<uint32_t *>(flags.p[r]) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const uint32_t *mine = reinterpret_cast<const uint32_t *>(flags.p[rank]) + r;
  const unsigned long long t0 = global_ns();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - epoch) >= 0) break;
    if (global_ns() - t0 > wait_ns) {
      if (status) atomicCAS(status, 0, kErrPeerBarrier);
      break;
    }
    __nanosleep(200);
  }
}

// Each thread: 8 consecutive columns of one row of this GPU's slice.  slots = [world][rows][n] fp32 in this GPU's
// memory (slot s = the partial sums GPU s computed for these rows).
template <typename Tout>
__global__ void __launch_bounds__(256)
reduce_gather_kernel(const float *__restrict__ slots, int world, int rank, int64_t rows, int64_t n, const void *bias,
                     int bias_bf16, PeerPtrs out) {
  const int64_t vec_per_row = n / 8;
  const int64_t total = rows * vec_per_row;
  const int64_t slot_elems = rows * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / vec_per_row, col = (i - row * vec_per_row) * 8;
    const int64_t off = row * n + col;
    float acc[8];
    {
      const float4 a = __ldcs(reinterpret_cast<const float4 *>(slots + off));
      const float4 b = __ldcs(reinterpret_cast<const float4 *>(slots + off) + 1);
      acc[0] = a.x, acc[1] = a.y, acc[2] = a.z, acc[3] = a.w, acc[4] = b.x, acc[5] = b.y, acc[6] = b.z, acc[7] = b.w;
    }
    for (int s = 1; s < world; ++s) {  // rank order: the sum does not depend on arrival times
      const float4 a = __ldcs(reinterpret_cast<const float4 *>(slots + s * slot_elems + off));
      const float4 b = __ldcs(reinterpret_cast<const float4 *>(slots + s * slot_elems + off) + 1);
      acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w, acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
    }
    if (bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        acc[j] += bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(bias)[col + j])
                            : reinterpret_cast<const float *>(bias)[col + j];
    }
    const int64_t dst = ((int64_t)rank * rows + row) * n + col;  // position in the full [world * rows, n] output
    if constexpr (sizeof(Tout) == 2) {
      uint4 v;
      __nv_bfloat162 h;
      h = __floats2bfloat162_rn(acc[0], acc[1]), v.x = *reinterpret_cast<uint32_t *>(&h);
      h = __floats2bfloat162_rn(acc[2], acc[3]), v.y = *reinterpret_cast<uint32_t *>(&h);
      h = __floats2bfloat162_rn(acc[4], acc[5]), v.z = *reinterpret_cast<uint32_t *>(&h);
      h = __floats2bfloat162_rn(acc[6], acc[7]), v.w = *reinterpret_cast<uint32_t *>(&h);
      for (int g = 0; g < world; ++g) *reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(out.p[g]) + dst) = v;
    } else {
      const float4 lo = make_float4(acc[0], acc[1], acc[2], acc[3]), hi = make_float4(acc[4], acc[5], acc[6], acc[7]);
      for (int g = 0; g < world; ++g) {
        float4 *q = reinterpret_cast<float4 *>(reinterpret_cast<float *>(out.p[g]) + dst);
        q[0] = lo, q[1] = hi;
      }
    }
  }
}

// byte offset of the E8M0 scale of (row, block kb of 32 along K) in the tensor-core scale layout
__device__ __forceinline__ int64_t scale_offset(int64_t row, int64_t kb, int64_t k_chunks) {
  return ((row >> 7) * k_chunks + (kb >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kb & 3);
}

// The same reduction, but what goes to every GPU is the next layer's activation operand: the reduced row slice is
// rounded to bf16 (the value a separate output tensor would hold), MXFP(E, F)-quantized in blocks of 32 along the row
// exactly as the activation pack does, and written as E4M3 bytes + E8M0 scale chunks into every GPU's operand buffers
// (and, when out.p[0] is set, also as bf16 into every GPU's output).  Half the all-gather bytes and no pack kernel in
// the consumer.  Each thread: 16 consecutive columns (half a block) of one row; the two lanes of a block are neighbours.
template <int E, int F>
__global__ void __launch_bounds__(256)
reduce_gather_pack_kernel(const float *__restrict__ slots, int world, int rank, int64_t rows, int64_t n, const void *bias,
                          int bias_bf16, PeerPtrs codes, PeerPtrs scales, PeerPtrs out,
                          const __grid_constant__ mxq::Log2Tab tab) {
  const int64_t unit_per_row = n / 16;
  const int64_t total = rows * unit_per_row;
  const int64_t slot_elems = rows * n;
  const int64_t k_chunks = (n + 127) / 128;
  const int64_t padded = ((total + 31) / 32) * 32;  // whole warps run the shuffles inside pack_bf16
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < padded; i += (int64_t)gridDim.x * blockDim.x) {
    const bool live = i < total;
    const int64_t row = live ? i / unit_per_row : 0, col = live ? (i - row * unit_per_row) * 16 : 0;
    const int64_t off = row * n + col;
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.f;
    if (live) {
      for (int s = 0; s < world; ++s) {  // rank order: the sum does not depend on arrival times
        const float4 *q = reinterpret_cast<const float4 *>(slots + s * slot_elems + off);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const float4 a = __ldcs(q + v);
          if (s == 0)
            acc[4 * v] = a.x, acc[4 * v + 1] = a.y, acc[4 * v + 2] = a.z, acc[4 * v + 3] = a.w;
          else
            acc[4 * v] += a.x, acc[4 * v + 1] += a.y, acc[4 * v + 2] += a.z, acc[4 * v + 3] += a.w;
        }
      }
      if (bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          acc[j] += bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(bias)[col + j])
                              : reinterpret_cast<const float *>(bias)[col + j];
      }
    }
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
    const uint4 lo = make_uint4(w[0], w[1], w[2], w[3]), hi = make_uint4(w[4], w[5], w[6], w[7]);
    int scale;
    const uint4 c16 = mxq::pack_bf16<E, F>(lo, hi, tab, scale);  // all lanes take part (shuffle inside)
    if (!live) continue;
    const int64_t grow = (int64_t)rank * rows + row;  // row in the full [world * rows, n] matrix
    const int64_t dst = grow * n + col;
    const int64_t sdst = scale_offset(grow, col >> 5, k_chunks);
    for (int g = 0; g < world; ++g) {
      *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(codes.p[g]) + dst) = c16;
      if ((threadIdx.x & 1) == 0) reinterpret_cast<uint8_t *>(scales.p[g])[sdst] = (uint8_t)scale;
      if (out.p[0] != nullptr) {
        uint4 *q = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(out.p[g]) + dst);
        q[0] = lo, q[1] = hi;
      }
    }
  }
}

}  // namespace peer
}  // namespace mxq

using namespace mxq::peer;

extern "C" {

int mxq_gemm_mxf8_scatter(const uint8_t *a_codes, const uint8_t *a_scales, const uint8_t *b_codes, const uint8_t *b_scales,
                          int b_format, void *const *slot_ptrs, int world, int rank, int64_t M, int64_t N, int64_t K,
                          int *status, const mxq_gemm_options *options, void *stream) {
  if (!slot_ptrs) return MXQ_ERR_NULL;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return MXQ_ERR_SHAPE;
  if (M <= 0 || N <= 0 || M % world || (M / world) % 256 || N % 4) return MXQ_ERR_UNSUPPORTED;
  if (b_format != MXQ_CODES_E4M3 && b_format != MXQ_CODES_E2M1X2) return MXQ_ERR_FORMAT;
  mxq::gemm::Opts o = mxq::gemm::make_opts(options);
  o.b_fp4 = b_format == MXQ_CODES_E2M1X2;
  o.scatter_world = world;
  o.scatter_rank = rank;
  const int64_t slot_bytes = (M / world) * N * 4;  // this rank's slot inside every GPU's buffer
  for (int r = 0; r < world; ++r) {
    if (!slot_ptrs[r] || (reinterpret_cast<uintptr_t>(slot_ptrs[r]) & 15u)) return MXQ_ERR_ALIGN;
    o.scatter_dst[r] = static_cast<uint8_t *>(slot_ptrs[r]) + rank * slot_bytes;
  }
  return mxq::gemm::gemm_mxf8(a_codes, a_scales, b_codes, b_scales, o.scatter_dst[rank], nullptr, MXQ_F32, MXQ_F32, M, N, K,
                              status, o, (cudaStream_t)stream);
}

int mxq_peer_barrier(void *const *flag_ptrs, int world, int rank, uint32_t epoch, int *status, int64_t wait_limit_ns,
                     void *stream) {
  if (!flag_ptrs) return MXQ_ERR_NULL;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return MXQ_ERR_SHAPE;
  PeerPtrs f = {};
  for (int r = 0; r < world; ++r) {
    if (!flag_ptrs[r]) return MXQ_ERR_NULL;
    f.p[r] = flag_ptrs[r];
  }
  const unsigned long long limit = wait_limit_ns > 0 ? (unsigned long long)wait_limit_ns : mxq::gemm::kDefaultWaitNs;
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, world, rank, epoch, status, limit);
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

int mxq_reduce_gather(const void *slots, int world, int rank, int64_t rows, int64_t n, const void *bias, int bias_dtype,
                      void *const *out_ptrs, int out_dtype, int max_ctas, void *stream) {
  if (rows == 0 || n == 0) return MXQ_OK;
  if (!slots || !out_ptrs) return MXQ_ERR_NULL;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || rows < 0 || n < 0 || n % 8) return MXQ_ERR_SHAPE;
  if (out_dtype != MXQ_F32 && out_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  if (bias && bias_dtype != MXQ_F32 && bias_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  if (reinterpret_cast<uintptr_t>(slots) & 15u) return MXQ_ERR_ALIGN;
  PeerPtrs out = {};
  for (int r = 0; r < world; ++r) {
    if (!out_ptrs[r] || (reinterpret_cast<uintptr_t>(out_ptrs[r]) & 15u)) return MXQ_ERR_ALIGN;
    out.p[r] = out_ptrs[r];
  }
  const int64_t total = rows * (n / 8);
  int64_t grid = (total + 255) / 256;
  const int64_t cap = max_ctas > 0 ? max_ctas : (int64_t)mxq::gemm::sm_count() * 4;
  if (grid > cap) grid = cap;
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dtype == MXQ_BF16)
    reduce_gather_kernel<__nv_bfloat16><<<(int)grid, 256, 0, st>>>((const float *)slots, world, rank, rows, n, bias,
                                                                   bias_dtype == MXQ_BF16, out);
  else
    reduce_gather_kernel<float><<<(int)grid, 256, 0, st>>>((const float *)slots, world, rank, rows, n, bias,
                                                           bias_dtype == MXQ_BF16, out);
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

int mxq_reduce_gather_pack(const void *slots, int world, int rank, int64_t rows, int64_t n, const void *bias,
                           int bias_dtype, void *const *codes_ptrs, void *const *scales_ptrs, void *const *out_ptrs, int E,
                           int F, const uint8_t *floor_tab_host, int max_ctas, void *stream) {
  if (rows == 0 || n == 0) return MXQ_OK;
  if (!slots || !codes_ptrs || !scales_ptrs || !floor_tab_host) return MXQ_ERR_NULL;
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || rows < 0 || n < 0 || n % 128) return MXQ_ERR_SHAPE;
  if (bias && bias_dtype != MXQ_F32 && bias_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  if (reinterpret_cast<uintptr_t>(slots) & 15u) return MXQ_ERR_ALIGN;
  PeerPtrs codes = {}, scales = {}, out = {};
  for (int r = 0; r < world; ++r) {
    if (!codes_ptrs[r] || !scales_ptrs[r] || (reinterpret_cast<uintptr_t>(codes_ptrs[r]) & 15u)) return MXQ_ERR_ALIGN;
    codes.p[r] = codes_ptrs[r], scales.p[r] = scales_ptrs[r];
    if (out_ptrs) {
      if (!out_ptrs[r] || (reinterpret_cast<uintptr_t>(out_ptrs[r]) & 15u)) return MXQ_ERR_ALIGN;
      out.p[r] = out_ptrs[r];
    }
  }
  mxq::Log2Tab tab;
  for (int i = 0; i < 256; ++i) tab.t[i] = floor_tab_host[i];
  const int64_t total = rows * (n / 16);
  int64_t grid = (total + 255) / 256;
  const int64_t cap = max_ctas > 0 ? max_ctas : (int64_t)mxq::gemm::sm_count() * 4;
  if (grid > cap) grid = cap;
  cudaStream_t st = (cudaStream_t)stream;
#define MXQ_RGP(e, f)                                                                                                  \
  if (E == e && F == f) {                                                                                              \
    reduce_gather_pack_kernel<e, f><<<(int)grid, 256, 0, st>>>((const float *)slots, world, rank, rows, n, bias,       \
                                                               bias_dtype == MXQ_BF16, codes, scales, out, tab);       \
    return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;                                                \
  }
  MXQ_RGP(4, 3) MXQ_RGP(2, 3) MXQ_RGP(3, 2) MXQ_RGP(2, 1) MXQ_RGP(1, 2)
#undef MXQ_RGP
  return MXQ_ERR_FORMAT;
}

}  // extern "C"
