// Declarations shared by the translation units of libmxq that are not part of the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "mxq.h"

namespace mxq {
namespace gemm {

constexpr unsigned long long kDefaultWaitNs = 1000000000ull;  // 1 s per device-side wait unless the call says otherwise

// Per-call settings: mxq_gemm_options with the defaults filled in.
struct Opts {
  int max_ctas = 0;  // 0 = every SM
  int tiles = MXQ_TILES_AUTO;
  bool split_k = true;
  bool transposed = true;  // problems of at most 128 rows go to the transposed (weight-major) kernel
  unsigned long long wait_ns = kDefaultWaitNs;
  int test_hook = 0;
  bool b_fp4 = false;  // block-scaled kind: B (the weight) holds E2M1 elements, two per byte
  bool a_e5m2 = false, b_e5m2 = false;  // block-scaled kind: operand holds E5M2 bytes (MXQ_GEMM_A_E5M2 / MXQ_CODES_E5M2)
  bool static_b = false;  // B was complete before anything still running on the stream (MXQ_GEMM_STATIC_B)
  // reduce-scatter fused into the GEMM: fp32 slot buffer of every GPU of the group (rows M / scatter_world each)
  int scatter_world = 0;
  int scatter_rank = 0;
  void *scatter_dst[8] = {};
};

Opts make_opts(const mxq_gemm_options *o);

// SM count of the current device
int sm_count();

// mxq_gemm_mxf8 with the options resolved
int gemm_mxf8(const uint8_t *a_codes, const uint8_t *a_scales, const uint8_t *b_codes, const uint8_t *b_scales, void *d,
              const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int *status,
              const Opts &o, cudaStream_t st);

}  // namespace gemm

// The activation packs behind mxq_mxfp_pack_mma / mxq_silu_mul_pack_mma.  chained = launched with programmatic stream
// serialization from inside a fused Linear call: the kernel lets the GEMM behind it start at once and itself waits on
// the device for the kernel before it.  The plain entry points never chain: what they write may be a weight, which a
// GEMM that is told its weight is static fetches before any wait.
int pack_mxfp_mma(const void *x, uint8_t *codes, uint8_t *scales_mma, int in_dtype, int64_t rows, int64_t k, int E, int F,
                  const uint8_t *floor_tab_host, cudaStream_t st, bool chained);
int pack_silu_mul_mma(const void *gate, const void *up, int64_t ld, uint8_t *codes, uint8_t *scales_mma, int64_t rows,
                      int64_t k, int E, int F, const uint8_t *floor_tab_host, cudaStream_t st, bool chained);

}  // namespace mxq
