// Declarations shared by the translation units of libmxq that are not part of the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "mxq.h"

namespace mxq {
namespace gemm {

constexpr unsigned long long kDefaultWaitNs = 1000000000ull;  // 1 s per device-side wait unless the call says otherwise

// Per-call settings (mxq_gemm_options with the defaults filled in) plus what mxq_mx_linear adds for a GEMM that runs
// next to its activation pack.
struct Opts {
  int max_ctas = 0;  // 0 = every SM
  int tiles = MXQ_TILES_AUTO;
  bool split_k = true;
  bool overlap = true;
  bool transposed = true;  // problems of at most 128 rows go to the transposed (weight-major) kernel
  unsigned long long wait_ns = kDefaultWaitNs;
  int test_hook = 0;
  const uint32_t *panel_ready = nullptr;  // counters of the concurrent pack, one per 128-row panel of A
  uint32_t units_per_row = 0;             // 32-byte units of bf16 input per row: a full panel counts 128 of these
};

Opts make_opts(const mxq_gemm_options *o);

// SM count of the current device
int sm_count();

// mxq_gemm_mxf8 with the options resolved
int gemm_mxf8(const uint8_t *a_codes, const uint8_t *a_scales, const uint8_t *b_codes, const uint8_t *b_scales, void *d,
              const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int *status,
              const Opts &o, cudaStream_t st);

}  // namespace gemm

// mxq_mxfp_pack_mma for bf16 input whose kernel stays resident as a whole (so that a dependent launch may start right
// away) and raises panel_ready[row / 128] by the 32-byte units it has stored, with release semantics.  The counters
// must be zero when the kernel starts.  Returns MXQ_ERR_UNSUPPORTED for inputs this variant does not take.
int pack_mma_signal(const void *x, uint8_t *codes, uint8_t *scales_mma, int64_t rows, int64_t k, int E, int F,
                    const uint8_t *floor_tab_host, uint32_t *panel_ready, cudaStream_t st);

}  // namespace mxq
