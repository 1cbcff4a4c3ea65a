// Forward of an MX Linear layer in one call: quantize the activations to MXFP along K into a caller-provided
// workspace (E4M3 bytes + E8M0 scale chunks), then run the block-scaled tensor-core GEMM against a weight that was
// packed once with mxq_mxfp_pack_mma.  Both steps are enqueued on the caller's stream.

#include <cuda_runtime.h>
#include <stdint.h>

#include "mxq.h"

static inline int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

extern "C" {

int64_t mxq_mx_linear_workspace_bytes(int64_t M, int64_t K) {
  if (M < 0 || K < 0) return MXQ_ERR_SHAPE;
  const int64_t sf = mxq_mma_scale_bytes(M, K);
  if (sf < 0) return sf;
  return align256(M * K) + align256(sf);
}

int mxq_mx_linear(const void *x, int in_dtype, const uint8_t *w_codes, const uint8_t *w_scales, void *d, const void *bias,
                  int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int E, int F,
                  const uint8_t *floor_tab_host, void *workspace, int64_t workspace_bytes, int *status, void *stream) {
  if (M == 0 || N == 0) return MXQ_OK;
  if (!workspace) return MXQ_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MXQ_ERR_ALIGN;
  const int64_t need = mxq_mx_linear_workspace_bytes(M, K);
  if (need < 0) return (int)need;
  if (workspace_bytes < need) return MXQ_ERR_SHAPE;
  uint8_t *a_codes = static_cast<uint8_t *>(workspace);
  uint8_t *a_scales = a_codes + align256(M * K);
  int rc = mxq_mxfp_pack_mma(x, a_codes, a_scales, in_dtype, M, K, E, F, floor_tab_host, stream);
  if (rc != MXQ_OK) return rc;
  return mxq_gemm_mxf8(a_codes, a_scales, w_codes, w_scales, d, bias, out_dtype, bias_dtype, M, N, K, status, stream);
}

}  // extern "C"
