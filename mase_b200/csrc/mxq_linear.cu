// Forward of an MX Linear layer in one call: quantize the activations to MXFP along K into a caller-provided
// workspace (E4M3 bytes + E8M0 scale chunks), then run the block-scaled tensor-core GEMM against a weight that was
// packed once with mxq_mxfp_pack_mma.  Both kernels are launched with programmatic stream serialization on the
// caller's stream: the pack may start under the tail of the previous kernel (it waits for it on the device) and lets
// the GEMM start at once; the GEMM sets up -- and, for few rows, fetches its weight, which by contract is older than
// anything in flight -- while the pack runs, and waits on the device for the packed activations.

#include <cuda_runtime.h>
#include <stdint.h>

#include "mxq.h"
#include "mxq_internal.h"

#include <mutex>

static inline int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

// The weight of a Linear layer was packed at load time: the small-M GEMM may fetch it before the stream dependency.
static mxq_gemm_options with_static_weight(const mxq_gemm_options *options) {
  mxq_gemm_options o = {};
  if (options) o = *options;
  o.flags |= MXQ_GEMM_STATIC_B;
  return o;
}

// Scratch for mxq_mx_linear_static.  The array lives in the device image of this library: every GPU that loads
// libmxq holds MXQ_STATIC_SCRATCH_BYTES of its memory from the first use of the library until the process exits.
// In host code the name below is only a handle for cudaGetSymbolAddress, never a pointer a kernel may be given.
static __device__ __align__(256) uint8_t g_static_scratch[MXQ_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device, looked up once per device.
static int static_scratch_address(uint8_t **out) {
  constexpr int kMaxDevices = 64;
  static uint8_t *cached[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return MXQ_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return MXQ_ERR_LAUNCH;
    cached[dev] = static_cast<uint8_t *>(ptr);
  }
  *out = cached[dev];
  return MXQ_OK;
}

extern "C" {

int64_t mxq_mx_linear_workspace_bytes(int64_t M, int64_t K) {
  if (M < 0 || K < 0) return MXQ_ERR_SHAPE;
  const int64_t sf = mxq_mma_scale_bytes(M, K);
  if (sf < 0) return sf;
  return align256(M * K) + align256(sf);  // codes, scale chunks
}

int mxq_mx_linear(const void *x, int in_dtype, const uint8_t *w_codes, const uint8_t *w_scales, int w_format, void *d,
                  const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int E, int F,
                  const uint8_t *floor_tab_host, void *workspace, int64_t workspace_bytes, int *status,
                  const mxq_gemm_options *options, void *stream) {
  if (M == 0 || N == 0) return MXQ_OK;
  if (!workspace) return MXQ_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MXQ_ERR_ALIGN;
  const int64_t need = mxq_mx_linear_workspace_bytes(M, K);
  if (need < 0) return (int)need;
  if (workspace_bytes < need) return MXQ_ERR_SHAPE;
  uint8_t *a_codes = static_cast<uint8_t *>(workspace);
  uint8_t *a_scales = a_codes + align256(M * K);
  const int rc = mxq::pack_mxfp_mma(x, a_codes, a_scales, in_dtype, M, K, E, F, floor_tab_host, (cudaStream_t)stream, true);
  if (rc != MXQ_OK) return rc;
  mxq_gemm_options o = with_static_weight(options);
  if (E == 5 && F == 2) o.flags |= MXQ_GEMM_A_E5M2;  // the pack wrote hardware E5M2 bytes
  return mxq_gemm_mxf8(a_codes, a_scales, w_codes, w_scales, w_format, d, bias, out_dtype, bias_dtype, M, N, K, status, &o,
                       stream);
}

int mxq_mx_gated_linear(const void *gate, const void *up, int64_t ld, const uint8_t *w_codes, const uint8_t *w_scales,
                        int w_format, void *d, const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int E,
                        int F, const uint8_t *floor_tab_host, void *workspace, int64_t workspace_bytes, int *status,
                        const mxq_gemm_options *options, void *stream) {
  if (M == 0 || N == 0) return MXQ_OK;
  if (!workspace) return MXQ_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MXQ_ERR_ALIGN;
  const int64_t need = mxq_mx_linear_workspace_bytes(M, K);
  if (need < 0) return (int)need;
  if (workspace_bytes < need) return MXQ_ERR_SHAPE;
  uint8_t *a_codes = static_cast<uint8_t *>(workspace);
  uint8_t *a_scales = a_codes + align256(M * K);
  const int rc = mxq::pack_silu_mul_mma(gate, up, ld, a_codes, a_scales, M, K, E, F, floor_tab_host, (cudaStream_t)stream,
                                         true);
  if (rc != MXQ_OK) return rc;
  const mxq_gemm_options o = with_static_weight(options);
  return mxq_gemm_mxf8(a_codes, a_scales, w_codes, w_scales, w_format, d, bias, out_dtype, bias_dtype, M, N, K, status, &o,
                       stream);
}

int mxq_mx_linear_static(const void *x, int in_dtype, const uint8_t *w_codes, const uint8_t *w_scales, int w_format, void *d,
                         const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int E, int F,
                         const uint8_t *floor_tab_host, int *status, const mxq_gemm_options *options, void *stream) {
  if (M == 0 || N == 0) return MXQ_OK;
  const int64_t need = mxq_mx_linear_workspace_bytes(M, K);
  if (need < 0) return (int)need;
  if (need > (int64_t)MXQ_STATIC_SCRATCH_BYTES) return MXQ_ERR_TOO_LARGE;
  uint8_t *scratch = nullptr;
  const int rc = static_scratch_address(&scratch);  // first call on a device resolves the symbol's address
  if (rc != MXQ_OK) return rc;
  // The array keeps the previous call's bytes.  This call rewrites the M * K code bytes and the scale bytes of its M
  // rows before reading them; scale bytes of the padding rows (up to the next multiple of 256) may be an earlier call's
  // and are read by the tensor cores, but only scale accumulator rows >= M, which are never stored; scale bytes of K
  // blocks past the end of a row are cleared by the pack step whenever K % 128 != 0.
  return mxq_mx_linear(x, in_dtype, w_codes, w_scales, w_format, d, bias, out_dtype, bias_dtype, M, N, K, E, F, floor_tab_host,
                       scratch, MXQ_STATIC_SCRATCH_BYTES, status, options, stream);
}

}  // extern "C"
