// Thin torch binding over the C ABI for the calls whose per-call host cost matters (a few rows through a Linear
// layer take less device time than Python + ctypes need to issue them).  It checks the tensors, allocates the
// output and the activation scratch from torch's allocator, takes torch's current stream and calls libmxq; nothing
// here computes.  mase_b200.gemm uses it when it is built and otherwise issues the same C calls through ctypes.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "mxq.h"

namespace {

int dtype_code(at::ScalarType t) {
  if (t == at::kFloat) return MXQ_F32;
  if (t == at::kBFloat16) return MXQ_BF16;
  TORCH_CHECK_NOT_IMPLEMENTED(false, "mase_b200: dtype ", t, " is not supported (float32 and bfloat16 are)");
}

void check_rc(int rc, const char *what) {
  TORCH_CHECK(rc == MXQ_OK, what, " failed: ", mxq_error_string(rc), " (code ", rc, ")");
}

// LinearMXFP.forward on packed weights: quantize x along K into scratch, block-scaled GEMM, one C call.
at::Tensor mx_linear(const at::Tensor &x, const at::Tensor &w_codes, const at::Tensor &w_scales, int64_t w_format,
                     int64_t n_out, const c10::optional<at::Tensor> &bias, int64_t exp_bits, int64_t frac_bits,
                     c10::optional<at::ScalarType> out_dtype, int64_t floor_tab_ptr, const at::Tensor &status,
                     int64_t options_ptr) {
  TORCH_CHECK(x.is_cuda(), "mx_linear: tensor is on '", x.device(), "'; mase_b200 runs on CUDA devices only");
  const int64_t K = x.size(-1);
  at::Tensor a = x.reshape({-1, K});
  if (!a.is_contiguous()) a = a.contiguous();
  if (reinterpret_cast<uintptr_t>(a.data_ptr()) % 16) a = a.clone();
  const int64_t M = a.size(0);
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t ws_bytes = mxq_mx_linear_workspace_bytes(M, K);
  TORCH_CHECK(ws_bytes >= 0, "mx_linear: bad shape");
  at::Tensor ws = at::empty({ws_bytes}, x.options().dtype(at::kByte));
  const at::ScalarType odt = out_dtype.value_or(x.scalar_type());
  at::Tensor out = at::empty({M, n_out}, x.options().dtype(odt));
  const void *bias_ptr = nullptr;
  int bias_dt = 0;
  at::Tensor b;
  if (bias.has_value() && bias->defined()) {
    b = bias->contiguous();
    bias_ptr = b.data_ptr();
    bias_dt = dtype_code(b.scalar_type());
  }
  const int rc = mxq_mx_linear(a.data_ptr(), dtype_code(a.scalar_type()), static_cast<const uint8_t *>(w_codes.data_ptr()),
                               static_cast<const uint8_t *>(w_scales.data_ptr()), (int)w_format, out.data_ptr(), bias_ptr,
                               dtype_code(odt), bias_dt, M, n_out, K, (int)exp_bits, (int)frac_bits,
                               reinterpret_cast<const uint8_t *>(floor_tab_ptr), ws.data_ptr(), ws_bytes,
                               static_cast<int *>(status.data_ptr()),
                               reinterpret_cast<const mxq_gemm_options *>(options_ptr),
                               at::cuda::getCurrentCUDAStream(x.device().index()).stream());
  check_rc(rc, "mxq_mx_linear");
  std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end() - 1);
  shape.push_back(n_out);
  return out.reshape(shape);
}

// F.linear on operands that already hold quantized values (bf16 exactly, fp32 as tf32).
at::Tensor dense_linear(const at::Tensor &x, const at::Tensor &weight, const c10::optional<at::Tensor> &bias,
                        c10::optional<at::ScalarType> out_dtype, const at::Tensor &status, int64_t options_ptr) {
  TORCH_CHECK(x.is_cuda(), "linear_forward: tensor is on '", x.device(), "'; mase_b200 runs on CUDA devices only");
  TORCH_CHECK(x.scalar_type() == weight.scalar_type(), "expected input and weight to have the same dtype");
  const int64_t K = x.size(-1), N = weight.size(0);
  TORCH_CHECK(weight.size(1) == K, "mat1 and mat2 shapes cannot be multiplied");
  TORCH_CHECK(K % (x.scalar_type() == at::kBFloat16 ? 8 : 4) == 0, "dense_linear: rows must be 16-byte multiples");
  at::Tensor a = x.reshape({-1, K});
  if (!a.is_contiguous()) a = a.contiguous();
  if (reinterpret_cast<uintptr_t>(a.data_ptr()) % 16) a = a.clone();
  at::Tensor w = weight.is_contiguous() ? weight : weight.contiguous();
  const int64_t M = a.size(0);
  const c10::cuda::CUDAGuard guard(x.device());
  const at::ScalarType odt = out_dtype.value_or(x.scalar_type());
  at::Tensor out = at::empty({M, N}, x.options().dtype(odt));
  const void *bias_ptr = nullptr;
  int bias_dt = 0;
  at::Tensor b;
  if (bias.has_value() && bias->defined()) {
    b = bias->contiguous();
    bias_ptr = b.data_ptr();
    bias_dt = dtype_code(b.scalar_type());
  }
  const int rc = mxq_gemm_dense(a.data_ptr(), w.data_ptr(), out.data_ptr(), bias_ptr, dtype_code(a.scalar_type()),
                                dtype_code(odt), bias_dt, M, N, K, static_cast<int *>(status.data_ptr()),
                                reinterpret_cast<const mxq_gemm_options *>(options_ptr),
                                at::cuda::getCurrentCUDAStream(x.device().index()).stream());
  check_rc(rc, "mxq_gemm_dense");
  std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end() - 1);
  shape.push_back(N);
  return out.reshape(shape);
}

// MXFP / MXINT quantize-dequantize of a tensor that already is a run of blocks (contiguous, blocks along the last
// dimension).  kind 0: MXFP (p0 = E, p1 = F, floor table); kind 1: MXINT (p0 = bits, ceil table of x's dtype).
at::Tensor mx_fake(const at::Tensor &x, int64_t kind, int64_t block, int64_t p0, int64_t p1,
                   c10::optional<at::ScalarType> out_dtype, int64_t tab_ptr) {
  TORCH_CHECK(x.is_cuda(), "mx_fake: tensor is on '", x.device(), "'; mase_b200 runs on CUDA devices only");
  TORCH_CHECK(x.is_contiguous() && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "mx_fake: contiguous, aligned input");
  const int64_t n = x.numel();
  TORCH_CHECK(block > 0 && n % block == 0, "Input tensor size ", n, " is not divisible by block size ", block, ".");
  const c10::cuda::CUDAGuard guard(x.device());
  const at::ScalarType odt = out_dtype.value_or(x.scalar_type());
  at::Tensor y = at::empty(x.sizes(), x.options().dtype(odt));
  void *stream = at::cuda::getCurrentCUDAStream(x.device().index()).stream();
  const uint8_t *tab = reinterpret_cast<const uint8_t *>(tab_ptr);
  int rc;
  if (kind == 0)
    rc = mxq_mxfp_fake(x.data_ptr(), y.data_ptr(), dtype_code(x.scalar_type()), dtype_code(odt), n / block, (int)block,
                       (int)p0, (int)p1, tab, stream);
  else
    rc = mxq_mxint_fake(x.data_ptr(), y.data_ptr(), dtype_code(x.scalar_type()), dtype_code(odt), n / block, (int)block,
                        (int)p0, tab, stream);
  check_rc(rc, kind == 0 ? "mxq_mxfp_fake" : "mxq_mxint_fake");
  return y;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("mx_fake", &mx_fake, "MXFP / MXINT quantize-dequantize of a contiguous run of blocks");
  m.def("mx_linear", &mx_linear, "LinearMXFP forward on packed weights (mxq_mx_linear)");
  m.def("dense_linear", &dense_linear, "F.linear of quantized bf16 / fp32 operands (mxq_gemm_dense)");
}
