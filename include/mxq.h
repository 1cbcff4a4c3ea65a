/*
 * mxq.h -- C ABI of libmxq, the sm_100a implementation of MASE's MX / block-floating-point
 * quantizers and of the forward GEMM of its MX Linear modules.
 *
 * Conventions
 *   - every pointer named x/y/codes/scales/... is DEVICE memory owned by the caller; the library never
 *     allocates or frees device memory, keeps no caller pointer past the call, and never synchronises the host with
 *     the device.  The one piece of device memory it owns is the fixed scratch array of mxq_mx_linear_static
 *     (MXQ_STATIC_SCRATCH_BYTES per GPU, part of the library's device image, used by that entry point only);
 *   - the library has no mutable process-wide settings: per-call behaviour travels in mxq_gemm_options;
 *   - every kernel is enqueued on `stream` (a cudaStream_t passed as void*; NULL = legacy default stream);
 *   - log2 tables are HOST pointers to 256 bytes, copied by value into the launch;
 *   - functions return MXQ_OK (0) or a negative MXQ_ERR_* code; nothing throws or exits.
 *
 * Each entry point cites the MASE function it replaces (paths inside the MASE repository).
 */
#ifndef MXQ_H_
#define MXQ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXQ_VERSION 1

/* element types of float tensors */
#define MXQ_F32 0
#define MXQ_BF16 1

#define MXQ_OK 0
#define MXQ_ERR_DTYPE (-1)     /* unsupported element type */
#define MXQ_ERR_SHAPE (-2)     /* sizes out of range or not divisible as required */
#define MXQ_ERR_FORMAT (-3)    /* unsupported (exponent, fraction) or bit width */
#define MXQ_ERR_ALIGN (-4)     /* pointer not aligned to 16 bytes */
#define MXQ_ERR_NULL (-5)      /* required pointer is NULL */
#define MXQ_ERR_LAUNCH (-6)    /* the CUDA runtime reported an error at launch */
#define MXQ_ERR_UNSUPPORTED (-7)
#define MXQ_ERR_DEVICE (-8)    /* a kernel reported a device-side error status (bounded wait ran out) */
#define MXQ_ERR_TOO_LARGE (-9) /* problem needs more scratch than MXQ_STATIC_SCRATCH_BYTES (mxq_mx_linear_static) */

int mxq_version(void);
const char *mxq_error_string(int code);

/*
 * log2 tables.  The reference picks the shared exponent as ceil(log2(amax)) or floor(log2(amax)) with
 * `torch.log2` evaluated on the host in fp32 or bf16; its rounding is observable next to powers of two.
 * The kernels compute the exact integer result from the bits of amax and correct it with a table indexed
 * by the biased exponent `ex` of amax (1..254):
 *   ceil tables  (MXINT, block-fp): mantissas 1..t[ex] (23-bit units for fp32 input, 7-bit units for bf16
 *                input) give ceil(log2(amax)) == ex-127 instead of ex-126;
 *   floor table  (MXFP):            the top t[ex] mantissas (2^23 - t[ex] .. 2^23 - 1) give
 *                floor(log2(amax)) == ex-126 instead of ex-127.
 * The host-side package builds them from the host's own torch.log2.
 */

/* MXINT quantize-dequantize.  Replaces chop/nn/quantizers/mxint/mxint.py:145-171 (mxint_quantizer_sim,
 * non-search branch) = extract_mxint_components + compose_mxint_tensor (mxint/fake.py:11-80) on a tensor
 * already flattened so that each block is `block` consecutive elements.
 * x: n_blocks*block elements of in_dtype; y: same count of out_dtype.  2 <= bits <= 8. */
int mxq_mxint_fake(const void *x, void *y, int in_dtype, int out_dtype, int64_t n_blocks, int block, int bits,
                   const uint8_t *ceil_tab_host, void *stream);

/* MXINT codes.  Replaces extract_mxint_components (mxint/fake.py:11-56).  mant: int8 [n_blocks*block] in
 * [-2^(bits-1), 2^(bits-1)-1]; scales: uint8 [n_blocks] = clamp(ceil(log2(amax)) + 127, 0, 255). */
int mxq_mxint_extract(const void *x, int8_t *mant, uint8_t *scales, int in_dtype, int64_t n_blocks, int block,
                      int bits, const uint8_t *ceil_tab_host, void *stream);

/* Replaces compose_mxint_tensor (mxint/fake.py:59-80). */
int mxq_mxint_compose(const int8_t *mant, const uint8_t *scales, void *y, int out_dtype, int64_t n_blocks,
                      int block, int bits, void *stream);

/* MXINT clipping search.  Replaces the quantile_search branch of mxint_quantizer_sim without activations
 * (mxint/mxint.py:40-136): per block, eleven candidate exponents from the quantiles 1.0, 0.995, 0.99, 0.97, 0.95,
 * 0.93, 0.90, 0.80, 0.70, 0.60, 0.50 of |x| (linear interpolation), the one with the smallest 2-norm error wins
 * (the first of equals).  x, y: n_blocks*32 elements of `dtype`; choice (may be NULL): uint8 [n_blocks], index of
 * the winning quantile.  block must be 32 (MXQ_ERR_UNSUPPORTED otherwise). */
int mxq_mxint_clip_search(const void *x, void *y, uint8_t *choice, int dtype, int64_t n_blocks, int block, int bits,
                          const uint8_t *ceil_tab_host, void *stream);

/* MXFP clipping search.  Replaces the quantile_search branch of mxfp_quantizer_sim without activations
 * (mxfp/mxfp.py:40-104), including its error measure (raw code bytes scaled in uint8 arithmetic) and its strict
 * "better than everything before" acceptance.  candidate < 0: search; 0..10: evaluate only that quantile
 * (extract_mxfp_components with percentile, mxfp/fake.py:57).  y: dequantized result in out_dtype; metric (may be
 * NULL): in_dtype [n_blocks*32], the values the error compares with x; choice (may be NULL): uint8 [n_blocks]. */
int mxq_mxfp_clip_search(const void *x, void *y, void *metric, uint8_t *choice, int in_dtype, int out_dtype,
                         int64_t n_blocks, int block, int E, int F, int candidate, const uint8_t *floor_tab_host,
                         void *stream);

/* MXFP quantize-dequantize with E exponent and F fraction bits per element, E8M0 shared scale.
 * Replaces chop/nn/quantizers/mxfp/mxfp.py:14-115 (mxfp_quantizer_sim, non-search branch) =
 * extract_mxfp_components + compose_mxfp_tensor (mxfp/fake.py:12-104) with the element codec of
 * _minifloat_mx/fake.py:11-149 (is_finite=True, round-to-nearest).
 * (E,F) in {(4,3),(5,2),(2,3),(3,2),(2,1),(1,2)}. */
int mxq_mxfp_fake(const void *x, void *y, int in_dtype, int out_dtype, int64_t n_blocks, int block, int E, int F,
                  const uint8_t *floor_tab_host, void *stream);

/* MXFP codes.  Replaces extract_mxfp_components (mxfp/fake.py:12-72).  codes: uint8 [n_blocks*block], one
 * element per byte (sign | exponent | fraction in the low 1+E+F bits); scales: uint8 [n_blocks] (E8M0). */
int mxq_mxfp_extract(const void *x, uint8_t *codes, uint8_t *scales, int in_dtype, int64_t n_blocks, int block,
                     int E, int F, const uint8_t *floor_tab_host, void *stream);

/* Replaces compose_mxfp_tensor (mxfp/fake.py:75-104). */
int mxq_mxfp_compose(const uint8_t *codes, const uint8_t *scales, void *y, int out_dtype, int64_t n_blocks,
                     int block, int E, int F, void *stream);

/* Element-wise minifloat quantize-dequantize.  Replaces minifloat_quantizer_sim
 * (_minifloat_mx/minifloat.py:12-33) for is_finite=True, round-to-nearest.  E >= 1, F >= 1, E + F <= 15 (the range of
 * the reference's MinifloatMeta: 8-bit formats as well as fp16-like E5M10 or bf16-like E8M7). */
int mxq_minifloat_fake(const void *x, void *y, int in_dtype, int out_dtype, int64_t n, int E, int F, void *stream);

/* Block floating point with tiles of `bs` consecutive elements of the last dimension (a ragged last tile is
 * padded with zeros).  Replaces _block_fp_quantize (chop/nn/quantizers/block_fp.py:7-82) for the tilings in
 * which a tile lies inside one row: 1-D tensors, 2-D activations, and block shapes [1, bs].
 * x, y: rows*cols elements of `dtype`.  width = mantissa bits + sign; exponent in
 * [-exp_bias, 2^exp_width - 1 - exp_bias]. */
int mxq_bfp_fake(const void *x, void *y, int dtype, int64_t rows, int64_t cols, int bs, int width, int exp_width,
                 int exp_bias, const uint8_t *ceil_tab_host, void *stream);

/* Block floating point with two-dimensional tiles of bh x bw over the last two dimensions of x[batch, rows, cols]
 * (ragged edges are zero padding).  Replaces _block_fp_quantize (chop/nn/quantizers/block_fp.py:7-82) for the tilings
 * that go through F.unfold / F.fold: 2-D weights with skip_first_dim=False (chop/nn/quantizers/utils.py:228-276) and
 * 3-D activations (utils.py:278-323).  A result of -0.0 is returned as +0.0, as after the reference's fold. */
int mxq_bfp_fake_tiles(const void *x, void *y, int dtype, int64_t batch, int64_t rows, int64_t cols, int bh, int bw,
                       int width, int exp_width, int exp_bias, const uint8_t *ceil_tab_host, void *stream);

/*
 * Forward GEMM of the quantized Linear modules: D[M,N] = A[M,K] * B[N,K]^T (+ bias[N]), fp32 accumulation on the
 * tcgen05 tensor cores.  Replaces the `F.linear(x, self.weight, self.bias)` at the end of LinearMXFP.forward,
 * LinearMXInt.forward (chop/nn/quantized/modules/linear.py:895, :972) and linearBlockFP
 * (chop/nn/quantized/functional/linear.py:278).
 *
 * `status` is an optional device int (zero it once): a kernel whose bounded waits run out stores a non-zero code
 * there instead of hanging; the caller reads it when it next synchronises.
 */

/*
 * Per-call options of the GEMM entry points (mxq_gemm_dense, mxq_gemm_mxf8, mxq_mx_linear, mxq_mx_linear_static).
 * No counterpart in the reference.  The library keeps no mutable process-wide state: everything that steers a launch
 * travels with the call, so calls from different threads or streams never influence one another.  Pass NULL for the
 * defaults; a zero-filled struct means the same.  The struct is read during the call and not kept.
 */
typedef struct mxq_gemm_options {
  /* Upper bound on the CTAs (= SMs) the launch occupies; 0 = every SM.  The GEMM kernels are persistent, one CTA per
   * SM, each holding nearly all of the SM's shared memory, so a kernel of another stream (an NCCL collective, say)
   * cannot start on an SM until a GEMM CTA leaves it; a caller that overlaps such a kernel leaves it some SMs. */
  int32_t max_ctas;
  /* Tile scheme for problems of more than 128 rows and columns.
   *   MXQ_TILES_AUTO    CTA pairs on 256 x 256 tiles (thread-block clusters of two, tcgen05 cta_group::2) when such
   *                     tiles fill the GPU, one CTA per 128 x 256 tile otherwise;
   *   MXQ_TILES_SINGLE  one CTA per tile only;
   *   MXQ_TILES_PAIRS   CTA pairs for every such problem, however small (for tests).
   * The schemes accumulate in the same order: results are bit-identical. */
  int32_t tiles;
  /* Small problems (at most 128 rows): K is split over the CTAs of a thread-block cluster, which hand their fp32
   * partial sums over through distributed shared memory in a fixed order (repeatable results).  0 = let the library
   * decide, 1 = never. */
  int32_t no_split_k;
  /* Bit flags.
   *   MXQ_GEMM_STATIC_B   operand B (the weight) was complete before the launch of every kernel that may still be
   *                       running on the stream -- packed at load time, say.  The small-M kernel then fetches it
   *                       ahead of the stream dependency, under the tail of the previous kernel.  Without the flag
   *                       nothing is read before the previous kernel of the stream has finished.  mxq_mx_linear,
   *                       mxq_mx_gated_linear and mxq_mx_linear_static imply it: their weight argument is by contract
   *                       a weight packed earlier, not the product of a kernel in flight.
   *   MXQ_GEMM_A_E5M2     mxq_gemm_mxf8: operand A holds E5M2 bytes (packed with E = 5, F = 2) instead of E4M3. */
  int32_t flags;
  /* Limit of every device-side wait in nanoseconds; 0 = one second.  When a wait runs out the kernel stores a
   * non-zero code in the status word, lets its copies in flight land, frees its tensor memory and returns. */
  int64_t wait_limit_ns;
  /* Test hook: MXQ_TEST_DROP_LAST_LOAD makes the loader skip the last operand tile of the launch, so that the wait of
   * the MMA issuer runs out and the error path above is taken (no fault is involved; the output is left incomplete
   * and the status word reads 2).  Leave 0 otherwise. */
  int32_t test_hook;
  /* Problems of at most 128 rows run a transposed kernel: the weight is the 128-row operand of the MMA, the few
   * activation rows are its narrow one, and K is split over a cluster of up to 8 CTAs.  1 = use the regular tiles
   * instead (for comparisons). */
  int32_t no_transposed;
} mxq_gemm_options;

#define MXQ_GEMM_STATIC_B 1
#define MXQ_GEMM_A_E5M2 4
#define MXQ_TILES_AUTO 0
#define MXQ_TILES_SINGLE 1
#define MXQ_TILES_PAIRS 2
#define MXQ_TEST_DROP_LAST_LOAD 1

/* sizeof(mxq_gemm_options) as the library was built, for bindings that mirror the struct by hand. */
int mxq_gemm_options_size(void);

/* Operands that already hold quantized values in bf16 (exact for every MX / block-fp format with <= 8 significant
 * bits) or fp32 (multiplied as tf32: exact for up to 11 significant bits).  A: [M,K], B: [N,K], row-major,
 * 16-byte aligned rows (K % 8 == 0 for bf16, K % 4 == 0 for fp32).  D: [M,N] of out_dtype. */
int mxq_gemm_dense(const void *a, const void *b, void *d, const void *bias, int in_dtype, int out_dtype, int bias_dtype,
                   int64_t M, int64_t N, int64_t K, int *status, const mxq_gemm_options *options, void *stream);

/* A batch of independent dense products D[i] = A[i] B[i]^T, i < batch, in one launch: A[i] = a + i * stride_a is
 * [M, K], B[i] = b + i * stride_b is [N, K], D[i] = d + i * stride_d is [M, N], all row-major (strides in elements,
 * at least one matrix apart; rows and the strides of a and b must be multiples of 16 bytes).  Element types and
 * accumulation as mxq_gemm_dense; no bias.  Replaces the torch.matmul / torch.bmm behind the quantized matmul and bmm
 * wrappers (chop/nn/quantized/functional/matmul.py:437-512) and behind the quantized attention products
 * (chop/nn/quantized/modules/llama/attention.py:334-394) once both operands are fake-quantized.  The tensor maps carry
 * the matrix index as a third coordinate, so tiles at a matrix edge read zeros and store nothing beyond it. */
int mxq_gemm_dense_batched(const void *a, const void *b, void *d, int in_dtype, int out_dtype, int64_t batch, int64_t M,
                           int64_t N, int64_t K, int64_t stride_a, int64_t stride_b, int64_t stride_d, int *status,
                           const mxq_gemm_options *options, void *stream);

/* Size in bytes of the scale array that mxq_mxfp_pack_mma writes for a [rows, k] operand. */
int64_t mxq_mma_scale_bytes(int64_t rows, int64_t k);

/* Quantize a [rows, k] matrix to MXFP (E, F) with blocks of 32 along k -- the same codes and scales as
 * extract_mxfp_components (chop/nn/quantizers/mxfp/fake.py:12-72) -- and store them as tensor-core operands:
 * hardware E4M3 bytes [rows, k] plus E8M0 scales in 512-byte chunks per 128 rows x 128 columns.  E <= 4, F <= 3,
 * or E = 5, F = 2.  A block that holds the reference's top E4M3 code (480, NaN in hardware) is stored one binade
 * lower with its scale raised by one.  E = 5, F = 2 writes hardware E5M2 bytes instead, every block one scale step up
 * with halved values (the reference's top exponent code 31 is inf / nan in hardware); the GEMM is told through
 * MXQ_CODES_E5M2 (operand B) or MXQ_GEMM_A_E5M2 (operand A).  The scale array is padded to whole 256-row tiles; scale bytes of rows past `rows` are left
 * unset (they only reach accumulator rows that the GEMM never stores), scale bytes of K blocks past `k` are zero. */
int mxq_mxfp_pack_mma(const void *x, uint8_t *codes, uint8_t *scales_mma, int in_dtype, int64_t rows, int64_t k, int E,
                      int F, const uint8_t *floor_tab_host, void *stream);

/* The same for MXFP4 (E2M1) only, with the codes nibble-packed: codes4 is [rows, k/2] bytes, element 2i of a row in
 * the low nibble of byte i and element 2i+1 in the high nibble, each nibble the reference's code sign|exponent|fraction
 * (chop/nn/quantizers/_minifloat_mx/fake.py:90-91), which is the hardware's FP4 encoding as it stands.  Scales as
 * above.  Weight storage of 0.53 bytes per element: the copy engine expands the nibbles on their way into shared
 * memory, so the GEMM also moves half the weight bytes.  k % 128 == 0; codes4 32-byte aligned. */
int mxq_mxfp4_pack_mma(const void *x, uint8_t *codes4, uint8_t *scales_mma, int in_dtype, int64_t rows, int64_t k,
                       const uint8_t *floor_tab_host, void *stream);

/* layout of the codes of a GEMM operand */
#define MXQ_CODES_E4M3 0    /* one hardware E4M3 byte per element (mxq_mxfp_pack_mma) */
#define MXQ_CODES_E2M1X2 1  /* two E2M1 nibbles per byte (mxq_mxfp4_pack_mma); B operand only */
#define MXQ_CODES_E5M2 2    /* hardware E5M2 bytes (mxq_mxfp_pack_mma with E = 5, F = 2) */

/* Block-scaled GEMM on operands produced by mxq_mxfp_pack_mma / mxq_mxfp4_pack_mma (kind::mxf8f6f4, one E8M0 scale
 * per 32 elements of K).  A is always E4M3 bytes; b_format says how B (the weight) is stored.  Replaces
 * quantize-activations + F.linear of LinearMXFP.forward (chop/nn/quantized/modules/linear.py:877-895). */
int mxq_gemm_mxf8(const uint8_t *a_codes, const uint8_t *a_scales, const uint8_t *b_codes, const uint8_t *b_scales,
                  int b_format, void *d, const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K,
                  int *status, const mxq_gemm_options *options, void *stream);

/* LinearMXFP.forward in one call (chop/nn/quantized/modules/linear.py:877-895): quantize x[M,K] to MXFP(E,F),
 * block 32 along K, into `workspace` (scratch owned by the caller, 256-byte aligned, at least
 * mxq_mx_linear_workspace_bytes(M, K) bytes), then D = x_q * W_q^T (+ bias) with the block-scaled GEMM.
 * w_codes / w_scales come from mxq_mxfp_pack_mma (w_format MXQ_CODES_E4M3) or mxq_mxfp4_pack_mma (MXQ_CODES_E2M1X2) on
 * the [N,K] weight. */
int64_t mxq_mx_linear_workspace_bytes(int64_t M, int64_t K);
int mxq_mx_linear(const void *x, int in_dtype, const uint8_t *w_codes, const uint8_t *w_scales, int w_format, void *d,
                  const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int E, int F,
                  const uint8_t *floor_tab_host, void *workspace, int64_t workspace_bytes, int *status,
                  const mxq_gemm_options *options, void *stream);

/* Hidden state of a gated MLP as tensor-core operands in one pass: h = silu(gate) * up, then the MXFP(E, F) pack of
 * mxq_mxfp_pack_mma on h.  Replaces the elementwise `act_fn(gate) * up` between the projections
 * (chop/nn/quantized/modules/llama/mlp.py:56-61, the unquantized-SiLU form) followed by the activation quantization
 * of the down projection (chop/nn/quantized/modules/linear.py:877-890).  gate and up are bf16 [rows, k] views with
 * a common row stride of `ld` elements (ld >= k, ld % 8 == 0, both 16-byte aligned): the two halves of one
 * [rows, 2k] GEMM output, for instance.  h is rounded as the framework's elementwise kernels round it: silu in fp32
 * as g / (1 + exp(-g)) -> bf16, product in fp32 -> bf16. */
int mxq_silu_mul_pack_mma(const void *gate, const void *up, int64_t ld, uint8_t *codes, uint8_t *scales_mma,
                          int64_t rows, int64_t k, int E, int F, const uint8_t *floor_tab_host, void *stream);

/* Second half of a gated MLP in one call: D[M,N] = MXFP(silu(gate) * up)[M,K] * W_q[N,K]^T (+ bias), i.e.
 * mxq_silu_mul_pack_mma into `workspace` followed by the block-scaled GEMM.  Workspace size and the other arguments
 * as for mxq_mx_linear (K = columns of gate / up). */
int mxq_mx_gated_linear(const void *gate, const void *up, int64_t ld, const uint8_t *w_codes, const uint8_t *w_scales,
                        int w_format, void *d, const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int E,
                        int F, const uint8_t *floor_tab_host, void *workspace, int64_t workspace_bytes, int *status,
                        const mxq_gemm_options *options, void *stream);

/* Softmax over the last dimension of rows that are MX-quantized first, in one pass: replaces softmax_mxfp /
 * softmax_mxint / softmax_minifloat (chop/nn/quantized/functional/softmax.py:10-57: quantize along the last dimension,
 * softmax in fp32, cast back).  x, y: [rows, cols] of `dtype`, contiguous.  quantizer: 0 = MXFP (p0 = E, p1 = F, floor
 * table), 1 = MXINT (p0 = bits, ceil table of x's dtype), 2 = element-wise minifloat (p0 = E, p1 = F, no table, block
 * ignored).  cols % block == 0 and cols <= 12288 (the row is kept in shared memory), else MXQ_ERR_SHAPE /
 * MXQ_ERR_UNSUPPORTED. */
int mxq_softmax_quant(const void *x, void *y, int dtype, int64_t rows, int64_t cols, int quantizer, int block, int p0,
                      int p1, const uint8_t *tab_host, void *stream);

/* The softmax of an attention block with what surrounds it, one warp per row, one pass over HBM.  Replaces, with the
 * roundings of the separate tensor operations (T = dtype),
 *     s = matmul_result * scaling; s = s + causal_mask; p = softmax_minifloat(s) (or the fp32 softmax); p = quantizer(p)
 * of chop/nn/quantized/modules/llama/attention.py:352-388:
 *     s = round_T(x * scale) when use_scale; s = round_T(s + mask[b, 0, i, :]) when mask != NULL
 *     q = quantizer(s): 0 MXFP(p0 = E, p1 = F), 1 MXINT(p0 = bits), 2 element-wise minifloat(p0 = E, p1 = F), 3 none
 *     p = round_T(softmax over the row of fp32(q))
 *     y = out_quantizer(p): 0 MXFP, 1 MXINT, 3 none
 * x, y: [rows, cols] of dtype, rows = batch * heads * mask_rows in that order; mask: dtype [batch, 1, mask_rows, >= cols]
 * with row stride mask_ld (elements) and batch stride mask_rows * mask_ld, finite values.  The MX quantizers work on
 * blocks of 32 along the row (block / out_block must be 32) with the host log2 tables of the plain quantizers.
 * cols % 32 == 0 and cols <= 2048, else MXQ_ERR_UNSUPPORTED (compose the operations instead). */
int mxq_attention_softmax(const void *x, void *y, int dtype, int64_t rows, int64_t cols, int use_scale, float scale,
                          const void *mask, int64_t mask_ld, int64_t mask_rows, int64_t heads, int quantizer, int block,
                          int p0, int p1, const uint8_t *tab_host, int out_quantizer, int out_block, int out_p0,
                          int out_p1, const uint8_t *out_tab_host, void *stream);

/* Rotary position embedding y = x * cos + rotate_half(x) * sin in one pass.  Replaces _apply_rope
 * (chop/nn/quantized/functional/rope.py:17-28; the rope_mxfp / rope_mxint / rope_minifloat wrappers quantize the
 * tables first and then call it).  x: [batch, heads, seq, dim] of `dtype` with a contiguous last dimension and the
 * element strides given (a transposed view of a [batch, seq, heads * dim] projection, for instance); y: the same shape,
 * contiguous, not overlapping x -- the layout the attention products read; cos, sin:
 * [batch or 1, seq, dim] of `table_dtype` (table_stride_b = 0 for tables shared by the batch).  dim % 16 == 0.
 * Tables of the tensor's dtype: each product and the sum are rounded to it, as the framework's elementwise kernels
 * do; fp32 tables with a bf16 tensor: evaluated in fp32 and rounded once. */
int mxq_rope(const void *x, void *y, const void *cos, const void *sin, int dtype, int table_dtype, int64_t batch,
             int64_t heads, int64_t seq, int64_t dim, int64_t x_stride_b, int64_t x_stride_h, int64_t x_stride_s,
             int64_t table_stride_b, int64_t table_stride_s, void *stream);

/*
 * Row-parallel Linear over the GPUs of one node (tensor parallelism).  The reference reaches this point through
 * DTensor redistribution (chop/distributed/tensor/_redistribute.py:189-245: partial -> replicate = all-reduce); here
 * the reduction is part of the GEMM and of one small kernel, over peer memory.  All buffers are symmetric
 * allocations of the caller: `*_ptrs` are HOST arrays of `world` device pointers, entry r = the buffer of GPU r as
 * mapped in this process; the calling process owns GPU `rank`.
 *
 *   slots    fp32 [world][M / world][N] per GPU: slot s of GPU r receives GPU s's partial sums of GPU r's row slice
 *   out      [M][N] of out_dtype per GPU: every GPU's copy of the reduced result
 *   flags    uint32 [world] per GPU, zero before the first barrier; `epoch` grows by one per barrier
 *
 * Sequence on every GPU, one stream: mxq_gemm_mxf8_scatter, mxq_peer_barrier(epoch), mxq_reduce_gather,
 * mxq_peer_barrier(epoch + 1); afterwards `out` is complete on every GPU.
 */

/* Block-scaled GEMM of this GPU's K shard whose epilogue stores every fp32 tile directly into the slot of the GPU
 * that owns the tile's rows (bulk tensor stores over NVLink; no multicast, no collective): the reduce-scatter
 * travels under the MMAs.  Needs (M / world) % 256 == 0; MXQ_ERR_UNSUPPORTED otherwise (use a collective). */
int mxq_gemm_mxf8_scatter(const uint8_t *a_codes, const uint8_t *a_scales, const uint8_t *b_codes, const uint8_t *b_scales,
                          int b_format, void *const *slot_ptrs, int world, int rank, int64_t M, int64_t N, int64_t K,
                          int *status, const mxq_gemm_options *options, void *stream);

/* Every GPU publishes `epoch` to all others (after a system-wide fence: its earlier stores are visible) and waits
 * until it has received theirs.  The wait is bounded (wait_limit_ns, 0 = one second): when a GPU does not arrive the
 * kernel stores 7 in the status word and returns.  One warp. */
int mxq_peer_barrier(void *const *flag_ptrs, int world, int rank, uint32_t epoch, int *status, int64_t wait_limit_ns,
                     void *stream);

/* This GPU's row slice: sum of its `world` slots in rank order (repeatable) + bias, one rounding to out_dtype,
 * written to rows [rank * rows, (rank + 1) * rows) of every GPU's `out` (peer stores): reduce + all-gather.
 * n % 8 == 0.  max_ctas caps the grid (0 = no cap) so that it can run beside a GEMM. */
int mxq_reduce_gather(const void *slots, int world, int rank, int64_t rows, int64_t n, const void *bias, int bias_dtype,
                      void *const *out_ptrs, int out_dtype, int max_ctas, void *stream);

/* mxq_reduce_gather for an output that the next layer consumes as an MXFP(E, F) activation (blocks of 32 along n):
 * the reduced slice is rounded to bf16 -- the value a separate output tensor would hold -- quantized exactly as
 * mxq_mxfp_pack_mma quantizes that tensor, and written as E4M3 bytes [world * rows, n] + scale chunks
 * (mxq_mma_scale_bytes(world * rows, n)) into every GPU's operand buffers; with out_ptrs != NULL the bf16 rows are
 * written as well.  Half the all-gather bytes, and the consumer needs no pack.  n % 128 == 0. */
int mxq_reduce_gather_pack(const void *slots, int world, int rank, int64_t rows, int64_t n, const void *bias,
                           int bias_dtype, void *const *codes_ptrs, void *const *scales_ptrs, void *const *out_ptrs, int E,
                           int F, const uint8_t *floor_tab_host, int max_ctas, void *stream);

/* Allocation-free variant of mxq_mx_linear.  It has no counterpart in the reference.
 *
 * Some callers are not in a position to hand over scratch memory: code that runs where the allocator must not be
 * touched (inside a serving loop with a frozen memory pool, in a plugin that only receives input and output
 * buffers from its host application, or in a process whose device memory is fully pre-partitioned), for whom a
 * cudaMalloc -- or a caching allocator falling back to one -- is either forbidden or an unpredictable stall.  For
 * them the packed activations go into a fixed array that is part of the library's device image:
 * MXQ_STATIC_SCRATCH_BYTES (40 MiB) on every GPU that loads the library, held until the process exits.
 *
 *   - needs mxq_mx_linear_workspace_bytes(M, K) <= MXQ_STATIC_SCRATCH_BYTES (e.g. M = 8192, K = 4096 fits); larger
 *     problems return MXQ_ERR_TOO_LARGE and must use mxq_mx_linear with their own workspace;
 *   - calls no cudaMalloc / cudaFree and no allocating library routine; inputs and the output are the caller's;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and caches it: make that first call with the right device current and before any stream capture;
 *   - every call on a device shares the one array, which keeps whatever the last call left in it.  A call overwrites
 *     the M x K code bytes and the scale bytes of its M rows before it reads them.  The
 *     scale bytes of the padding rows (M rounded up to 256) are NOT rewritten and may hold an earlier call's bytes:
 *     the tensor cores do read them, but they only scale accumulator rows >= M, which are never stored.  Scale bytes
 *     of K blocks past the end of a row (K not a multiple of 128) are cleared by every call, because there a stale
 *     0xFF (NaN) would meet the zero-filled codes of rows that are stored.  So leftovers are harmless, but two calls
 *     that overlap in time on the same GPU (different streams or threads) race on the array and corrupt each
 *     other's result: serialise them.
 * Arguments and results are otherwise those of mxq_mx_linear. */
#define MXQ_STATIC_SCRATCH_BYTES (40u << 20)
int mxq_mx_linear_static(const void *x, int in_dtype, const uint8_t *w_codes, const uint8_t *w_scales, int w_format, void *d,
                         const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int E, int F,
                         const uint8_t *floor_tab_host, int *status, const mxq_gemm_options *options, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MXQ_H_ */
