// Block quantizer kernels (MXINT, MXFP, minifloat, block floating point) and their C entry points.
//
// Fast path: the tensor is a flat run of blocks of B consecutive elements, B a power of two.  Every
// thread owns one 16-byte vector (4 fp32 or 8 bf16 elements) per step, so a block is shared by
// G = B / vector-length neighbouring lanes; the block maximum is found with log2(G) xor-shuffles, the
// shared exponent is derived from its bits, and elements are encoded in registers.  Loads and stores are
// 128-bit, fully coalesced and streaming (evict-first); a CTA handles kUnroll independent vectors per
// thread per step to keep enough bytes in flight for HBM3e.
//
// Generic path: any other block size (smaller than a vector, not a power of two, wider than a warp's
// span, or a ragged row tail for block-fp) is handled by one thread per block with scalar accesses.

#include "mxq_common.cuh"
#include "mxq_internal.h"
#include "mxq_pack.cuh"

namespace mxq {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

enum class Mode { kFake, kCodes };

// ---------------------------------------------------------------------------------------------------
// MXINT
// ---------------------------------------------------------------------------------------------------
template <typename Tin, typename Tout, Mode kMode>
__global__ void __launch_bounds__(kThreads)
mxint_kernel(const Tin *__restrict__ x, Tout *__restrict__ y, int8_t *__restrict__ mant, uint8_t *__restrict__ scales,
             int64_t n_vec, int group, int bits, const __grid_constant__ Log2Tab tab) {
  constexpr int N = Elem<Tin>::kVec;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x);
  const int64_t step = (int64_t)gridDim.x * kThreads * kUnroll;
  for (int64_t base = (int64_t)blockIdx.x * kThreads * kUnroll; base < n_vec; base += step) {
    uint4 raw[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + u * kThreads + threadIdx.x;
      raw[u] = i < n_vec ? ld_stream(xv + i) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + u * kThreads + threadIdx.x;
      uint32_t b[N];
      unpack(raw[u], b);
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < N; ++k) amax = fmaxf(amax, fabsf(__uint_as_float(b[k])));
      amax = group_max(amax, group);
      const MxintBlock p = mxint_block<Elem<Tin>::kBf16>(amax, bits, tab);
      if (i >= n_vec) continue;
      if constexpr (kMode == Mode::kFake) {
        float out[N];
#pragma unroll
        for (int k = 0; k < N; ++k) out[k] = mxint_dequant(mxint_mant(__uint_as_float(b[k]), p), p);
        store_vals(y, i * N, out);
      } else {
        uint32_t c[N];
#pragma unroll
        for (int k = 0; k < N; ++k) c[k] = (uint32_t)(int)mxint_mant(__uint_as_float(b[k]), p) & 0xFFu;
        store_bytes(reinterpret_cast<uint8_t *>(mant), i * N, c);
        if ((threadIdx.x & (group - 1)) == 0) scales[i / group] = (uint8_t)p.scale;
      }
    }
  }
}

template <typename Tin, typename Tout, Mode kMode>
__global__ void __launch_bounds__(kThreads)
mxint_generic_kernel(const Tin *__restrict__ x, Tout *__restrict__ y, int8_t *__restrict__ mant,
                     uint8_t *__restrict__ scales, int64_t n_blocks, int block, int bits,
                     const __grid_constant__ Log2Tab tab) {
  for (int64_t blk = (int64_t)blockIdx.x * kThreads + threadIdx.x; blk < n_blocks;
       blk += (int64_t)gridDim.x * kThreads) {
    const Tin *xb = x + blk * block;
    float amax = 0.f;
    for (int k = 0; k < block; ++k) amax = fmaxf(amax, fabsf(load_scalar(xb + k)));
    const MxintBlock p = mxint_block<Elem<Tin>::kBf16>(amax, bits, tab);
    for (int k = 0; k < block; ++k) {
      const float m = mxint_mant(load_scalar(xb + k), p);
      if constexpr (kMode == Mode::kFake)
        store_scalar(y + blk * block + k, mxint_dequant(m, p));
      else
        mant[blk * block + k] = (int8_t)(int)m;
    }
    if constexpr (kMode == Mode::kCodes) scales[blk] = (uint8_t)p.scale;
  }
}

template <typename Tout>
__global__ void __launch_bounds__(kThreads)
mxint_compose_kernel(const int8_t *__restrict__ mant, const uint8_t *__restrict__ scales, Tout *__restrict__ y,
                     int64_t n, int block, int bits) {
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads) {
    const int k = (int)scales[i / block] - 127;
    const float m = (float)mant[i];
    // mant / 2**(bits-1) * 2**(scale-127); 2**128 is inf in the reference's working dtype
    const float v = k >= 128 ? m * __int_as_float(0x7F800000) : m * pow2f(k - (bits - 1));
    store_scalar(y + i, v);
  }
}

// ---------------------------------------------------------------------------------------------------
// MXFP
// ---------------------------------------------------------------------------------------------------
template <typename Tin, typename Tout, Mode kMode, int E, int F>
__global__ void __launch_bounds__(kThreads)
mxfp_kernel(const Tin *__restrict__ x, Tout *__restrict__ y, uint8_t *__restrict__ codes, uint8_t *__restrict__ scales,
            int64_t n_vec, int group, const __grid_constant__ Log2Tab tab) {
  constexpr int N = Elem<Tin>::kVec;
  constexpr bool kBf16In = Elem<Tin>::kBf16;
  constexpr int kTop = (1 << E) - 1;
  constexpr int kBias = (1 << (E - 1)) - 1;
  constexpr int kEmax = kTop - kBias;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x);
  const int64_t step = (int64_t)gridDim.x * kThreads * kUnroll;
  for (int64_t base = (int64_t)blockIdx.x * kThreads * kUnroll; base < n_vec; base += step) {
    uint4 raw[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + u * kThreads + threadIdx.x;
      raw[u] = i < n_vec ? ld_stream(xv + i) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + u * kThreads + threadIdx.x;
      const uint32_t r[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
      // ---- block maximum of |x| as an fp32 bit pattern (0 when every element is zero or an fp32 subnormal) ----
      uint32_t a[4], amax;
      if constexpr (kBf16In) {
        __nv_bfloat162 m2 = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&(a[0] = r[0] & 0x7FFF7FFFu)),
                                    *reinterpret_cast<const __nv_bfloat162 *>(&(a[1] = r[1] & 0x7FFF7FFFu)));
        m2 = __hmax2(m2, __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&(a[2] = r[2] & 0x7FFF7FFFu)),
                                 *reinterpret_cast<const __nv_bfloat162 *>(&(a[3] = r[3] & 0x7FFF7FFFu))));
        const uint32_t mb = *reinterpret_cast<uint32_t *>(&m2);
        const uint32_t m = group_max(max(mb & 0xFFFFu, mb >> 16), group);
        amax = (m >> 7) ? (m << 16) : 0u;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] = r[k] & 0x7FFFFFFFu;
        const uint32_t m = group_max(max(max(a[0], a[1]), max(a[2], a[3])), group);
        amax = (m >> 23) ? m : 0u;
      }
      if (i >= n_vec) continue;
      const int exm = (int)(amax >> 23);
      int up = 0;  // host log2 rounds up to the next integer for fp32 maxima a few ulps below a power of two
      if constexpr (!kBf16In) {
        const uint32_t man = amax & 0x7FFFFFu;
        if (man >= 0x7FFF00u) up = (0x7FFFFFu - man) < tab.t[exm] ? 1 : 0;
      }
      const int K = exm + up - kTop;
      // `fast`: every element has a normal code (ye >= 1).  `sub`: some have subnormal codes or underflow, and the
      // vector still avoids clamped scales and inf / nan; fake-quantization then stays on the bit patterns too.
      // Narrow-exponent formats (E <= 3) meet small codes in almost every vector and skip the first test.
      constexpr bool kSubPath = kMode == Mode::kFake;
      constexpr bool kTryFast = !kSubPath || E >= 4;
      bool fast = kTryFast && K >= 1;
      const bool sub = kSubPath && K >= 1 && exm != 255;
      uint32_t yq[N];  // rounded |x| as fp32 bit patterns (bf16 input: two bf16 patterns per word in yq[0..3])
      if constexpr (kBf16In) {
        if constexpr (kTryFast) {
          const uint32_t t1 = (uint32_t)((K + 1) << 7) * 0x00010001u;
          const __nv_bfloat162 t1v = *reinterpret_cast<const __nv_bfloat162 *>(&t1);
#pragma unroll
          for (int k = 0; k < 4; ++k) fast = fast && __hbge2(*reinterpret_cast<const __nv_bfloat162 *>(&a[k]), t1v);
        }
        const uint32_t kodd2 = (K & 1) ? 0x00800080u : 0u;
        if (fast) {
#pragma unroll
          for (int k = 0; k < 4; ++k) yq[k] = mxfp_round_pair<F>(a[k], kodd2);
          if constexpr (kSubPath) {
#pragma unroll
            for (int k = 0; k < 4; ++k) yq[k] |= r[k] & 0x80008000u;
          }
        } else if (sub) {
          const SubThresholds2 th = sub_thresholds2<E, F>(K);
#pragma unroll
          for (int k = 0; k < 4; ++k) yq[k] = mxfp_round_pair_sub<F>(r[k], kodd2, th);
        }
      } else {
        if constexpr (kTryFast) {
          const uint32_t t1 = (uint32_t)(K + 1) << 23;
#pragma unroll
          for (int k = 0; k < 4; ++k) fast = fast && a[k] >= t1;
        }
        if (fast) {
          const uint32_t kodd = (K & 1) ? 0x00800000u : 0u;
#pragma unroll
          for (int k = 0; k < 4; ++k) yq[k] = mxfp_round_one<F>(a[k] & 0x7FFFFF00u, kodd);
          if constexpr (kSubPath) {
#pragma unroll
            for (int k = 0; k < 4; ++k) yq[k] |= r[k] & 0x80000000u;
          }
        } else if (sub) {
#pragma unroll
          for (int k = 0; k < 4; ++k) yq[k] = mxfp_round_one_sub<E, F>(r[k], K);
        }
      }
      if (fast || sub) {
        if constexpr (kMode == Mode::kFake) {  // yq holds the signed results
          if constexpr (kBf16In && Elem<Tout>::kBf16) {
            st_stream(reinterpret_cast<uint4 *>(y) + i, make_uint4(yq[0], yq[1], yq[2], yq[3]));
          } else {
            float out[N];
            if constexpr (kBf16In) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                out[2 * k] = __uint_as_float(yq[k] << 16), out[2 * k + 1] = __uint_as_float(yq[k] & 0xFFFF0000u);
              }
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) out[k] = __uint_as_float(yq[k]);
            }
            store_vals(y, i * N, out);
          }
        } else {
          // code = sign | ((ye << F) | f) with ye = ex - K: the rounded pattern shifted down, minus K << F
          if constexpr (kBf16In) {
            uint32_t c2[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              c2[k] = ((yq[k] >> (7 - F)) - (uint32_t)(K << F) * 0x00010001u) |
                      ((r[k] >> (15 - (E + F))) & ((1u << (E + F)) * 0x00010001u));
            __stcs(reinterpret_cast<uint2 *>(codes + i * N),
                   make_uint2(__byte_perm(c2[0], c2[1], 0x6420), __byte_perm(c2[2], c2[3], 0x6420)));
          } else {
            uint32_t c[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              c[k] = ((yq[k] >> (23 - F)) - (uint32_t)(K << F)) | ((r[k] >> (31 - (E + F))) & (1u << (E + F)));
            store_bytes(codes, i * N, c);
          }
          if ((threadIdx.x & (group - 1)) == 0) scales[i / group] = (uint8_t)(exm + up - kEmax);
        }
      } else {
        // ---- general path: subnormal / underflowing / flushed elements, all-zero blocks, clamped scales ----
        uint32_t b[N];
        unpack(raw[u], b);
#pragma unroll
        for (int k = 0; k < N; ++k)
          if (((b[k] & 0x7FFFFFFFu) >> 23) == 0) b[k] = 0;  // fp32 subnormals and -0 are flushed to +0
        const MxfpBlock p = mxfp_block(amax, E, tab);
        if constexpr (kMode == Mode::kFake) {
          float out[N];
#pragma unroll
          for (int k = 0; k < N; ++k) out[k] = mxfp_decode(mxfp_encode(b[k], p.sh, E, F), E, F) * p.scale_f;
          store_vals(y, i * N, out);
        } else {
          uint32_t c[N];
#pragma unroll
          for (int k = 0; k < N; ++k) c[k] = mxfp_encode(b[k], p.sh, E, F);
          store_bytes(codes, i * N, c);
          if ((threadIdx.x & (group - 1)) == 0) scales[i / group] = (uint8_t)p.scale;
        }
      }
    }
  }
}

// byte offset of the E8M0 scale of (row, block kb of 32 along K) in the tensor-core scale layout
template <typename I>
__device__ __forceinline__ I mma_scale_offset(I row, I kb, I k_chunks) {
  return ((row >> 7) * k_chunks + (kb >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kb & 3);
}

// fp32 tensors: one 16-byte vector (4 elements) per lane and step, 8 lanes per block
template <int E, int F>
__global__ void __launch_bounds__(kThreads)
mxfp_pack_mma_f32_kernel(const float *__restrict__ x, uint8_t *__restrict__ codes, uint8_t *__restrict__ scales,
                         int64_t n_vec, uint32_t vec_per_row, int64_t k_chunks, const __grid_constant__ Log2Tab tab) {
  constexpr int kU = 2;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x);
  const int64_t step = (int64_t)gridDim.x * kThreads * kU;
  for (int64_t base = (int64_t)blockIdx.x * kThreads * kU; base < n_vec; base += step) {
    uint4 raws[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t i = base + u * kThreads + threadIdx.x;
      raws[u] = i < n_vec ? ld_stream(xv + i) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t i = base + u * kThreads + threadIdx.x;
      int scale;
      const uint32_t c4 = pack_f32<E, F>(raws[u], tab, scale);  // every lane of the warp takes part (shuffles inside)
      if (i >= n_vec) continue;
      __stcs(reinterpret_cast<uint32_t *>(codes + i * 4), c4);
      if ((threadIdx.x & 7) == 0) {
        const int64_t row = i / vec_per_row, vcol = i - row * vec_per_row;
        scales[mma_scale_offset<int64_t>(row, vcol >> 3, k_chunks)] = (uint8_t)scale;
      }
    }
  }
}

// bf16 tensors: 32 bytes (16 elements, half a block) per lane and step.  The position of a unit in the matrix is
// carried along by additions: `jump` = (rows, units) to add per kThreads units, `stride` = the same per grid step.
struct UnitStep {
  uint32_t rows, units;
};
template <bool kWide>
__device__ __forceinline__ void load_unit(const __nv_bfloat16 *x, int64_t unit, uint4 &lo, uint4 &hi) {
  if constexpr (kWide) {  // one 32-byte load (the pointer is 32-byte aligned)
    asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(x + unit * 16));
  } else {
    const uint4 *p = reinterpret_cast<const uint4 *>(x) + unit * 2;
    lo = ld_stream(p), hi = ld_stream(p + 1);
  }
}
// I = uint32_t when unit indices and scale offsets fit in 32 bits (the usual case), else int64_t.
template <int E, int F, bool kWide, typename I>
__global__ void __launch_bounds__(kThreads, 4)
mxfp_pack_mma_bf16_kernel(const __nv_bfloat16 *__restrict__ x, uint8_t *__restrict__ codes,
                          uint8_t *__restrict__ scales, int64_t n_unit64, uint32_t unit_per_row, int64_t k_chunks,
                          UnitStep jump, UnitStep stride, const __grid_constant__ Log2Tab tab, uint32_t chained) {
  constexpr int kU = 2;
  // Inside a fused Linear call: the GEMM that follows in the stream may be launched from now on (it sets up its
  // barriers and tensor memory, and may fetch its weight, while this kernel runs, and waits on the device for the
  // operands written here); this kernel itself may have been launched under the tail of the previous one and waits
  // for it before reading x or writing the scratch that kernel may still be reading.
  if (chained) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  const I n_unit = (I)n_unit64;
  const I step = (I)gridDim.x * kThreads * kU;
  I base = (I)blockIdx.x * kThreads * kU;
  // (row, unit in row) of this lane's first unit
  I row;
  uint32_t col;
  {
    const I j = base + threadIdx.x;
    if (j <= (I)0x7FFFFFFF) {
      const uint32_t q = (uint32_t)j / unit_per_row;
      row = q, col = (uint32_t)j - q * unit_per_row;
    } else {
      row = j / unit_per_row, col = (uint32_t)(j - row * unit_per_row);
    }
  }
  for (; base < n_unit; base += step) {
    uint4 raws[kU][2];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const I j = base + u * kThreads + threadIdx.x;
      if (j < n_unit)
        load_unit<kWide>(x, (int64_t)j, raws[u][0], raws[u][1]);
      else
        raws[u][0] = raws[u][1] = make_uint4(0, 0, 0, 0);
    }
    I r = row;
    uint32_t c = col;
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const I j = base + u * kThreads + threadIdx.x;
      int scale;
      const uint4 c16 = pack_bf16<E, F>(raws[u][0], raws[u][1], tab, scale);  // all lanes take part (shuffle inside)
      if (j < n_unit) {
        __stcs(reinterpret_cast<uint4 *>(codes) + j, c16);
        if ((threadIdx.x & 1) == 0) scales[mma_scale_offset<I>(r, (I)(c >> 1), (I)k_chunks)] = (uint8_t)scale;
      }
      c += jump.units, r += jump.rows;
      if (c >= unit_per_row) c -= unit_per_row, ++r;
    }
    col += stride.units, row += stride.rows;
    if (col >= unit_per_row) col -= unit_per_row, ++row;
  }
}

// Gated-MLP hidden state straight into tensor-core operands: h = silu(gate) * up in bf16 exactly as the framework's
// elementwise kernels compute it (silu evaluated in fp32 as g / (1 + exp(-g)) and rounded to bf16, the product
// evaluated in fp32 and rounded to bf16), then the MXFP pack of the kernel above on h.  gate and up are [rows, k]
// views with a common row stride (the two halves of one [rows, 2k] GEMM output, for instance).  One unit = 16
// elements per lane and step.
__device__ __forceinline__ uint32_t silu_mul_pair(uint32_t g2, uint32_t u2) {
  float g0 = __uint_as_float(g2 << 16), g1 = __uint_as_float(g2 & 0xFFFF0000u);
  float u0 = __uint_as_float(u2 << 16), u1 = __uint_as_float(u2 & 0xFFFF0000u);
  const float s0 = __bfloat162float(__float2bfloat16_rn(g0 / (1.0f + expf(-g0))));
  const float s1 = __bfloat162float(__float2bfloat16_rn(g1 / (1.0f + expf(-g1))));
  const __nv_bfloat162 h = __floats2bfloat162_rn(s0 * u0, s1 * u1);
  return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ uint4 silu_mul_vec(const uint4 &g, const uint4 &u) {
  return make_uint4(silu_mul_pair(g.x, u.x), silu_mul_pair(g.y, u.y), silu_mul_pair(g.z, u.z), silu_mul_pair(g.w, u.w));
}
template <int E, int F>
__global__ void __launch_bounds__(kThreads, 4)
silu_mul_pack_mma_kernel(const __nv_bfloat16 *__restrict__ gate, const __nv_bfloat16 *__restrict__ up, int64_t ld,
                         uint8_t *__restrict__ codes, uint8_t *__restrict__ scales, int64_t n_unit,
                         uint32_t unit_per_row, int64_t k_chunks, const __grid_constant__ Log2Tab tab, uint32_t chained) {
  if (chained) {  // see mxfp_pack_mma_bf16_kernel
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  const int64_t step = (int64_t)gridDim.x * kThreads;
  for (int64_t base = (int64_t)blockIdx.x * kThreads; base < n_unit; base += step) {
    const int64_t j = base + threadIdx.x;
    const bool live = j < n_unit;
    int64_t row = 0;
    uint32_t col = 0;
    uint4 h_lo = make_uint4(0, 0, 0, 0), h_hi = h_lo;
    if (live) {
      row = j / unit_per_row, col = (uint32_t)(j - row * unit_per_row);
      const uint4 *pg = reinterpret_cast<const uint4 *>(gate + row * ld + (int64_t)col * 16);
      const uint4 *pu = reinterpret_cast<const uint4 *>(up + row * ld + (int64_t)col * 16);
      const uint4 g_lo = ld_stream(pg), g_hi = ld_stream(pg + 1), u_lo = ld_stream(pu), u_hi = ld_stream(pu + 1);
      h_lo = silu_mul_vec(g_lo, u_lo), h_hi = silu_mul_vec(g_hi, u_hi);
    }
    int scale;
    const uint4 c16 = pack_bf16<E, F>(h_lo, h_hi, tab, scale);  // all lanes take part (shuffle inside)
    if (live) {
      __stcs(reinterpret_cast<uint4 *>(codes) + j, c16);
      if ((threadIdx.x & 1) == 0) scales[mma_scale_offset<int64_t>(row, (int64_t)(col >> 1), k_chunks)] = (uint8_t)scale;
    }
  }
}

// MXFP4 (E2M1) weights as nibble-packed tensor-core operands: one thread per block of 32 elements, the element codec
// of the generic path, two codes per byte (element 2i in the low nibble), the scale in the tensor-core chunk layout.
// Runs once per weight at load time.
template <typename Tin>
__global__ void __launch_bounds__(kThreads)
mxfp4_pack_mma_kernel(const Tin *__restrict__ x, uint8_t *__restrict__ codes4, uint8_t *__restrict__ scales,
                      int64_t n_blocks, int64_t blocks_per_row, int64_t k_chunks, const __grid_constant__ Log2Tab tab) {
  for (int64_t blk = (int64_t)blockIdx.x * kThreads + threadIdx.x; blk < n_blocks;
       blk += (int64_t)gridDim.x * kThreads) {
    const Tin *xb = x + blk * 32;
    uint32_t bits[32];
    uint32_t amax = 0;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      uint32_t b = __float_as_uint(load_scalar(xb + k));
      if (((b & 0x7FFFFFFFu) >> 23) == 0) b = 0;  // zero and fp32-subnormal inputs are flushed
      bits[k] = b;
      amax = max(amax, b & 0x7FFFFFFFu);
    }
    const MxfpBlock p = mxfp_block(amax, 2, tab);
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t word = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) word |= (mxfp_encode(bits[8 * q + k], p.sh, 2, 1) & 0xFu) << (4 * k);
      w[q] = word;
    }
    *reinterpret_cast<uint4 *>(codes4 + blk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    const int64_t row = blk / blocks_per_row, kb = blk - row * blocks_per_row;
    scales[mma_scale_offset<int64_t>(row, kb, k_chunks)] = (uint8_t)p.scale;
  }
}

// MXINT mantissas and shared exponents of bf16 tensors in blocks of 32: the same half-block-per-lane scheme.
template <bool kWide>
__global__ void __launch_bounds__(kThreads, 4)
mxint_codes_bf16_kernel(const __nv_bfloat16 *__restrict__ x, int8_t *__restrict__ mant, uint8_t *__restrict__ scales,
                        int64_t n_unit, int bits, const __grid_constant__ Log2Tab tab) {
  constexpr int kU = 2;
  const int64_t step = (int64_t)gridDim.x * kThreads * kU;
  for (int64_t base = (int64_t)blockIdx.x * kThreads * kU; base < n_unit; base += step) {
    uint4 raws[kU][2];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t j = base + u * kThreads + threadIdx.x;
      if (j < n_unit)
        load_unit<kWide>(x, j, raws[u][0], raws[u][1]);
      else
        raws[u][0] = raws[u][1] = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t j = base + u * kThreads + threadIdx.x;
      int scale;
      const uint4 c16 = mxint_codes_bf16(raws[u][0], raws[u][1], tab, bits, scale);  // all lanes take part
      if (j < n_unit) {
        __stcs(reinterpret_cast<uint4 *>(mant) + j, c16);
        if ((threadIdx.x & 1) == 0) scales[j >> 1] = (uint8_t)scale;
      }
    }
  }
}

// Reference codes and E8M0 scales of bf16 tensors in blocks of 32: 32 bytes (half a block) per lane and step, codes
// stored 16 bytes per lane, one scale byte per pair of lanes.
template <int E, int F, bool kWide>
__global__ void __launch_bounds__(kThreads, 4)
mxfp_codes_bf16_kernel(const __nv_bfloat16 *__restrict__ x, uint8_t *__restrict__ codes, uint8_t *__restrict__ scales,
                       int64_t n_unit, const __grid_constant__ Log2Tab tab) {
  constexpr int kU = 2;
  const int64_t step = (int64_t)gridDim.x * kThreads * kU;
  for (int64_t base = (int64_t)blockIdx.x * kThreads * kU; base < n_unit; base += step) {
    uint4 raws[kU][2];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t j = base + u * kThreads + threadIdx.x;
      if (j < n_unit)
        load_unit<kWide>(x, j, raws[u][0], raws[u][1]);
      else
        raws[u][0] = raws[u][1] = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t j = base + u * kThreads + threadIdx.x;
      int scale;
      const uint4 c16 = codes_bf16<E, F>(raws[u][0], raws[u][1], tab, scale);  // all lanes take part (shuffle inside)
      if (j < n_unit) {
        __stcs(reinterpret_cast<uint4 *>(codes) + j, c16);
        if ((threadIdx.x & 1) == 0) scales[j >> 1] = (uint8_t)scale;
      }
    }
  }
}

template <typename Tin, typename Tout, Mode kMode>
__global__ void __launch_bounds__(kThreads)
mxfp_generic_kernel(const Tin *__restrict__ x, Tout *__restrict__ y, uint8_t *__restrict__ codes,
                    uint8_t *__restrict__ scales, int64_t n_blocks, int block, int E, int F,
                    const __grid_constant__ Log2Tab tab) {
  for (int64_t blk = (int64_t)blockIdx.x * kThreads + threadIdx.x; blk < n_blocks;
       blk += (int64_t)gridDim.x * kThreads) {
    const Tin *xb = x + blk * block;
    uint32_t amax = 0;
    for (int k = 0; k < block; ++k) {
      const uint32_t a = __float_as_uint(load_scalar(xb + k)) & 0x7FFFFFFFu;
      amax = max(amax, (a >> 23) == 0 ? 0u : a);
    }
    const MxfpBlock p = mxfp_block(amax, E, tab);
    for (int k = 0; k < block; ++k) {
      uint32_t b = __float_as_uint(load_scalar(xb + k));
      if (((b & 0x7FFFFFFFu) >> 23) == 0) b = 0;
      const uint32_t c = mxfp_encode(b, p.sh, E, F);
      if constexpr (kMode == Mode::kFake)
        store_scalar(y + blk * block + k, mxfp_decode(c, E, F) * p.scale_f);
      else
        codes[blk * block + k] = (uint8_t)c;
    }
    if constexpr (kMode == Mode::kCodes) scales[blk] = (uint8_t)p.scale;
  }
}

template <typename Tout>
__global__ void __launch_bounds__(kThreads)
mxfp_compose_kernel(const uint8_t *__restrict__ codes, const uint8_t *__restrict__ scales, Tout *__restrict__ y,
                    int64_t n, int block, int E, int F) {
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads) {
    const float sf = pow2f((int)scales[i / block] - 127);
    store_scalar(y + i, mxfp_decode(codes[i], E, F) * sf);
  }
}

// element-wise minifloat: the MXFP codec with a unit scale; input subnormals flush, sign follows x < 0
template <typename Tin, typename Tout>
__global__ void __launch_bounds__(kThreads)
minifloat_kernel(const Tin *__restrict__ x, Tout *__restrict__ y, int64_t n, int E, int F) {
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads) {
    const uint32_t b = __float_as_uint(load_scalar(x + i));
    uint32_t c = mxfp_encode(b & 0x7FFFFFFFu, 0, E, F);
    if ((b >> 31) && (b & 0x7FFFFFFFu) != 0) c |= 1u << (E + F);  // x < 0, also for flushed subnormals
    store_scalar(y + i, mxfp_decode(c, E, F));
  }
}

// ---------------------------------------------------------------------------------------------------
// block floating point
// ---------------------------------------------------------------------------------------------------
// Fast path of block floating point: when the tile exponent e leaves 2**(mb-e) and 2**(e-mb) in the normal
// fp32 range and every element is either exactly zero or large enough that the reference's "+1e-9" and its
// "close to zero" pass-through cannot matter (bf16: |x| >= 2**-21; fp32: |x| > 1e-8, where the addition is kept),
// the result is sign(x) * min(rint(val * 2**(mb-e)), hi) * 2**(e-mb).  Other vectors take bfp_elem().
template <typename T>
__global__ void __launch_bounds__(kThreads)
bfp_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t n_vec, int group, int width, int exp_width, int exp_bias,
           const __grid_constant__ Log2Tab tab) {
  constexpr int N = Elem<T>::kVec;
  constexpr bool kBf16 = Elem<T>::kBf16;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x);
  const int64_t step = (int64_t)gridDim.x * kThreads * kUnroll;
  const int mb = width - 1;
  const int e_lo = -exp_bias, e_hi = (1 << exp_width) - 1 - exp_bias;
  const float hi = round_to<T>((float)((1 << mb) - 1));
  // smallest |x| bit pattern that stays on the fast path, minus one (so that 0 - 1 wraps and passes too)
  const uint32_t thr_m1 = kBf16 ? ((uint32_t)(127 - 21) << 23) - 1u : __float_as_uint(1e-8f);
  for (int64_t base = (int64_t)blockIdx.x * kThreads * kUnroll; base < n_vec; base += step) {
    uint4 raw[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + u * kThreads + threadIdx.x;
      raw[u] = i < n_vec ? ld_stream(xv + i) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + u * kThreads + threadIdx.x;
      uint32_t b[N];
      unpack(raw[u], b);
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < N; ++k) amax = fmaxf(amax, fabsf(__uint_as_float(b[k])));
      amax = group_max(amax, group);
      if (i >= n_vec) continue;
      int e = 0;
      bool fast = (__float_as_uint(amax) >> 23) != 0;
      if (fast) {
        e = min(max(ceil_log2_ref<kBf16>(amax, tab), e_lo), e_hi);
        fast = e <= 127 && e >= mb - 28 && mb <= 16;
      }
#pragma unroll
      for (int k = 0; k < N; ++k) fast = fast && ((b[k] & 0x7FFFFFFFu) - 1u) >= thr_m1;
      float out[N];
      if (fast) {
        const float c1 = __int_as_float((mb - e + 127) << 23), c2 = __int_as_float((e - mb + 127) << 23);
#pragma unroll
        for (int k = 0; k < N; ++k) {
          const float xf = __uint_as_float(b[k]);
          const float val = kBf16 ? fabsf(xf) : fabsf(xf) + 1e-9f;
          const float q = fminf(rintf(val * c1), hi) * c2;
          out[k] = copysignf(q, xf + 0.f);  // x = -0 gives +0, a negative x that rounds to zero gives -0
        }
      } else {
        const BfpBlock p = bfp_block<T>(amax, width, exp_width, exp_bias, tab);
#pragma unroll
        for (int k = 0; k < N; ++k) out[k] = bfp_elem<T>(__uint_as_float(b[k]), p);
      }
      store_vals(y, i * N, out);
    }
  }
}

// one thread per tile; tiles never cross a row, the last tile of a row may be short
template <typename T>
__global__ void __launch_bounds__(kThreads)
bfp_generic_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int64_t cols, int bs, int width,
                   int exp_width, int exp_bias, const __grid_constant__ Log2Tab tab) {
  const int64_t tiles_per_row = (cols + bs - 1) / bs;
  const int64_t n_tiles = rows * tiles_per_row;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < n_tiles; t += (int64_t)gridDim.x * kThreads) {
    const int64_t r = t / tiles_per_row, c0 = (t % tiles_per_row) * bs;
    const int len = (int)min((int64_t)bs, cols - c0);
    const T *xb = x + r * cols + c0;
    float amax = 0.f;
    for (int k = 0; k < len; ++k) amax = fmaxf(amax, fabsf(load_scalar(xb + k)));
    const BfpBlock p = bfp_block<T>(amax, width, exp_width, exp_bias, tab);
    for (int k = 0; k < len; ++k) store_scalar(y + r * cols + c0 + k, bfp_elem<T>(load_scalar(xb + k), p));
  }
}

// Tiles of bh x bw over the last two dimensions of x[batch, rows, cols] (ragged edges count as zero padding).
// A group of G threads owns one tile: a warp for tiles of up to 2048 elements, a whole CTA above that.  Pass 1 finds
// the tile maximum, pass 2 re-reads the tile (from L1/L2) and applies the element-wise restatement of the reference.
template <typename T, int G>
__global__ void __launch_bounds__(kThreads)
bfp_tile_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t batch, int rows, int cols, int bh, int bw, int width,
                int exp_width, int exp_bias, const __grid_constant__ Log2Tab tab) {
  __shared__ float warp_max[kThreads / 32];
  const int tiles_r = (rows + bh - 1) / bh, tiles_c = (cols + bw - 1) / bw;
  const int64_t n_tiles = batch * tiles_r * tiles_c;
  const int groups_per_cta = kThreads / G;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  for (int64_t tile0 = (int64_t)blockIdx.x * groups_per_cta; tile0 < n_tiles; tile0 += (int64_t)gridDim.x * groups_per_cta) {
    const int64_t tile = tile0 + g;
    const bool live = tile < n_tiles;
    int64_t b = 0;
    int r0 = 0, c0 = 0, vh = 0, vw = 1;
    if (live) {
      b = tile / (tiles_r * tiles_c);
      const int rem = (int)(tile - b * (tiles_r * tiles_c));
      r0 = (rem / tiles_c) * bh, c0 = (rem % tiles_c) * bw;
      vh = min(bh, rows - r0), vw = min(bw, cols - c0);
    }
    const T *xt = x + (b * rows + r0) * (int64_t)cols + c0;
    T *yt = y + (b * rows + r0) * (int64_t)cols + c0;
    const int n = vh * vw;
    float amax = 0.f;
    for (int e = t; e < n; e += G) amax = fmaxf(amax, fabsf(load_scalar(xt + (int64_t)(e / vw) * cols + e % vw)));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if constexpr (G > 32) {
      __syncthreads();  // previous iteration's readers are done
      if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
      __syncthreads();
      amax = 0.f;
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) amax = fmaxf(amax, warp_max[w]);
    }
    const BfpBlock p = bfp_block<T>(amax, width, exp_width, exp_bias, tab);
    for (int e = t; e < n; e += G) {
      const int64_t off = (int64_t)(e / vw) * cols + e % vw;
      // the reference folds tiles back by adding them into zeros: -0.0 comes out as +0.0
      store_scalar(yt + off, bfp_elem<T>(load_scalar(xt + off), p) + 0.f);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
static int grid_for(int64_t work_items, int per_cta) {
  int64_t g = (work_items + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)mxq::gemm::sm_count() * 16;  // a few waves of resident CTAs; the kernels loop beyond that
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}
static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }
static int check_launch() { return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH; }
static Log2Tab load_tab(const uint8_t *host) {
  Log2Tab t;
  for (int i = 0; i < 256; ++i) t.t[i] = host ? host[i] : 0;
  return t;
}
static bool legal_ef(int E, int F) {
  return (E == 4 && F == 3) || (E == 5 && F == 2) || (E == 2 && F == 3) || (E == 3 && F == 2) || (E == 2 && F == 1) ||
         (E == 1 && F == 2);
}
// lanes sharing one block, or 0 when the fast path does not apply
// MXFP8 with E5M2 elements as tensor-core operands: one thread per block of 32, the element codec of the generic path.
// The hardware reads exponent code 31 as inf / nan while the reference uses it as a normal binade -- and its shared
// exponent puts every block's maximum exactly there -- so each block is stored one scale step up with its values
// halved (exponent codes one lower).  Halving is exact except for elements in the two lowest binades of the format
// whose last fraction bit is set; those are rounded to nearest by the hardware conversion, an error of at most
// 2**-17 of the block scale against a block maximum of at least 2**15.
template <typename Tin>
__global__ void __launch_bounds__(kThreads)
mxfp_pack_mma_e5m2_kernel(const Tin *__restrict__ x, uint8_t *__restrict__ codes, uint8_t *__restrict__ scales,
                          int64_t n_blocks, int64_t blocks_per_row, int64_t k_chunks, const __grid_constant__ Log2Tab tab) {
  for (int64_t blk = (int64_t)blockIdx.x * kThreads + threadIdx.x; blk < n_blocks;
       blk += (int64_t)gridDim.x * kThreads) {
    const Tin *xb = x + blk * 32;
    uint32_t bits[32];
    uint32_t amax = 0;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      uint32_t b = __float_as_uint(load_scalar(xb + k));
      if (((b & 0x7FFFFFFFu) >> 23) == 0) b = 0;  // zero and fp32-subnormal inputs are flushed
      bits[k] = b;
      amax = max(amax, b & 0x7FFFFFFFu);
    }
    const MxfpBlock p = mxfp_block(amax, 5, tab);
    uint32_t w[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      uint32_t word = 0;
#pragma unroll
      for (int k = 0; k < 4; k += 2) {
        const float v0 = mxfp_decode(mxfp_encode(bits[4 * q + k], p.sh, 5, 2), 5, 2) * 0.5f;
        const float v1 = mxfp_decode(mxfp_encode(bits[4 * q + k + 1], p.sh, 5, 2), 5, 2) * 0.5f;
        word |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v0, v1), __NV_SATFINITE, __NV_E5M2) << (8 * k);
      }
      w[q] = word;
    }
    uint4 *dst = reinterpret_cast<uint4 *>(codes + blk * 32);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]), dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    const int64_t row = blk / blocks_per_row, kb = blk - row * blocks_per_row;
    scales[mma_scale_offset<int64_t>(row, kb, k_chunks)] = (uint8_t)(p.scale + 1);
  }
}

template <typename Tin>
static int fast_group(int block) {
  constexpr int N = Elem<Tin>::kVec;
  if (!is_pow2(block) || block < N || block > 32 * N) return 0;
  return block / N;
}

template <typename Tin, typename Tout, Mode kMode>
static int launch_mxint(const void *x, void *y, int8_t *mant, uint8_t *scales, int64_t n_blocks, int block, int bits,
                        const Log2Tab &tab, cudaStream_t st) {
  const int group = fast_group<Tin>(block);
  if constexpr (kMode == Mode::kCodes && Elem<Tin>::kBf16) {
    if (block == 32 && aligned16(x) && aligned16(mant)) {
      const int64_t n_unit = n_blocks * 2;
      const int grid = grid_for(n_unit, kThreads * 2);
      if ((reinterpret_cast<uintptr_t>(x) & 31) == 0)
        mxint_codes_bf16_kernel<true><<<grid, kThreads, 0, st>>>((const __nv_bfloat16 *)x, mant, scales, n_unit, bits, tab);
      else
        mxint_codes_bf16_kernel<false><<<grid, kThreads, 0, st>>>((const __nv_bfloat16 *)x, mant, scales, n_unit, bits, tab);
      return check_launch();
    }
  }
  if (group && aligned16(x) && (kMode == Mode::kCodes ? aligned16(mant) : aligned16(y))) {
    const int64_t n_vec = n_blocks * group;
    mxint_kernel<Tin, Tout, kMode><<<grid_for(n_vec, kThreads * kUnroll), kThreads, 0, st>>>(
        (const Tin *)x, (Tout *)y, mant, scales, n_vec, group, bits, tab);
  } else {
    mxint_generic_kernel<Tin, Tout, kMode><<<grid_for(n_blocks, kThreads), kThreads, 0, st>>>(
        (const Tin *)x, (Tout *)y, mant, scales, n_blocks, block, bits, tab);
  }
  return check_launch();
}

template <typename Tin, typename Tout, Mode kMode, int E, int F>
static int launch_mxfp_ef(const void *x, void *y, uint8_t *codes, uint8_t *scales, int64_t n_blocks, int block,
                          const Log2Tab &tab, cudaStream_t st) {
  const int group = fast_group<Tin>(block);
  if constexpr (kMode == Mode::kCodes && Elem<Tin>::kBf16) {
    if (block == 32 && aligned16(x) && aligned16(codes)) {
      const int64_t n_unit = n_blocks * 2;
      const int grid = grid_for(n_unit, kThreads * 2);
      if ((reinterpret_cast<uintptr_t>(x) & 31) == 0)
        mxfp_codes_bf16_kernel<E, F, true><<<grid, kThreads, 0, st>>>((const __nv_bfloat16 *)x, codes, scales, n_unit, tab);
      else
        mxfp_codes_bf16_kernel<E, F, false><<<grid, kThreads, 0, st>>>((const __nv_bfloat16 *)x, codes, scales, n_unit, tab);
      return check_launch();
    }
  }
  if (group && aligned16(x) && (kMode == Mode::kCodes ? aligned16(codes) : aligned16(y))) {
    const int64_t n_vec = n_blocks * group;
    mxfp_kernel<Tin, Tout, kMode, E, F><<<grid_for(n_vec, kThreads * kUnroll), kThreads, 0, st>>>(
        (const Tin *)x, (Tout *)y, codes, scales, n_vec, group, tab);
  } else {
    mxfp_generic_kernel<Tin, Tout, kMode><<<grid_for(n_blocks, kThreads), kThreads, 0, st>>>(
        (const Tin *)x, (Tout *)y, codes, scales, n_blocks, block, E, F, tab);
  }
  return check_launch();
}

template <typename Tin, typename Tout, Mode kMode>
static int launch_mxfp(const void *x, void *y, uint8_t *codes, uint8_t *scales, int64_t n_blocks, int block, int E,
                       int F, const Log2Tab &tab, cudaStream_t st) {
#define MXQ_EF(e, f) \
  if (E == e && F == f) return launch_mxfp_ef<Tin, Tout, kMode, e, f>(x, y, codes, scales, n_blocks, block, tab, st);
  MXQ_EF(4, 3) MXQ_EF(5, 2) MXQ_EF(2, 3) MXQ_EF(3, 2) MXQ_EF(2, 1) MXQ_EF(1, 2)
#undef MXQ_EF
  return MXQ_ERR_FORMAT;
}

}  // namespace mxq

using namespace mxq;

// dispatch on (input type, output type)
#define MXQ_DISPATCH_IO(in_dtype, out_dtype, CALL)                                    \
  if (in_dtype == MXQ_F32 && out_dtype == MXQ_F32) { CALL(float, float) }             \
  if (in_dtype == MXQ_BF16 && out_dtype == MXQ_BF16) { CALL(__nv_bfloat16, __nv_bfloat16) } \
  if (in_dtype == MXQ_F32 && out_dtype == MXQ_BF16) { CALL(float, __nv_bfloat16) }    \
  if (in_dtype == MXQ_BF16 && out_dtype == MXQ_F32) { CALL(__nv_bfloat16, float) }    \
  return MXQ_ERR_DTYPE;

extern "C" {

int mxq_version(void) { return MXQ_VERSION; }

const char *mxq_error_string(int code) {
  switch (code) {
    case MXQ_OK: return "ok";
    case MXQ_ERR_DTYPE: return "unsupported element type";
    case MXQ_ERR_SHAPE: return "bad shape or size";
    case MXQ_ERR_FORMAT: return "unsupported number format";
    case MXQ_ERR_ALIGN: return "pointer is not 16-byte aligned";
    case MXQ_ERR_NULL: return "null pointer";
    case MXQ_ERR_LAUNCH: return "CUDA launch failed";
    case MXQ_ERR_UNSUPPORTED: return "unsupported configuration";
    case MXQ_ERR_DEVICE: return "device-side error status";
    case MXQ_ERR_TOO_LARGE: return "problem exceeds the built-in scratch of mxq_mx_linear_static (MXQ_STATIC_SCRATCH_BYTES)";
    default: return "unknown error";
  }
}

int mxq_mxint_fake(const void *x, void *y, int in_dtype, int out_dtype, int64_t n_blocks, int block, int bits,
                   const uint8_t *ceil_tab_host, void *stream) {
  if (n_blocks == 0) return MXQ_OK;
  if (!x || !y || !ceil_tab_host) return MXQ_ERR_NULL;
  if (n_blocks < 0 || block < 1) return MXQ_ERR_SHAPE;
  if (bits < 2 || bits > 8) return MXQ_ERR_FORMAT;
  const Log2Tab tab = load_tab(ceil_tab_host);
#define CALL(TI, TO) \
  return launch_mxint<TI, TO, Mode::kFake>(x, y, nullptr, nullptr, n_blocks, block, bits, tab, (cudaStream_t)stream);
  MXQ_DISPATCH_IO(in_dtype, out_dtype, CALL)
#undef CALL
}

int mxq_mxint_extract(const void *x, int8_t *mant, uint8_t *scales, int in_dtype, int64_t n_blocks, int block, int bits,
                      const uint8_t *ceil_tab_host, void *stream) {
  if (n_blocks == 0) return MXQ_OK;
  if (!x || !mant || !scales || !ceil_tab_host) return MXQ_ERR_NULL;
  if (n_blocks < 0 || block < 1) return MXQ_ERR_SHAPE;
  if (bits < 2 || bits > 8) return MXQ_ERR_FORMAT;
  const Log2Tab tab = load_tab(ceil_tab_host);
  if (in_dtype == MXQ_F32)
    return launch_mxint<float, float, Mode::kCodes>(x, nullptr, mant, scales, n_blocks, block, bits, tab,
                                                    (cudaStream_t)stream);
  if (in_dtype == MXQ_BF16)
    return launch_mxint<__nv_bfloat16, float, Mode::kCodes>(x, nullptr, mant, scales, n_blocks, block, bits, tab,
                                                            (cudaStream_t)stream);
  return MXQ_ERR_DTYPE;
}

int mxq_mxint_compose(const int8_t *mant, const uint8_t *scales, void *y, int out_dtype, int64_t n_blocks, int block,
                      int bits, void *stream) {
  if (n_blocks == 0) return MXQ_OK;
  if (!mant || !scales || !y) return MXQ_ERR_NULL;
  if (n_blocks < 0 || block < 1) return MXQ_ERR_SHAPE;
  if (bits < 2 || bits > 8) return MXQ_ERR_FORMAT;
  const int64_t n = n_blocks * block;
  const int grid = grid_for(n, kThreads);
  if (out_dtype == MXQ_F32)
    mxint_compose_kernel<float><<<grid, kThreads, 0, (cudaStream_t)stream>>>(mant, scales, (float *)y, n, block, bits);
  else if (out_dtype == MXQ_BF16)
    mxint_compose_kernel<__nv_bfloat16>
        <<<grid, kThreads, 0, (cudaStream_t)stream>>>(mant, scales, (__nv_bfloat16 *)y, n, block, bits);
  else
    return MXQ_ERR_DTYPE;
  return check_launch();
}

int mxq_mxfp_fake(const void *x, void *y, int in_dtype, int out_dtype, int64_t n_blocks, int block, int E, int F,
                  const uint8_t *floor_tab_host, void *stream) {
  if (n_blocks == 0) return MXQ_OK;
  if (!x || !y || !floor_tab_host) return MXQ_ERR_NULL;
  if (n_blocks < 0 || block < 1) return MXQ_ERR_SHAPE;
  if (!legal_ef(E, F)) return MXQ_ERR_FORMAT;
  const Log2Tab tab = load_tab(floor_tab_host);
#define CALL(TI, TO) \
  return launch_mxfp<TI, TO, Mode::kFake>(x, y, nullptr, nullptr, n_blocks, block, E, F, tab, (cudaStream_t)stream);
  MXQ_DISPATCH_IO(in_dtype, out_dtype, CALL)
#undef CALL
}

int mxq_mxfp_extract(const void *x, uint8_t *codes, uint8_t *scales, int in_dtype, int64_t n_blocks, int block, int E,
                     int F, const uint8_t *floor_tab_host, void *stream) {
  if (n_blocks == 0) return MXQ_OK;
  if (!x || !codes || !scales || !floor_tab_host) return MXQ_ERR_NULL;
  if (n_blocks < 0 || block < 1) return MXQ_ERR_SHAPE;
  if (!legal_ef(E, F)) return MXQ_ERR_FORMAT;
  const Log2Tab tab = load_tab(floor_tab_host);
  if (in_dtype == MXQ_F32)
    return launch_mxfp<float, float, Mode::kCodes>(x, nullptr, codes, scales, n_blocks, block, E, F, tab,
                                                   (cudaStream_t)stream);
  if (in_dtype == MXQ_BF16)
    return launch_mxfp<__nv_bfloat16, float, Mode::kCodes>(x, nullptr, codes, scales, n_blocks, block, E, F, tab,
                                                           (cudaStream_t)stream);
  return MXQ_ERR_DTYPE;
}

int mxq_mxfp_pack_mma(const void *x, uint8_t *codes, uint8_t *scales_mma, int in_dtype, int64_t rows, int64_t k, int E, int F,
                      const uint8_t *floor_tab_host, void *stream) {
  return mxq::pack_mxfp_mma(x, codes, scales_mma, in_dtype, rows, k, E, F, floor_tab_host, (cudaStream_t)stream, false);
}

int mxq_silu_mul_pack_mma(const void *gate, const void *up, int64_t ld, uint8_t *codes, uint8_t *scales_mma,
                          int64_t rows, int64_t k, int E, int F, const uint8_t *floor_tab_host, void *stream) {
  return mxq::pack_silu_mul_mma(gate, up, ld, codes, scales_mma, rows, k, E, F, floor_tab_host, (cudaStream_t)stream,
                                false);
}

}  // extern "C"

namespace mxq {

// Plain launch, or (chained) one with programmatic stream serialization: the kernel may then start under the tail of
// the previous kernel of the stream and waits for it on the device.
template <typename... KArgs, typename... Args>
static void launch_pack(void (*kernel)(KArgs...), int grid, cudaStream_t st, bool chained, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid), cfg.blockDim = dim3((unsigned)kThreads), cfg.dynamicSmemBytes = 0, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = chained ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, args..., (uint32_t)(chained ? 1 : 0));
}

int pack_mxfp_mma(const void *x, uint8_t *codes, uint8_t *scales_mma, int in_dtype, int64_t rows, int64_t k, int E, int F,
                  const uint8_t *floor_tab_host, cudaStream_t st, bool chained) {
  if (rows == 0 || k == 0) return MXQ_OK;
  if (!x || !codes || !scales_mma || !floor_tab_host) return MXQ_ERR_NULL;
  if (rows < 0 || k < 0 || k % 32) return MXQ_ERR_SHAPE;
  const bool e5m2 = E == 5 && F == 2;
  if (!legal_ef(E, F) || (!e5m2 && (E > 4 || F > 3))) return MXQ_ERR_FORMAT;
  if (!aligned16(x) || !aligned16(codes)) return MXQ_ERR_ALIGN;
  const Log2Tab tab = load_tab(floor_tab_host);
  const int64_t k_chunks = (k + 127) / 128;
  const int64_t sf_bytes = ((rows + 255) / 256) * 2 * k_chunks * 512;
  // Scales of K blocks past the end of a row (K not a multiple of 128) must be finite: the codes there read as zero,
  // and zero times an unset scale byte (0xFF is NaN) would poison valid outputs.  Scales of rows past the end only
  // reach accumulator rows that are never stored, so they may stay unset.
  if (k % 128 && cudaMemsetAsync(scales_mma, 0, sf_bytes, st) != cudaSuccess) return MXQ_ERR_LAUNCH;
  if (e5m2) {  // hardware E5M2 bytes, every block at scale + 1: the element codec, one thread per block
    const int64_t n_blocks = rows * (k / 32);
    const int grid = grid_for(n_blocks, kThreads);
    if (in_dtype == MXQ_F32)
      mxfp_pack_mma_e5m2_kernel<float><<<grid, kThreads, 0, st>>>((const float *)x, codes, scales_mma, n_blocks, k / 32, k_chunks,
                                                                tab);
    else if (in_dtype == MXQ_BF16)
      mxfp_pack_mma_e5m2_kernel<__nv_bfloat16>
          <<<grid, kThreads, 0, st>>>((const __nv_bfloat16 *)x, codes, scales_mma, n_blocks, k / 32, k_chunks, tab);
    else
      return MXQ_ERR_DTYPE;
    return check_launch();
  }
  if (in_dtype == MXQ_F32) {
    const int64_t n_vec = rows * k / 4;
#define MXQ_PACK(e, f)                                                                                  \
  if (E == e && F == f) {                                                                               \
    mxfp_pack_mma_f32_kernel<e, f><<<grid_for(n_vec, kThreads * 2), kThreads, 0, st>>>(                 \
        (const float *)x, codes, scales_mma, n_vec, (uint32_t)(k / 4), k_chunks, tab);                  \
    return check_launch();                                                                              \
  }
    MXQ_PACK(4, 3) MXQ_PACK(2, 3) MXQ_PACK(3, 2) MXQ_PACK(2, 1) MXQ_PACK(1, 2)
#undef MXQ_PACK
  } else if (in_dtype == MXQ_BF16) {
    const int64_t n_unit = rows * k / 16;
    const uint32_t upr = (uint32_t)(k / 16);
    const int grid = grid_for(n_unit, kThreads * 2);
    const int64_t step = (int64_t)grid * kThreads * 2;
    const UnitStep jump = {(uint32_t)(kThreads / upr), (uint32_t)(kThreads % upr)};
    const UnitStep stride = {(uint32_t)(step / upr), (uint32_t)(step % upr)};
    const bool wide = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    // 32-bit indices: unit numbers (with a grid step of headroom) and scale offsets stay below 2**31
    const bool small = n_unit + step < (1ll << 31) && sf_bytes < (1ll << 31);
#define MXQ_PACK_ARGS (const __nv_bfloat16 *)x, codes, scales_mma, n_unit, upr, k_chunks, jump, stride, tab
#define MXQ_PACK(e, f)                                                                                   \
  if (E == e && F == f) {                                                                                \
    if (wide && small)                                                                                   \
      launch_pack(mxfp_pack_mma_bf16_kernel<e, f, true, uint32_t>, grid, st, chained, MXQ_PACK_ARGS);    \
    else if (wide)                                                                                       \
      launch_pack(mxfp_pack_mma_bf16_kernel<e, f, true, int64_t>, grid, st, chained, MXQ_PACK_ARGS);     \
    else if (small)                                                                                      \
      launch_pack(mxfp_pack_mma_bf16_kernel<e, f, false, uint32_t>, grid, st, chained, MXQ_PACK_ARGS);   \
    else                                                                                                 \
      launch_pack(mxfp_pack_mma_bf16_kernel<e, f, false, int64_t>, grid, st, chained, MXQ_PACK_ARGS);    \
    return check_launch();                                                                               \
  }
    MXQ_PACK(4, 3) MXQ_PACK(2, 3) MXQ_PACK(3, 2) MXQ_PACK(2, 1) MXQ_PACK(1, 2)
  } else {
    return MXQ_ERR_DTYPE;
  }
#undef MXQ_PACK
#undef MXQ_PACK_ARGS
  return MXQ_ERR_FORMAT;
}

}  // namespace mxq

extern "C" {

int mxq_mxfp4_pack_mma(const void *x, uint8_t *codes4, uint8_t *scales_mma, int in_dtype, int64_t rows, int64_t k,
                       const uint8_t *floor_tab_host, void *stream) {
  if (rows == 0 || k == 0) return MXQ_OK;
  if (!x || !codes4 || !scales_mma || !floor_tab_host) return MXQ_ERR_NULL;
  if (rows < 0 || k < 0 || k % 128) return MXQ_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(codes4) & 31u) return MXQ_ERR_ALIGN;
  const Log2Tab tab = load_tab(floor_tab_host);
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t k_chunks = k / 128;
  const int64_t n_blocks = rows * (k / 32);
  if (in_dtype == MXQ_F32)
    mxfp4_pack_mma_kernel<float><<<grid_for(n_blocks, kThreads), kThreads, 0, st>>>((const float *)x, codes4, scales_mma,
                                                                                   n_blocks, k / 32, k_chunks, tab);
  else if (in_dtype == MXQ_BF16)
    mxfp4_pack_mma_kernel<__nv_bfloat16><<<grid_for(n_blocks, kThreads), kThreads, 0, st>>>(
        (const __nv_bfloat16 *)x, codes4, scales_mma, n_blocks, k / 32, k_chunks, tab);
  else
    return MXQ_ERR_DTYPE;
  return check_launch();
}

}  // extern "C"

int mxq::pack_silu_mul_mma(const void *gate, const void *up, int64_t ld, uint8_t *codes, uint8_t *scales_mma, int64_t rows,
                           int64_t k, int E, int F, const uint8_t *floor_tab_host, cudaStream_t st, bool chained) {
  using namespace mxq;
  if (rows == 0 || k == 0) return MXQ_OK;
  if (!gate || !up || !codes || !scales_mma || !floor_tab_host) return MXQ_ERR_NULL;
  if (rows < 0 || k < 0 || k % 32 || ld < k || ld % 8) return MXQ_ERR_SHAPE;
  if (!legal_ef(E, F) || E > 4 || F > 3) return MXQ_ERR_FORMAT;
  if (!aligned16(gate) || !aligned16(up) || !aligned16(codes)) return MXQ_ERR_ALIGN;
  const Log2Tab tab = load_tab(floor_tab_host);
  const int64_t k_chunks = (k + 127) / 128;
  const int64_t sf_bytes = ((rows + 255) / 256) * 2 * k_chunks * 512;
  // scale bytes of K blocks past the end of a row must be finite (see mxq_mxfp_pack_mma)
  if (k % 128 && cudaMemsetAsync(scales_mma, 0, sf_bytes, st) != cudaSuccess) return MXQ_ERR_LAUNCH;
  const int64_t n_unit = rows * k / 16;
  const uint32_t upr = (uint32_t)(k / 16);
  const int grid = grid_for(n_unit, kThreads);
#define MXQ_PACK(e, f)                                                                                          \
  if (E == e && F == f) {                                                                                       \
    launch_pack(silu_mul_pack_mma_kernel<e, f>, grid, st, chained, (const __nv_bfloat16 *)gate,                 \
                (const __nv_bfloat16 *)up, ld, codes, scales_mma, n_unit, upr, k_chunks, tab);                  \
    return check_launch();                                                                                      \
  }
  MXQ_PACK(4, 3) MXQ_PACK(2, 3) MXQ_PACK(3, 2) MXQ_PACK(2, 1) MXQ_PACK(1, 2)
#undef MXQ_PACK
  return MXQ_ERR_FORMAT;
}

extern "C" {

int mxq_mxfp_compose(const uint8_t *codes, const uint8_t *scales, void *y, int out_dtype, int64_t n_blocks, int block,
                     int E, int F, void *stream) {
  if (n_blocks == 0) return MXQ_OK;
  if (!codes || !scales || !y) return MXQ_ERR_NULL;
  if (n_blocks < 0 || block < 1) return MXQ_ERR_SHAPE;
  if (!legal_ef(E, F)) return MXQ_ERR_FORMAT;
  const int64_t n = n_blocks * block;
  const int grid = grid_for(n, kThreads);
  if (out_dtype == MXQ_F32)
    mxfp_compose_kernel<float><<<grid, kThreads, 0, (cudaStream_t)stream>>>(codes, scales, (float *)y, n, block, E, F);
  else if (out_dtype == MXQ_BF16)
    mxfp_compose_kernel<__nv_bfloat16>
        <<<grid, kThreads, 0, (cudaStream_t)stream>>>(codes, scales, (__nv_bfloat16 *)y, n, block, E, F);
  else
    return MXQ_ERR_DTYPE;
  return check_launch();
}

int mxq_minifloat_fake(const void *x, void *y, int in_dtype, int out_dtype, int64_t n, int E, int F, void *stream) {
  if (n == 0) return MXQ_OK;
  if (!x || !y) return MXQ_ERR_NULL;
  if (n < 0) return MXQ_ERR_SHAPE;
  if (E < 1 || F < 1 || E + F > 15) return MXQ_ERR_FORMAT;  // the reference's range: fewer than 16 bits after the sign
  const int grid = grid_for(n, kThreads);
#define CALL(TI, TO)                                                                                        \
  minifloat_kernel<TI, TO><<<grid, kThreads, 0, (cudaStream_t)stream>>>((const TI *)x, (TO *)y, n, E, F); \
  return check_launch();
  MXQ_DISPATCH_IO(in_dtype, out_dtype, CALL)
#undef CALL
}

int mxq_bfp_fake(const void *x, void *y, int dtype, int64_t rows, int64_t cols, int bs, int width, int exp_width,
                 int exp_bias, const uint8_t *ceil_tab_host, void *stream) {
  if (rows == 0 || cols == 0) return MXQ_OK;
  if (!x || !y || !ceil_tab_host) return MXQ_ERR_NULL;
  if (rows < 0 || cols < 0 || bs < 1) return MXQ_ERR_SHAPE;
  if (width < 2 || width > 24 || exp_width < 1 || exp_width > 8) return MXQ_ERR_FORMAT;
  const Log2Tab tab = load_tab(ceil_tab_host);
  cudaStream_t st = (cudaStream_t)stream;
  if (bs > cols) bs = (int)cols;
  if (dtype == MXQ_F32) {
    const int group = fast_group<float>(bs);
    if (group && cols % bs == 0 && aligned16(x) && aligned16(y)) {
      const int64_t n_vec = rows * cols / 4;
      bfp_kernel<float><<<grid_for(n_vec, kThreads * kUnroll), kThreads, 0, st>>>(
          (const float *)x, (float *)y, n_vec, group, width, exp_width, exp_bias, tab);
    } else {
      bfp_generic_kernel<float><<<grid_for(rows * ((cols + bs - 1) / bs), kThreads), kThreads, 0, st>>>(
          (const float *)x, (float *)y, rows, cols, bs, width, exp_width, exp_bias, tab);
    }
  } else if (dtype == MXQ_BF16) {
    const int group = fast_group<__nv_bfloat16>(bs);
    if (group && cols % bs == 0 && aligned16(x) && aligned16(y)) {
      const int64_t n_vec = rows * cols / 8;
      bfp_kernel<__nv_bfloat16><<<grid_for(n_vec, kThreads * kUnroll), kThreads, 0, st>>>(
          (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, n_vec, group, width, exp_width, exp_bias, tab);
    } else {
      bfp_generic_kernel<__nv_bfloat16><<<grid_for(rows * ((cols + bs - 1) / bs), kThreads), kThreads, 0, st>>>(
          (const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, rows, cols, bs, width, exp_width, exp_bias, tab);
    }
  } else {
    return MXQ_ERR_DTYPE;
  }
  return check_launch();
}

int mxq_bfp_fake_tiles(const void *x, void *y, int dtype, int64_t batch, int64_t rows, int64_t cols, int bh, int bw,
                       int width, int exp_width, int exp_bias, const uint8_t *ceil_tab_host, void *stream) {
  if (batch == 0 || rows == 0 || cols == 0) return MXQ_OK;
  if (!x || !y || !ceil_tab_host) return MXQ_ERR_NULL;
  if (batch < 0 || rows < 0 || cols < 0 || rows > INT32_MAX || cols > INT32_MAX || bh < 1 || bw < 1) return MXQ_ERR_SHAPE;
  if (width < 2 || width > 24 || exp_width < 1 || exp_width > 8) return MXQ_ERR_FORMAT;
  if (bh > rows) bh = (int)rows;
  if (bw > cols) bw = (int)cols;
  const Log2Tab tab = load_tab(ceil_tab_host);
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t n_tiles = batch * ((rows + bh - 1) / bh) * ((cols + bw - 1) / bw);
  const bool small = (int64_t)bh * bw <= 2048;
  const int grid = grid_for(n_tiles, small ? kThreads / 32 : 1);
#define MXQ_TILES(T)                                                                                            \
  if (small)                                                                                                    \
    bfp_tile_kernel<T, 32><<<grid, kThreads, 0, st>>>((const T *)x, (T *)y, batch, (int)rows, (int)cols, bh, bw, \
                                                      width, exp_width, exp_bias, tab);                         \
  else                                                                                                          \
    bfp_tile_kernel<T, kThreads><<<grid, kThreads, 0, st>>>((const T *)x, (T *)y, batch, (int)rows, (int)cols, bh, \
                                                            bw, width, exp_width, exp_bias, tab);
  if (dtype == MXQ_F32) {
    MXQ_TILES(float)
  } else if (dtype == MXQ_BF16) {
    MXQ_TILES(__nv_bfloat16)
  } else {
    return MXQ_ERR_DTYPE;
  }
#undef MXQ_TILES
  return check_launch();
}

}  // extern "C"
