// D[M,N] = A[M,K] * B[N,K]^T (+ bias[N]) on the 5th-generation tensor cores of sm_100a.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0     TMA producer: 128-byte-swizzled K-major tiles of A (128 rows) and B (BN rows) and, for the
//              block-scaled kind, the E8M0 scale chunks, into a shared-memory ring (mbarrier transaction counts
//              signal arrival);
//   warp 1     MMA issuer: tcgen05.mma (M=128, N=BN, 32 bytes of K per instruction) with fp32 accumulators in tensor
//              memory; tcgen05.commit releases ring slots and publishes finished accumulators;
//   warps 2..5 epilogue: tcgen05.ld the accumulator (each warp owns the 32 TMEM lanes of its quarter), add the bias,
//              convert, stage in shared memory and store with TMA.
// Warps 0 and 1 run their loops with all lanes on identical values and elect one lane per instruction group, so that
// the operands of the TMA / tcgen05 instructions live in uniform registers.
// Kinds: bf16 x bf16 (kind::f16), fp32 x fp32 rounded to tf32 (kind::tf32) and MXFP8 E4M3 x E4M3 with one E8M0
// scale per 32 elements of K (kind::mxf8f6f4.block_scale).  Accumulators are double-buffered so that the epilogue of
// a tile overlaps the main loop of the next one (for the block-scaled 256-column tile the two overlap by 64 columns,
// see the kernel).  A second kernel runs all kinds on CTA pairs (cta_group::2, 256 x 256 tiles).
//
// Every load targets one CTA only (no cluster-wide broadcast loads).  Every wait on an mbarrier is bounded: when it runs out the CTA raises an abort
// flag, records an error code in the caller's status word, waits (bounded) for its own bulk copies in flight, frees
// its tensor memory and returns.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "mxq.h"
#include "mxq_internal.h"

namespace mxq {
namespace gemm {

constexpr int BM = 128;
constexpr int kMaxStages = 8;
constexpr int kThreads = 192;
constexpr int kRowBytes = 128;            // bytes of K per row per stage = one 128B swizzle atom
constexpr int kTmemCols = 512;

enum Kind { kBf16 = 0, kTf32 = 1, kMxf8 = 2 };

// error codes written to the status word
constexpr int kErrProducerWait = 1, kErrMmaWaitFull = 2, kErrMmaWaitAcc = 3, kErrEpilogueWait = 4;

// ---- PTX wrappers -----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another one ran out of time).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code,
                                          unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xFFu) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}
// the same for a whole warp: every lane waits, and all lanes get the same answer
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                               int code, unsigned long long limit_ns) {
  return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag, status, code, limit_ns));
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// the same with a third coordinate: (k, row, matrix of a batch)
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// ---- thread-block clusters ----
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}
// true in exactly one lane of a fully active warp (the same lane every time)
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// shared-memory matrix descriptor: K-major tile of rows x 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// descriptor of a 32 x 16-byte scale-factor chunk (no swizzle, 8-row groups 128 bytes apart)
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
template <int kKind>
__device__ __forceinline__ void umma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc, uint32_t sfa,
                                     uint32_t sfb) {
  if constexpr (kKind == kBf16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc)
        : "memory");
  } else if constexpr (kKind == kTf32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
        : "memory");
  }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Wait for the outstanding tcgen05.ld.  The registers of `r` only hold data after the wait, which the compiler cannot
// know: the empty statements re-define them after the (volatile, hence ordered) wait so that no use is hoisted above it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                    "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :: "memory");
  asm volatile("" : "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]),
                    "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]),
                    "+r"(r[31])
               :: "memory");
}

// element format codes of the block-scaled kind's instruction descriptor (A: bits 7-9, B: bits 10-12); E4M3 is 0
constexpr uint32_t kFormatE2M1 = 5;
constexpr uint32_t kFormatE5M2 = 1;

// instruction descriptor: fp32 accumulate, K-major A and B, M = 128, N = BN
template <int kKind, int BN>
__device__ __forceinline__ uint32_t make_idesc() {
  uint32_t d = ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  if constexpr (kKind == kBf16) d |= (1u << 4) | (1u << 7) | (1u << 10);   // D fp32, A bf16, B bf16
  if constexpr (kKind == kTf32) d |= (1u << 4) | (2u << 7) | (2u << 10);   // D fp32, A tf32, B tf32
  if constexpr (kKind == kMxf8) d |= (0u << 7) | (0u << 10) | (1u << 23);  // A, B E4M3; scales E8M0
  return d;
}

// Operand ring and 2 store boxes per epilogue warp.  256-column tiles: 4 slots of 48 KB (a 3-slot ring with a store
// staging area for a whole tile was measured slower).  Narrow tiles serve small problems whose time is the latency
// of streaming the weight through the ring once, so they get 8 slots.
template <int BN, bool kScaled, bool kSplit = false>
struct Layout {
  // kSplit: two CTAs of a cluster share one narrow tile, each taking half of K; the second one hands its fp32
  // accumulator over through a column-major exchange buffer in its shared memory (128 rows x BN columns)
  static constexpr int kStages = kSplit ? 6 : (BN <= 64 ? 8 : 4);
  static constexpr int kStoreBufs = 2;  // 2048-byte store boxes per epilogue warp
  static constexpr int kA = BM * kRowBytes;
  static constexpr int kB = BN * kRowBytes;
  static constexpr int kSfa = kScaled ? 512 : 0;
  static constexpr int kSfbChunks = (BN + 127) / 128;    // 128-row scale chunks that cover the BN rows of a B tile
  static constexpr int kSfb = kScaled ? kSfbChunks * 512 : 0;
  static constexpr int kAB = kA + kB;                   // operand tiles of one stage; a multiple of 1024 bytes
  static constexpr int kSf = kSfa + kSfb;               // scale chunks of one stage
  static constexpr int kStage = kAB + kSf;              // bytes that arrive per stage (the transaction count)
  static constexpr int kSfBase = kStages * kAB;         // scale chunks live after all operand tiles
  static constexpr int kStaging = (kStages * kStage + 1023) & ~1023;  // epilogue: 4 warps x kStoreBufs x 2048 bytes
  static constexpr int kXbuf = kStaging + 4 * kStoreBufs * 2048;
  static constexpr int kBarriers = kXbuf + (kSplit ? BM * BN * 4 : 0);  // full[], empty[], acc_full[2], acc_empty[2]
  static constexpr int kTotal = kBarriers + 32 * 8 + 16 + 1024;  // + tmem slot, abort flag, alignment slack
};

struct Params {
  const uint8_t *sfa;   // scale factors of A in 512-byte chunks [rows/128][k/128] (block-scaled kind only)
  const uint8_t *sfb;
  void *d;
  const void *bias;
  int *status;
  int M, N, K;          // K in elements
  int k_chunks;         // ceil(K * element_size / 128)
  int out_bf16;         // output element type: 1 bf16, 0 fp32
  int bias_bf16;        // bias element type
  int tma_store;        // output rows are 16-byte multiples: the epilogue writes through TMA stores
  int a_box_bytes;      // bytes one A load delivers: fewer than 128 rows when M is small (single-CTA kernel)
  unsigned long long wait_ns;  // limit of every wait
  int drop_last_load;   // test hook: CTA 0 never loads the last K chunk of its first tile
  uint32_t b_fp4;       // block-scaled kind: B holds E2M1 elements (two per byte in global memory) instead of E4M3 bytes
  uint32_t fmt_bits = 0;  // block-scaled kind: element formats of A (bits 7-9) and B (bits 10-12) that are not E4M3 / E2M1
  uint32_t tx_less;     // a 4-bit box counts its packed bytes on the barrier, half of what lands in shared memory
  // Row-parallel GEMM fused with the reduce-scatter (CTA-pair kernel): rows [r * scatter_rows, (r + 1) * scatter_rows)
  // of the fp32 result go to store map r, which covers a buffer in GPU r's memory.  0 = one output, map 0.
  int scatter_rows;
  // Rows of 256-row tiles by which the CTA-pair kernel's tile order is rotated.  With a scatter every GPU of the group
  // starts with the rows of a different owner (its successor's), so that at any time the GPUs store into different
  // peers instead of all into the same one.
  int m_rotate;
  // Batch of independent products (single-CTA kernel, dense kinds): the maps of A, B and D carry the matrix index as a
  // third coordinate, tiles are numbered matrix by matrix.  0 = one product, two-dimensional maps.
  int batch = 0;
  long long d_batch_stride = 0;  // elements between consecutive outputs (direct stores)
};

// Store maps of the CTA-pair kernel: one output, or one slot buffer per GPU of a tensor-parallel group.
constexpr int kMaxPeers = 8;
struct StoreMaps {
  CUtensorMap m[kMaxPeers];
};

// Epilogue of one tile for one warp: drains the warp's 32 TMEM lanes (= 32 tile rows starting at row0) of the
// accumulator at t_acc in chunks of 32 columns, starting with chunk `first`.  A chunk is converted, written to a
// 64-byte-swizzled staging buffer in shared memory (32 rows x 64 bytes, kStoreBufs buffers per warp) and handed to a
// TMA store, which writes whole lines and clips at the matrix edges; output matrices whose rows are not 16-byte
// multiples take direct predicated stores.  With overlapping accumulators `shared_columns_read` is called (lane 0)
// once the first two chunks -- the columns both accumulators share -- are in registers.
struct NoCombine {
  __device__ __forceinline__ void operator()(uint32_t (&)[32], int) const {}
};
template <int BN, bool kOverlap, int kStoreBufs, typename F, typename C = NoCombine>
__device__ __forceinline__ void drain_accumulator(const Params &p, const CUtensorMap *map_d, uint32_t t_acc, int first,
                                                  int row0, int n0, int lane, uint8_t *stage_buf, int &buf,
                                                  F shared_columns_read, C combine = C(), int z = -1) {
  // two chunks in flight: the TMEM load of chunk c+1 is issued before chunk c is converted and stored
  // chunk order: with overlapping accumulators the 64 shared columns go first (the last two chunks of
  // accumulator 0, the first two of accumulator 1)
  uint32_t vv[2][32];
  tmem_ld32(t_acc + (uint32_t)(first * 32), vv[0]);
  tmem_ld_wait(vv[0]);
#pragma unroll
  for (int ci = 0; ci < BN / 32; ++ci) {
    const int c = ((ci + first) % (BN / 32)) * 32;
    const bool active = n0 + c < p.N;  // uniform across the warp; chunks past the edge are read but not stored
    uint32_t(&v)[32] = vv[ci & 1];
    if (ci + 1 < BN / 32) tmem_ld32(t_acc + (uint32_t)(((ci + 1 + first) % (BN / 32)) * 32), vv[(ci + 1) & 1]);
    combine(v, c);  // split-K: add the other CTA's partial sums of these 32 columns
    if (p.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int n = n0 + c + j;
        float b = 0.f;
        if (n < p.N)
          b = p.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p.bias)[n])
                          : reinterpret_cast<const float *>(p.bias)[n];
        v[j] = __float_as_uint(__uint_as_float(v[j]) + b);
      }
    }
    if (!active) {
      // nothing to store
    } else if (p.tma_store) {
      if (p.out_bf16) {
        uint32_t w[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * t]), __uint_as_float(v[2 * t + 1]));
          w[t] = *reinterpret_cast<uint32_t *>(&h);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kStoreBufs - 1) : "memory");
        __syncwarp();
        uint8_t *dst = stage_buf + buf * 2048 + lane * 64;
#pragma unroll
        for (int t = 0; t < 4; ++t)  // 16-byte chunk t of this row lands at chunk t ^ ((row >> 1) & 3)
          *reinterpret_cast<uint4 *>(dst + ((t ^ ((lane >> 1) & 3)) << 4)) =
              make_uint4(w[4 * t], w[4 * t + 1], w[4 * t + 2], w[4 * t + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (z >= 0)
            tma_store_3d(map_d, smem_u32(stage_buf + buf * 2048), n0 + c, row0, z);
          else
            tma_store_2d(map_d, smem_u32(stage_buf + buf * 2048), n0 + c, row0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        buf = (buf + 1) % kStoreBufs;
      } else {
        // fp32: one box of 32 columns (128 bytes per row, 128-byte swizzle) per chunk.  It takes both of the warp's
        // staging buffers, so the previous box must have been read out first; rows of 128 bytes matter when the
        // destination is another GPU (64-byte rows reached a quarter of the link's bandwidth).
        static_assert(kStoreBufs == 2, "the fp32 box spans both staging buffers");
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
        uint8_t *dst = stage_buf + lane * 128;
#pragma unroll
        for (int t = 0; t < 8; ++t)  // 16-byte chunk t of this row lands at chunk t ^ (row & 7)
          *reinterpret_cast<uint4 *>(dst + ((t ^ (lane & 7)) << 4)) =
              make_uint4(v[4 * t], v[4 * t + 1], v[4 * t + 2], v[4 * t + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (z >= 0)
            tma_store_3d(map_d, smem_u32(stage_buf), n0 + c, row0, z);
          else
            tma_store_2d(map_d, smem_u32(stage_buf), n0 + c, row0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        buf = 0;
      }
    } else if (row0 + lane < p.M) {
      const size_t off = (size_t)(row0 + lane) * p.N + n0 + c + (z > 0 ? (size_t)z * (size_t)p.d_batch_stride : 0);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (n0 + c + j < p.N) {
          if (p.out_bf16)
            reinterpret_cast<__nv_bfloat16 *>(p.d)[off + j] = __float2bfloat16_rn(__uint_as_float(v[j]));
          else
            reinterpret_cast<float *>(p.d)[off + j] = __uint_as_float(v[j]);
        }
      }
    }
    tmem_ld_wait(vv[(ci + 1) & 1]);
    if constexpr (kOverlap) {
      if (ci == 0) {  // chunks 0 and 1 of this order -- the shared columns -- are in registers now
        tc_fence_before();
        __syncwarp();
        if (lane == 0) shared_columns_read();
      }
    }
  }
}

template <int kKind, int BN, bool kSplit = false>
__global__ void __launch_bounds__(kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                 const __grid_constant__ CUtensorMap map_d, const Params p) {
  constexpr bool kScaled = kKind == kMxf8;
  constexpr int kSfbChunks = (BN + 127) / 128;
  constexpr int kSfColsPerStage = 4 + 4 * kSfbChunks;
  // two accumulators when they fit next to the scale-factor columns (always for the dense kinds)
  // Two accumulators of BN columns when they fit next to the scale-factor columns (always for the dense kinds).
  // The block-scaled 256-column tile does not fit twice (2 x 256 + 48 > 512): its two accumulators overlap by 64
  // columns -- [0, 256) and [192, 448), scale factors from column 448 -- and the epilogue drains the shared 64
  // columns first and says so on its own barrier, so that the next tile's MMAs wait for a quarter of the epilogue
  // instead of all of it.
  constexpr bool kOverlap = kScaled && BN == 256;
  constexpr int kAccCols = BN;                     // TMEM columns of one accumulator stage
  constexpr int kAccStages =
      kOverlap || 2 * kAccCols + (kScaled ? kMaxStages * kSfColsPerStage : 0) <= kTmemCols ? 2 : 1;
  constexpr int kAccStride = kOverlap ? 192 : kAccCols;  // first column of accumulator stage 1
  constexpr int kSfCol = kOverlap ? 448 : kAccStages * kAccCols;  // first TMEM column of the scale factors
  using L = Layout<BN, kScaled, kSplit>;
  constexpr int kStages = L::kStages;
  constexpr int kStoreBufs = L::kStoreBufs;
  constexpr int kElem = kKind == kBf16 ? 2 : (kKind == kTf32 ? 4 : 1);
  constexpr int kBlockK = kRowBytes / kElem;      // elements of K per stage

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + L::kBarriers;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
  const uint32_t overlap_bar = bar_base + 8u * (2 * kMaxStages + 4);  // shared accumulator columns drained
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kBarriers + 32 * 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kBarriers + 32 * 8 + 8);

  const int warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;  // warp: provably uniform
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int tiles_mn = tiles_m * tiles_n;
  const int n_tiles = tiles_mn * (p.batch > 0 ? p.batch : 1);
  // Split K (small problems, launched as clusters of two with one tile per cluster): CTA `rank` of the cluster takes
  // the K chunks [kc_begin, kc_end) of tile blockIdx.x / 2; rank 1 hands its accumulator to rank 0, which stores.
  const int rank = kSplit ? (int)cluster_rank() : 0;
  const int first_tile = kSplit ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = kSplit ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int kc_half = (p.k_chunks + 1) / 2;
  const int kc_begin = kSplit && rank == 1 ? kc_half : 0;
  const int kc_end = kSplit && rank == 0 ? kc_half : p.k_chunks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(full_bar(s), 1), mbar_init(empty_bar(s), 1);
    for (int a = 0; a < 2; ++a) mbar_init(acc_full_bar(a), 1), mbar_init(acc_empty_bar(a), 4);
    mbar_init(overlap_bar, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Launched with programmatic stream serialization: everything above (barriers, tensor memory) may run while the
  // previous kernel of the stream -- normally the activation pack -- is still finishing; its results are visible
  // from here on.  Without that launch attribute this is a no-op.
  grid_dependency_wait();

  // The producer and the MMA issuer run their loops with all 32 lanes of their warp on identical values and elect
  // one lane for the TMA / tcgen05 instructions themselves.  Those instructions take their operands from uniform
  // registers; in a loop that only one lane executes every operand would have to be moved there first, which made
  // each of them cost about 70 cycles to issue -- more per K chunk than its MMAs take to run.
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      if constexpr (kScaled) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfa) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfb) : "memory");
      }
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_d) : "memory");
    }
    uint32_t sa = s_base, ssf = s_base + L::kSfBase, full = full_bar(0), empty = empty_bar(0);
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step) {
      const int z = tile / tiles_mn, in_z = tile - z * tiles_mn;  // matrix of the batch, tile inside it
      const int m_blk = in_z / tiles_n, n_blk = in_z % tiles_n;
      const int row_a = m_blk * BM, row_b = n_blk * BN;
      // rows of the scale maps
      int chunk_a = m_blk * p.k_chunks + kc_begin, chunk_b = ((n_blk * BN) / 128) * p.k_chunks + kc_begin;
      int k0 = kc_begin * kBlockK;
      for (int kc = kc_begin; kc < kc_end; ++kc) {
        if (!mbar_wait_warp(empty, phase ^ 1u, abort_flag, p.status, kErrProducerWait, p.wait_ns)) {
          ok = false;
          break;
        }
        // test hook: this slot is never filled, so the MMA issuer's wait for it runs out
        if (p.drop_last_load && blockIdx.x == 0 && tile == first_tile && kc == kc_end - 1) break;
        if (elect_one()) {
          mbar_expect_tx(full, L::kStage - L::kA + p.a_box_bytes - p.tx_less);
          if (p.batch > 0) {
            tma_load_3d(sa, &map_a, full, k0, row_a, z);
            tma_load_3d(sa + L::kA, &map_b, full, k0, row_b, z);
          } else {
            tma_load_2d(sa, &map_a, full, k0, row_a);
            tma_load_2d(sa + L::kA, &map_b, full, k0, row_b);
          }
          if constexpr (kScaled) {
            tma_load_2d(ssf, &map_sfa, full, 0, chunk_a);
#pragma unroll
            for (int j = 0; j < kSfbChunks; ++j)
              tma_load_2d(ssf + 512 + 512 * j, &map_sfb, full, 0, chunk_b + j * p.k_chunks);
          }
        }
        k0 += kBlockK, ++chunk_a, ++chunk_b;
        sa += L::kAB, ssf += L::kSf, full += 8, empty += 8, ++issued;
        if (++stage == kStages)
          stage = 0, phase ^= 1u, sa = s_base, ssf = s_base + L::kSfBase, full = full_bar(0), empty = empty_bar(0);
      }
    }
    if (*abort_flag && lane == 0) {
      // let the copies that were already issued land before the CTA gives up its shared memory
      for (int s = 0; s < kStages && s < issued; ++s) {
        const int last = (issued - 1 - s) / kStages;  // index of the last fill of slot (issued - 1 - s) % kStages
        const unsigned long long t0 = global_ns();
        while (!mbar_try_wait(full_bar((issued - 1 - s) % kStages), (uint32_t)last & 1u) &&
               global_ns() - t0 < 20000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const uint32_t idesc = make_idesc<kKind, BN>() | (p.b_fp4 ? kFormatE2M1 << 10 : 0u) | p.fmt_bits;
    uint32_t idk[4];  // per 32 bytes of K: byte k of each scale word
#pragma unroll
    for (int k = 0; k < 4; ++k) idk[k] = kScaled ? idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4) : idesc;
    // running operand descriptors (the start-address field counts 16-byte units), barriers and TMEM columns
    constexpr uint32_t kDescStep = L::kAB >> 4, kSfDescStep = L::kSf >> 4;
    const uint64_t da0 = desc_sw128(s_base), db0 = desc_sw128(s_base + L::kA);
    const uint64_t dsf0 = desc_sf(s_base + L::kSfBase);
    uint64_t da = da0, db = db0, dsf = dsf0;
    uint32_t sf_t = tmem_base + (uint32_t)kSfCol;
    uint32_t full = full_bar(0), empty = empty_bar(0);
    int stage = 0;
    uint32_t phase = 0;
    int local = 0;
    bool ok = true;
    for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step, ++local) {
      const int acc = local % kAccStages;
      const uint32_t acc_phase = (uint32_t)(local / kAccStages) & 1u;
      if (!mbar_wait_warp(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, kErrMmaWaitAcc, p.wait_ns)) break;
      if constexpr (kOverlap) {  // the previous tile's epilogue has read the columns both accumulators share
        if (local > 0 && !mbar_wait_warp(overlap_bar, (uint32_t)(local - 1) & 1u, abort_flag, p.status, kErrMmaWaitAcc, p.wait_ns))
          break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kAccStride);
      // a B tile narrower than a 128-row scale chunk starts at one of the chunk's four 32-row TMEM columns
      const uint32_t sfb_col = (uint32_t)((((tile % tiles_n) * BN) & 127) >> 5);
      uint32_t accumulate = 0;  // the tile's first MMA overwrites the accumulator
      for (int kc = kc_begin; kc < kc_end; ++kc) {
        if (!mbar_wait_warp(full, phase, abort_flag, p.status, kErrMmaWaitFull, p.wait_ns)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one()) {
          if constexpr (kScaled) {
            tc_cp_sf(sf_t, dsf);
#pragma unroll
            for (int j = 0; j < kSfbChunks; ++j) tc_cp_sf(sf_t + 4 + 4 * j, dsf + 32u * (j + 1));  // 512 bytes on
          }
          // 32 bytes of K per instruction: advance the start-address field inside the swizzle atom
          umma<kKind>(d_tmem, da, db, idk[0], accumulate, sf_t, sf_t + 4 + sfb_col);
#pragma unroll
          for (int k = 1; k < 4; ++k) umma<kKind>(d_tmem, da + 2u * k, db + 2u * k, idk[k], 1u, sf_t, sf_t + 4 + sfb_col);
          tc_commit(empty);  // arrives when the MMAs that read this slot have completed
        }
        accumulate = 1;
        da += kDescStep, db += kDescStep, dsf += kSfDescStep, sf_t += kSfColsPerStage, full += 8, empty += 8;
        if (++stage == kStages) {
          stage = 0, phase ^= 1u;
          da = da0, db = db0, dsf = dsf0, sf_t = tmem_base + (uint32_t)kSfCol, full = full_bar(0), empty = empty_bar(0);
        }
      }
      if (ok && elect_one()) tc_commit(acc_full_bar(acc));
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    // Each warp drains the 32 TMEM lanes (= 32 tile rows) of its quarter in chunks of 32 columns.  A chunk is
    // converted, written to a 64-byte-swizzled staging buffer in shared memory (32 rows x 64 bytes, two buffers per
    // warp) and handed to a TMA store, which writes whole lines and clips at the matrix edges.  Output matrices
    // whose rows are not 16-byte multiples take direct predicated stores instead.
    const int quarter = warp & 3;  // TMEM lanes [32 * quarter, +32) are the ones this warp may read
    uint8_t *stage_buf = smem + L::kStaging + (warp - 2) * (kStoreBufs * 2048);
    int buf = 0;
    int local = 0;
    if constexpr (!kSplit) {
      for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++local) {
        const int z = tile / tiles_mn, in_z = tile - z * tiles_mn;
        const int m_blk = in_z / tiles_n, n_blk = in_z % tiles_n;
        const int acc = local % kAccStages;
        const uint32_t acc_phase = (uint32_t)(local / kAccStages) & 1u;
        if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_flag, p.status, kErrEpilogueWait, p.wait_ns)) break;
        tc_fence_after();
        drain_accumulator<BN, kOverlap, kStoreBufs>(
            p, &map_d, tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * kAccStride),
            kOverlap && acc == 0 ? BN / 32 - 2 : 0, m_blk * BM + quarter * 32, n_blk * BN, lane, stage_buf, buf,
            [&] { mbar_arrive(overlap_bar); }, NoCombine(), p.batch > 0 ? z : -1);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(acc));
      }
    } else if (rank == 1 && first_tile < n_tiles) {
      // split K, second CTA: park the fp32 accumulator in the exchange buffer, column-major (element (row, col) at
      // col * 128 + row) so that the 32 lanes of a warp, one row each, hit 32 different banks
      float *xbuf = reinterpret_cast<float *>(smem + L::kXbuf);
      if (mbar_wait(acc_full_bar(0), 0u, abort_flag, p.status, kErrEpilogueWait, p.wait_ns)) {
        tc_fence_after();
        const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld32(t_acc + (uint32_t)c, v);
          tmem_ld_wait(v);
#pragma unroll
          for (int j = 0; j < 32; ++j) xbuf[(c + j) * BM + quarter * 32 + lane] = __uint_as_float(v[j]);
        }
        tc_fence_before();
      }
    }
    if constexpr (!kSplit) {
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores done before the CTA exits
    }
  }

  if constexpr (kSplit) {
    // every thread of both CTAs: the second CTA's partial sums are in its exchange buffer
    cluster_sync();
    if (warp >= 2 && rank == 0 && first_tile < n_tiles) {
      const int quarter = warp & 3;
      uint8_t *stage_buf = smem + L::kStaging + (warp - 2) * (kStoreBufs * 2048);
      int buf = 0;
      const int tile = first_tile, m_blk = tile / tiles_n, n_blk = tile % tiles_n;
      if (mbar_wait(acc_full_bar(0), 0u, abort_flag, p.status, kErrEpilogueWait, p.wait_ns)) {
        tc_fence_after();
        const uint32_t peer = map_to_cta(s_base + L::kXbuf, 1u) + (uint32_t)(quarter * 32 + lane) * 4u;
        drain_accumulator<BN, false, kStoreBufs>(
            p, &map_d, tmem_base + ((uint32_t)(quarter * 32) << 16), 0, m_blk * BM + quarter * 32, n_blk * BN, lane,
            stage_buf, buf, [] {},
            [&](uint32_t(&v)[32], int c) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = __float_as_uint(__uint_as_float(v[j]) + ld_cluster_f32(peer + (uint32_t)((c + j) * BM) * 4u));
            });
        tc_fence_before();
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    cluster_sync();  // the second CTA keeps its shared memory until the first one has read it
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// =====================================================================================================================
// GEMM on CTA pairs (tcgen05 cta_group::2), all three kinds.
//
// Two CTAs of a cluster share a 256 x 256 output tile.  CTA r of the pair holds 128 rows of A (rows m0 + 128 r ...)
// and 128 rows of B (columns n0 + 128 r ... of the output) in its shared memory and accumulates its 128 x 256 half
// of the tile in its own tensor memory; one thread of the leader CTA (rank 0) issues M = 256 MMAs that run on both
// SMs, each reading its A rows and its half of B locally.  Per SM and MMA that is 8 KB of operand reads from shared
// memory instead of 12 KB for a lone CTA, and 32 KB instead of 48 KB per ring slot, which buys a 6-slot ring.
//
// Synchronisation (every wait bounded as in the single-CTA kernel):
//   full[s]      leader's barrier.  The leader's producer arrives with the byte count of BOTH CTAs' slot s; all loads
//                of both CTAs (cta_group::2 form of the TMA load, one destination CTA each) complete on it.
//   empty[s]     one per CTA; the leader commits the MMAs of slot s to its own and to the peer's barrier.
//   acc_full[a]  one per CTA, committed the same way when a tile's MMAs are done.
//   acc_empty[a], overlap: leader's barriers; the epilogue warps of both CTAs arrive (the peer's remotely).
// Scale factors (block-scaled kind): each CTA loads the chunk of its own A rows and both chunks of the tile's B columns;
// tcgen05.cp.cta_group::2 moves them from each CTA's shared memory into that CTA's tensor memory.
// Both CTAs take part in one cta_group::2 allocation of all 512 TMEM columns, so their accumulator and scale
// addresses agree (still checked at start-up: a mismatch is reported in the status word, nothing is computed).
// A cluster barrier before the CTAs free their tensor memory keeps each alive while the other may still touch its
// barriers or read its half of B.
// =====================================================================================================================
constexpr int kErrPairTmem = 5;

template <bool kScaled>
struct PairLayout {
  static constexpr int kStages = 6;
  static constexpr int kStoreBufs = 2;
  static constexpr int kA = BM * kRowBytes;            // this CTA's 128 rows of A
  static constexpr int kB = 128 * kRowBytes;           // this CTA's 128 rows of B
  static constexpr int kAB = kA + kB;
  static constexpr int kSf = kScaled ? 512 + 2 * 512 : 0;  // own A chunk, both B chunks
  static constexpr int kStageTx = 2 * (kAB + kSf);     // bytes of both CTAs that complete on the leader's barrier
  static constexpr int kSfBase = kStages * kAB;
  static constexpr int kStaging = (kStages * (kAB + kSf) + 1023) & ~1023;
  static constexpr int kBarriers = kStaging + 4 * kStoreBufs * 2048;
  static constexpr int kTotal = kBarriers + 32 * 8 + 16 + 1024;
};

// TMA load of a CTA pair: the data lands in this CTA's shared memory, the bytes complete on `bar`, which may be a
// barrier of the peer CTA (shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// the MMAs issued so far by this thread arrive on `bar` (shared::cluster address, either CTA of the pair) when done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
template <int kKind>
__device__ __forceinline__ void umma_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc, uint32_t sfa,
                                          uint32_t sfb) {
  if constexpr (kKind == kBf16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc)
        : "memory");
  } else if constexpr (kKind == kTf32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
        : "memory");
  }
}

template <int kKind>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                      const __grid_constant__ StoreMaps maps_d, const Params p) {
  constexpr bool kScaled = kKind == kMxf8;
  using L = PairLayout<kScaled>;
  constexpr int BN = 256;
  constexpr int kStages = L::kStages;
  constexpr int kStoreBufs = L::kStoreBufs;
  constexpr int kElem = kKind == kBf16 ? 2 : (kKind == kTf32 ? 4 : 1);
  constexpr int kBlockK = kRowBytes / kElem;  // elements of K per ring slot
  // block-scaled: accumulators [0, 256) and [192, 448) overlap, scale factors from column 448; dense: [0, 256), [256, 512)
  constexpr bool kOverlap = kScaled;
  constexpr int kAccStride = kScaled ? 192 : 256;
  constexpr int kSfCol = 448;
  constexpr int kSfSlots = 4;      // TMEM scale-factor slots of 12 columns, used round-robin per K chunk

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + L::kBarriers;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
  const uint32_t overlap_bar = bar_base + 8u * (2 * kMaxStages + 4);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kBarriers + 32 * 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kBarriers + 32 * 8 + 8);

  const int warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();  // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m = (p.M + 255) / 256, tiles_n = (p.N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(full_bar(s), 1), mbar_init(empty_bar(s), 1);
    for (int a = 0; a < 2; ++a) mbar_init(acc_full_bar(a), 1), mbar_init(acc_empty_bar(a), 8);
    mbar_init(overlap_bar, 8);  // 4 epilogue warps in each CTA
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    // every tcgen05 instruction of this kernel is the cta_group::2 form: one warp of each CTA of the pair takes
    // part in the allocation, which hands both CTAs the same columns
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers are initialised and both tensor-memory addresses are published
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();  // see the single-CTA kernel
  // the MMAs address both CTAs' tensor memory with one address: the two allocations must coincide
  if (ld_cluster_u32(map_to_cta(smem_u32(tmem_slot), rank ^ 1u)) != tmem_base) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kErrPairTmem);
  } else if (warp == 0) {
    // ---------------- TMA producer (both CTAs; warp-uniform loop, one elected lane issues) ----------------
    if (elect_one()) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      if constexpr (kScaled) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfa) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfb) : "memory");
      }
      asm volatile("prefetch.tensormap [%0];" ::"l"(&maps_d.m[0]) : "memory");
    }
    const uint32_t lead_full0 = map_to_cta(full_bar(0), 0);  // the leader's full[0] as a shared::cluster address
    uint32_t sa = s_base, ssf = s_base + L::kSfBase, full = full_bar(0), lead_full = lead_full0, empty = empty_bar(0);
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
      // (row of tiles, rotated when the epilogue scatters to other GPUs: see Params::m_rotate)
      const int m_blk = ((tile / tiles_n + p.m_rotate) % tiles_m) * 2 + (int)rank;  // 128-row block of A and its scales
      const int n_blk = (tile % tiles_n) * 2;                  // first of the tile's two 128-column blocks
      const int row_a = m_blk * BM, row_b = (n_blk + (int)rank) * 128;
      int chunk_a = m_blk * p.k_chunks, chunk_b = n_blk * p.k_chunks;
      int k0 = 0;
      for (int kc = 0; kc < p.k_chunks; ++kc) {
        if (!mbar_wait_warp(empty, phase ^ 1u, abort_flag, p.status, kErrProducerWait, p.wait_ns)) {
          ok = false;
          break;
        }
        if (elect_one()) {
          if (leader) mbar_expect_tx(full, L::kStageTx - p.tx_less);
          tma_load_2d_pair(sa, &map_a, lead_full, k0, row_a);
          tma_load_2d_pair(sa + L::kA, &map_b, lead_full, k0, row_b);
          if constexpr (kScaled) {
            tma_load_2d_pair(ssf, &map_sfa, lead_full, 0, chunk_a);
            tma_load_2d_pair(ssf + 512, &map_sfb, lead_full, 0, chunk_b);
            tma_load_2d_pair(ssf + 1024, &map_sfb, lead_full, 0, chunk_b + p.k_chunks);
          }
        }
        k0 += kBlockK, ++chunk_a, ++chunk_b;
        sa += L::kAB, ssf += L::kSf, full += 8, lead_full += 8, empty += 8, ++issued;
        if (++stage == kStages) {
          stage = 0, phase ^= 1u;
          sa = s_base, ssf = s_base + L::kSfBase, full = full_bar(0), lead_full = lead_full0, empty = empty_bar(0);
        }
      }
    }
    if (*abort_flag && leader && lane == 0) {
      // let the copies that were already issued land before the CTAs give up their shared memory
      for (int s = 0; s < kStages && s < issued; ++s) {
        const int last = (issued - 1 - s) / kStages;
        const unsigned long long t0 = global_ns();
        while (!mbar_try_wait(full_bar((issued - 1 - s) % kStages), (uint32_t)last & 1u) &&
               global_ns() - t0 < 20000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (leader) {
      // ---------------- MMA issuer (leader only; warp-uniform loop, one elected lane issues) ----------------
      // the single-CTA descriptor with M = 256 (both CTAs) instead of 128
      const uint32_t idesc = (make_idesc<kKind, BN>() & ~(0x1Fu << 24)) | ((uint32_t)(256 >> 4) << 24) |
                             (p.b_fp4 ? kFormatE2M1 << 10 : 0u) | p.fmt_bits;
      uint32_t idk[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)  // block-scaled: byte k of each scale word
        idk[k] = kScaled ? idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4) : idesc;
      constexpr uint32_t kDescStep = L::kAB >> 4, kSfDescStep = L::kSf >> 4;
      const uint64_t da0 = desc_sw128(s_base), db0 = desc_sw128(s_base + L::kA), dsf0 = desc_sf(s_base + L::kSfBase);
      const uint32_t my_empty0 = map_to_cta(empty_bar(0), rank), peer_empty0 = map_to_cta(empty_bar(0), rank ^ 1u);
      uint64_t da = da0, db = db0, dsf = dsf0;
      uint32_t full = full_bar(0), my_empty = my_empty0, peer_empty = peer_empty0;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      uint32_t slot = 0;  // TMEM scale-factor slot
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
        if (!mbar_wait_warp(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, kErrMmaWaitAcc, p.wait_ns)) break;
        if constexpr (kOverlap) {
          if (local > 0 &&
              !mbar_wait_warp(overlap_bar, (uint32_t)(local - 1) & 1u, abort_flag, p.status, kErrMmaWaitAcc, p.wait_ns))
            break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kAccStride);
        uint32_t accumulate = 0;
        for (int kc = 0; kc < p.k_chunks; ++kc) {
          if (!mbar_wait_warp(full, phase, abort_flag, p.status, kErrMmaWaitFull, p.wait_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sf_t = tmem_base + (uint32_t)kSfCol + slot * 12u;
          if (elect_one()) {
            if constexpr (kScaled) {
              tc_cp_sf_pair(sf_t, dsf);
              tc_cp_sf_pair(sf_t + 4, dsf + 32u);
              tc_cp_sf_pair(sf_t + 8, dsf + 64u);
            }
            umma_pair<kKind>(d_tmem, da, db, idk[0], accumulate, sf_t, sf_t + 4);
#pragma unroll
            for (int k = 1; k < 4; ++k) umma_pair<kKind>(d_tmem, da + 2u * k, db + 2u * k, idk[k], 1u, sf_t, sf_t + 4);
            // both CTAs' slot is free once these MMAs have completed
            tc_commit_pair(my_empty);
            tc_commit_pair(peer_empty);
          }
          accumulate = 1;
          slot = (slot + 1) % kSfSlots;
          da += kDescStep, db += kDescStep, dsf += kSfDescStep, full += 8, my_empty += 8, peer_empty += 8;
          if (++stage == kStages) {
            stage = 0, phase ^= 1u;
            da = da0, db = db0, dsf = dsf0, full = full_bar(0), my_empty = my_empty0, peer_empty = peer_empty0;
          }
        }
        if (ok && elect_one()) {
          tc_commit_pair(map_to_cta(acc_full_bar(acc), rank));
          tc_commit_pair(map_to_cta(acc_full_bar(acc), rank ^ 1u));
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs): this CTA's 128 rows of the tile ----------------
    const int quarter = warp & 3;
    uint8_t *stage_buf = smem + L::kStaging + (warp - 2) * (kStoreBufs * 2048);
    const uint32_t lead_overlap = map_to_cta(overlap_bar, 0);
    int buf = 0;
    int local = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++local) {
      const int m_blk = ((tile / tiles_n + p.m_rotate) % tiles_m) * 2 + (int)rank, n_blk = tile % tiles_n;
      const int acc = local & 1;
      const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
      if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_flag, p.status, kErrEpilogueWait, p.wait_ns)) break;
      tc_fence_after();
      // with a reduce-scatter fused in, the tile goes to the slot buffer of the GPU that owns its rows
      const int owner = p.scatter_rows ? (m_blk * BM) / p.scatter_rows : 0;
      drain_accumulator<BN, kOverlap, kStoreBufs>(
          p, &maps_d.m[owner], tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * kAccStride),
          kOverlap && acc == 0 ? BN / 32 - 2 : 0,
          m_blk * BM - owner * p.scatter_rows + quarter * 32, n_blk * BN, lane, stage_buf, buf,
          [&] { mbar_arrive_cluster(lead_overlap); });
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty_bar(acc), 0));
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores done before the CTA exits
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();  // neither CTA frees tensor memory or exits while the other may still use it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// =====================================================================================================================
// Few rows of activations against a large weight (M <= 128): the transposed product D^T[N, M] = W[N, K] X[M, K]^T.
//
// Such a problem is the latency of streaming the weight once.  Here the weight is the 128-row operand of the MMA and
// the activations are its narrow one (16, 32, 64 or 128 columns of the accumulator), so one instruction covers 128
// weight rows with a short pass through the tensor pipe, and a CTA's 128-row stripe of the weight is fetched by a
// producer that never waits for the activations: it initialises the barriers itself and issues its weight and
// weight-scale loads at once -- before the rest of the CTA has set up tensor memory and before the dependency wait on
// the previous kernel of the stream (the activation pack) -- and the activation loads behind that wait, into a ring
// deep enough to hold a CTA's whole share of K for the common shapes.  K is split over the 1, 2 or 4 CTAs of a
// thread-block cluster so that about every SM pulls on the weight; the other CTAs push their fp32 partial sums into
// the first CTA's shared memory (distributed shared memory stores, one cluster barrier), which adds them in rank
// order (repeatable), adds the bias and stores D transposed back: lane = weight row, so a warp writes 32 consecutive
// elements of one output row.
// =====================================================================================================================
constexpr int kSwapMaxStages = 12;

template <int BNX, bool kScaled>
struct SwapLayout {
  static constexpr int kMaxSplit = BNX <= 32 ? 4 : 2;  // shares of K (CTAs per cluster)
  static constexpr int kW = BM * kRowBytes;   // 128 weight rows
  static constexpr int kX = BNX * kRowBytes;  // activation rows (the ones past M are never stored)
  static constexpr int kWX = kW + kX;
  static constexpr int kSf = kScaled ? 1024 : 0;  // weight chunk, activation chunk
  // partial sums of the other CTAs of the cluster land here in the first CTA: [rank - 1][column][row] fp32
  static constexpr int kXbufBytes = (kMaxSplit - 1) * BNX * BM * 4;
  static constexpr int kRingSpace = 200 * 1024 - kXbufBytes;
  static constexpr int kFit = kRingSpace / (kWX + kSf);
  static constexpr int kStages = kFit < 10 ? kFit : 10;
  static constexpr int kSfBase = kStages * kWX;
  static constexpr int kXbuf = (kStages * (kWX + kSf) + 1023) & ~1023;
  static constexpr int kBarriers = kXbuf + kXbufBytes;  // full[], empty[], acc_full
  static constexpr int kTotal = kBarriers + (2 * kSwapMaxStages + 2) * 8 + 16 + 1024;
};

struct SwapParams {
  void *d;
  const void *bias;
  int *status;
  int M, N;
  int k_chunks;
  int split;         // CTAs per cluster = shares of K
  int x_box_bytes;   // bytes one activation load delivers
  int out_bf16, bias_bf16;
  uint32_t w_fp4;    // block-scaled kind: the weight holds E2M1 elements, two per byte in global memory
  uint32_t fmt_bits = 0;  // element formats other than E4M3 / E2M1: the weight's in bits 7-9, the activations' in bits 10-12
  uint32_t tx_less;  // a 4-bit box counts its packed bytes on the barrier, half of what lands in shared memory
  uint32_t early_w;  // the weight was complete before anything still running on the stream: fetch it ahead of the wait
  unsigned long long wait_ns;
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                    "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :: "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

template <int kKind, int BNX>
__global__ void __launch_bounds__(kThreads, 1)
umma_gemm_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const __grid_constant__ CUtensorMap map_sfw, const __grid_constant__ CUtensorMap map_sfx,
                      const SwapParams p) {
  constexpr bool kScaled = kKind == kMxf8;
  using L = SwapLayout<BNX, kScaled>;
  constexpr int kStages = L::kStages;
  constexpr int kElem = kKind == kBf16 ? 2 : (kKind == kTf32 ? 4 : 1);
  constexpr int kBlockK = kRowBytes / kElem;
  constexpr int kSfCol = 128;          // scale factors behind the (at most 128) accumulator columns
  // The next kernel of the stream may be scheduled from here on (it waits on the device before it touches anything
  // this launch reads or writes): its CTAs take over an SM the moment this launch's CTA leaves it and, for a launch of
  // this kernel with a static weight, start pulling the weight without waiting for the rest of this grid.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int kSwapTmemCols = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + L::kBarriers;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kSwapMaxStages + s); };
  const uint32_t acc_full = bar_base + 8u * (2 * kSwapMaxStages);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kBarriers + (2 * kSwapMaxStages + 2) * 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kBarriers + (2 * kSwapMaxStages + 2) * 8 + 8);

  const int warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int rank = p.split > 1 ? (int)cluster_rank() : 0;
  const int n_blk = (int)blockIdx.x / p.split;        // 128-row stripe of the weight
  // this CTA's share of the K chunks: the first `rem` ranks take one more
  const int base = p.k_chunks / p.split, rem = p.k_chunks % p.split;
  const int kc_begin = rank * base + (rank < rem ? rank : rem);
  const int kc_count = base + (rank < rem ? 1 : 0);
  const int first_pass = kc_count < kStages ? kc_count : kStages;
  const int row_w = n_blk * BM;
  const uint32_t stage_tx = (uint32_t)(L::kW + L::kSf) + (uint32_t)p.x_box_bytes - p.tx_less;
  // Every CTA of a cluster must be running before another one touches its shared memory: arrive now, wait (long
  // since satisfied) right before the partial sums are pushed.
  if (p.split > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

  if (warp == 0) {
    // The producer does not wait for the rest of the CTA: it initialises the barriers and starts the weight stream.
    if (lane == 0) {
      for (int s = 0; s < kStages; ++s) mbar_init(full_bar(s), 1), mbar_init(empty_bar(s), 1);
      mbar_init(acc_full, 1);
      *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    if (!p.early_w) grid_dependency_wait();  // the weight may be the product of a kernel that is still running
    for (int i = 0; i < first_pass; ++i) {
      if (elect_one()) {
        const int kc = kc_begin + i;
        mbar_expect_tx(full_bar(i), stage_tx);
        tma_load_2d(s_base + i * L::kWX, &map_w, full_bar(i), kc * kBlockK, row_w);
        if constexpr (kScaled) tma_load_2d(s_base + L::kSfBase + i * L::kSf, &map_sfw, full_bar(i), 0, n_blk * p.k_chunks + kc);
      }
    }
  } else if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kSwapTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();  // barriers initialised, tensor memory allocated
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer, continued ----------------
    grid_dependency_wait();  // the activations (and their scales) come from the previous kernel
    for (int i = 0; i < first_pass; ++i) {
      if (elect_one()) {
        const int kc = kc_begin + i;
        tma_load_2d(s_base + i * L::kWX + L::kW, &map_x, full_bar(i), kc * kBlockK, 0);
        if constexpr (kScaled) tma_load_2d(s_base + L::kSfBase + i * L::kSf + 512, &map_sfx, full_bar(i), 0, kc);
      }
    }
    int issued = first_pass;
    for (int i = first_pass; i < kc_count; ++i) {
      const int s = i % kStages;
      if (!mbar_wait_warp(empty_bar(s), (uint32_t)(i / kStages - 1) & 1u, abort_flag, p.status, kErrProducerWait, p.wait_ns))
        break;
      if (elect_one()) {
        const int kc = kc_begin + i;
        mbar_expect_tx(full_bar(s), stage_tx);
        tma_load_2d(s_base + s * L::kWX, &map_w, full_bar(s), kc * kBlockK, row_w);
        tma_load_2d(s_base + s * L::kWX + L::kW, &map_x, full_bar(s), kc * kBlockK, 0);
        if constexpr (kScaled) {
          tma_load_2d(s_base + L::kSfBase + s * L::kSf, &map_sfw, full_bar(s), 0, n_blk * p.k_chunks + kc);
          tma_load_2d(s_base + L::kSfBase + s * L::kSf + 512, &map_sfx, full_bar(s), 0, kc);
        }
      }
      ++issued;
    }
    if (*abort_flag && lane == 0) {
      // let the copies that were already issued land before the CTA gives up its shared memory
      for (int s = 0; s < kStages && s < issued; ++s) {
        const int last = (issued - 1 - s) / kStages;
        const unsigned long long t0 = global_ns();
        while (!mbar_try_wait(full_bar((issued - 1 - s) % kStages), (uint32_t)last & 1u) &&
               global_ns() - t0 < 20000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const uint32_t idesc = make_idesc<kKind, BNX>() | (p.w_fp4 ? kFormatE2M1 << 7 : 0u) | p.fmt_bits;  // the weight is operand A here
    uint32_t idk[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) idk[k] = kScaled ? idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4) : idesc;
    bool ok = true;
    for (int i = 0; i < kc_count; ++i) {
      const int s = i % kStages;
      if (!mbar_wait_warp(full_bar(s), (uint32_t)(i / kStages) & 1u, abort_flag, p.status, kErrMmaWaitFull, p.wait_ns)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (elect_one()) {
        const uint64_t dw = desc_sw128(s_base + s * L::kWX), dx = desc_sw128(s_base + s * L::kWX + L::kW);
        const uint32_t sf_t = tmem_base + (uint32_t)(kSfCol + 8 * s);
        if constexpr (kScaled) {
          const uint64_t dsf = desc_sf(s_base + L::kSfBase + s * L::kSf);
          tc_cp_sf(sf_t, dsf);
          tc_cp_sf(sf_t + 4, dsf + 32u);  // 512 bytes on: the activations' chunk
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma<kKind>(tmem_base, dw + 2u * k, dx + 2u * k, idk[k], (i | k) ? 1u : 0u, sf_t, sf_t + 4);
        tc_commit(empty_bar(s));
      }
    }
    if (ok && elect_one()) tc_commit(acc_full);
  }

  if (p.split > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // all CTAs of the cluster have started
  // ---------------- epilogue (warps 2..5): TMEM lane = weight row ----------------
  const int quarter = warp & 3;
  const int row_in_tile = quarter * 32 + lane;
  const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16);
  bool have_acc = false;
  if (warp >= 2) {
    have_acc = mbar_wait_warp(acc_full, 0u, abort_flag, p.status, kErrEpilogueWait, p.wait_ns);
    tc_fence_after();
    if (have_acc && rank != 0) {
      // push this CTA's partial sums into the first CTA's exchange buffer, column-major (element (row, col) at
      // col * 128 + row: the 32 lanes of a warp write 128 consecutive bytes)
      const uint32_t dst = map_to_cta(s_base + L::kXbuf, 0u) + (uint32_t)((rank - 1) * BNX * BM + row_in_tile) * 4u;
#pragma unroll
      for (int c = 0; c < BNX; c += 16) {
        if (c >= p.M) break;
        uint32_t v[16];
        tmem_ld16(t_acc + (uint32_t)c, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) st_cluster_f32(dst + (uint32_t)((c + j) * BM) * 4u, __uint_as_float(v[j]));
      }
      tc_fence_before();
    }
  }
  if (p.split > 1) cluster_sync();  // every thread of every CTA: the pushed sums are visible in the first CTA
  if (warp >= 2 && rank == 0 && have_acc) {
    grid_dependency_wait();  // nothing of the previous kernel may still be reading D
    const int n = n_blk * BM + row_in_tile;
    float bias = 0.f;
    if (p.bias != nullptr && n < p.N)
      bias = p.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p.bias)[n])
                         : reinterpret_cast<const float *>(p.bias)[n];
    const float *xbuf = reinterpret_cast<const float *>(smem + L::kXbuf) + row_in_tile;
#pragma unroll
    for (int c = 0; c < BNX; c += 16) {
      if (c >= p.M) break;
      uint32_t v[16];
      tmem_ld16(t_acc + (uint32_t)c, v);
      float f[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) f[j] = __uint_as_float(v[j]);
      for (int r = 1; r < p.split; ++r) {  // fixed order: repeatable sums
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] += xbuf[((r - 1) * BNX + c + j) * BM];
      }
      if (n < p.N) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = c + j;
          if (m < p.M) {
            const size_t off = (size_t)m * p.N + n;
            if (p.out_bf16)
              reinterpret_cast<__nv_bfloat16 *>(p.d)[off] = __float2bfloat16_rn(f[j] + bias);
            else
              reinterpret_cast<float *>(p.d)[off] = f[j] + bias;
          }
        }
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kSwapTmemCols) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn driver_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// A tensor map is a pure function of the arguments of cuTensorMapEncodeTiled (it holds an address and a geometry, no
// state), and a serving loop launches the same few problems over and over: every host thread keeps the maps it encoded
// last, keyed by all arguments, and a launch that finds its map copies 128 bytes instead of calling the driver.
struct MapKey {
  uint64_t v[16];
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kMapSlots = 128;
static CUresult encode_cached(CUtensorMap *map, CUtensorMapDataType dt, cuuint32_t rank, void *ptr, const cuuint64_t *dims,
                              const cuuint64_t *strides, const cuuint32_t *box, const cuuint32_t *estr,
                              CUtensorMapInterleave il, CUtensorMapSwizzle sw, CUtensorMapL2promotion promo,
                              CUtensorMapFloatOOBfill fill) {
  EncodeTiledFn fn = driver_encode_fn();
  if (rank < 1 || rank > 3) return fn(map, dt, rank, ptr, dims, strides, box, estr, il, sw, promo, fill);
  static thread_local MapSlot slots[kMapSlots] = {};
  MapKey k = {};
  k.v[0] = reinterpret_cast<uintptr_t>(ptr);
  k.v[1] = ((uint64_t)dt << 48) | ((uint64_t)rank << 40) | ((uint64_t)il << 32) | ((uint64_t)sw << 24) | ((uint64_t)promo << 16) |
           (uint64_t)fill;
  for (cuuint32_t i = 0; i < rank; ++i) k.v[2 + i] = dims[i], k.v[8 + i] = ((uint64_t)box[i] << 32) | estr[i];
  for (cuuint32_t i = 0; i + 1 < rank; ++i) k.v[5 + i] = strides[i];
  uint64_t h = 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < 11; ++i) h = (h ^ k.v[i]) * 0x100000001B3ull;
  MapSlot &s = slots[(h >> 20) % kMapSlots];
  if (s.valid && memcmp(&s.key, &k, sizeof(k)) == 0) {
    *map = s.map;
    return CUDA_SUCCESS;
  }
  const CUresult r = fn(map, dt, rank, ptr, dims, strides, box, estr, il, sw, promo, fill);
  if (r == CUDA_SUCCESS) s.key = k, s.map = *map, s.valid = true;
  return r;
}
static EncodeTiledFn encode_fn() { return driver_encode_fn() ? &encode_cached : nullptr; }

// tensor map of a K-major matrix [rows, k] with boxes of box_rows x 128 bytes, 128-byte swizzle, zero fill
static int make_map(CUtensorMap *map, const void *ptr, int kind, int64_t rows, int64_t k, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return MXQ_ERR_UNSUPPORTED;
  const int es = kind == kBf16 ? 2 : (kind == kTf32 ? 4 : 1);
  const CUtensorMapDataType dt = kind == kBf16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : kind == kTf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * es};
  cuuint32_t box[2] = {(cuuint32_t)(kRowBytes / es), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_LAUNCH;
}

// Tensor map of a K-major matrix [rows, k] of 4-bit elements stored two per byte: the copy engine expands each group
// of 16 elements (8 bytes in global memory) to 16 bytes of shared memory, the padded form in which the block-scaled
// MMA reads 4-bit operands.  A box is box_rows x 128 elements and lands as box_rows x 128 bytes, 128-byte swizzle --
// the footprint of an E4M3 box -- while only half the bytes travel (and half are counted on the mbarrier).  Needs
// k % 128 == 0 and a 32-byte aligned base.
static int make_map_fp4(CUtensorMap *map, const void *ptr, int64_t rows, int64_t k, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return MXQ_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k / 2};
  cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_UNSUPPORTED;
}

// tensor map of the output [rows, n] for stores of 32-row x 32-column boxes: 64-byte rows with 64-byte swizzle for
// bf16, 128-byte rows with 128-byte swizzle for fp32
static int make_store_map(CUtensorMap *map, void *ptr, bool bf16, int64_t rows, int64_t n) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return MXQ_ERR_UNSUPPORTED;
  const int es = bf16 ? 2 : 4;
  cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)n * es};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, bf16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_LAUNCH;
}

// tensor map over scale-factor chunks: [chunks, 512 bytes] as rows of 128 32-bit words, one chunk per box
static int make_sf_map(CUtensorMap *map, const void *ptr, int64_t chunks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return MXQ_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {128, (cuuint64_t)chunks};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_LAUNCH;
}

Opts make_opts(const mxq_gemm_options *o) {
  Opts r;
  if (o) {
    r.max_ctas = o->max_ctas > 0 ? o->max_ctas : 0;
    r.tiles = o->tiles == MXQ_TILES_SINGLE || o->tiles == MXQ_TILES_PAIRS ? o->tiles : MXQ_TILES_AUTO;
    r.split_k = o->no_split_k == 0;
    r.transposed = o->no_transposed == 0;
    if (o->wait_limit_ns > 0) r.wait_ns = (unsigned long long)o->wait_limit_ns;
    r.test_hook = o->test_hook;
    r.static_b = (o->flags & MXQ_GEMM_STATIC_B) != 0;
    r.a_e5m2 = (o->flags & MXQ_GEMM_A_E5M2) != 0;
  }
  return r;
}

static int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev;
}

// SM count of the current device (cached per device ordinal; the value never changes, so a racing first call writes
// the same number)
int sm_count() {
  static int cached[64] = {};
  const int dev = current_device();
  int &n = cached[dev & 63];
  if (n <= 0) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    n = v > 0 ? v : 148;
  }
  return n;
}

// Launch with programmatic stream serialization: the kernel may start while the previous kernel of the stream is
// still running (once that kernel has let its dependents go, or finished) and waits for it on the device.
template <typename... KArgs, typename... Args>
static cudaError_t launch_dependent(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t st,
                                    int cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid), cfg.blockDim = dim3((unsigned)block), cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  if (cluster > 1) {  // kernels without a compile-time cluster size: clusters of `cluster` CTAs along x
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cluster, attr[1].val.clusterDim.y = 1, attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Batches of matrices: the same boxes with the matrix index as a third coordinate (box extent 1), so that loads fill
// with zeros and stores clip at the edge of each matrix, not of the whole allocation.  Strides in elements.
struct Batch {
  int64_t count = 0;  // 0 = one product, two-dimensional maps
  int64_t stride_a = 0, stride_b = 0, stride_d = 0;
};
static int make_map3(CUtensorMap *map, const void *ptr, int kind, int64_t rows, int64_t k, int box_rows, int64_t batch,
                     int64_t stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return MXQ_ERR_UNSUPPORTED;
  const int es = kind == kBf16 ? 2 : 4;
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)k * es, (cuuint64_t)stride * es};
  cuuint32_t box[3] = {(cuuint32_t)(kRowBytes / es), (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, kind == kBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                  const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_LAUNCH;
}
static int make_store_map3(CUtensorMap *map, void *ptr, bool bf16, int64_t rows, int64_t n, int64_t batch, int64_t stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return MXQ_ERR_UNSUPPORTED;
  const int es = bf16 ? 2 : 4;
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)n * es, (cuuint64_t)stride * es};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ptr, dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, bf16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_LAUNCH;
}

template <int kKind, int BN, bool kSplit = false>
static int launch(const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb, void *d, const void *bias,
                  int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int *status, const Opts &o,
                  cudaStream_t st, const Batch &bt = Batch()) {
  using L = Layout<BN, kKind == kMxf8, kSplit>;
  if (bt.count > 0 && (kKind == kMxf8 || kSplit)) return MXQ_ERR_UNSUPPORTED;
  constexpr int es = kKind == kBf16 ? 2 : (kKind == kTf32 ? 4 : 1);
  CUtensorMap ma, mb, md;
  // With fewer than 128 rows the A load fetches only the rows that exist (rounded up to the 8-row swizzle atom): the
  // remaining rows of the tile in shared memory stay as they are, and the accumulator rows they produce are never
  // stored.  (Letting TMA zero-fill them costs time: M = 16 ran slower than M = 128.)
  const int a_rows = M < BM ? (int)((M + 7) / 8 * 8) : BM;
  int rc = bt.count > 0 ? make_map3(&ma, a, kKind, M, K, a_rows, bt.count, bt.stride_a) : make_map(&ma, a, kKind, M, K, a_rows);
  if (rc) return rc;
  rc = bt.count > 0 ? make_map3(&mb, b, kKind, N, K, BN, bt.count, bt.stride_b)
                    : (o.b_fp4 ? make_map_fp4(&mb, b, N, K, BN) : make_map(&mb, b, kKind, N, K, BN));
  if (rc) return rc;
  const bool out_bf16 = out_dtype == MXQ_BF16;
  const bool tma_store = (N * (out_bf16 ? 2 : 4)) % 16 == 0 && (bt.count == 0 || (bt.stride_d * (out_bf16 ? 2 : 4)) % 16 == 0);
  if (tma_store) {
    rc = bt.count > 0 ? make_store_map3(&md, d, out_bf16, M, N, bt.count, bt.stride_d) : make_store_map(&md, d, out_bf16, M, N);
    if (rc) return rc;
  } else {
    md = ma;  // unused by the kernel
  }
  Params p;
  p.batch = (int)bt.count, p.d_batch_stride = bt.stride_d;
  p.sfa = sfa, p.sfb = sfb, p.d = d, p.bias = bias, p.status = status;
  p.M = (int)M, p.N = (int)N, p.K = (int)K;
  p.k_chunks = (int)((K * es + kRowBytes - 1) / kRowBytes);
  p.out_bf16 = out_bf16, p.bias_bf16 = bias_dtype == MXQ_BF16, p.tma_store = tma_store;
  p.a_box_bytes = a_rows * kRowBytes;
  p.wait_ns = o.wait_ns, p.drop_last_load = !kSplit && o.test_hook == MXQ_TEST_DROP_LAST_LOAD;
  p.b_fp4 = o.b_fp4 ? 1u : 0u;
  p.fmt_bits = (o.a_e5m2 ? kFormatE5M2 << 7 : 0u) | (o.b_e5m2 ? kFormatE5M2 << 10 : 0u);
  p.tx_less = o.b_fp4 ? BN * (kRowBytes / 2) : 0;
  p.scatter_rows = 0, p.m_rotate = 0;
  CUtensorMap msa = ma, msb = ma;  // unused by the dense kinds
  if constexpr (kKind == kMxf8) {
    rc = make_sf_map(&msa, sfa, ((M + 255) / 256) * 2 * p.k_chunks);
    if (rc) return rc;
    rc = make_sf_map(&msb, sfb, ((N + 255) / 256) * 2 * p.k_chunks);
    if (rc) return rc;
  }
  static bool attr_done[64] = {};  // per device: function attributes belong to the device's context
  bool &attr_set = attr_done[current_device() & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(umma_gemm_kernel<kKind, BN, kSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) !=
        cudaSuccess)
      return MXQ_ERR_LAUNCH;
    attr_set = true;
  }
  const int64_t tiles64 = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * (bt.count > 0 ? bt.count : 1);
  if (tiles64 > INT32_MAX) return MXQ_ERR_SHAPE;
  const int tiles = (int)tiles64;
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (o.max_ctas > 0 && grid > o.max_ctas) grid = o.max_ctas;
  if (kSplit) {  // one tile per cluster of two; the caller checked that 2 * tiles CTAs fit
    grid = 2 * tiles;
    if (o.max_ctas > 0 && grid > o.max_ctas) return MXQ_ERR_UNSUPPORTED;
  }
  const cudaError_t err = launch_dependent(umma_gemm_kernel<kKind, BN, kSplit>, grid, kThreads, L::kTotal, st,
                                           kSplit ? 2 : 0, ma, mb, msa, msb, md, p);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return MXQ_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

// Block-scaled GEMM on CTA pairs; the scale buffers are padded to whole 256-row tiles (mxq_mma_scale_bytes).
template <int kKind>
static int launch_pair(const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb, void *d, const void *bias,
                       int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int *status, const Opts &o,
                       cudaStream_t st) {
  using L = PairLayout<kKind == kMxf8>;
  constexpr int es = kKind == kBf16 ? 2 : (kKind == kTf32 ? 4 : 1);
  CUtensorMap ma, mb, msa, msb;
  int rc = make_map(&ma, a, kKind, M, K, BM);
  if (rc) return rc;
  rc = o.b_fp4 ? make_map_fp4(&mb, b, N, K, 128) : make_map(&mb, b, kKind, N, K, 128);
  if (rc) return rc;
  const int64_t k_chunks = (K * es + kRowBytes - 1) / kRowBytes;
  msa = ma, msb = ma;  // unused by the dense kinds
  if constexpr (kKind == kMxf8) {
    rc = make_sf_map(&msa, sfa, ((M + 255) / 256) * 2 * k_chunks);
    if (rc) return rc;
    rc = make_sf_map(&msb, sfb, ((N + 255) / 256) * 2 * k_chunks);
    if (rc) return rc;
  }
  const bool out_bf16 = out_dtype == MXQ_BF16;
  const bool tma_store = (N * (out_bf16 ? 2 : 4)) % 16 == 0;
  StoreMaps maps;
  for (int r = 0; r < kMaxPeers; ++r) maps.m[r] = ma;  // placeholders
  if (o.scatter_world > 0) {
    // one fp32 slot buffer [scatter_rows, N] per GPU of the group; d is unused
    if (!tma_store || out_bf16 || M % o.scatter_world || (M / o.scatter_world) % 256) return MXQ_ERR_UNSUPPORTED;
    for (int r = 0; r < o.scatter_world; ++r) {
      rc = make_store_map(&maps.m[r], o.scatter_dst[r], false, M / o.scatter_world, N);
      if (rc) return rc;
    }
  } else if (tma_store) {
    rc = make_store_map(&maps.m[0], d, out_bf16, M, N);
    if (rc) return rc;
  }
  Params p;
  p.sfa = sfa, p.sfb = sfb, p.d = d, p.bias = bias, p.status = status;
  p.M = (int)M, p.N = (int)N, p.K = (int)K;
  p.k_chunks = (int)k_chunks;
  p.out_bf16 = out_bf16, p.bias_bf16 = bias_dtype == MXQ_BF16, p.tma_store = tma_store;
  p.a_box_bytes = BM * kRowBytes;
  p.wait_ns = o.wait_ns, p.drop_last_load = 0;
  p.b_fp4 = o.b_fp4 ? 1u : 0u;
  p.fmt_bits = (o.a_e5m2 ? kFormatE5M2 << 7 : 0u) | (o.b_e5m2 ? kFormatE5M2 << 10 : 0u);
  p.tx_less = o.b_fp4 ? 2 * 128 * (kRowBytes / 2) : 0;  // the B boxes of both CTAs
  p.scatter_rows = o.scatter_world > 0 ? (int)(M / o.scatter_world) : 0;
  p.m_rotate = o.scatter_world > 0 ? (int)((((int64_t)o.scatter_rank + 1) % o.scatter_world) * (M / o.scatter_world / 256)) : 0;
  static bool attr_done[64] = {};  // per device: function attributes belong to the device's context
  bool &attr_set = attr_done[current_device() & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(umma_gemm_pair_kernel<kKind>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) !=
        cudaSuccess)
      return MXQ_ERR_LAUNCH;
    attr_set = true;
  }
  const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
  int grid = sm_count();
  if (o.max_ctas > 0 && grid > o.max_ctas) grid = o.max_ctas;
  if (2 * tiles < grid) grid = (int)(2 * tiles);
  grid &= ~1;
  if (grid < 2) return MXQ_ERR_UNSUPPORTED;
  const cudaError_t err = launch_dependent(umma_gemm_pair_kernel<kKind>, grid, kThreads, L::kTotal, st, 0, ma, mb, msa, msb, maps, p);
  if (err != cudaSuccess) {
    cudaGetLastError();  // clear it: the caller falls back to single-CTA tiles
    return MXQ_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

// Transposed kernel for M <= 128 (see umma_gemm_swap_kernel): a = activations [M, K], b = weight [N, K].
template <int kKind, int BNX>
static int launch_swap(const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb, void *d, const void *bias,
                       int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int *status, const Opts &o,
                       cudaStream_t st) {
  using L = SwapLayout<BNX, kKind == kMxf8>;
  constexpr int es = kKind == kBf16 ? 2 : (kKind == kTf32 ? 4 : 1);
  const int64_t k_chunks = (K * es + kRowBytes - 1) / kRowBytes;
  const int x_rows = (int)((M + 7) / 8 * 8) < BNX ? (int)((M + 7) / 8 * 8) : BNX;
  CUtensorMap mw, mx, msw, msx;
  int rc = o.b_fp4 ? make_map_fp4(&mw, b, N, K, BM) : make_map(&mw, b, kKind, N, K, BM);
  if (rc) return rc;
  rc = make_map(&mx, a, kKind, M, K, x_rows);
  if (rc) return rc;
  msw = mw, msx = mw;  // unused by the dense kinds
  if constexpr (kKind == kMxf8) {
    rc = make_sf_map(&msw, sfb, ((N + 255) / 256) * 2 * k_chunks);
    if (rc) return rc;
    rc = make_sf_map(&msx, sfa, ((M + 255) / 256) * 2 * k_chunks);
    if (rc) return rc;
  }
  const int64_t tiles = (N + BM - 1) / BM;
  const int sms = o.max_ctas > 0 && o.max_ctas < sm_count() ? o.max_ctas : sm_count();
  // shares of K: as many CTAs as there are SMs, at least 4 chunks each
  int split = 1;
  while (o.split_k && split < L::kMaxSplit && tiles * split * 2 <= sms && k_chunks / (split * 2) >= 4) split *= 2;
  SwapParams p;
  p.d = d, p.bias = bias, p.status = status, p.M = (int)M, p.N = (int)N, p.k_chunks = (int)k_chunks, p.split = split;
  p.x_box_bytes = x_rows * kRowBytes;
  p.out_bf16 = out_dtype == MXQ_BF16, p.bias_bf16 = bias_dtype == MXQ_BF16, p.wait_ns = o.wait_ns;
  p.w_fp4 = o.b_fp4 ? 1u : 0u;
  p.fmt_bits = (o.b_e5m2 ? kFormatE5M2 << 7 : 0u) | (o.a_e5m2 ? kFormatE5M2 << 10 : 0u);  // operands swapped
  p.tx_less = o.b_fp4 ? BM * (kRowBytes / 2) : 0;
  p.early_w = o.static_b ? 1u : 0u;
  static bool attr_done[64] = {};  // per device: function attributes belong to the device's context
  bool &attr_set = attr_done[current_device() & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(umma_gemm_swap_kernel<kKind, BNX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             L::kTotal) != cudaSuccess)
      return MXQ_ERR_LAUNCH;
    attr_set = true;
  }
  const cudaError_t err = launch_dependent(umma_gemm_swap_kernel<kKind, BNX>, (int)(tiles * split), kThreads,
                                           L::kTotal, st, split, mw, mx, msw, msx, p);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return MXQ_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? MXQ_OK : MXQ_ERR_LAUNCH;
}

template <int kKind>
static int launch_swap_any(const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb, void *d, const void *bias,
                           int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int *status, const Opts &o,
                           cudaStream_t st) {
#define MXQ_SWAP(bnx) \
  return launch_swap<kKind, bnx>(a, b, sfa, sfb, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st)
  if (M <= 16) MXQ_SWAP(16);
  if (M <= 32) MXQ_SWAP(32);
  if (M <= 64) MXQ_SWAP(64);
  MXQ_SWAP(128);
#undef MXQ_SWAP
}

// Tile width: 256 columns when that already gives every SM a tile; narrower tiles for small problems (few rows of
// activations against a large weight are bound by streaming the weight, which needs many SMs pulling at once).
template <int kKind>
static int launch_any(const void *a, const void *b, const uint8_t *sfa, const uint8_t *sfb, void *d, const void *bias,
                      int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int *status, const Opts &o,
                      cudaStream_t st) {
  const int64_t tiles_m = (M + BM - 1) / BM;
  const int sms = sm_count();
  if (o.scatter_world > 0)  // reduce-scatter fused into the epilogue: CTA pairs only
    return launch_pair<kKind>(a, b, sfa, sfb, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
  if (M <= BM && o.transposed && o.test_hook == 0) {
    // few rows: the weight streams through as the 128-row operand (a context that cannot place the clusters falls
    // back to the tiles below)
    const int rc = launch_swap_any<kKind>(a, b, sfa, sfb, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
    if (rc != MXQ_ERR_LAUNCH && rc != MXQ_ERR_UNSUPPORTED) return rc;
  }
  const bool wide = tiles_m * ((N + 255) / 256) * 2 > sms || N <= 64;
  if (M > 128 && N > 128 && ((o.tiles == MXQ_TILES_AUTO && wide) || o.tiles == MXQ_TILES_PAIRS)) {
    // a context that cannot place clusters of two such CTAs falls back to one CTA per tile
    const int rc = launch_pair<kKind>(a, b, sfa, sfb, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
    if (rc != MXQ_ERR_LAUNCH && rc != MXQ_ERR_UNSUPPORTED) return rc;
  }
  if (wide) return launch<kKind, 256>(a, b, sfa, sfb, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
  // The block-scaled MMA takes its B scales from TMEM columns whose offset inside a 128-row chunk must be even
  // (0 or 2), so its narrowest tile is 64 columns; the dense kinds go down to 32.
  if (kKind == kMxf8 || tiles_m * ((N + 63) / 64) * 2 > sms || N <= 32) {
    // one row of tiles that leaves at least half of the SMs idle and a long K: two CTAs per tile, half of K each
    constexpr int es = kKind == kBf16 ? 2 : (kKind == kTf32 ? 4 : 1);
    const int64_t tiles = tiles_m * ((N + 63) / 64), k_chunks = (K * es + kRowBytes - 1) / kRowBytes;
    // (the hand-over costs ~2 us: measured slower below 32 chunks of K, 7 % faster at 32, 26 % at 64)
    if (o.split_k && tiles_m == 1 && 2 * tiles <= sms && k_chunks >= 32) {
      const int rc = launch<kKind, 64, true>(a, b, sfa, sfb, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
      if (rc != MXQ_ERR_LAUNCH && rc != MXQ_ERR_UNSUPPORTED) return rc;
    }
    return launch<kKind, 64>(a, b, sfa, sfb, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
  }
  if constexpr (kKind != kMxf8)
    return launch<kKind, 32>(a, b, sfa, sfb, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
  return MXQ_ERR_UNSUPPORTED;
}

template <int kKind>
static int launch_batched(const void *a, const void *b, void *d, int out_dtype, int64_t M, int64_t N, int64_t K, int *status,
                          const Opts &o, cudaStream_t st, const Batch &bt) {
  // tile width by the output's width: the batch supplies the parallelism
  if (N > 128) return launch<kKind, 256>(a, b, nullptr, nullptr, d, nullptr, out_dtype, MXQ_F32, M, N, K, status, o, st, bt);
  if (N > 32) return launch<kKind, 64>(a, b, nullptr, nullptr, d, nullptr, out_dtype, MXQ_F32, M, N, K, status, o, st, bt);
  return launch<kKind, 32>(a, b, nullptr, nullptr, d, nullptr, out_dtype, MXQ_F32, M, N, K, status, o, st, bt);
}

}  // namespace gemm
}  // namespace mxq

using namespace mxq::gemm;

extern "C" {

int mxq_gemm_options_size(void) { return (int)sizeof(mxq_gemm_options); }

int64_t mxq_mma_scale_bytes(int64_t rows, int64_t k) {
  if (rows < 0 || k < 0) return MXQ_ERR_SHAPE;
  const int64_t row_chunks = ((rows + 255) / 256) * 2;  // padded to whole 256-row tiles
  const int64_t k_chunks = (k + 127) / 128;
  return row_chunks * k_chunks * 512;
}

int mxq_gemm_dense_batched(const void *a, const void *b, void *d, int in_dtype, int out_dtype, int64_t batch, int64_t M,
                           int64_t N, int64_t K, int64_t stride_a, int64_t stride_b, int64_t stride_d, int *status,
                           const mxq_gemm_options *options, void *stream) {
  if (batch == 0 || M == 0 || N == 0) return MXQ_OK;
  if (!a || !b || !d) return MXQ_ERR_NULL;
  Opts o = make_opts(options);
  o.test_hook = 0;
  if (batch < 0 || M < 0 || N < 0 || K <= 0 || batch > INT32_MAX || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return MXQ_ERR_SHAPE;
  if (stride_a < M * K || stride_b < N * K || stride_d < M * N) return MXQ_ERR_SHAPE;
  if (out_dtype != MXQ_F32 && out_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  if (in_dtype != MXQ_F32 && in_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  const int es = in_dtype == MXQ_BF16 ? 2 : 4;
  if ((K * es) % 16 || (stride_a * es) % 16 || (stride_b * es) % 16) return MXQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(d)) & 15u)
    return MXQ_ERR_ALIGN;
  Batch bt;
  bt.count = batch, bt.stride_a = stride_a, bt.stride_b = stride_b, bt.stride_d = stride_d;
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == MXQ_BF16) return launch_batched<kBf16>(a, b, d, out_dtype, M, N, K, status, o, st, bt);
  return launch_batched<kTf32>(a, b, d, out_dtype, M, N, K, status, o, st, bt);
}

int mxq_gemm_dense(const void *a, const void *b, void *d, const void *bias, int in_dtype, int out_dtype, int bias_dtype,
                   int64_t M, int64_t N, int64_t K, int *status, const mxq_gemm_options *options, void *stream) {
  if (M == 0 || N == 0) return MXQ_OK;
  if (!a || !b || !d) return MXQ_ERR_NULL;
  const Opts o = make_opts(options);
  if (M < 0 || N < 0 || K <= 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return MXQ_ERR_SHAPE;
  if (out_dtype != MXQ_F32 && out_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  if (bias && bias_dtype != MXQ_F32 && bias_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(d)) & 15u)
    return MXQ_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == MXQ_BF16) {
    if (K % 8) return MXQ_ERR_SHAPE;  // rows must be 16-byte multiples for the tensor map
    return launch_any<kBf16>(a, b, nullptr, nullptr, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
  }
  if (in_dtype == MXQ_F32) {
    if (K % 4) return MXQ_ERR_SHAPE;
    return launch_any<kTf32>(a, b, nullptr, nullptr, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
  }
  return MXQ_ERR_DTYPE;
}

int mxq_gemm_mxf8(const uint8_t *a_codes, const uint8_t *a_scales, const uint8_t *b_codes, const uint8_t *b_scales,
                  int b_format, void *d, const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K,
                  int *status, const mxq_gemm_options *options, void *stream) {
  Opts o = make_opts(options);
  if (b_format != MXQ_CODES_E4M3 && b_format != MXQ_CODES_E2M1X2 && b_format != MXQ_CODES_E5M2) return MXQ_ERR_FORMAT;
  o.b_fp4 = b_format == MXQ_CODES_E2M1X2;
  o.b_e5m2 = b_format == MXQ_CODES_E5M2;
  return mxq::gemm::gemm_mxf8(a_codes, a_scales, b_codes, b_scales, d, bias, out_dtype, bias_dtype, M, N, K, status, o,
                              (cudaStream_t)stream);
}

}  // extern "C"

namespace mxq {
namespace gemm {

// mxq_gemm_mxf8 with the options resolved
int gemm_mxf8(const uint8_t *a_codes, const uint8_t *a_scales, const uint8_t *b_codes, const uint8_t *b_scales, void *d,
              const void *bias, int out_dtype, int bias_dtype, int64_t M, int64_t N, int64_t K, int *status,
              const Opts &o, cudaStream_t st) {
  if (M == 0 || N == 0) return MXQ_OK;
  if (!a_codes || !a_scales || !b_codes || !b_scales || !d) return MXQ_ERR_NULL;
  if (M < 0 || N < 0 || K <= 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || K % 32) return MXQ_ERR_SHAPE;
  if (o.b_fp4 && (K % 128 || (reinterpret_cast<uintptr_t>(b_codes) & 31u))) return MXQ_ERR_SHAPE;
  if (out_dtype != MXQ_F32 && out_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  if (bias && bias_dtype != MXQ_F32 && bias_dtype != MXQ_BF16) return MXQ_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(a_codes) | reinterpret_cast<uintptr_t>(b_codes) | reinterpret_cast<uintptr_t>(d) |
       reinterpret_cast<uintptr_t>(a_scales) | reinterpret_cast<uintptr_t>(b_scales)) & 15u)
    return MXQ_ERR_ALIGN;
  return launch_any<kMxf8>(a_codes, b_codes, a_scales, b_scales, d, bias, out_dtype, bias_dtype, M, N, K, status, o, st);
}

}  // namespace gemm
}  // namespace mxq
