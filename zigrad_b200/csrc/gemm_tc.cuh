// tcgen05 / TMEM / TMA GEMM for sm_100a.
//
//   C[b] = epilogue(alpha * op(A[b % nA]) * op(B[b % nB]) + beta * C[b])
//
// One CTA computes one 128 x BN tile of C (optionally one K-split of it).
// Roles inside the CTA (8 warps):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A and B
//               k-slabs into a ring of shared-memory stages (128-byte swizzle)
//   warp 1      MMA issuer: the whole warp walks the k loop (so waits and
//               descriptor arithmetic stay warp-uniform; a loop run by a single
//               lane measured 55 cycles per tcgen05.mma issued against 20 this
//               way), one elected lane issues tcgen05.mma with the accumulator
//               in tensor memory; also owns the TMEM allocation
//   warps 2-7   FP32X3 mode only: for every fp32 operand slab write the
//               remainder lo = x - tf32(x) to a second buffer.  The MMA reads
//               only the top 19 bits of an fp32 word (measured: results do not
//               change when the low 13 bits are cleared first), so the fetched
//               slab itself serves as "hi" and Ahi*Bhi + Alo*Bhi + Ahi*Blo
//               recovers fp32-level accuracy.  With a K-major A (hi and lo of A
//               go to tensor memory) and tiles of up to 64 columns, warps 4-7
//               split A, warps 2-3 most of B, each fetching its part of the
//               next slab before it hands the current one over; one mbarrier
//               arrival per warp
//   warps 4-7   epilogue: tcgen05.ld of the accumulator (warp q reads TMEM
//               lanes 32q..32q+31, one row per thread), alpha/beta/bias/ReLU/
//               mask in registers, 128-bit row-contiguous global accesses
//
// Operand layouts.  A row-major matrix whose contiguous dimension is K is a
// "K-major" UMMA operand; one whose contiguous dimension is M (or N) is
// "MN-major".  Both are fetched by TMA into the canonical 128-byte-swizzled
// layouts that the shared-memory matrix descriptors name:
//   K-major  : slab = rows x 128 bytes of K; 8-row groups are 1024 bytes apart
//              (SBO); the k-th MMA inside the slab starts 32 bytes further
//   MN-major : slab = column blocks of 128 bytes of M/N; inside a block the
//              k rows are 128 bytes apart, swizzle-row groups are SBO apart,
//              column blocks BK*128 bytes apart (LBO).  16-bit types use the
//              plain 128-byte swizzle (8-row groups, SBO 1024); 32-bit types
//              must use the 128-byte swizzle with 32-byte atoms (4-row groups,
//              SBO 512) -- the only MN-major layout tcgen05 accepts for tf32
//
// Every wait on an mbarrier is bounded: when the limit is reached the CTA
// raises a flag in global memory, stops issuing work, and still releases its
// tensor memory before it returns.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>

#include "common.cuh"

namespace zg {
namespace tc {

constexpr int kBM = 128;
constexpr int kThreadsTc = 256;
constexpr int kSplitThreads = kThreadsTc - 64;  // warps 2-7
__host__ __device__ constexpr int tc_threads(int /*mode*/) { return kThreadsTc; }
constexpr int kSlabBytes = 128;          // bytes of the contiguous dimension per smem row
constexpr uint32_t kSpinLimit = 1u << 24;  // polls per wait before giving up

enum Mode { kTF32 = 0, kFP32X3 = 1, kBF16 = 2 };

struct Params {
  float* C;             // fp32 output (or nullptr when Cb is used)
  __nv_bfloat16* Cb;    // bf16 output
  const float* bias;    // [n] or nullptr
  float* colsum;        // [n] or nullptr: column sums of the stored values are ADDED here (fp32 atomics)
  const float* mask;    // fp32 mask source with C's layout (when C is fp32)
  const __nv_bfloat16* maskb;
  uint64_t c_batch_stride;  // elements
  uint32_t m, n, k;
  uint32_t ldc;
  uint32_t nA, nB;      // operand batch counts (index wraps)
  uint32_t splits;      // K splits (gridDim.z = batches * splits)
  uint32_t k_per_split; // multiple of BK
  float alpha, beta;
  int epilogue;
  int vec_ok;           // C (and mask, bias) rows allow 16-byte accesses at every 32-column boundary
  int* error_flag;      // set to 1 when a bounded wait ran out
  // Epilogue through the C tensor map (fp32 C with 16-byte-aligned rows): each epilogue warp stages its
  // 32 rows of a 32-column chunk in shared memory (128-byte swizzle) and one lane hands the box to the
  // TMA unit -- 1: plain store (no split-K, beta == 0, epilogue NONE / BIAS / BIAS_RELU, no column
  // sums), 2: reduce-add into C (split-K partial products; C pre-scaled by beta).  Whole 128-byte
  // lines leave the SM instead of 16-byte pieces of 32 different lines per instruction, and boxes that
  // hang over the edge of C are clipped by the unit.  0: register path below.
  int tma_epilogue;
  // Split-K with a fused epilogue: the partial products are added into C (which
  // the launcher scaled by beta first) with the epilogue switched off; every CTA
  // then takes a ticket of its tile, and the one that draws the last applies
  // bias / ReLU / mask / column sums to the finished sums.  One counter per
  // output tile, zero before and after the launch.
  unsigned* tile_tickets;
  int deferred_epilogue;  // what to apply at the end (epilogue is NONE and colsum NULL during accumulation)
  float* deferred_colsum;
};

// ------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while when the phase is
// still open; a look-ahead must not)
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises *failed) when the limit is hit or
// another role already failed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) {
      if (*failed) return false;
      __nanosleep(40);
    }
  }
  *failed = 1;
  return false;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]
template <bool BF16>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (BF16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// One lane of a converged warp (the same lane every time for the full mask)
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
// mbarrier arrives once all previously issued MMAs of this thread are done
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t gets row (lane base + t)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 32 lanes x 32 consecutive 32-bit columns: thread t writes row (lane base + t)
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem desc], tf32: A is read from tensor memory (row m in lane m, one k element per column)
__device__ __forceinline__ void umma_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor (tcgen05): start address, leading-dimension
// byte offset and stride byte offset in 16-byte units, descriptor version 1,
// 128-byte swizzle.
// `layout`: 2 = 128-byte swizzle, 1 = 128-byte swizzle with 32-byte atoms.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // version (Blackwell)
  d |= (uint64_t)layout << 61;
  return d;
}

// The same descriptor as two 32-bit halves: the upper half is a compile-time
// constant of the layout, the lower half is (address >> 4) | (LBO >> 4) << 16,
// so stepping to the next MMA inside a slab is ONE integer add on the lower
// half (the MMA-issuing thread is a single in-order thread; this keeps its
// work per tcgen05.mma at a few instructions).
__host__ __device__ constexpr uint32_t desc_hi32(uint32_t sbo_bytes, uint32_t layout) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (layout << 29);
}
__device__ __forceinline__ uint32_t desc_lo32(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint64_t desc_pack(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor: fp32 accumulate, A/B format (tf32 = 2, bf16 = 1),
// operand majors, N >> 3, M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, bool a_mn_major, bool b_mn_major, int N) {
  return (1u << 4) | ((bf16 ? 1u : 2u) << 7) | ((bf16 ? 1u : 2u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

// shared -> global through a tensor map, tracked by the issuing thread's bulk async-group
__device__ __forceinline__ void tma_store_box(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_box(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until the bulk operations of this thread have READ their shared-memory source (their global writes are
// complete when the grid completes, which is what a dependent kernel waits for)
__device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

template <int MODE>
struct ModeTraits {
  static constexpr bool kBf16 = (MODE == kBF16);
  static constexpr int kElem = kBf16 ? 2 : 4;
  static constexpr int kBK = kSlabBytes / kElem;       // elements of K per stage: 32 (fp32) / 64 (bf16)
  static constexpr int kUmmaK = 32 / kElem;            // K per MMA: 8 (tf32) / 16 (bf16)
  static constexpr int kAtomMN = kSlabBytes / kElem;   // M/N elements per 128-byte column block
  static constexpr int kBufs = (MODE == kFP32X3) ? 2 : 1;  // hi (+ lo) copies of each operand slab
};

// Epilogue of one 32-column chunk of one accumulator row (registers r, raw
// fp32 bits): alpha/beta/bias/ReLU/mask, the store (or the split-K reduction
// into C), and the optional column sums.  `o` = element offset of (row, col0)
// in C; warp-collective when p.colsum is set.
__device__ __forceinline__ void epilogue_chunk(const Params& p, const uint32_t (&r)[32], bool row_ok, uint64_t o, uint32_t col0, int lane) {
  if (!row_ok && !p.colsum) return;
  const bool need_c = p.beta != 0.f, need_m = p.epilogue == ZG_EPI_RELU_MASK;
  const bool has_bias = p.epilogue == ZG_EPI_BIAS || p.epilogue == ZG_EPI_BIAS_RELU;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
  const bool full = p.vec_ok && (col0 + 32 <= p.n);
  if (!row_ok) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = 0.f;
  } else if (full) {
    if (p.splits > 1) {
      // C was pre-scaled by beta on the host side; no fused epilogue with split-K
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p.C + o + j), "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3]) : "memory");
      return;
    }
    if (p.C) {  // fp32 C / mask
      if (need_c) {
        float4 cv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) cv[j] = *reinterpret_cast<const float4*>(p.C + o + 4 * j);
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[4 * j] += p.beta * cv[j].x; v[4 * j + 1] += p.beta * cv[j].y; v[4 * j + 2] += p.beta * cv[j].z; v[4 * j + 3] += p.beta * cv[j].w; }
      }
      if (has_bias) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col0) + j);
          v[4 * j] += bv.x; v[4 * j + 1] += bv.y; v[4 * j + 2] += bv.z; v[4 * j + 3] += bv.w;
        }
        if (p.epilogue == ZG_EPI_BIAS_RELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
        }
      } else if (need_m) {
        float4 mv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) mv[j] = *reinterpret_cast<const float4*>(p.mask + o + 4 * j);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (mv[j].x <= 0.f) v[4 * j] = 0.f;
          if (mv[j].y <= 0.f) v[4 * j + 1] = 0.f;
          if (mv[j].z <= 0.f) v[4 * j + 2] = 0.f;
          if (mv[j].w <= 0.f) v[4 * j + 3] = 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(p.C + o + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {  // bf16 C / mask: 32 values = 64 bytes = 4 x 16-byte accesses
      if (need_c) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 u = *reinterpret_cast<const uint4*>(p.Cb + o + 8 * j);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int t = 0; t < 4; ++t) { const float2 f = __bfloat1622float2(h[t]); v[8 * j + 2 * t] += p.beta * f.x; v[8 * j + 2 * t + 1] += p.beta * f.y; }
        }
      }
      if (has_bias) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col0) + j);
          v[4 * j] += bv.x; v[4 * j + 1] += bv.y; v[4 * j + 2] += bv.z; v[4 * j + 3] += bv.w;
        }
        if (p.epilogue == ZG_EPI_BIAS_RELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
        }
      } else if (need_m) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 u = *reinterpret_cast<const uint4*>(p.maskb + o + 8 * j);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = __bfloat1622float2(h[t]);
            if (f.x <= 0.f) v[8 * j + 2 * t] = 0.f;
            if (f.y <= 0.f) v[8 * j + 2 * t + 1] = 0.f;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int t = 0; t < 4; ++t) h[t] = __floats2bfloat162_rn(v[8 * j + 2 * t], v[8 * j + 2 * t + 1]);
        *reinterpret_cast<uint4*>(p.Cb + o + 8 * j) = u;
      }
    }
  } else {
    // ragged edge or unaligned C: element-wise with a column bound
    const uint32_t ncol = (p.n - col0) < 32u ? (p.n - col0) : 32u;
#pragma unroll
    for (uint32_t j = 0; j < 32; ++j) {
      if (j < ncol) {
        float x = v[j];
        if (p.splits > 1) { atomicAdd(p.C + o + j, x); continue; }
        if (need_c) x += p.beta * (p.C ? p.C[o + j] : __bfloat162float(p.Cb[o + j]));
        if (has_bias) { x += p.bias[col0 + j]; if (p.epilogue == ZG_EPI_BIAS_RELU) x = x > 0.f ? x : 0.f; }
        else if (need_m) { if ((p.mask ? p.mask[o + j] : __bfloat162float(p.maskb[o + j])) <= 0.f) x = 0.f; }
        if (p.C) p.C[o + j] = x;
        else p.Cb[o + j] = __float2bfloat16_rn(x);
        v[j] = x;
      } else {
        v[j] = 0.f;
      }
    }
  }
  if (p.colsum) {
    // Column sums of this warp's 32 x 32 block without shared memory: five
    // exchange rounds, each halving the columns a lane still carries (a lane
    // keeps the half selected by its own bit); lane j ends with column j.
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int j = 0; j < off; ++j) {
        const float send = upper ? v[j] : v[j + off];
        const float keep = upper ? v[j + off] : v[j];
        v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
    if (col0 + lane < p.n) atomicAdd(p.colsum + col0 + lane, v[0]);
  }
}

// One row of an fp32 A slab (32 k values of row `row` of the 128-row tile) from its shared-memory stage.
// K-major: the row is 128 contiguous bytes whose 16-byte chunks sit at position c ^ (row % 8).
// MN-major: the stage holds four column blocks of 32 rows; a block is 32 k-rows of 128 bytes (32
// consecutive rows of A) whose 32-byte atoms sit at position atom ^ (k % 4); the read transposes.
template <bool A_KMAJOR>
__device__ __forceinline__ void load_a_row(const uint8_t* a_stage, int row, float4 (&v)[8]) {
  if constexpr (A_KMAJOR) {
    const uint8_t* rp = a_stage + row * kSlabBytes;
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const float4*>(rp + ((c ^ (row & 7)) << 4));
  } else {
    const uint8_t* bp = a_stage + (row >> 5) * (32 * kSlabBytes) + ((row & 7) << 2);
    const int atom = (row >> 3) & 3;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      v[c].x = *reinterpret_cast<const float*>(bp + (4 * c + 0) * kSlabBytes + ((atom ^ 0) << 5));
      v[c].y = *reinterpret_cast<const float*>(bp + (4 * c + 1) * kSlabBytes + ((atom ^ 1) << 5));
      v[c].z = *reinterpret_cast<const float*>(bp + (4 * c + 2) * kSlabBytes + ((atom ^ 2) << 5));
      v[c].w = *reinterpret_cast<const float*>(bp + (4 * c + 3) * kSlabBytes + ((atom ^ 3) << 5));
    }
  }
}

// ATM: FP32X3 keeps the hi and lo parts of the A operand in TENSOR
// MEMORY (written by the split warps with tcgen05.st, read by the MMA from
// there): shared memory then holds A once per stage (the fetched slab) and no
// MMA reads it, which takes 64 of the 144 KB per 128x64x32 slab off the
// shared-memory data pipe -- the unit that bounds this mode.
template <int BN, int MODE, bool ATM = false>
struct SmemLayout {
  using MT = ModeTraits<MODE>;
  static constexpr int kABytes = kBM * kSlabBytes;   // 16 KB
  static constexpr int kBBytes = BN * kSlabBytes;
  static constexpr int kStageBytes = ATM ? (kABytes + 2 * kBBytes) : (kABytes + kBBytes) * MT::kBufs;
  static constexpr int kEpiBytes = 0;
  static constexpr int kBudget = 220 * 1024;
  static constexpr int kAccCols = BN < 32 ? 32 : BN;
  static constexpr int kATmemCols = 64;              // per stage: 32 columns hi + 32 columns lo
  static constexpr int kStagesSmem = (kBudget - kEpiBytes - 1024) / kStageBytes;
  static constexpr int kStagesTmem = ATM ? (512 - kAccCols) / kATmemCols : 8;
  static constexpr int kStagesRaw = kStagesSmem < kStagesTmem ? kStagesSmem : kStagesTmem;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kTmemNeed = ATM ? kAccCols + kATmemCols * kStages : kAccCols;
  static constexpr int kTmemCols = kTmemNeed <= 32 ? 32 : (kTmemNeed <= 64 ? 64 : (kTmemNeed <= 128 ? 128 : (kTmemNeed <= 256 ? 256 : 512)));
  static constexpr int kTotal = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  // ATM: 16-byte words of a B slab per thread of the two B warps / of the four A warps
  // (BN 128: 8 + 4, BN 64: 6 + 1, BN 32: 4 + 0; 64 * kBWordsB + 128 * kBWordsA = BN * 8)
  static constexpr int kBWordsA = BN >= 128 ? 4 : (BN >= 64 ? 1 : 0);
  static constexpr int kBWordsB = (BN * 8 - 128 * kBWordsA) / 64;
};

template <int BN, bool A_KMAJOR, bool B_KMAJOR, int MODE, bool ATM = false>
__global__ void __launch_bounds__(tc_threads(MODE), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
               const Params p) {
  static_assert(!ATM || MODE == kFP32X3, "A through tensor memory: FP32X3 only");
  using MT = ModeTraits<MODE>;
  using SL = SmemLayout<BN, MODE, ATM>;
  constexpr int S = SL::kStages;
  constexpr bool X3 = (MODE == kFP32X3);
  // an A operand in tensor memory is K-major by construction (row m in lane m, one k element per column)
  constexpr uint32_t kIdesc = make_idesc(MT::kBf16, ATM ? false : !A_KMAJOR, !B_KMAJOR, BN);
  constexpr uint32_t kTmemCols = SL::kTmemCols;

  extern __shared__ uint8_t smem_raw[];
  // stages need 1024-byte alignment (swizzle atoms)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * SL::kStageBytes + SL::kEpiBytes);
  uint64_t* full = bars;            // [S] TMA bytes landed
  uint64_t* ready = bars + S;       // [S] (X3) split done
  uint64_t* empty = bars + 2 * S;   // [S] MMAs that read the stage retired
  uint64_t* accum = bars + 3 * S;   // accumulator complete
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tile_n = blockIdx.x, tile_m = blockIdx.y;
  const uint32_t batch = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
  const uint32_t k_begin = split * p.k_per_split;
  uint32_t k_end = k_begin + p.k_per_split;
  if (k_end > p.k) k_end = p.k;
  const int KT = (k_end > k_begin) ? (int)((k_end - k_begin + MT::kBK - 1) / MT::kBK) : 0;

  if (threadIdx.x == 0) {
    failed = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&ready[s], kSplitThreads / 32);  // one arrival per split warp
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (p.tma_epilogue) prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base_slot;
  pdl_sync();  // everything above overlaps the previous kernel's tail

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      const int za = (int)(batch % p.nA), zb = (int)(batch % p.nB);
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % S;
        if (kt >= S && !mbar_wait(&empty[s], ((kt / S) & 1) ^ 1, &failed)) break;
        uint8_t* st = stage_base + s * SL::kStageBytes;
        uint8_t* a_dst = st;
        uint8_t* b_dst = st + (ATM ? SL::kABytes : SL::kABytes * MT::kBufs);
        mbar_expect_tx(&full[s], SL::kABytes + SL::kBBytes);
        const int k0 = (int)k_begin + kt * MT::kBK;
        if (A_KMAJOR) {
          tma_load_3d(a_dst, &tmA, &full[s], k0, (int)(tile_m * kBM), za);
        } else {
#pragma unroll
          for (int j = 0; j < kBM / MT::kAtomMN; ++j)
            tma_load_3d(a_dst + j * MT::kBK * kSlabBytes, &tmA, &full[s], (int)(tile_m * kBM) + j * MT::kAtomMN, k0, za);
        }
        if (B_KMAJOR) {
          tma_load_3d(b_dst, &tmB, &full[s], k0, (int)(tile_n * BN), zb);
        } else {
#pragma unroll
          for (int j = 0; j < BN / MT::kAtomMN; ++j)
            tma_load_3d(b_dst + j * MT::kBK * kSlabBytes, &tmB, &full[s], (int)(tile_n * BN) + j * MT::kAtomMN, k0, zb);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // The whole warp walks the loop (waits and descriptor arithmetic stay
    // warp-uniform); one elected lane issues the MMAs and their commit.
    // The barrier of the next slab is polled once before this slab's MMAs go
    // out, so that in steady state no wait sits between two slabs.
    {
      bool have = false;
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % S;
        if (!have) {
          const bool got = mbar_wait(X3 ? &ready[s] : &full[s], (kt / S) & 1, &failed);
          if (!__all_sync(0xffffffffu, got)) break;
        }
        bool next_seen = false;  // consumed after the MMAs of this slab are out
        if (kt + 1 < KT) {
          const int s1 = (kt + 1) % S;
          next_seen = mbar_test(X3 ? &ready[s1] : &full[s1], ((kt + 1) / S) & 1);
        }
        tc_fence_after();
        uint8_t* st = stage_base + s * SL::kStageBytes;
        const uint32_t a_hi = smem_u32(st), a_lo = a_hi + SL::kABytes;
        const uint32_t b_hi = a_hi + (ATM ? SL::kABytes : SL::kABytes * MT::kBufs), b_lo = b_hi + SL::kBBytes;
        const uint32_t a_tm = tmem_d + SL::kAccCols + (uint32_t)s * SL::kATmemCols;  // ATM: hi at +0, lo at +32
        // K-major: the next MMA starts 32 bytes further inside the 128-byte rows;
        // MN-major: kUmmaK k-rows (128 bytes each) further.  MN-major 32-bit
        // operands use the 32-byte-atom swizzle with 4-row groups.
        constexpr uint32_t a_step = (A_KMAJOR ? 32u : (uint32_t)(MT::kUmmaK * kSlabBytes)) >> 4;
        constexpr uint32_t b_step = (B_KMAJOR ? 32u : (uint32_t)(MT::kUmmaK * kSlabBytes)) >> 4;
        constexpr uint32_t a_lbo = A_KMAJOR ? 16u : (uint32_t)(MT::kBK * kSlabBytes);
        constexpr uint32_t b_lbo = B_KMAJOR ? 16u : (uint32_t)(MT::kBK * kSlabBytes);
        constexpr uint32_t a_lay = (!A_KMAJOR && !MT::kBf16) ? 1u : 2u, b_lay = (!B_KMAJOR && !MT::kBf16) ? 1u : 2u;
        constexpr uint32_t a_h32 = desc_hi32(a_lay == 1u ? 512u : 1024u, a_lay), b_h32 = desc_hi32(b_lay == 1u ? 512u : 1024u, b_lay);
        const uint32_t da0 = desc_lo32(a_hi, a_lbo), dal0 = desc_lo32(a_lo, a_lbo);
        const uint32_t db0 = desc_lo32(b_hi, b_lbo), dbl0 = desc_lo32(b_lo, b_lbo);
        if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < MT::kBK / MT::kUmmaK; ++kk) {
          const uint64_t db = desc_pack(db0 + kk * b_step, b_h32);
          const uint32_t acc = (kt > 0 || kk > 0) ? 1u : 0u;
          if constexpr (ATM) {
            const uint64_t dbl = desc_pack(dbl0 + kk * b_step, b_h32);
            const uint32_t ta_hi = a_tm + kk * MT::kUmmaK, ta_lo = ta_hi + 32;
            umma_tmem_a(tmem_d, ta_lo, db, kIdesc, acc);   // Alo * Bhi
            umma_tmem_a(tmem_d, ta_hi, dbl, kIdesc, 1u);   // Ahi * Blo
            umma_tmem_a(tmem_d, ta_hi, db, kIdesc, 1u);    // Ahi * Bhi
          } else if constexpr (X3) {
            const uint64_t da = desc_pack(da0 + kk * a_step, a_h32);
            const uint64_t dal = desc_pack(dal0 + kk * a_step, a_h32);
            const uint64_t dbl = desc_pack(dbl0 + kk * b_step, b_h32);
            umma<false>(tmem_d, dal, db, kIdesc, acc);   // Alo * Bhi
            umma<false>(tmem_d, da, dbl, kIdesc, 1u);    // Ahi * Blo
            umma<false>(tmem_d, da, db, kIdesc, 1u);     // Ahi * Bhi
          } else {
            const uint64_t da = desc_pack(da0 + kk * a_step, a_h32);
            umma<MT::kBf16>(tmem_d, da, db, kIdesc, acc);
          }
        }
        umma_commit(&empty[s]);  // stage reusable once these MMAs have read it
        }
        have = __all_sync(0xffffffffu, next_seen);
      }
      if (elect_one()) umma_commit(accum);
    }
  } else if (X3) {
    // ------------------------------------------- hi/lo split (warps 2..7)
    const int t = threadIdx.x - 64;
    const bool a_warp = warp >= 4;  // ATM: the four warps that cover the TMEM lane quadrants (warp % 4)
    constexpr int NT = kSplitThreads;
    // Narrow tiles run the pipelined role loops below; with BN = 128 the MMAs' operand reads load the
    // shared-memory pipe so heavily that the plain lock-step split measured faster.
    constexpr bool PIPE = ATM && BN <= 64;
    if (PIPE && a_warp) {
      // Four warps (TMEM lane quadrant = warp % 4), thread = row of the A slab.  The row's eight
      // 16-byte chunks sit at chunk position c ^ (row % 8) (128-byte swizzle); hi = the fetched
      // word itself, lo = x - tf32(x); both go to tensor memory.  The row of the NEXT slab is
      // fetched while the stores of this one drain, so a warp's chain per slab is
      // split -> store -> (load next) -> wait -> arrive.
      const int row = (warp & 3) * 32 + lane;
      const uint32_t ta0 = tmem_d + SL::kAccCols + ((uint32_t)((warp & 3) * 32) << 16);
      float4 v[8];
      bool have = false;
      auto load_row = [&](int stage) { load_a_row<A_KMAJOR>(stage_base + stage * SL::kStageBytes, row, v); };
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % S;
        if (!have) {
          const bool got = mbar_wait(&full[s], (kt / S) & 1, &failed);
          if (!__all_sync(0xffffffffu, got)) break;
          load_row(s);
        }
        uint32_t hi[32], lo[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float x[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t h = __float_as_uint(x[e]) & 0xFFFFE000u;
            hi[4 * c + e] = __float_as_uint(x[e]);
            lo[4 * c + e] = __float_as_uint(x[e] - __uint_as_float(h));
          }
        }
        const uint32_t ta = ta0 + (uint32_t)s * SL::kATmemCols;
        tmem_st32(ta, hi);
        tmem_st32(ta + 32, lo);
        if constexpr (SL::kBWordsA > 0) {
          // this warp's share of the B split (the words after those of the two B warps)
          float4* bh = reinterpret_cast<float4*>(stage_base + s * SL::kStageBytes + SL::kABytes);
          float4* bl = bh + SL::kBBytes / 16;
#pragma unroll
          for (int j = 0; j < SL::kBWordsA; ++j) {
            const int i = 64 * SL::kBWordsB + (threadIdx.x - 128) + 128 * j;
            const float4 b = bh[i];
            float4 l;
            l.x = b.x - __uint_as_float(__float_as_uint(b.x) & 0xFFFFE000u);
            l.y = b.y - __uint_as_float(__float_as_uint(b.y) & 0xFFFFE000u);
            l.z = b.z - __uint_as_float(__float_as_uint(b.z) & 0xFFFFE000u);
            l.w = b.w - __uint_as_float(__float_as_uint(b.w) & 0xFFFFE000u);
            bl[i] = l;
          }
        }
        have = false;
        if (kt + 1 < KT) {
          const int s1 = (kt + 1) % S;
          have = __all_sync(0xffffffffu, mbar_test(&full[s1], ((kt + 1) / S) & 1));
          if (have) load_row(s1);
        }
        if constexpr (SL::kBWordsA > 0) fence_async_smem();
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ready[s]);
      }
    } else if (PIPE) {
      // The two other warps split B: lo = x - tf32(x) into the second B buffer of the stage.
      // Like the A warps they fetch the next slab's part before they hand this one over.
      constexpr int NB = SL::kBWordsB;  // 16-byte words per thread and slab
      float4 v[NB];
      bool have = false;
      auto b_hi_of = [&](int stage) { return reinterpret_cast<float4*>(stage_base + stage * SL::kStageBytes + SL::kABytes); };
      auto load_b = [&](int stage) {
        const float4* src = b_hi_of(stage);
#pragma unroll
        for (int j = 0; j < NB; ++j) v[j] = src[t + 64 * j];
      };
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % S;
        if (!have) {
          const bool got = mbar_wait(&full[s], (kt / S) & 1, &failed);
          if (!__all_sync(0xffffffffu, got)) break;
          load_b(s);
        }
        float4* dst = b_hi_of(s) + SL::kBBytes / 16;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          float4 l;
          l.x = v[j].x - __uint_as_float(__float_as_uint(v[j].x) & 0xFFFFE000u);
          l.y = v[j].y - __uint_as_float(__float_as_uint(v[j].y) & 0xFFFFE000u);
          l.z = v[j].z - __uint_as_float(__float_as_uint(v[j].z) & 0xFFFFE000u);
          l.w = v[j].w - __uint_as_float(__float_as_uint(v[j].w) & 0xFFFFE000u);
          dst[t + 64 * j] = l;
        }
        have = false;
        if (kt + 1 < KT) {
          const int s1 = (kt + 1) % S;
          have = __all_sync(0xffffffffu, mbar_test(&full[s1], ((kt + 1) / S) & 1));
          if (have) load_b(s1);
        }
        fence_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&ready[s]);
      }
    } else
    for (int kt = 0; kt < KT; ++kt) {
      const int s = kt % S;
      if (!mbar_wait(&full[s], (kt / S) & 1, &failed)) break;
      uint8_t* st = stage_base + s * SL::kStageBytes;
      float4* a_hi = reinterpret_cast<float4*>(st);
      float4* a_lo = reinterpret_cast<float4*>(st + SL::kABytes);
      float4* b_hi = reinterpret_cast<float4*>(st + (ATM ? SL::kABytes : SL::kABytes * 2));
      float4* b_lo = b_hi + SL::kBBytes / 16;
      if constexpr (ATM) {
        if (a_warp) {  // thread = row of the A slab, as in the pipelined loop above
          const int row = (warp & 3) * 32 + lane;
          float4 va[8];
          load_a_row<A_KMAJOR>(st, row, va);
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float x[4] = {va[c].x, va[c].y, va[c].z, va[c].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const uint32_t h = __float_as_uint(x[e]) & 0xFFFFE000u;
              hi[4 * c + e] = __float_as_uint(x[e]);
              lo[4 * c + e] = __float_as_uint(x[e] - __uint_as_float(h));
            }
          }
          const uint32_t ta = tmem_d + SL::kAccCols + (uint32_t)s * SL::kATmemCols + ((uint32_t)((warp & 3) * 32) << 16);
          tmem_st32(ta, hi);
          tmem_st32(ta + 32, lo);
          tmem_st_wait();
          tc_fence_before();
        }
      }
      // the split is position independent, so the swizzle does not matter here
#pragma unroll 4
      for (int i = t; i < (ATM ? 0 : SL::kABytes / 16); i += NT) {
        const float4 v = a_hi[i];
        float4 h, l;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u); l.x = v.x - h.x;
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u); l.y = v.y - h.y;
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u); l.z = v.z - h.z;
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u); l.w = v.w - h.w;
        a_lo[i] = l;
      }
#pragma unroll 4
      for (int i = t; i < SL::kBBytes / 16; i += NT) {
        const float4 v = b_hi[i];
        float4 h, l;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u); l.x = v.x - h.x;
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u); l.y = v.y - h.y;
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u); l.z = v.z - h.z;
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u); l.w = v.w - h.w;
        b_lo[i] = l;
      }
      fence_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&ready[s]);
    }
  }

  // ---------------------------------------------------------------- epilogue
  // Each epilogue thread owns one accumulator row: 32 consecutive columns per
  // tcgen05.ld, i.e. one full 128-byte line of C, read (beta / mask) and
  // written with 128-bit accesses straight from registers.
  if (warp >= 4 && warp < 8) {
    const int q = warp - 4;  // TMEM lane quadrant
    const bool have_acc = (KT > 0) && mbar_wait(accum, 0, &failed);
    tc_fence_after();
    const uint32_t row = tile_m * kBM + q * 32 + lane;
    const uint64_t c_off = (uint64_t)batch * p.c_batch_stride + (uint64_t)row * p.ldc;
    const bool row_ok = row < p.m;
    if (p.tma_epilogue && (KT == 0 || have_acc)) {
      // The stage ring is idle by now (every fetched slab was consumed by MMAs that have completed):
      // its first bytes stage the output, 4 KB per warp and chunk, 1024-byte aligned for the swizzle.
      uint8_t* stg = stage_base + q * (BN / 32) * 4096;
      const bool has_bias = p.epilogue == ZG_EPI_BIAS || p.epilogue == ZG_EPI_BIAS_RELU;
      int chunks = 0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const uint32_t col0 = tile_n * BN + c * 32;
        if (col0 >= p.n) break;  // uniform across the warp
        uint32_t r[32];
        if (KT > 0) {
          tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
        if (has_bias) {
          if (col0 + 32 <= p.n) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col0) + j);
              v[4 * j] += bv.x; v[4 * j + 1] += bv.y; v[4 * j + 2] += bv.z; v[4 * j + 3] += bv.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.n) v[j] += __ldg(p.bias + col0 + j);
          }
          if (p.epilogue == ZG_EPI_BIAS_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
          }
        }
        uint8_t* rowp = stg + c * 4096 + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        ++chunks;
      }
      fence_async_smem();  // generic-proxy writes -> visible to the TMA unit
      __syncwarp();
      if (lane == 0 && tile_m * kBM + q * 32 < p.m) {
        for (int c = 0; c < chunks; ++c) {
          const int x = (int)(tile_n * BN) + c * 32, y = (int)(tile_m * kBM) + q * 32;
          if (p.tma_epilogue == 2) tma_reduce_add_box(&tmC, stg + c * 4096, x, y, (int)batch);
          else tma_store_box(&tmC, stg + c * 4096, x, y, (int)batch);
        }
        bulk_commit_group();
        bulk_wait_group_read();
      }
      __syncwarp();
    } else if (KT == 0 || have_acc) {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const uint32_t col0 = tile_n * BN + c * 32;
        if (col0 >= p.n) break;  // uniform across the warp
        uint32_t r[32];
        if (KT > 0) {
          tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);  // warp-collective
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        epilogue_chunk(p, r, row_ok, c_off + col0, col0, lane);
      }
      if (p.tile_tickets) {
        // ---- deferred epilogue of a split-K tile (warps 4-7 only: named barrier 1)
        __shared__ int is_last;
        __threadfence();  // this thread's reductions into C are visible device-wide
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 128) {
          unsigned* ticket = p.tile_tickets + ((size_t)batch * gridDim.y + tile_m) * gridDim.x + tile_n;
          const unsigned t = atomicAdd(ticket, 1u);
          is_last = (t == p.splits - 1) ? 1 : 0;
          if (is_last) *ticket = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (is_last) {
          __threadfence();
          Params q = p;
          q.alpha = 1.f; q.beta = 0.f; q.splits = 1; q.epilogue = p.deferred_epilogue; q.colsum = p.deferred_colsum;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const uint32_t col0 = tile_n * BN + c * 32;
            if (col0 >= p.n) break;
            uint32_t r[32];
            const uint64_t o = c_off + col0;
            if (row_ok && p.vec_ok && col0 + 32 <= p.n) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(p.C + o) + j);
                r[4 * j] = __float_as_uint(v.x); r[4 * j + 1] = __float_as_uint(v.y);
                r[4 * j + 2] = __float_as_uint(v.z); r[4 * j + 3] = __float_as_uint(v.w);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = (row_ok && col0 + j < p.n) ? __float_as_uint(__ldcg(p.C + o + j)) : 0u;
            }
            epilogue_chunk(q, r, row_ok, o, col0, lane);
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_d, kTmemCols);
  }
  if (threadIdx.x == 0 && failed && p.error_flag) *p.error_flag = 1;
}

}  // namespace tc
}  // namespace zg
