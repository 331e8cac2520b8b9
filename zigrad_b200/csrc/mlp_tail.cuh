// The middle of an MLP training step in ONE kernel, for the layer widths of the
// MNIST model (.. -> 128 -> 64 -> C, C <= 16; examples/mnist/src/model.zig:34-55):
//
//   act1    = relu(act0 W1^T + b1)                     [rows, 64]     Linear + ReLU
//   logits  = act1 W2^T + b2                           [rows, C]      Linear
//   loss, dlogits = softmax cross-entropy fwd + bwd    (src/nn/loss.zig:130-215)
//   db2    += column sums of dlogits                                  (src/ndtensor.zig:783-788)
//   dact1   = (dlogits W2) where act1 > 0, db1 += column sums         (BmmAccBwd dX + relu_inplace_bwd,
//   dact0   = (dact1  W1) where act0 > 0, db0 += column sums           src/ndtensor.zig:1092-1136)
//
// As separate launches these are six dependent kernels whose operands (act0:
// 64 KB per 128 rows, W1: 32 KB, W2: 2.5 KB) would fit on one SM: each costs a
// launch, a first round trip to memory and a drain.  Here a CTA owns 128 rows and
// walks the whole chain with its operands on chip:
//
//   * act0 tile and W1 arrive by TMA (128-byte swizzle); W1 twice, once K-major
//     (B of act0 W1^T) and once N-major (B of dact1 W1).  Weights, biases and
//     labels are fetched -- and W1 split -- BEFORE the dependency wait when the
//     caller vouches that the preceding kernel does not write them;
//   * the two 128 x 64 x 128 products run on the tensor cores as 3xTF32
//     (Alo Bhi + Ahi Blo + Ahi Bhi): the A operand (act0, later dact1) is split
//     into hi/lo by the threads that own the row and goes to TENSOR MEMORY
//     (tcgen05.st), W1's lo parts are formed in shared memory by helper warps,
//     accumulators live in tensor memory;
//   * the per-row work between the products is latency-bound (a chain of a few
//     thousand dependent instructions per row), so FOUR threads share a row:
//     thread (row, q) owns columns 16q..16q+15 of the 64-wide tensors, k-slab q of
//     act0 and column block q of dact0.  The full act1 row is exchanged through the
//     shared-memory tile that also feeds its TMA store; thread q forms the logits
//     of classes q, q+4, .. in FFMA against W2 in shared memory (broadcast reads);
//     the C logits are exchanged through the logits staging tile; every thread takes
//     the row's maximum and sum of exponentials itself and then the loss terms and
//     dlogits of ITS classes, which meet in the dlogits staging tile;
//   * every output tile leaves through shared memory: act1, dact1 and dact0 as TMA
//     stores of swizzled [128 x 32] slabs (dact0 overwrites the act0 slab it was
//     masked with), logits / dlogits as a copy by the row threads while the second
//     product runs;
//   * bias gradients: the helper warps add the staged tiles up column by column
//     in row order and issue one fp32 atomic per column and CTA; the loss leaves as
//     one partial per CTA with a ticket drawn while the second product runs, and the
//     CTA that drew the last ticket folds the partials in a fixed order at its end.
//
// Roles (20 warps): 0-15 own the rows (warp w: TMEM lanes 32(w%4).., quarter w/4),
// 16-18 helpers (staging, W1 split, column sums, copy-out), 19 issues the TMA
// loads and the MMAs and owns the tensor-memory allocation.  Every mbarrier wait
// is bounded and reports through the time-out flag; after a failed wait a thread
// skips its work but still takes part in every CTA barrier, so the CTA always
// reaches its TMEM release.
#pragma once

#include "gemm_tc.cuh"

namespace zg {
namespace tail {

using namespace tc;

constexpr int kH1 = 128;       // width of act0
constexpr int kH2 = 64;        // width of act1
constexpr int kRows = 128;     // rows per CTA
constexpr int kRowThreads = 512;
constexpr int kHelperThreads = 96;
constexpr int kThreads = kRowThreads + kHelperThreads + 32;   // 640
constexpr int kCMax = 16;

// shared memory (byte offsets from a 1024-byte aligned base)
constexpr int kOffA = 0;                       // act0 tile: 4 k-slabs of [128 rows x 128 B]; later dact0
constexpr int kOffW1kHi = 65536;               // W1 K-major: 4 k-slabs of [64 rows x 128 B]
constexpr int kOffW1kLo = kOffW1kHi + 32768;
constexpr int kOffW1nHi = kOffW1kLo + 32768;   // W1 N-major: 2 k-stages of 4 column blocks of [32 k-rows x 128 B]
constexpr int kOffW1nLo = kOffW1nHi + 32768;
constexpr int kOffW2 = kOffW1nLo + 32768;      // [kCMax][64] floats
constexpr int kOffB1 = kOffW2 + kCMax * kH2 * 4;
constexpr int kOffB2 = kOffB1 + kH2 * 4;
constexpr int kOffRed = kOffB2 + kCMax * 4;    // [32] floats
constexpr int kOffBars = kOffRed + 128;        // 13 mbarriers
constexpr int kOffLg = kOffBars + 16 * 8;      // [128][ld_out <= 16] logits on their way out
constexpr int kOffDl = kOffLg + kRows * kCMax * 4;   // the same for dlogits
constexpr int kOffT = kOffDl + kRows * kCMax * 4;    // [128][C] one-hot label rows
constexpr int kSmemBytes = kOffT + kRows * kCMax * 4 + 1024 /*alignment slack*/;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
// After the first product W1's K-major copy is dead: its hi half stages act1, its lo half dact1 (two
// k-slabs of [128 rows x 128 B] each, the layout of the TMA store); dact0 overwrites the act0 tile slab by slab.
constexpr int kOffAct1 = kOffW1kHi, kOffDact1 = kOffW1kLo;

// tensor memory (columns): the two accumulators and the hi/lo parts of the A operand (64 columns per 32-deep k-stage)
constexpr uint32_t kTmAcc1 = 0, kTmAcc2 = 64, kTmA = 192, kTmCols = 512;

struct Params {
  const float* W2;        // [C, 64]
  const float* b1;        // [64]
  const float* b2;        // [C]
  const void* labels;     // fp32 [rows, C] one-hot / probability rows, or u64 [rows] class indices
  int label_index;
  float* logits;          // [rows, ld_out]
  float* dlogits;         // [rows, ld_out]
  float* db2;             // [C]   column sums are ADDED (the gradient buffer is zero at the start of a step)
  float* db1;             // [64]
  float* db0;             // [128]
  float* loss_out;        // one scalar, overwritten
  float* loss_partial;    // workspace: one float per CTA
  unsigned* counter;      // workspace: ticket, zero before and after
  uint32_t rows, C, ld_out;
  float divisor, inv_divisor;
  int exact_inv;
  int early_weights;      // weights, biases and labels may be fetched before the dependency wait
  int* error_flag;
};

constexpr float kLogPMin = -16.11809565f;     // logf(1e-7f): the reference clamps p to [1e-7, 1 - 1e-7] before the log
constexpr float kLogPMax = -1.1920929e-07f;   // logf(1.0f - 1e-7f)

// shared -> global through a tensor map (rows beyond the tensor's extent are clipped), tracked by the
// issuing thread's bulk async-group
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until the bulk stores of this thread have READ their shared-memory source (their global writes are complete
// when the grid completes, which is what a dependent kernel waits for)
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// named CTA barriers: arrive does not block, sync does; `n` = threads taking part
__device__ __forceinline__ void bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// 32 lanes x 16 consecutive 32-bit columns of tensor memory
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ float lo_part(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

// Address of 16-byte chunk `c` (0..7) of row `row` inside a K-major k-slab ([128 rows x 128 B], chunk c at position c ^ (row % 8))
__device__ __forceinline__ float4* slab_chunk(uint8_t* slab, int row, int c) {
  return reinterpret_cast<float4*>(slab + row * kSlabBytes + ((c ^ (row & 7)) << 4));
}

// Column sums of a staged [128 rows x 32 columns] slab in row order: lane = column.  Conflict-free: for a
// fixed row the 32 lanes read the eight chunks at their swizzled positions, i.e. all 32 banks.
__device__ __forceinline__ float slab_column_sum(uint8_t* slab, int lane) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  const int c = lane >> 2, e = lane & 3;
#pragma unroll 4
  for (int r = 0; r < kRows; r += 4) {
    s0 += reinterpret_cast<const float*>(slab_chunk(slab, r, c))[e];
    s1 += reinterpret_cast<const float*>(slab_chunk(slab, r + 1, c))[e];
    s2 += reinterpret_cast<const float*>(slab_chunk(slab, r + 2, c))[e];
    s3 += reinterpret_cast<const float*>(slab_chunk(slab, r + 3, c))[e];
  }
  return (s0 + s1) + (s2 + s3);
}

template <int CP>  // C rounded up to 4, 8, 12 or 16
__global__ void __launch_bounds__(kThreads, 1)
mlp_tail_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW1k, const __grid_constant__ CUtensorMap tmW1n,
                const __grid_constant__ CUtensorMap tmAct1, const __grid_constant__ CUtensorMap tmDact1,
                const __grid_constant__ CUtensorMap tmDact0, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* W2s = reinterpret_cast<float*>(smem + kOffW2);
  float* b1s = reinterpret_cast<float*>(smem + kOffB1);
  float* b2s = reinterpret_cast<float*>(smem + kOffB2);
  float* red = reinterpret_cast<float*>(smem + kOffRed);
  float* lgs = reinterpret_cast<float*>(smem + kOffLg);
  float* dls = reinterpret_cast<float*>(smem + kOffDl);
  float* Ts = reinterpret_cast<float*>(smem + kOffT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* barA = bars;            // [4] act0 k-slab landed
  uint64_t* barW1k = bars + 4;      // W1 (K-major copy) landed
  uint64_t* barW1n = bars + 5;      // W1 (N-major copy) landed
  uint64_t* barW1kLo = bars + 6;    // its lo part written (3 helper warps)
  uint64_t* barW1nLo = bars + 7;
  uint64_t* barSplit1 = bars + 8;   // act0 hi/lo in tensor memory (16 row warps)
  uint64_t* barAcc1 = bars + 9;     // first product complete
  uint64_t* barSplit2 = bars + 10;  // dact1 hi/lo in tensor memory
  uint64_t* barAcc2 = bars + 11;    // second product complete
  uint64_t* barStaged = bars + 12;  // W2, biases and labels in shared memory (3 helper warps)
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;
  __shared__ int is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row0 = blockIdx.x * kRows;
  const uint32_t nrows = (p.rows - row0) < (uint32_t)kRows ? (p.rows - row0) : (uint32_t)kRows;
  const int C = (int)p.C;
  const int ld = (int)p.ld_out;
  constexpr int kIssuer = kThreads / 32 - 1;                   // warp 19
  constexpr int kHelper0 = kRowThreads / 32;                   // warps 16..18
  // named barriers: 1 = the row threads among themselves; 2 = act1 / dact1 / dlogits staged (rows arrive, helpers and
  // the issuer wait); 3 = dact0 staged (likewise)
  constexpr int kBar2 = kThreads, kBar3 = kThreads;

  if (threadIdx.x == 0) {
    failed = 0;
    for (int s = 0; s < 4; ++s) mbar_init(&barA[s], 1);
    mbar_init(barW1k, 1);
    mbar_init(barW1n, 1);
    mbar_init(barW1kLo, kHelperThreads / 32);
    mbar_init(barW1nLo, kHelperThreads / 32);
    mbar_init(barSplit1, kRowThreads / 32);
    mbar_init(barAcc1, 1);
    mbar_init(barSplit2, kRowThreads / 32);
    mbar_init(barAcc2, 1);
    mbar_init(barStaged, kHelperThreads / 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmW1k);
    prefetch_tmap(&tmW1n);
    prefetch_tmap(&tmAct1);
    prefetch_tmap(&tmDact1);
    prefetch_tmap(&tmDact0);
  }
  if (warp == kIssuer) {
    tmem_alloc(&tmem_base_slot, kTmCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;

  if (warp == kIssuer) {
    // =========================================================== TMA loads and MMAs
    // The weights are fetched before the dependency wait when the caller vouches that the kernel
    // launched just before this one does not write them (in a training step that kernel is the
    // preceding layer's forward GEMM; the optimizer ran a whole step earlier).
    auto fetch_w1 = [&]() {
      if (lane == 0) {
        mbar_expect_tx(barW1k, 32768);
        for (int s = 0; s < 4; ++s) tma_load_3d(smem + kOffW1kHi + s * 8192, &tmW1k, barW1k, s * 32, 0, 0);
        mbar_expect_tx(barW1n, 32768);
        for (int ks = 0; ks < 2; ++ks)
          for (int j = 0; j < 4; ++j) tma_load_3d(smem + kOffW1nHi + ks * 16384 + j * 4096, &tmW1n, barW1n, j * 32, ks * 32, 0);
      }
    };
    if (p.early_weights) fetch_w1();
    pdl_sync();  // act0 is the output of the preceding kernel
    if (!p.early_weights) fetch_w1();
    if (lane == 0) {
      for (int s = 0; s < 4; ++s) {
        mbar_expect_tx(&barA[s], 16384);
        tma_load_3d(smem + kOffA + s * 16384, &tmA, &barA[s], s * 32, (int)row0, 0);
      }
    }
    __syncwarp();
    constexpr uint32_t kIdesc1 = make_idesc(false, false, false, kH2);   // A tensor memory, B K-major, N = 64
    constexpr uint32_t kIdesc2 = make_idesc(false, false, true, kH1);    // A tensor memory, B N-major, N = 128
    constexpr uint32_t kHi1 = desc_hi32(1024u, 2u), kHi2 = desc_hi32(512u, 1u);
    bool ok = mbar_wait(barSplit1, 0, &failed) && mbar_wait(barW1kLo, 0, &failed);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok && elect_one()) {
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint32_t bh = desc_lo32(smem_u32(smem + kOffW1kHi + s * 8192), 16u), bl = desc_lo32(smem_u32(smem + kOffW1kLo + s * 8192), 16u);
        const uint32_t ta = tmem + kTmA + (uint32_t)s * 64;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t db = desc_pack(bh + kk * 2, kHi1), dbl = desc_pack(bl + kk * 2, kHi1);
          const uint32_t ta_hi = ta + kk * 8, ta_lo = ta_hi + 32;
          umma_tmem_a(tmem + kTmAcc1, ta_lo, db, kIdesc1, (s > 0 || kk > 0) ? 1u : 0u);  // Alo * Bhi
          umma_tmem_a(tmem + kTmAcc1, ta_hi, dbl, kIdesc1, 1u);                            // Ahi * Blo
          umma_tmem_a(tmem + kTmAcc1, ta_hi, db, kIdesc1, 1u);                             // Ahi * Bhi
        }
      }
      umma_commit(barAcc1);
    }
    __syncwarp();
    ok = ok && mbar_wait(barSplit2, 0, &failed) && mbar_wait(barW1nLo, 0, &failed);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok && elect_one()) {
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const uint32_t bh = desc_lo32(smem_u32(smem + kOffW1nHi + ks * 16384), 4096u), bl = desc_lo32(smem_u32(smem + kOffW1nLo + ks * 16384), 4096u);
        const uint32_t ta = tmem + kTmA + (uint32_t)ks * 64;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t db = desc_pack(bh + kk * 64, kHi2), dbl = desc_pack(bl + kk * 64, kHi2);  // 8 k-rows of 128 bytes further
          const uint32_t ta_hi = ta + kk * 8, ta_lo = ta_hi + 32;
          umma_tmem_a(tmem + kTmAcc2, ta_lo, db, kIdesc2, (ks > 0 || kk > 0) ? 1u : 0u);
          umma_tmem_a(tmem + kTmAcc2, ta_hi, dbl, kIdesc2, 1u);
          umma_tmem_a(tmem + kTmAcc2, ta_hi, db, kIdesc2, 1u);
        }
      }
      umma_commit(barAcc2);
    }
    __syncwarp();
    // act1 / dact1 are staged (the row threads arrived on barrier 2 before barSplit2 completed): send them off
    bar_sync(2, kBar2);
    if (!failed && lane == 0) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tma_store_3d(&tmAct1, smem + kOffAct1 + h * 16384, h * 32, (int)row0, 0);
        tma_store_3d(&tmDact1, smem + kOffDact1 + h * 16384, h * 32, (int)row0, 0);
      }
      bulk_commit();
    }
    __syncwarp();
    // dact0 staged: send it off; db0, last column block
    bar_sync(3, kBar3);
    if (!failed) {
      if (lane == 0) {
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_store_3d(&tmDact0, smem + kOffA + c * 16384, c * 32, (int)row0, 0);
        bulk_commit();
      }
      __syncwarp();
      atomicAdd(p.db0 + 96 + lane, slab_column_sum(smem + kOffA + 3 * 16384, lane));
    }
    if (lane == 0) bulk_wait_read();
  } else if (warp >= kHelper0) {
    // ===================================================================== helpers
    const int t = threadIdx.x - kRowThreads;   // 0..95
    const int hw = warp - kHelper0;            // 0..2
    // W2, biases, labels: every load of a thread is issued before the first store (one round trip)
    auto stage_small = [&]() {
      constexpr int kW2Per = (kCMax * kH2 + kHelperThreads - 1) / kHelperThreads;   // 11
      float w[kW2Per];
#pragma unroll
      for (int i = 0; i < kW2Per; ++i) {
        const int e = t + i * kHelperThreads;
        w[i] = (e < C * kH2) ? __ldg(p.W2 + e) : 0.f;
      }
      const float bv1 = (t < kH2) ? __ldg(p.b1 + t) : 0.f;
      const float bv2 = (t < C) ? __ldg(p.b2 + t) : 0.f;
      constexpr int kTPer = (kRows * kCMax + kHelperThreads - 1) / kHelperThreads;  // 22
      float tv[kTPer];
      const uint32_t nt = p.label_index ? 0u : nrows * (uint32_t)C;
      const float* tsrc = static_cast<const float*>(p.labels) + (size_t)row0 * C;
#pragma unroll
      for (int i = 0; i < kTPer; ++i) {
        const uint32_t e = (uint32_t)(t + i * kHelperThreads);
        tv[i] = (e < nt) ? __ldg(tsrc + e) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < kW2Per; ++i) {
        const int e = t + i * kHelperThreads;
        if (e < kCMax * kH2) W2s[e] = w[i];
      }
      if (t < kH2) b1s[t] = bv1;
      if (t < kCMax) b2s[t] = bv2;
#pragma unroll
      for (int i = 0; i < kTPer; ++i) {
        const uint32_t e = (uint32_t)(t + i * kHelperThreads);
        if (e < nt) Ts[e] = tv[i];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(barStaged);
    };
    auto split_region = [&](int off_hi, int off_lo) {
      const float4* hi = reinterpret_cast<const float4*>(smem + off_hi);
      float4* lo = reinterpret_cast<float4*>(smem + off_lo);
#pragma unroll 8
      for (int i = t; i < 32768 / 16; i += kHelperThreads) {
        const float4 v = hi[i];
        lo[i] = make_float4(lo_part(v.x), lo_part(v.y), lo_part(v.z), lo_part(v.w));
      }
      fence_async_smem();  // generic-proxy writes -> visible to the tensor core's async proxy
      __syncwarp();
    };
    auto split_w1 = [&]() {
      if (__all_sync(0xffffffffu, mbar_wait(barW1k, 0, &failed))) {
        split_region(kOffW1kHi, kOffW1kLo);
        if (lane == 0) mbar_arrive(barW1kLo);
      }
      if (__all_sync(0xffffffffu, mbar_wait(barW1n, 0, &failed))) {
        split_region(kOffW1nHi, kOffW1nLo);
        if (lane == 0) mbar_arrive(barW1nLo);
      }
    };
    if (p.early_weights) { stage_small(); split_w1(); }
    pdl_sync();
    if (!p.early_weights) { stage_small(); split_w1(); }
    // ---- act1 / dact1 / logits / dlogits staged by the row threads
    bar_sync(2, kBar2);
    if (!failed) {
      if (hw < 2) {
        atomicAdd(p.db1 + hw * 32 + lane, slab_column_sum(smem + kOffDact1 + hw * 16384, lane));
      } else if (lane < C) {
        float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
        for (int r = 0; r < kRows; r += 2) { s0 += dls[r * ld + lane]; s1 += dls[(r + 1) * ld + lane]; }
        atomicAdd(p.db2 + lane, s0 + s1);
      }
    }
    // ---- dact0 staged
    bar_sync(3, kBar3);
    if (!failed) atomicAdd(p.db0 + hw * 32 + lane, slab_column_sum(smem + kOffA + hw * 16384, lane));
  } else {
    // =================================================================== row threads
    const int q = warp >> 2;                       // quarter of the row's columns
    const int row = (warp & 3) * 32 + lane;
    const bool row_ok = (uint32_t)row < nrows;
    const uint32_t lanebits = (uint32_t)((warp & 3) * 32) << 16;
    pdl_sync();
    bool ok = true;
    float loss_row = 0.f;
    // ---- k-slab q of the act0 row -> hi/lo in tensor memory
    ok = __all_sync(0xffffffffu, mbar_wait(&barA[q], 0, &failed));
    if (ok) {
      float4 v[8];
      load_a_row<true>(smem + kOffA + q * 16384, row, v);
      uint32_t hi[32], lo[32];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        hi[4 * c] = __float_as_uint(v[c].x); lo[4 * c] = __float_as_uint(lo_part(v[c].x));
        hi[4 * c + 1] = __float_as_uint(v[c].y); lo[4 * c + 1] = __float_as_uint(lo_part(v[c].y));
        hi[4 * c + 2] = __float_as_uint(v[c].z); lo[4 * c + 2] = __float_as_uint(lo_part(v[c].z));
        hi[4 * c + 3] = __float_as_uint(v[c].w); lo[4 * c + 3] = __float_as_uint(lo_part(v[c].w));
      }
      tmem_st32(tmem + kTmA + lanebits + (uint32_t)q * 64, hi);
      tmem_st32(tmem + kTmA + lanebits + (uint32_t)q * 64 + 32, lo);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(barSplit1);
    }
    // ---- act1 quarter = relu(acc1 + b1)
    ok = ok && __all_sync(0xffffffffu, mbar_wait(barAcc1, 0, &failed) && mbar_wait(barStaged, 0, &failed));
    tc_fence_after();
    float a1[16];
    const int slab_h = q >> 1, cbase = (q & 1) * 4;   // where columns 16q.. sit inside the [128 x 32] slabs
    if (ok) {
      uint32_t r[16];
      tmem_ld16(tmem + kTmAcc1 + lanebits + (uint32_t)q * 16, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float v = __uint_as_float(r[j]) + b1s[q * 16 + j];
        a1[j] = v > 0.f ? v : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *slab_chunk(smem + kOffAct1 + slab_h * 16384, row, cbase + j) = make_float4(a1[4 * j], a1[4 * j + 1], a1[4 * j + 2], a1[4 * j + 3]);
    }
    bar_sync(1, kRowThreads);
    // ---- logits of classes q, q + 4, .. : the whole act1 row (read back from the staged tile) against W2.
    // (Loops are kept rolled on purpose: this code runs once per launch, so every instruction is fetched
    // cold -- the fully unrolled form spent a quarter of its issue slots waiting for instructions.)
    if (ok) {
      float acc[CP / 4];
#pragma unroll
      for (int i = 0; i < CP / 4; ++i) acc[i] = 0.f;
#pragma unroll 2
      for (int jc = 0; jc < 16; ++jc) {
        const float4 av = *slab_chunk(smem + kOffAct1 + (jc >> 3) * 16384, row, jc & 7);
#pragma unroll
        for (int i = 0; i < CP / 4; ++i) {
          const float4 wv = *reinterpret_cast<const float4*>(W2s + (q + 4 * i) * kH2 + jc * 4);
          acc[i] = fmaf(av.x, wv.x, acc[i]);
          acc[i] = fmaf(av.y, wv.y, acc[i]);
          acc[i] = fmaf(av.z, wv.z, acc[i]);
          acc[i] = fmaf(av.w, wv.w, acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < CP / 4; ++i) {
        const int c = q + 4 * i;
        if (c < C) lgs[row * ld + c] = acc[i] + b2s[c];
      }
    }
    bar_sync(1, kRowThreads);
    // ---- softmax cross-entropy forward and backward for the row: each of its four threads takes the row's maximum
    // and sum of exponentials (ten loads and exponentials: cheaper than exchanging them) and then the loss terms and
    // dlogits of ITS classes q, q + 4, ..; the dlogits meet in shared memory.
    if (ok) {
      const float* lrow = lgs + row * ld;
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < C; ++c) mx = fmaxf(mx, lrow[c]);
      float se = 0.f;
#pragma unroll 1
      for (int c = 0; c < C; ++c) se += __expf(lrow[c] - mx);
      const float inv = 1.f / se, lse = logf(se);
      int lab = -1;
      if (p.label_index && row_ok) {
        const len_t l = static_cast<const len_t*>(p.labels)[row0 + row];
        lab = l < (len_t)C ? (int)l : -1;
      }
#pragma unroll
      for (int i = 0; i < CP / 4; ++i) {
        const int c = q + 4 * i;
        if (c < C) {
          const float dc = lrow[c] - mx;
          float gc = 0.f;
          if (row_ok) {
            const float t = p.label_index ? ((c == lab) ? 1.f : 0.f) : Ts[row * C + c];
            if (t != 0.f) loss_row -= t * fminf(fmaxf(dc - lse, kLogPMin), kLogPMax);
            const float diff = __expf(dc) * inv - t;
            gc = p.exact_inv ? diff * p.inv_divisor : diff / p.divisor;
          }
          dls[row * ld + c] = gc;
        }
      }
    }
    bar_sync(1, kRowThreads);
    // ---- the row's dact1 quarter = (dlogits W2) where act1 > 0.  One rolled loop over the C classes.
    if (ok) {
      const float* drow = dls + row * ld;
      float x[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) x[j] = 0.f;
#pragma unroll 2
      for (int c = 0; c < C; ++c) {
        const float gc = drow[c];
        const float4* w = reinterpret_cast<const float4*>(W2s + c * kH2 + q * 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 wv = w[j];
          x[4 * j] = fmaf(gc, wv.x, x[4 * j]);
          x[4 * j + 1] = fmaf(gc, wv.y, x[4 * j + 1]);
          x[4 * j + 2] = fmaf(gc, wv.z, x[4 * j + 2]);
          x[4 * j + 3] = fmaf(gc, wv.w, x[4 * j + 3]);
        }
      }
      // staged for its TMA store, hi/lo to tensor memory
      uint32_t hi[16], lo[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (!(a1[j] > 0.f)) x[j] = 0.f;
        hi[j] = __float_as_uint(x[j]);
        lo[j] = __float_as_uint(lo_part(x[j]));
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *slab_chunk(smem + kOffDact1 + slab_h * 16384, row, cbase + j) = make_float4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
      const uint32_t ta = tmem + kTmA + lanebits + (uint32_t)slab_h * 64 + (uint32_t)(q & 1) * 16;
      tmem_st16(ta, hi);
      tmem_st16(ta + 32, lo);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(barSplit2);
    }
    // loss terms of this warp's (row, class) pairs, handed to thread 0 across the barrier below
    {
      const float ws = warp_sum(loss_row);
      if (lane == 0) red[warp] = ws;  // all 16 row warps: every thread holds the loss terms of its classes
    }
    fence_async_smem();  // the staged tiles -> visible to the copy engine
    bar_arrive(2, kBar2);
    // logits / dlogits leave while the second product runs: thread (row, q) copies columns q, q + 4, ..
    bar_sync(1, kRowThreads);
    // loss: CTA partial -> workspace and a ticket, while the second product runs; the CTA that drew the
    // last ticket folds the partials at the end of the kernel
    if (threadIdx.x == 0) {
      float cta_loss = 0.f;
#pragma unroll
      for (int w = 0; w < kRowThreads / 32; ++w) cta_loss += red[w];
      p.loss_partial[blockIdx.x] = cta_loss;
      __threadfence();
      const unsigned t = atomicAdd(p.counter, 1u);
      is_last = (t == gridDim.x - 1) ? 1 : 0;
      if (is_last) *p.counter = 0;
    }
    if (ok && row_ok) {
      float* gl = p.logits + (size_t)(row0 + row) * ld;
      float* gd = p.dlogits + (size_t)(row0 + row) * ld;
#pragma unroll
      for (int i = 0; i < CP / 4; ++i) {
        const int c = q + 4 * i;
        if (c < C) { gl[c] = lgs[row * ld + c]; gd[c] = dls[row * ld + c]; }
      }
    }
    // ---- dact0 column block q = acc2 where act0 > 0, written over the act0 slab it was masked with
    ok = ok && __all_sync(0xffffffffu, mbar_wait(barAcc2, 0, &failed));
    tc_fence_after();
    if (ok) {
      uint32_t r[32];
      tmem_ld32(tmem + kTmAcc2 + lanebits + (uint32_t)q * 32, r);
      float4 av[8];
      load_a_row<true>(smem + kOffA + q * 16384, row, av);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 o;
        o.x = (row_ok && av[j].x > 0.f) ? __uint_as_float(r[4 * j]) : 0.f;
        o.y = (row_ok && av[j].y > 0.f) ? __uint_as_float(r[4 * j + 1]) : 0.f;
        o.z = (row_ok && av[j].z > 0.f) ? __uint_as_float(r[4 * j + 2]) : 0.f;
        o.w = (row_ok && av[j].w > 0.f) ? __uint_as_float(r[4 * j + 3]) : 0.f;
        *slab_chunk(smem + kOffA + q * 16384, row, j) = o;
      }
    }
    fence_async_smem();
    bar_arrive(3, kBar3);
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kIssuer) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmCols);
  }
  if (threadIdx.x == 0 && failed && p.error_flag) *p.error_flag = 1;
  // loss: the CTA that drew the last ticket (all partials are in the workspace then) folds them in a fixed order
  if (is_last) {
    __threadfence();
    float v = 0.f;
    for (unsigned k = threadIdx.x; k < gridDim.x; k += kThreads) v += __ldcg(p.loss_partial + k);
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int w = 0; w < kThreads / 32; ++w) s += red[w];
      *p.loss_out = s / p.divisor;
    }
  }
}

}  // namespace tail
}  // namespace zg
