// Persistent tcgen05 GEMM for large problems (bf16 and single-pass TF32).
//
// One CTA per SM walks a list of 128 x 256 output tiles.  Compared with the
// one-tile-per-CTA kernel of gemm_tc.cuh:
//   * the tile is twice as wide, so one k-slab of operands (A 16 KB + B 32 KB)
//     feeds twice the tensor work: shared-memory traffic per flop drops by a
//     quarter, which is what bounds the narrower tile;
//   * the accumulator is double-buffered in tensor memory (2 x 256 columns =
//     all 512): the epilogue warps drain tile i while the MMA warp already
//     accumulates tile i+1, and the TMA ring never drains between tiles;
//   * set-up (barriers, TMEM allocation, descriptor prefetch) is paid once per
//     SM instead of once per tile.
// Tiles are visited in groups of kGroupM row-tiles x all column-tiles so that
// the CTAs running at the same time share operand slabs in L2.  The schedule
// is dynamic: the producer thread draws the next work item from a counter in
// global memory and hands it to the other roles through a small ring in
// shared memory, so a CTA that starts late (SMs held by a kernel of another
// stream, e.g. a collective) simply finds less work left instead of delaying
// a fixed share of the tiles.  The CTA that draws the last ticket of the
// launch (n_items + gridDim.x - 1) resets the counter for the next launch.
//
// K may be split (weight gradients: fp32 C, no fused epilogue): a work item is
// then one K range of one tile and its epilogue adds into C with vector
// reductions, which evens out the last wave when the tile count is a poor
// multiple of the SM count.
//
// Roles (12 warps): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner,
// warps 4-11 epilogue in two groups (warp w drains TMEM lanes 32(w%4)..+31;
// group 0 takes the even 32-column chunks of a tile, group 1 the odd ones, so
// two chunks' global loads and stores are in flight at once).  Every mbarrier
// wait is bounded (see mbar_wait); after a failed wait all roles stop and the
// CTA still frees its tensor memory.
#pragma once

#include "gemm_tc.cuh"

namespace zg {
namespace tc {

constexpr int kPBN = 256;      // tile width
constexpr int kGroupM = 16;    // row-tiles per scheduling group
constexpr int kThreadsPersistent = 384;
constexpr int kEpiThreads = kThreadsPersistent - 128;
constexpr int kSchedDepth = 4;                  // work items in flight between the roles
constexpr uint32_t kNoTile = 0xFFFFFFFFu;       // end of work

template <int MODE>
struct PersistentSmem {
  using MT = ModeTraits<MODE>;
  static constexpr int kABytes = kBM * kSlabBytes;    // 16 KB
  static constexpr int kBBytes = kPBN * kSlabBytes;   // 32 KB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = 4;
  static constexpr int kTotal = kStages * kStageBytes + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

struct TileCoord { uint32_t m, n, batch, split; };

// tile index -> (row-tile, column-tile, batch); groups of kGroupM row-tiles, row-tile fastest inside a group
__device__ __forceinline__ TileCoord tile_coord(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t splits) {
  TileCoord c;
  c.split = t % splits;  // the K ranges of a tile are neighbours in the list: they run at the same time
  t /= splits;
  const uint32_t per_batch = tiles_m * tiles_n;
  c.batch = t / per_batch;
  t -= c.batch * per_batch;
  const uint32_t group_sz = kGroupM * tiles_n;
  const uint32_t g = t / group_sz, in_g = t - g * group_sz;
  const uint32_t m0 = g * kGroupM;
  const uint32_t gm = (tiles_m - m0) < (uint32_t)kGroupM ? (tiles_m - m0) : (uint32_t)kGroupM;
  c.n = in_g / gm;
  c.m = m0 + (in_g - c.n * gm);
  return c;
}

template <bool A_KMAJOR, bool B_KMAJOR, int MODE>
__global__ void __launch_bounds__(kThreadsPersistent, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p,
                          const uint32_t tiles_m, const uint32_t tiles_n, const uint32_t n_tiles, unsigned* sched_counter) {
  static_assert(MODE == kBF16 || MODE == kTF32, "the persistent kernel has no operand-split warps");
  using MT = ModeTraits<MODE>;
  using SL = PersistentSmem<MODE>;
  constexpr int S = SL::kStages;
  constexpr int BN = kPBN;
  constexpr uint32_t kIdesc = make_idesc(MT::kBf16, !A_KMAJOR, !B_KMAJOR, BN);
  constexpr uint32_t kTmemCols = 512;  // two 256-column accumulators

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * SL::kStageBytes);
  uint64_t* full = bars;                 // [S] TMA bytes landed
  uint64_t* empty = bars + S;            // [S] MMAs that read the stage retired
  uint64_t* acc_full = bars + 2 * S;     // [2] accumulator complete
  uint64_t* acc_empty = bars + 2 * S + 2;  // [2] accumulator drained by the epilogue
  uint64_t* sched_full = bars + 2 * S + 4;                 // [kSchedDepth] work item published
  uint64_t* sched_empty = bars + 2 * S + 4 + kSchedDepth;  // [kSchedDepth] read by the MMA thread and every epilogue warp
  __shared__ uint32_t sched_tile[kSchedDepth];
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // k-slabs of K range `split` (p.k_per_split is a multiple of the slab depth)
  auto slabs_of = [&](uint32_t split) -> int {
    const uint32_t kb = split * p.k_per_split;
    if (kb >= p.k) return 0;
    const uint32_t ke = (kb + p.k_per_split < p.k) ? kb + p.k_per_split : p.k;
    return (int)((ke - kb + MT::kBK - 1) / MT::kBK);
  };

  if (threadIdx.x == 0) {
    failed = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kEpiThreads);  // every epilogue thread arrives
    }
    for (int j = 0; j < kSchedDepth; ++j) {
      mbar_init(&sched_full[j], 1);
      mbar_init(&sched_empty[j], 1 + kEpiThreads / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_sync();  // everything above overlaps the previous kernel's tail

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t it = 0;  // k-slabs issued so far (ring position)
      bool ok = true;
      for (uint32_t i = 0; ok; ++i) {
        const int j = (int)(i % kSchedDepth);
        if (i >= (uint32_t)kSchedDepth && !mbar_wait(&sched_empty[j], ((i / kSchedDepth) & 1) ^ 1, &failed)) break;
        uint32_t t = atomicAdd(sched_counter, 1u);
        if (t == n_tiles + gridDim.x - 1) atomicExch(sched_counter, 0u);  // the last draw of the launch
        if (t >= n_tiles) t = kNoTile;
        sched_tile[j] = t;
        mbar_arrive(&sched_full[j]);
        if (t == kNoTile) break;
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n, p.splits);
        const int za = (int)(tc.batch % p.nA), zb = (int)(tc.batch % p.nB);
        const int KT = slabs_of(tc.split);
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const int s = (int)(it % S);
          if (it >= (uint32_t)S && !mbar_wait(&empty[s], ((it / S) & 1) ^ 1, &failed)) { ok = false; break; }
          uint8_t* a_dst = smem + s * SL::kStageBytes;
          uint8_t* b_dst = a_dst + SL::kABytes;
          mbar_expect_tx(&full[s], SL::kStageBytes);
          const int k0 = (int)(tc.split * p.k_per_split) + kt * MT::kBK;
          if (A_KMAJOR) {
            tma_load_3d(a_dst, &tmA, &full[s], k0, (int)(tc.m * kBM), za);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / MT::kAtomMN; ++j)
              tma_load_3d(a_dst + j * MT::kBK * kSlabBytes, &tmA, &full[s], (int)(tc.m * kBM) + j * MT::kAtomMN, k0, za);
          }
          if (B_KMAJOR) {
            // a TMA box holds at most 256 rows: one load for the whole 256-row slab
            tma_load_3d(b_dst, &tmB, &full[s], k0, (int)(tc.n * BN), zb);
          } else {
#pragma unroll
            for (int j = 0; j < BN / MT::kAtomMN; ++j)
              tma_load_3d(b_dst + j * MT::kBK * kSlabBytes, &tmB, &full[s], (int)(tc.n * BN) + j * MT::kAtomMN, k0, zb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // The whole warp walks the loops (waits and descriptor arithmetic stay
    // warp-uniform), one elected lane issues the MMAs and the commits; the
    // barrier of the next ring position is tested before this slab's MMAs go out.
    {
      uint32_t it = 0, tcount = 0;
      bool ok = true, have = false;
      for (; ok; ++tcount) {
        const int j = (int)(tcount % kSchedDepth);
        bool got = mbar_wait(&sched_full[j], (tcount / kSchedDepth) & 1, &failed);
        if (!__all_sync(0xffffffffu, got)) break;
        const uint32_t t = sched_tile[j];
        __syncwarp();
        if (lane == 0) mbar_arrive(&sched_empty[j]);
        if (t == kNoTile) break;
        const uint32_t buf = tcount & 1;
        if (tcount >= 2) {
          got = mbar_wait(&acc_empty[buf], ((tcount >> 1) & 1) ^ 1, &failed);
          if (!__all_sync(0xffffffffu, got)) break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        const int KT = slabs_of(tile_coord(t, tiles_m, tiles_n, p.splits).split);
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const int s = (int)(it % S);
          if (!have) {
            got = mbar_wait(&full[s], (it / S) & 1, &failed);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
          }
          const uint32_t it1 = it + 1;
          const bool next_seen = mbar_test(&full[it1 % S], (it1 / S) & 1);
          tc_fence_after();
          const uint32_t a_s = smem_u32(smem + s * SL::kStageBytes), b_s = a_s + SL::kABytes;
          constexpr uint32_t a_step = (A_KMAJOR ? 32u : (uint32_t)(MT::kUmmaK * kSlabBytes)) >> 4;
          constexpr uint32_t b_step = (B_KMAJOR ? 32u : (uint32_t)(MT::kUmmaK * kSlabBytes)) >> 4;
          constexpr uint32_t a_lbo = A_KMAJOR ? 16u : (uint32_t)(MT::kBK * kSlabBytes);
          constexpr uint32_t b_lbo = B_KMAJOR ? 16u : (uint32_t)(MT::kBK * kSlabBytes);
          constexpr uint32_t a_lay = (!A_KMAJOR && !MT::kBf16) ? 1u : 2u, b_lay = (!B_KMAJOR && !MT::kBf16) ? 1u : 2u;
          constexpr uint32_t a_h32 = desc_hi32(a_lay == 1u ? 512u : 1024u, a_lay), b_h32 = desc_hi32(b_lay == 1u ? 512u : 1024u, b_lay);
          const uint32_t da0 = desc_lo32(a_s, a_lbo), db0 = desc_lo32(b_s, b_lbo);
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < MT::kBK / MT::kUmmaK; ++kk)
              umma<MT::kBf16>(tmem_d, desc_pack(da0 + kk * a_step, a_h32), desc_pack(db0 + kk * b_step, b_h32), kIdesc,
                              (kt > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&empty[s]);
          }
          have = __all_sync(0xffffffffu, next_seen);
        }
        if (ok && elect_one()) umma_commit(&acc_full[buf]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3, group = (warp - 4) >> 2;
    uint32_t tcount = 0;
    for (;; ++tcount) {
      const int j = (int)(tcount % kSchedDepth);
      if (!mbar_wait(&sched_full[j], (tcount / kSchedDepth) & 1, &failed)) break;
      const uint32_t t = sched_tile[j];
      __syncwarp();
      if (lane == 0) mbar_arrive(&sched_empty[j]);
      if (t == kNoTile) break;
      const uint32_t buf = tcount & 1;
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n, p.splits);
      const int KT = slabs_of(tc.split);
      if (!mbar_wait(&acc_full[buf], (tcount >> 1) & 1, &failed)) break;
      tc_fence_after();
      const uint32_t row = tc.m * kBM + q * 32 + lane;
      const uint64_t c_off = (uint64_t)tc.batch * p.c_batch_stride + (uint64_t)row * p.ldc;
      const bool row_ok = row < p.m;
#pragma unroll 1
      for (int c = group; c < BN / 32; c += 2) {
        const uint32_t col0 = tc.n * BN + c * 32;
        if (col0 >= p.n) break;  // uniform across the warp
        uint32_t r[32];
        if (KT > 0) {
          tmem_ld32(tmem_base + buf * BN + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        epilogue_chunk(p, r, row_ok, c_off + col0, col0, lane);
      }
      // all tcgen05.ld of this thread have completed (wait::ld): hand the accumulator back
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && failed && p.error_flag) *p.error_flag = 1;
}

}  // namespace tc
}  // namespace zg
