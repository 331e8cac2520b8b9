// Losses: fused row-softmax + cross-entropy (forward and backward in one
// pass over the logits), smooth-L1, and the softmax / NLL entry points of
// include/nn_conflux.h.  Semantics: src/nn/loss.zig:130-215, :259-305.
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstring>

#include "common.cuh"
#include "async_copy.cuh"
#include "../../include/nn_conflux.h"

namespace zg {

constexpr int kLThreads = 256;

// Adds `v` over the whole grid into *out (overwriting it): CTA partials go to
// the workspace, the last CTA folds them in index order -> deterministic.
__device__ __forceinline__ void grid_sum_store(float v, float* sm32, float* partial, unsigned* counter, float* out, float divisor) {
  const float bs = block_sum<float>(v, sm32);
  if (threadIdx.x == 0) partial[blockIdx.x] = bs;
  __threadfence();
  __shared__ bool last;
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(counter, 1u);
    last = (t == gridDim.x - 1);
    if (last) *counter = 0;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  float s = 0.f;
  for (unsigned k = threadIdx.x; k < gridDim.x; k += blockDim.x) s += __ldcg(partial + k);
  s = block_sum<float>(s, sm32);
  if (threadIdx.x == 0 && out) *out = s / divisor;
}

struct SmceArgs {
  const float* logits;   // [rows, ld]
  const void* labels;    // fp32 [rows, C] (contiguous) or u64 [rows]
  size_t rows;
  int C;
  size_t ld;             // row stride of logits / dlogits / probs, in elements
  float divisor;
  float inv_divisor;     // 1 / divisor
  int exact_inv;         // divisor is a power of two: multiplying by inv_divisor equals dividing
  float* loss_out;
  float* dlogits;        // [rows, ld] or nullptr
  int accumulate;
  float* probs_out;      // [rows, ld] or nullptr
  float* dbias;          // [C] or nullptr: column sums of (p - t)/divisor
  float* partial;        // workspace: gridDim.x loss partials, then gridDim.x * C bias partials
  int fold_bias_inline;  // the last CTA folds the bias partials into dbias (else a later launch does)
  unsigned* counter_error;  // raised when a bounded wait of the staged kernel runs out
  unsigned* counter;
};

// Column sums over the whole grid of per-thread values acc[i] (column lane+32i):
// CTA partials in a fixed warp order -> workspace -> folded by the last CTA
// (the caller guarantees that this runs in the last CTA only after all
// partials are visible).
template <int ITEMS>
__device__ __forceinline__ void cta_column_partials(const float (&acc)[ITEMS], float* colsum /*smem [32*ITEMS]*/, float* out, int C) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int w = 0; w < kLThreads / 32; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int j = lane + 32 * i;
        if (j < C) colsum[j] = (w == 0 ? 0.f : colsum[j]) + acc[i];
      }
    }
    __syncthreads();
  }
  for (int j = threadIdx.x; j < C; j += blockDim.x) out[j] = colsum[j];
}

// Tail shared by the softmax-CE kernels: per-CTA loss partial -> workspace; the
// last CTA (atomic ticket) folds the loss partials and, when requested, the
// per-CTA bias-gradient partials that every CTA has already written to
// partial[gridDim.x + cta*C ...], both in a fixed order.
__device__ __forceinline__ void smce_finish(const SmceArgs& a, float loss_acc, float* sm32) {
  const int C = a.C;
  float* bias_partial = a.partial + gridDim.x;
  const float bs = block_sum<float>(loss_acc, sm32);
  if (threadIdx.x == 0) a.partial[blockIdx.x] = bs;
  __threadfence();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(a.counter, 1u);
    last = (t == gridDim.x - 1);
    if (last) *a.counter = 0;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  float s = 0.f;
  for (unsigned k = threadIdx.x; k < gridDim.x; k += blockDim.x) s += __ldcg(a.partial + k);
  s = block_sum<float>(s, sm32);
  if (threadIdx.x == 0 && a.loss_out) *a.loss_out = s / a.divisor;
  if (a.dbias && a.fold_bias_inline) {
    // `parts` threads per column, each over every parts-th CTA partial, then a shuffle tree
    const unsigned parts = (C * 8 <= (int)blockDim.x) ? 8u : ((C * 4 <= (int)blockDim.x) ? 4u : ((C * 2 <= (int)blockDim.x) ? 2u : 1u));
    const unsigned part = threadIdx.x % parts;
    const int per_trip = blockDim.x / parts;
    for (int base = 0; base < C; base += per_trip) {
      const int j = base + threadIdx.x / parts;
      float v = 0.f;
      if (j < C)
        for (unsigned k = part; k < gridDim.x; k += parts) v += __ldcg(bias_partial + (size_t)k * C + j);
      for (unsigned o = parts >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (j < C && part == 0) a.dbias[j] = v;
    }
  }
}

// log of the probability clamp of the reference loss (p limited to [1e-7, 1 - 1e-7]):
// log(clamp(p)) == clamp(log p), and log p = (x - max) - log(sum exp) needs no log per element
constexpr float kLogPMin = -16.11809565f;     // logf(1e-7f)
constexpr float kLogPMax = -1.1920929e-07f;   // logf(1.0f - 1e-7f)
__device__ __forceinline__ float clamp_logp(float lp) { return fminf(fmaxf(lp, kLogPMin), kLogPMax); }

// exp of a non-positive shifted logit: one multiply and the hardware base-2
// exponential (relative error about 2^-22 plus 2^-24 |d| from the rounded
// product; the softmax that comes out agrees with an exact one to ~1e-6)
__device__ __forceinline__ float fast_exp(float d) { return __expf(d); }
// exp(x - m) as 2^(x log2(e) - m log2(e)): one fused multiply-add and one ex2.approx (nm2 = -m log2(e))
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float fast_exp_shifted(float x, float nm2) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fmaf(x, kLog2e, nm2)));
  return r;
}

// FAST: dlogits written (not accumulated), no probabilities wanted, divisor a power of two
template <bool FAST>
__device__ __forceinline__ float grad_scale(const SmceArgs& a, float d) {
  if (FAST) return d * a.inv_divisor;
  return a.exact_inv ? d * a.inv_divisor : d / a.divisor;
}

// One warp per row, ROWS rows per trip; ITEMS = ceil(C/32) logits per lane and
// row held in registers, so the logits are read from memory exactly once and
// dlogits written once.  All loads of a trip are issued before the first
// shuffle, the ROWS independent reductions overlap, and the element loops are
// branch-free (index labels) so that the compiler can interleave them.
template <int ITEMS, int ROWS, bool INDEX_LABELS, bool FAST>
__global__ void __launch_bounds__(kLThreads) softmax_ce_kernel(const SmceArgs a) {
  __shared__ float sm32[32];
  __shared__ float colsum[32 * ITEMS];
  const int lane = threadIdx.x & 31;
  const int C = a.C;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  pdl_sync();
  float loss_acc = 0.f;
  float bias_acc[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) bias_acc[i] = 0.f;
  for (size_t r0 = (((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * ROWS; r0 < a.rows; r0 += warps * ROWS) {
    float x[ROWS][ITEMS];
    float mx[ROWS], se[ROWS], dlab[ROWS];
    int lab[ROWS];
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      const bool ok = r0 + k < a.rows;
      const float* xr = a.logits + (r0 + k) * a.ld;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int j = lane + 32 * i;
        x[k][i] = (ok && j < C) ? xr[j] : -INFINITY;
      }
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      lab[k] = -1;
      if (INDEX_LABELS && r0 + k < a.rows) {
        const len_t l = static_cast<const len_t*>(a.labels)[r0 + k];
        lab[k] = l < (len_t)C ? (int)l : -1;
      }
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      float m = x[k][0];
#pragma unroll
      for (int i = 1; i < ITEMS; ++i) m = fmaxf(m, x[k][i]);
      mx[k] = m;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int k = 0; k < ROWS; ++k) mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], o));
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      float sacc = 0.f;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        x[k][i] = fast_exp(x[k][i] - mx[k]);          // -inf in the padding lanes gives 0
        sacc += x[k][i];
      }
      se[k] = sacc;
    }
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      // the lane that owns the label column fetches that logit again (a cache hit)
      dlab[k] = 0.f;
      if (INDEX_LABELS && lab[k] >= 0 && (lab[k] & 31) == lane) dlab[k] = a.logits[(r0 + k) * a.ld + lab[k]] - mx[k];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int k = 0; k < ROWS; ++k) se[k] += __shfl_xor_sync(0xffffffffu, se[k], o);
#pragma unroll
    for (int k = 0; k < ROWS; ++k) {
      if (r0 + k >= a.rows) continue;
      const size_t r = r0 + k;
      const float inv = 1.f / se[k];
      const float lse = logf(se[k]);
      if (INDEX_LABELS && lab[k] >= 0 && (lab[k] & 31) == lane) loss_acc -= clamp_logp(dlab[k] - lse);
      const float* tr = INDEX_LABELS ? nullptr : static_cast<const float*>(a.labels) + r * (size_t)C;
      float* dl = a.dlogits + r * a.ld;
      // FAST: the divisor is a power of two, so (e * inv - t) * 2^-k == e * (inv * 2^-k) - t * 2^-k bit for bit
      const float sc = inv * a.inv_divisor;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int j = lane + 32 * i;
        if (j < C) {
          float g;
          if (FAST && INDEX_LABELS) {
            g = x[k][i] * sc;
            if (j == lab[k]) g -= a.inv_divisor;
          } else {
            const float p = x[k][i] * inv;
            float t;
            if (INDEX_LABELS) t = (j == lab[k]) ? 1.f : 0.f;
            else {
              t = tr[j];
              if (t != 0.f) loss_acc -= t * clamp_logp(logf(p));
            }
            g = grad_scale<FAST>(a, p - t);
            if (!FAST && a.probs_out) a.probs_out[r * a.ld + j] = p;
          }
          bias_acc[i] += g;
          if (FAST) dl[j] = g;
          else if (a.dlogits) dl[j] = a.accumulate ? dl[j] + g : g;
        }
      }
    }
  }
  float* bias_partial = a.partial + gridDim.x;
  if (a.dbias) cta_column_partials<ITEMS>(bias_acc, colsum, bias_partial + (size_t)blockIdx.x * C, C);
  smce_finish(a, loss_acc, sm32);
}

// Wide rows with index labels, staged: the logits travel through a ring of
// shared-memory stages filled by bulk asynchronous copies (a group of whole rows
// and their labels per stage), each consumer warp works on rows of the current
// stage in place, and the gradient leaves through a bulk store of the same
// stage.  Memory latency is hidden by the ring instead of by occupancy.
//
// Roles: warps 0..15 compute; one lane of warp 16 drives the copies.  The
// consumers of a stage wait on its `full` barrier (bytes landed), compute, make
// their writes visible to the copy engine and arrive on its `done` barrier; the
// copy lane waits on `done`, issues the bulk store, waits until the store has
// read the stage and refills it with the group n_stages further on.  No
// CTA-wide barrier sits on this path: warps run ahead into the next stage while
// the previous one drains.  Whole groups only go through the ring; the ragged
// last group of the problem is copied by the threads of one CTA after its ring.
// FAST form only (dlogits written, power-of-two divisor, no probabilities);
// unpadded rows (ld == C, C % 4 == 0) and 16-byte aligned bases.
constexpr int kStThreads = 512;  // consumer threads
constexpr int kStLaunchThreads = kStThreads + 32;
constexpr int kStMaxStages = 8;

//
// SUBL > 0 selects the sub-warp form for rows of up to 128 columns: SUBL lanes
// (8 or 16) share a row, each holding 8 consecutive columns (two 128-bit
// shared-memory accesses), a warp works on 32 / SUBL rows at once and the row
// reductions take log2(SUBL) shuffle rounds for all of them together; the
// lane-per-column form spends 10 shuffles on every 64-column row and is bound
// by the shuffle/shared-memory pipe there.  ROWS must then be 32 / SUBL.
template <int ITEMS, int ROWS, int SUBL = 0>
__global__ void __launch_bounds__(kStLaunchThreads, 1) softmax_ce_staged_kernel(const SmceArgs a, const int group_rows, const int n_stages) {
  extern __shared__ __align__(128) unsigned char st_raw[];
  __shared__ uint64_t full[kStMaxStages], done[kStMaxStages];
  __shared__ float sm32[32];
  __shared__ float colsum[32 * ITEMS];
  __shared__ int failed;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int kWarps = kStThreads / 32;
  const int C = a.C;
  const size_t ld = a.ld;
  const size_t stage_floats = (size_t)group_rows * ld;
  // a stage = the logits of a group of rows followed by their labels (u64 each)
  const size_t stage_bytes = stage_floats * sizeof(float) + (size_t)group_rows * sizeof(len_t);
  const size_t n_full = a.rows / (size_t)group_rows;
  const int tail_rows = (int)(a.rows - n_full * (size_t)group_rows);
  const size_t my_groups = n_full > blockIdx.x ? (n_full - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  auto stage_logits = [&](int s) -> float* { return reinterpret_cast<float*>(st_raw + (size_t)s * stage_bytes); };
  auto stage_labels = [&](int s) -> len_t* { return reinterpret_cast<len_t*>(st_raw + (size_t)s * stage_bytes + stage_floats * sizeof(float)); };
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      ac::mbar_init(&full[s], 1);
      ac::mbar_init(&done[s], kWarps);
    }
    ac::mbar_fence_init();
    failed = 0;
  }
  __syncthreads();
  pdl_sync();
  float loss_acc = 0.f;
  constexpr int kAcc = SUBL > 0 ? 8 : ITEMS;
  float bias_acc[kAcc];
#pragma unroll
  for (int i = 0; i < kAcc; ++i) bias_acc[i] = 0.f;
  volatile int* failed_v = &failed;
  const int warps_per_group = (group_rows + ROWS - 1) / ROWS < kWarps ? (group_rows + ROWS - 1) / ROWS : 0;

  // ---- the rows [0, nrows) of one stage, ROWS per warp and trip, in place
  auto compute_rows = [&](float* st, const len_t* lst, const int nrows, const int warp) {
    if constexpr (SUBL > 0) {
      static_assert(ROWS * SUBL == 32, "sub-warp form: ROWS == 32 / SUBL");
      const int sub = lane / SUBL, c0 = (lane % SUBL) * 8;
      for (int r0 = warp * ROWS; r0 < nrows; r0 += kWarps * ROWS) {
        const int r = r0 + sub;
        const bool ok = r < nrows;
        float* xr = st + (size_t)(ok ? r : 0) * ld + c0;
        const bool v0 = ok && c0 < C, v1 = ok && c0 + 4 < C;  // C % 4 == 0: a quad lies wholly inside or outside the row
        const float4 q0 = v0 ? *reinterpret_cast<const float4*>(xr) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        const float4 q1 = v1 ? *reinterpret_cast<const float4*>(xr + 4) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        float x[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        int lab = -1;
        if (ok) {
          const len_t l = lst[r];
          lab = l < (len_t)C ? (int)l : -1;
        }
        float m = x[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) m = fmaxf(m, x[i]);
#pragma unroll
        for (int o = SUBL / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (!ok) m = 0.f;  // an idle row slot: keep the arithmetic finite
        const bool owner = lab >= c0 && lab < c0 + 8;
        const float dlab = owner ? st[(size_t)r * ld + lab] - m : 0.f;
        float se = 0.f;
        const float nm2 = -m * kLog2e;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          x[i] = fast_exp_shifted(x[i], nm2);
          se += x[i];
        }
#pragma unroll
        for (int o = SUBL / 2; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
        if (ok) {
          if (owner) loss_acc -= clamp_logp(dlab - __logf(se));
          const float sc = __fdividef(a.inv_divisor, se);
          const int li = lab - c0;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            x[i] *= sc;
            if (i == li) x[i] -= a.inv_divisor;
          }
          if (v0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) bias_acc[i] += x[i];
            *reinterpret_cast<float4*>(xr) = make_float4(x[0], x[1], x[2], x[3]);
          }
          if (v1) {
#pragma unroll
            for (int i = 4; i < 8; ++i) bias_acc[i] += x[i];
            *reinterpret_cast<float4*>(xr + 4) = make_float4(x[4], x[5], x[6], x[7]);
          }
        }
      }
    } else {
    for (int r0 = warp * ROWS; r0 < nrows; r0 += kWarps * ROWS) {
      float x[ROWS][ITEMS];
      float mx[ROWS], se[ROWS];
      int lab[ROWS];
#pragma unroll
      for (int k = 0; k < ROWS; ++k) {
        const bool ok = r0 + k < nrows;
        const float* xr = st + (size_t)(r0 + k) * ld;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          const int j = lane + 32 * i;
          x[k][i] = (ok && j < C) ? xr[j] : -INFINITY;
        }
        lab[k] = -1;
        if (ok) {
          const len_t l = lst[r0 + k];
          lab[k] = l < (len_t)C ? (int)l : -1;
        }
      }
#pragma unroll
      for (int k = 0; k < ROWS; ++k) {
        float m = x[k][0];
#pragma unroll
        for (int i = 1; i < ITEMS; ++i) m = fmaxf(m, x[k][i]);
        mx[k] = m;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < ROWS; ++k) mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], o));
      float dlab[ROWS];
#pragma unroll
      for (int k = 0; k < ROWS; ++k) {
        float sacc = 0.f;
        dlab[k] = 0.f;
        if (lab[k] >= 0 && (lab[k] & 31) == lane) dlab[k] = st[(size_t)(r0 + k) * ld + lab[k]] - mx[k];
        const float nm2 = -mx[k] * kLog2e;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          x[k][i] = fast_exp_shifted(x[k][i], nm2);
          sacc += x[k][i];
        }
        se[k] = sacc;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < ROWS; ++k) se[k] += __shfl_xor_sync(0xffffffffu, se[k], o);
#pragma unroll
      for (int k = 0; k < ROWS; ++k) {
        if (r0 + k >= nrows) continue;
        const float lse = __logf(se[k]);
        if (lab[k] >= 0 && (lab[k] & 31) == lane) loss_acc -= clamp_logp(dlab[k] - lse);
        const float sc = __fdividef(a.inv_divisor, se[k]);
        float* out = st + (size_t)(r0 + k) * ld;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          const int j = lane + 32 * i;
          if (j < C) {
            float gv = x[k][i] * sc;
            if (j == lab[k]) gv -= a.inv_divisor;
            bias_acc[i] += gv;
            out[j] = gv;
          }
        }
      }
    }
    }
  };

  if (warp == kWarps) {
    // ---- the copy lane
    if (lane == 0) {
      const uint32_t bytes = (uint32_t)(stage_floats * sizeof(float)), lbytes = (uint32_t)((size_t)group_rows * sizeof(len_t));
      auto issue_load = [&](size_t it) {
        const size_t g = blockIdx.x + it * gridDim.x;
        const int s = (int)(it % (size_t)n_stages);
        ac::mbar_expect_tx(&full[s], bytes + lbytes);
        ac::bulk_load(stage_logits(s), a.logits + g * stage_floats, bytes, &full[s]);
        ac::bulk_load(stage_labels(s), static_cast<const len_t*>(a.labels) + g * (size_t)group_rows, lbytes, &full[s]);
      };
      for (size_t it = 0; it < (size_t)n_stages && it < my_groups; ++it) issue_load(it);
      for (size_t it = 0; it < my_groups; ++it) {
        const int s = (int)(it % (size_t)n_stages);
        if (!ac::mbar_wait(&done[s], (uint32_t)((it / (size_t)n_stages) & 1))) { *failed_v = 1; break; }
        if (*failed_v) break;
        ac::bulk_store(a.dlogits + (blockIdx.x + it * gridDim.x) * stage_floats, stage_logits(s), bytes);
        ac::bulk_commit();
        if (it + n_stages < my_groups) {
          ac::bulk_wait_read<0>();  // the store has read the stage: it can take the next group
          issue_load(it + n_stages);
        }
      }
      ac::bulk_wait_all<0>();  // every store has landed before the CTA retires its shared memory
    }
  } else {
    // ---- the consumers
    for (size_t it = 0; it < my_groups; ++it) {
      const int s = (int)(it % (size_t)n_stages);
      if (!ac::mbar_wait(&full[s], (uint32_t)((it / (size_t)n_stages) & 1))) { *failed_v = 1; break; }
      if (*failed_v) break;
      // a group smaller than one trip of all warps: successive groups go to successive sets of warps
      compute_rows(stage_logits(s), stage_labels(s), group_rows, (int)((warp + it * (size_t)warps_per_group) % kWarps));
      ac::fence_async_smem();
      __syncwarp();
      if (lane == 0) ac::mbar_arrive(&done[s]);
    }
  }
  __syncthreads();
  // ---- the ragged last group: one CTA, plain loads and stores through stage 0
  if (tail_rows > 0 && blockIdx.x == (unsigned)(n_full % gridDim.x) && !failed) {
    float* st = stage_logits(0);
    len_t* lst = stage_labels(0);
    const size_t first = n_full * (size_t)group_rows;
    const float* src = a.logits + first * ld;
    for (size_t e = threadIdx.x; e < (size_t)tail_rows * ld; e += blockDim.x) st[e] = src[e];
    for (int e = threadIdx.x; e < tail_rows; e += blockDim.x) lst[e] = static_cast<const len_t*>(a.labels)[first + e];
    __syncthreads();
    if (warp < kWarps) compute_rows(st, lst, tail_rows, warp);
    __syncthreads();
    float* dst = a.dlogits + first * ld;
    for (size_t e = threadIdx.x; e < (size_t)tail_rows * ld; e += blockDim.x) dst[e] = st[e];
  }
  if (threadIdx.x == 0 && failed) *a.counter_error = 1;
  float* bias_partial = a.partial + gridDim.x;
  if (a.dbias) {
    if constexpr (SUBL > 0) {
      // the row slots of a warp hold the same columns: fold them onto slot 0 first
#pragma unroll
      for (int o = SUBL; o < 32; o <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i) bias_acc[i] += __shfl_xor_sync(0xffffffffu, bias_acc[i], o);
    }
    // per-CTA column partials, warps in a fixed order
    for (int w = 0; w < kWarps; ++w) {
      if (warp == w) {
        if constexpr (SUBL > 0) {
          if (lane < SUBL) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int j = lane * 8 + i;
              if (j < C) colsum[j] = (w == 0 ? 0.f : colsum[j]) + bias_acc[i];
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < ITEMS; ++i) {
            const int j = lane + 32 * i;
            if (j < C) colsum[j] = (w == 0 ? 0.f : colsum[j]) + bias_acc[i];
          }
        }
      }
      __syncthreads();
    }
    for (int j = threadIdx.x; j < C; j += blockDim.x) bias_partial[(size_t)blockIdx.x * C + j] = colsum[j];
  }
  smce_finish(a, loss_acc, sm32);
}

// Narrow rows (C <= 32): one THREAD per row, rows staged through shared memory.
// A CTA walks blocks of 128 rows: the block is copied in with coalesced
// (128-bit where the layout allows) loads into a shared array whose odd row
// stride keeps the thread-per-row reads conflict-free, every thread computes
// its row in registers, the gradient goes back through the same array and out
// with coalesced stores.  The bias gradient is kept per thread over all blocks
// and folded once per CTA by a 32x32 exchange-reduce per warp.
constexpr int kRowThreads = 128;
constexpr int kRowMaxW = 36;  // widest staged row: C <= 32 plus padding up to ld = 36

// global [nrows x W] (row stride ld; one contiguous block when ld == W) -> shared (row stride S)
__device__ __forceinline__ void stage_load(float* sm, int S, const float* __restrict__ g, size_t ld, int W, int nrows) {
  const int total = nrows * W;
  if (ld == (size_t)W && aligned16(g)) {
    const int nv = total >> 2;
    int r = (threadIdx.x * 4) / W, j = (threadIdx.x * 4) % W;
    const int dj = (kRowThreads * 4) % W, dr = (kRowThreads * 4) / W;
    for (int v = threadIdx.x; v < nv; v += kRowThreads) {
      const float4 q = __ldg(reinterpret_cast<const float4*>(g) + v);
      int rr = r, jj = j;
      sm[rr * S + jj] = q.x; if (++jj == W) { jj = 0; ++rr; }
      sm[rr * S + jj] = q.y; if (++jj == W) { jj = 0; ++rr; }
      sm[rr * S + jj] = q.z; if (++jj == W) { jj = 0; ++rr; }
      sm[rr * S + jj] = q.w;
      j += dj; r += dr;
      if (j >= W) { j -= W; ++r; }
    }
    for (int e = (nv << 2) + threadIdx.x; e < total; e += kRowThreads) sm[(e / W) * S + e % W] = g[e];
  } else {
    int r = threadIdx.x / W, j = threadIdx.x % W;
    const int dj = kRowThreads % W, dr = kRowThreads / W;
    for (int e = threadIdx.x; e < total; e += kRowThreads) {
      sm[r * S + j] = g[(size_t)r * ld + j];
      j += dj; r += dr;
      if (j >= W) { j -= W; ++r; }
    }
  }
}

// shared (row stride S) -> global [nrows x C] (row stride ld); adds into global when `accumulate`
__device__ __forceinline__ void stage_store(const float* sm, int S, float* g, size_t ld, int C, int nrows, bool accumulate) {
  const int total = nrows * C;
  if (ld == (size_t)C && aligned16(g)) {
    const int nv = total >> 2;
    int r = (threadIdx.x * 4) / C, j = (threadIdx.x * 4) % C;
    const int dj = (kRowThreads * 4) % C, dr = (kRowThreads * 4) / C;
    for (int v = threadIdx.x; v < nv; v += kRowThreads) {
      float4 q;
      int rr = r, jj = j;
      q.x = sm[rr * S + jj]; if (++jj == C) { jj = 0; ++rr; }
      q.y = sm[rr * S + jj]; if (++jj == C) { jj = 0; ++rr; }
      q.z = sm[rr * S + jj]; if (++jj == C) { jj = 0; ++rr; }
      q.w = sm[rr * S + jj];
      float4* dst = reinterpret_cast<float4*>(g) + v;
      if (accumulate) { const float4 o = *dst; q.x += o.x; q.y += o.y; q.z += o.z; q.w += o.w; }
      *dst = q;
      j += dj; r += dr;
      if (j >= C) { j -= C; ++r; }
    }
    for (int e = (nv << 2) + threadIdx.x; e < total; e += kRowThreads) {
      const float v = sm[(e / C) * S + e % C];
      g[e] = accumulate ? g[e] + v : v;
    }
  } else {
    int r = threadIdx.x / C, j = threadIdx.x % C;
    const int dj = kRowThreads % C, dr = kRowThreads / C;
    for (int e = threadIdx.x; e < total; e += kRowThreads) {
      const size_t o = (size_t)r * ld + j;
      const float v = sm[r * S + j];
      g[o] = accumulate ? g[o] + v : v;
      j += dj; r += dr;
      if (j >= C) { j -= C; ++r; }
    }
  }
}

__host__ __device__ constexpr int pow2_at_least(int v) { return v <= 4 ? 4 : (v <= 8 ? 8 : (v <= 16 ? 16 : 32)); }

template <int CP, bool INDEX_LABELS, bool FAST>  // CP: C rounded up to 4, 8, 12, 16, 24 or 32
__global__ void __launch_bounds__(kRowThreads) softmax_ce_row_kernel(const SmceArgs a) {
  constexpr int P2 = pow2_at_least(CP);
  __shared__ float sm32[32];
  __shared__ float wsum[kRowThreads / 32][32];
  __shared__ __align__(16) float stage[kRowThreads * (kRowMaxW + 1)];
  __shared__ __align__(16) float tstage[INDEX_LABELS ? 4 : kRowThreads * 33];
  const int C = a.C;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool block_rows = a.ld <= (size_t)kRowMaxW;  // rows and their padding form one contiguous block
  const int W = block_rows ? (int)a.ld : C;
  const int S = W | 1, ST = C | 1;
  pdl_sync();
  float gacc[P2];
#pragma unroll
  for (int j = 0; j < P2; ++j) gacc[j] = 0.f;
  float loss_acc = 0.f;
  for (size_t base = (size_t)blockIdx.x * kRowThreads; base < a.rows; base += (size_t)gridDim.x * kRowThreads) {
    const int nrows = (int)((a.rows - base) < (size_t)kRowThreads ? (a.rows - base) : (size_t)kRowThreads);
    stage_load(stage, S, a.logits + base * a.ld, a.ld, W, nrows);
    if (!INDEX_LABELS) stage_load(tstage, ST, static_cast<const float*>(a.labels) + base * (size_t)C, (size_t)C, C, nrows);
    __syncthreads();
    if ((int)threadIdx.x < nrows) {
      const size_t r = base + threadIdx.x;
      float* xs = stage + threadIdx.x * S;
      const float* tr = tstage + threadIdx.x * ST;
      float d[CP], e[CP];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < CP; ++j) {
        d[j] = (j < C) ? xs[j] : -INFINITY;
        mx = fmaxf(mx, d[j]);
      }
      int lab = -1;
      if (INDEX_LABELS) {
        const len_t l = static_cast<const len_t*>(a.labels)[r];
        lab = l < (len_t)C ? (int)l : -1;
      }
      float se = 0.f;
      const float dlab = (INDEX_LABELS && lab >= 0) ? xs[lab] - mx : 0.f;
#pragma unroll
      for (int j = 0; j < CP; ++j) {
        d[j] -= mx;                       // -inf in the padding columns: exp gives 0
        e[j] = fast_exp(d[j]);
        se += e[j];
      }
      const float inv = 1.f / se;
      const float lse = logf(se);
      if (INDEX_LABELS && lab >= 0) loss_acc -= clamp_logp(dlab - lse);
      const float sc = inv * a.inv_divisor;  // FAST: exact power-of-two scaling (see the warp kernel)
#pragma unroll
      for (int j = 0; j < CP; ++j) {
        if (j < C) {
          float g;
          if (FAST && INDEX_LABELS) {
            g = e[j] * sc;
            if (j == lab) g -= a.inv_divisor;
          } else {
            const float p = e[j] * inv;
            float t;
            if (INDEX_LABELS) t = (j == lab) ? 1.f : 0.f;
            else {
              t = tr[j];
              loss_acc -= t * clamp_logp(d[j] - lse);
            }
            if (!FAST && a.probs_out) a.probs_out[r * a.ld + j] = p;
            g = grad_scale<FAST>(a, p - t);
          }
          gacc[j] += g;
          xs[j] = g;
        }
      }
    }
    __syncthreads();
    if (FAST || a.dlogits) stage_store(stage, S, a.dlogits + base * a.ld, a.ld, C, nrows, FAST ? false : a.accumulate != 0);
    __syncthreads();
  }
  if (a.dbias) {
    // log2(P2) exchange rounds: lane l ends with the sum of column (l mod P2)
    // over the P2 lanes of its group in gacc[0]
#pragma unroll
    for (int off = P2 / 2; off >= 1; off >>= 1) {
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int j = 0; j < off; ++j) {
        const float send = upper ? gacc[j] : gacc[j + off];
        const float keep = upper ? gacc[j + off] : gacc[j];
        gacc[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
    // groups (lanes that agree modulo P2) hold partial sums of the same column
#pragma unroll
    for (int off = 16; off >= P2; off >>= 1) gacc[0] += __shfl_xor_sync(0xffffffffu, gacc[0], off);
    wsum[warp][lane] = gacc[0];
    __syncthreads();
    if ((int)threadIdx.x < C) {
      float s = 0.f;
      for (int w = 0; w < kRowThreads / 32; ++w) s += wsum[w][threadIdx.x];
      a.partial[gridDim.x + (size_t)blockIdx.x * C + threadIdx.x] = s;
    }
  }
  smce_finish(a, loss_acc, sm32);
}

// Narrow rows at scale (index labels, FAST form, unpadded 16-byte aligned
// rows): the same thread-per-row arithmetic, but the blocks of rows travel
// through a ring of shared-memory stages with bulk asynchronous copies (as in
// softmax_ce_staged_kernel) instead of being copied by the threads -- the
// staging arithmetic was about half of the narrow kernel's instructions.  A stage
// holds kNrRows rows exactly as they lie in memory (row stride C); a thread
// takes rows t, t + 128, ...  With stride C the thread-per-row reads conflict
// gcd(C, 32) ways, so the launcher uses this kernel when that is at most 4.
constexpr int kNrRows = 512;     // rows per stage
constexpr int kNrStages = 3;

template <int CP>
__global__ void __launch_bounds__(kRowThreads) softmax_ce_rows_staged_kernel(const SmceArgs a) {
  constexpr int P2 = pow2_at_least(CP);
  extern __shared__ __align__(128) unsigned char nr_raw[];
  __shared__ uint64_t full[kNrStages];
  __shared__ float sm32[32];
  __shared__ float wsum[kRowThreads / 32][32];
  __shared__ int failed;
  const int C = a.C;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t stage_floats = (size_t)kNrRows * C;
  const size_t stage_bytes = stage_floats * sizeof(float) + (size_t)kNrRows * sizeof(len_t);  // logits, then the rows' labels
  const size_t n_groups = (a.rows + kNrRows - 1) / kNrRows;
  auto stage_logits = [&](int s) -> float* { return reinterpret_cast<float*>(nr_raw + (size_t)s * stage_bytes); };
  auto stage_labels = [&](int s) -> len_t* { return reinterpret_cast<len_t*>(nr_raw + (size_t)s * stage_bytes + stage_floats * sizeof(float)); };
  if (threadIdx.x == 0) {
    for (int s = 0; s < kNrStages; ++s) ac::mbar_init(&full[s], 1);
    ac::mbar_fence_init();
    failed = 0;
  }
  __syncthreads();
  pdl_sync();
  auto rows_of = [&](size_t g) -> int { const size_t r0 = g * kNrRows; return (int)((a.rows - r0) < (size_t)kNrRows ? (a.rows - r0) : (size_t)kNrRows); };
  auto bulk_ok = [&](int nrows) -> bool { return ((size_t)nrows * C) % 4 == 0 && nrows % 2 == 0; };  // whole groups always; the ragged last one maybe not
  auto issue_load = [&](size_t g, int s) {
    const int nrows = rows_of(g);
    if (!bulk_ok(nrows)) return;
    const uint32_t bytes = (uint32_t)((size_t)nrows * C * sizeof(float)), lbytes = (uint32_t)(nrows * sizeof(len_t));
    ac::mbar_expect_tx(&full[s], bytes + lbytes);
    ac::bulk_load(stage_logits(s), a.logits + g * stage_floats, bytes, &full[s]);
    ac::bulk_load(stage_labels(s), static_cast<const len_t*>(a.labels) + g * (size_t)kNrRows, lbytes, &full[s]);
  };
  float gacc[P2];
#pragma unroll
  for (int j = 0; j < P2; ++j) gacc[j] = 0.f;
  float loss_acc = 0.f;
  if (threadIdx.x == 0) {
    for (int k = 0; k < kNrStages - 1; ++k) {
      const size_t g = blockIdx.x + (size_t)k * gridDim.x;
      if (g < n_groups) issue_load(g, k);
    }
  }
  size_t it = 0;
  for (size_t g = blockIdx.x; g < n_groups; g += gridDim.x, ++it) {
    const int s = (int)(it % kNrStages);
    const int nrows = rows_of(g);
    float* st = stage_logits(s);
    len_t* lst = stage_labels(s);
    if (threadIdx.x == 0) {
      const size_t gn = g + (size_t)(kNrStages - 1) * gridDim.x;
      if (gn < n_groups) {
        ac::bulk_wait_read<0>();  // the store of the group that used that stage has finished reading it
        issue_load(gn, (int)((it + kNrStages - 1) % kNrStages));
      }
    }
    if (bulk_ok(nrows)) {
      // (only the very last group can be ragged and skip the barrier, so the parity is a function of `it`)
      if (!ac::mbar_wait(&full[s], (uint32_t)((it / kNrStages) & 1))) failed = 1;
    } else {
      const float* src = a.logits + g * stage_floats;
      for (size_t e = threadIdx.x; e < (size_t)nrows * C; e += kRowThreads) st[e] = src[e];
      for (int e = threadIdx.x; e < nrows; e += kRowThreads) lst[e] = static_cast<const len_t*>(a.labels)[g * (size_t)kNrRows + e];
    }
    __syncthreads();
    if (failed) break;
    for (int rr = threadIdx.x; rr < nrows; rr += kRowThreads) {
      float* xs = st + (size_t)rr * C;
      float d[CP], e[CP];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < CP; ++j) {
        d[j] = (j < C) ? xs[j] : -INFINITY;
        mx = fmaxf(mx, d[j]);
      }
      const len_t l = lst[rr];
      const int lab = l < (len_t)C ? (int)l : -1;
      const float dlab = lab >= 0 ? xs[lab] - mx : 0.f;
      float se = 0.f;
#pragma unroll
      for (int j = 0; j < CP; ++j) {
        e[j] = fast_exp(d[j] - mx);
        se += e[j];
      }
      const float lse = logf(se);
      if (lab >= 0) loss_acc -= clamp_logp(dlab - lse);
      const float sc = (1.f / se) * a.inv_divisor;
#pragma unroll
      for (int j = 0; j < CP; ++j) {
        if (j < C) {
          float gv = e[j] * sc;
          if (j == lab) gv -= a.inv_divisor;
          gacc[j] += gv;
          xs[j] = gv;
        }
      }
    }
    if (bulk_ok(nrows) && (reinterpret_cast<uintptr_t>(a.dlogits) & 15u) == 0) {
      ac::fence_async_smem();
      __syncthreads();
      if (threadIdx.x == 0) {
        ac::bulk_store(a.dlogits + g * stage_floats, st, (uint32_t)((size_t)nrows * C * sizeof(float)));
        ac::bulk_commit();
      }
    } else {
      __syncthreads();
      float* dst = a.dlogits + g * stage_floats;
      for (size_t e2 = threadIdx.x; e2 < (size_t)nrows * C; e2 += kRowThreads) dst[e2] = st[e2];
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) {
    ac::bulk_wait_all<0>();
    if (failed) *a.counter_error = 1;
  }
  if (a.dbias) {
#pragma unroll
    for (int off = P2 / 2; off >= 1; off >>= 1) {
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int j = 0; j < off; ++j) {
        const float send = upper ? gacc[j] : gacc[j + off];
        const float keep = upper ? gacc[j + off] : gacc[j];
        gacc[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
#pragma unroll
    for (int off = 16; off >= P2; off >>= 1) gacc[0] += __shfl_xor_sync(0xffffffffu, gacc[0], off);
    wsum[warp][lane] = gacc[0];
    __syncthreads();
    if ((int)threadIdx.x < C) {
      float sres = 0.f;
      for (int w = 0; w < kRowThreads / 32; ++w) sres += wsum[w][threadIdx.x];
      a.partial[gridDim.x + (size_t)blockIdx.x * C + threadIdx.x] = sres;
    }
  }
  smce_finish(a, loss_acc, sm32);
}

// Rows wider than 1024: three passes over the row (values come back from L1/L2).
template <bool INDEX_LABELS>
__global__ void __launch_bounds__(kLThreads) softmax_ce_wide_kernel(const SmceArgs a) {
  __shared__ float sm32[32];
  const int lane = threadIdx.x & 31;
  const int C = a.C;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  float loss_acc = 0.f;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < a.rows; r += warps) {
    const float* xr = a.logits + r * a.ld;
    float mx = -INFINITY;
    for (int j = lane; j < C; j += 32) mx = fmaxf(mx, xr[j]);
    mx = warp_max(mx);
    float se = 0.f;
    for (int j = lane; j < C; j += 32) se += expf(xr[j] - mx);
    se = warp_sum(se);
    const float lse = mx + logf(se);
    size_t label_idx = 0;
    if (INDEX_LABELS) label_idx = static_cast<const len_t*>(a.labels)[r];
    const float* tr = INDEX_LABELS ? nullptr : static_cast<const float*>(a.labels) + r * (size_t)C;
    for (int j = lane; j < C; j += 32) {
      const float p = expf(xr[j] - lse);
      const float t = INDEX_LABELS ? ((size_t)j == label_idx ? 1.f : 0.f) : tr[j];
      const float safe = fminf(fmaxf(p, 1e-7f), 1.0f - 1e-7f);
      if (t != 0.f) loss_acc -= t * logf(safe);
      const size_t o = r * a.ld + j;
      if (a.probs_out) a.probs_out[o] = p;
      if (a.dlogits) {
        const float g = (p - t) / a.divisor;
        a.dlogits[o] = a.accumulate ? a.dlogits[o] + g : g;
      }
    }
  }
  grid_sum_store(loss_acc, sm32, a.partial, a.counter, a.loss_out, a.divisor);
}

__global__ void __launch_bounds__(kLThreads) smooth_l1_kernel(const float* __restrict__ pred, const float* __restrict__ target, size_t n,
                                                              float beta, float* loss_out, float* grad, float* partial, unsigned* counter) {
  __shared__ float sm32[32];
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  const float fn = (float)n;
  float acc = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth) {
    const float d = pred[i] - target[i];
    const float ad = fabsf(d);
    if (ad < beta) {
      acc += 0.5f * (d * d) / beta;
      if (grad) grad[i] += d / (beta * fn);
    } else {
      acc += ad - (0.5f * beta);
      if (grad) grad[i] += (float)((d > 0.f) - (d < 0.f)) / fn;
    }
  }
  grid_sum_store(acc, sm32, partial, counter, loss_out, fn);
}

// Plain row softmax / log-softmax (one warp per row, any width).
__global__ void __launch_bounds__(kLThreads) softmax_rows_kernel(const float* x, float* y, size_t rows, int C, int log_mode) {
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const float* xr = x + r * (size_t)C;
    float* yr = y + r * (size_t)C;
    float mx = -INFINITY;
    for (int j = lane; j < C; j += 32) mx = fmaxf(mx, xr[j]);
    mx = warp_max(mx);
    float se = 0.f;
    for (int j = lane; j < C; j += 32) se += expf(xr[j] - mx);
    se = warp_sum(se);
    const float lse = mx + logf(se);
    for (int j = lane; j < C; j += 32) {
      const float v = xr[j] - lse;
      yr[j] = log_mode ? v : expf(v);
    }
  }
}

// x_grd += y * (y_grd - sum_j y_j * y_grd_j) per row
__global__ void __launch_bounds__(kLThreads) softmax_rows_bwd_kernel(const float* __restrict__ y, const float* __restrict__ yg, float* xg, size_t rows, int C) {
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const size_t o = r * (size_t)C;
    float s = 0.f;
    for (int j = lane; j < C; j += 32) s += y[o + j] * yg[o + j];
    s = warp_sum(s);
    for (int j = lane; j < C; j += 32) xg[o + j] += y[o + j] * (yg[o + j] - s);
  }
}

__global__ void nll_index_fwd_kernel(const float* src, len_t trg, float* dst, len_t n, int mean) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *dst = mean ? -src[trg] / (float)n : -src[trg];
}
__global__ void nll_encode_fwd_kernel(const float* src, const float* trg, float* dst, len_t n, int mean) {
  __shared__ float sm32[32];
  float acc = 0.f;
  for (len_t i = threadIdx.x; i < n; i += blockDim.x) acc -= trg[i] * src[i];
  acc = block_sum<float>(acc, sm32);
  if (threadIdx.x == 0) *dst = mean ? acc / (float)n : acc;
}
__global__ void __launch_bounds__(kLThreads) nll_bwd_kernel(const float* __restrict__ x, const float* __restrict__ onehot, len_t trg, float* xg, len_t n, float denom) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth) {
    const float t = onehot ? onehot[i] : (i == trg ? 1.f : 0.f);
    xg[i] = (x[i] - t) / denom;
  }
}

// CTAs of `kernel` that fit on the device at once (the kernels below walk
// their rows with a grid-stride loop, so a grid of exactly this size runs as
// one wave without a tail)
template <typename K>
static unsigned resident_ctas(K kernel, int threads) {
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, 0) != cudaSuccess || occ < 1) {
    (void)cudaGetLastError();
    occ = 1;
  }
  return (unsigned)occ * (unsigned)sm_count();
}

template <int CP, bool IDX, bool FAST>
static void launch_smce_rows(cudaStream_t s, SmceArgs a) {
  static const unsigned resident = resident_ctas(softmax_ce_row_kernel<CP, IDX, FAST>, kRowThreads);
  const unsigned gr = (unsigned)std::min<size_t>((a.rows + kRowThreads - 1) / kRowThreads, resident);
  unsigned* counters = nullptr;
  float* partial = static_cast<float*>(workspace(s, sizeof(float) * ((size_t)gr + (a.dbias ? (size_t)gr * a.C : 0)), &counters));
  if (!partial) return;
  a.partial = partial;
  a.counter = counters;
  a.fold_bias_inline = 1;
  launch_pdl(softmax_ce_row_kernel<CP, IDX, FAST>, dim3(gr), dim3(kRowThreads), 0, s, a);
}

template <int ITEMS, int ROWS, bool IDX, bool FAST>
static void launch_smce_warps(cudaStream_t s, SmceArgs a) {
  static const unsigned resident = resident_ctas(softmax_ce_kernel<ITEMS, ROWS, IDX, FAST>, kLThreads);
  const int C = a.C;
  const size_t rows_per_cta = (size_t)(kLThreads / 32) * ROWS;
  unsigned g = (unsigned)std::min<size_t>((a.rows + rows_per_cta - 1) / rows_per_cta, resident);
  // The bias gradient leaves the kernel as one partial row per CTA.  Few of
  // them are folded by the last CTA to finish; many (wide rows on a large grid)
  // by a second, multi-CTA column-sum launch over the partials.
  const bool separate_fold = a.dbias && (size_t)g * C > 32768;
  unsigned* counters = nullptr;
  float* partial = static_cast<float*>(workspace(s, sizeof(float) * ((size_t)g + (a.dbias ? (size_t)g * C : 0)), &counters, separate_fold ? 1 : 0));
  if (!partial) return;
  a.partial = partial;
  a.counter = counters;
  a.fold_bias_inline = separate_fold ? 0 : 1;
  if (!launch_pdl(softmax_ce_kernel<ITEMS, ROWS, IDX, FAST>, dim3(g), dim3(kLThreads), 0, s, a)) return;
  if (separate_fold) fold_rows_f32(s, partial + g, a.dbias, g, (size_t)C);
}

template <int ITEMS, int ROWS, int SUBL = 0>
static void launch_smce_staged(cudaStream_t s, SmceArgs a) {
  const int C = a.C;
  constexpr int kWarps = kStThreads / 32;
  // rows per stage: about 32 KB (small stages keep the copies flowing smoothly), whole trips of
  // all warps, or for wide rows a power-of-two fraction of one trip; four stages (measured best: 32 KB x 4)
  static const size_t stage_target = [] { const char* e = getenv("ZG_SMCE_STAGE_KB"); return (size_t)(e ? atoi(e) : 32) * 1024; }();
  static const int max_stages = [] { const char* e = getenv("ZG_SMCE_STAGES"); const int v = e ? atoi(e) : 4; return v < 2 ? 2 : (v > kStMaxStages ? kStMaxStages : v); }();
  const size_t row_bytes = (size_t)a.ld * sizeof(float);
  constexpr int kTrip = kWarps * ROWS;
  int group_rows = (int)(stage_target / row_bytes);
  if (group_rows >= kTrip) {
    group_rows = group_rows / kTrip * kTrip;
  } else {
    int gr = kTrip;
    while (gr > 2 && gr > ROWS && (size_t)gr * row_bytes > stage_target) gr /= 2;
    group_rows = gr;
  }
  const size_t stage_bytes = (size_t)group_rows * row_bytes + (size_t)group_rows * sizeof(len_t);
  int n_stages = (int)std::min<size_t>((size_t)max_stages, ((size_t)200 * 1024) / stage_bytes);
  if (n_stages < 2) { set_error(kUnsupported, "zg_softmax_ce_fwd_bwd: rows too wide for the staged kernel"); return; }
  const size_t smem = (size_t)n_stages * stage_bytes;
  auto kern = softmax_ce_staged_kernel<ITEMS, ROWS, SUBL>;
  static bool attr_set = false;
  if (!attr_set) {
    if (!ZG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024))) return;
    attr_set = true;
  }
  const size_t n_groups = (a.rows + group_rows - 1) / group_rows;
  const unsigned g = (unsigned)std::min<size_t>(n_groups, (size_t)sm_count());
  const bool separate_fold = a.dbias && (size_t)g * C > 32768;
  unsigned* counters = nullptr;
  float* partial = static_cast<float*>(workspace(s, sizeof(float) * ((size_t)g + (a.dbias ? (size_t)g * C : 0)), &counters, separate_fold ? 1 : 0));
  if (!partial) return;
  a.partial = partial;
  a.counter = counters;
  a.fold_bias_inline = separate_fold ? 0 : 1;
  a.counter_error = reinterpret_cast<unsigned*>(kernel_timeout_flag());
  if (!a.counter_error) return;
  if (!launch_pdl(kern, dim3(g), dim3(kStLaunchThreads), smem, s, a, group_rows, n_stages)) return;
  if (separate_fold) fold_rows_f32(s, partial + g, a.dbias, g, (size_t)C);
}

template <int CP>
static void launch_smce_rows_staged(cudaStream_t s, SmceArgs a) {
  const int C = a.C;
  const size_t smem = (size_t)kNrStages * ((size_t)kNrRows * C * sizeof(float) + (size_t)kNrRows * sizeof(len_t));
  auto kern = softmax_ce_rows_staged_kernel<CP>;
  static bool attr_set = false;
  static unsigned per_sm = 1;
  if (!attr_set) {
    if (!ZG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024))) return;
    attr_set = true;
  }
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kRowThreads, smem) != cudaSuccess || occ < 1) { (void)cudaGetLastError(); occ = 1; }
  per_sm = (unsigned)occ;
  const size_t n_groups = (a.rows + kNrRows - 1) / kNrRows;
  const unsigned g = (unsigned)std::min<size_t>(n_groups, (size_t)sm_count() * per_sm);
  unsigned* counters = nullptr;
  float* partial = static_cast<float*>(workspace(s, sizeof(float) * ((size_t)g + (a.dbias ? (size_t)g * C : 0)), &counters));
  if (!partial) return;
  a.partial = partial;
  a.counter = counters;
  a.fold_bias_inline = 1;
  a.counter_error = reinterpret_cast<unsigned*>(kernel_timeout_flag());
  if (!a.counter_error) return;
  launch_pdl(kern, dim3(g), dim3(kRowThreads), smem, s, a);
}

template <bool IDX>
static void launch_softmax_ce(cudaStream_t s, SmceArgs a) {
  const int C = a.C;
  int e = 0;
  a.inv_divisor = 1.f / a.divisor;
  a.exact_inv = (std::frexp(a.divisor, &e) == 0.5f && std::isnormal(a.inv_divisor)) ? 1 : 0;
  const bool fast = a.exact_inv && a.dlogits && !a.accumulate && !a.probs_out;
#define ZG_ROWS(CPV) return fast ? launch_smce_rows<CPV, IDX, true>(s, a) : launch_smce_rows<CPV, IDX, false>(s, a)
#define ZG_WARPS(I, R) return fast ? launch_smce_warps<I, R, IDX, true>(s, a) : launch_smce_warps<I, R, IDX, false>(s, a)
  // large index-label problems with unpadded, 16-byte aligned rows: the staged kernel
  if (IDX && fast && C > 32 && C <= 1024 && C % 4 == 0 && a.ld == (size_t)C && host_aligned16(a.logits) && host_aligned16(a.dlogits) && host_aligned16(a.labels) &&
      a.rows * (size_t)C >= ((size_t)1 << 20) && (size_t)2 * 2 * C * (sizeof(float) + 2) <= 196 * 1024) {
    if (C <= 64) return launch_smce_staged<4, 4, 8>(s, a);
    if (C <= 128) return launch_smce_staged<4, 2, 16>(s, a);
    if (C <= 256) return launch_smce_staged<8, 2>(s, a);
    if (C <= 512) return launch_smce_staged<16, 1>(s, a);
    return launch_smce_staged<32, 1>(s, a);
  }
  // narrow rows at scale: the bulk-copy ring (see softmax_ce_rows_staged_kernel for the conditions)
  {
    int gcd = C, b32 = 32;
    while (b32) { const int t = gcd % b32; gcd = b32; b32 = t; }
    if (IDX && fast && C <= 32 && a.ld == (size_t)C && gcd <= 4 && host_aligned16(a.logits) && host_aligned16(a.dlogits) && host_aligned16(a.labels) &&
        a.rows * (size_t)C >= ((size_t)1 << 20)) {
      if (C <= 4) return launch_smce_rows_staged<4>(s, a);
      if (C <= 8) return launch_smce_rows_staged<8>(s, a);
      if (C <= 12) return launch_smce_rows_staged<12>(s, a);
      if (C <= 16) return launch_smce_rows_staged<16>(s, a);
      if (C <= 24) return launch_smce_rows_staged<24>(s, a);
      return launch_smce_rows_staged<32>(s, a);
    }
  }
  if (C <= 4) ZG_ROWS(4);
  if (C <= 8) ZG_ROWS(8);
  if (C <= 12) ZG_ROWS(12);
  if (C <= 16) ZG_ROWS(16);
  if (C <= 24) ZG_ROWS(24);
  if (C <= 32) ZG_ROWS(32);
  if (C <= 64) ZG_WARPS(2, 8);
  if (C <= 128) ZG_WARPS(4, 4);
  if (C <= 256) ZG_WARPS(8, 2);
  if (C <= 512) ZG_WARPS(16, 2);
  if (C <= 1024) ZG_WARPS(32, 1);
#undef ZG_ROWS
#undef ZG_WARPS
  if (a.dbias) { set_error(kUnsupported, "zg_softmax_ce_fwd_bwd: the fused bias gradient supports C <= 1024"); return; }
  unsigned g = grid_for(a.rows, kLThreads / 32, 8);
  unsigned* counters = nullptr;
  float* partial = static_cast<float*>(workspace(s, sizeof(float) * (size_t)g, &counters));
  if (!partial) return;
  a.partial = partial;
  a.counter = counters;
  softmax_ce_wide_kernel<IDX><<<g, kLThreads, 0, s>>>(a);
  ZG_LAUNCH_CHECK();
}

}  // namespace zg

using namespace zg;

extern "C" void zg_softmax_ce_fwd_bwd(dtype id, StreamWrapper w, const void* logits, const void* labels, int label_kind, len_t rows,
                                      len_t C, len_t ld, double loss_div, void* loss_out, void* dlogits, int accumulate,
                                      void* probs_out, void* dbias) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_softmax_ce_fwd_bwd: only SINGLE is implemented"); return; }
  if (rows == 0 || C == 0) return;
  if (C > (len_t)0x7fffffff) { set_error(kBadArgument, "zg_softmax_ce_fwd_bwd: C too large"); return; }
  if (ld == 0) ld = C;
  if (ld < C) { set_error(kBadArgument, "zg_softmax_ce_fwd_bwd: ld %lu < C %lu", ld, C); return; }
  SmceArgs a;
  a.logits = (const float*)logits; a.labels = labels; a.rows = rows; a.C = (int)C; a.ld = ld; a.divisor = (float)loss_div;
  a.loss_out = (float*)loss_out; a.dlogits = (float*)dlogits; a.accumulate = accumulate; a.probs_out = (float*)probs_out;
  a.dbias = (float*)dbias; a.partial = nullptr; a.counter = nullptr; a.fold_bias_inline = 1;
  cudaStream_t s = as_stream(w);
  if (label_kind == ZG_LABEL_INDEX) launch_softmax_ce<true>(s, a);
  else if (label_kind == ZG_LABEL_ONEHOT) launch_softmax_ce<false>(s, a);
  else set_error(kBadArgument, "zg_softmax_ce_fwd_bwd: unknown label kind %d", label_kind);
}

extern "C" void zg_smooth_l1_fwd_bwd(dtype id, StreamWrapper w, const void* pred, const void* target, len_t n, double beta,
                                     void* loss_out, void* grad) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_smooth_l1_fwd_bwd: only SINGLE is implemented"); return; }
  if (n == 0) return;
  cudaStream_t s = as_stream(w);
  unsigned g = grid_for(n, kLThreads * 4, 4);
  if (g > 1024) g = 1024;
  unsigned* counters = nullptr;
  float* partial = static_cast<float*>(workspace(s, sizeof(float) * g, &counters));
  if (!partial) return;
  smooth_l1_kernel<<<g, kLThreads, 0, s>>>((const float*)pred, (const float*)target, n, (float)beta, (float*)loss_out, (float*)grad, partial, counters);
  ZG_LAUNCH_CHECK();
}

static void softmax_rows(const char* name, dtype id, cudaStream_t s, const void* x, void* y, len_t m, len_t n, int log_mode) {
  if (id != SINGLE) { set_error(kUnsupported, "%s: only SINGLE is implemented", name); return; }
  if (m == 0 || n == 0) return;
  softmax_rows_kernel<<<grid_for(m, kLThreads / 32), kLThreads, 0, s>>>((const float*)x, (float*)y, m, (int)n, log_mode);
  ZG_LAUNCH_CHECK();
}
static void softmax_rows_bwd(const char* name, dtype id, cudaStream_t s, const void* y, const void* yg, void* xg, len_t m, len_t n) {
  if (id != SINGLE) { set_error(kUnsupported, "%s: only SINGLE is implemented", name); return; }
  if (m == 0 || n == 0) return;
  softmax_rows_bwd_kernel<<<grid_for(m, kLThreads / 32), kLThreads, 0, s>>>((const float*)y, (const float*)yg, (float*)xg, m, (int)n);
  ZG_LAUNCH_CHECK();
}

extern "C" void smax_vec_fwd(dtype id, CudnnWrapper w, const void* x, void* y, len_t n, smaxtype smaxop) {
  softmax_rows("smax_vec_fwd", id, as_stream(w), x, y, 1, n, smaxop == SMAX_LOG);
}
extern "C" void smax_vec_bwd(dtype id, CudnnWrapper w, const void* y_val, const void* y_grd, void* x_grd, len_t n) {
  softmax_rows_bwd("smax_vec_bwd", id, as_stream(w), y_val, y_grd, x_grd, 1, n);
}
extern "C" void smax_2D_row_fwd(dtype id, CudnnWrapper w, const void* x, void* y, len_t m, len_t n) {
  softmax_rows("smax_2D_row_fwd", id, as_stream(w), x, y, m, n, 0);
}
extern "C" void smax_2D_row_bwd(dtype id, CudnnWrapper w, const void* y_val, const void* y_grd, void* x_grd, len_t m, len_t n) {
  softmax_rows_bwd("smax_2D_row_bwd", id, as_stream(w), y_val, y_grd, x_grd, m, n);
}

extern "C" void nll_loss_1D_index_fwd(dtype id, CudnnWrapper w, void* src, len_t trg, void* dst, len_t n, bool inplace_smax, reduxtype reduxop) {
  if (id != SINGLE) { set_error(kUnsupported, "nll_loss_1D_index_fwd: only SINGLE is implemented"); return; }
  if (n == 0 || trg >= n) { set_error(kBadArgument, "nll_loss_1D_index_fwd: target %lu out of range %lu", trg, n); return; }
  if (inplace_smax) smax_vec_fwd(id, w, src, src, n, SMAX_LOG);
  nll_index_fwd_kernel<<<1, 32, 0, as_stream(w)>>>((const float*)src, trg, (float*)dst, n, reduxop != RDX_SUM);
  ZG_LAUNCH_CHECK();
}
extern "C" void nll_loss_1D_index_bwd(dtype id, CudnnWrapper w, const void* x_val, void* x_grd, len_t trg, len_t n, reduxtype reduxop) {
  if (id != SINGLE) { set_error(kUnsupported, "nll_loss_1D_index_bwd: only SINGLE is implemented"); return; }
  if (n == 0) return;
  nll_bwd_kernel<<<grid_for(n, kLThreads), kLThreads, 0, as_stream(w)>>>((const float*)x_val, nullptr, trg, (float*)x_grd, n, reduxop == RDX_SUM ? 1.f : (float)n);
  ZG_LAUNCH_CHECK();
}
extern "C" void nll_loss_1D_encode_fwd(dtype id, CudnnWrapper w, void* src, const void* trg, void* dst, len_t n, bool inplace_smax, reduxtype reduxop) {
  if (id != SINGLE) { set_error(kUnsupported, "nll_loss_1D_encode_fwd: only SINGLE is implemented"); return; }
  if (n == 0) return;
  if (inplace_smax) smax_vec_fwd(id, w, src, src, n, SMAX_LOG);
  nll_encode_fwd_kernel<<<1, kLThreads, 0, as_stream(w)>>>((const float*)src, (const float*)trg, (float*)dst, n, reduxop != RDX_SUM);
  ZG_LAUNCH_CHECK();
}
extern "C" void nll_loss_1D_encode_bwd(dtype id, CudnnWrapper w, const void* x_val, const void* y_val, void* x_grd, len_t n, reduxtype reduxop) {
  if (id != SINGLE) { set_error(kUnsupported, "nll_loss_1D_encode_bwd: only SINGLE is implemented"); return; }
  if (n == 0) return;
  nll_bwd_kernel<<<grid_for(n, kLThreads), kLThreads, 0, as_stream(w)>>>((const float*)x_val, (const float*)y_val, 0, (float*)x_grd, n, reduxop == RDX_SUM ? 1.f : (float)n);
  ZG_LAUNCH_CHECK();
}
