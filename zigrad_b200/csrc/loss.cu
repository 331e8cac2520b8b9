// Losses: fused row-softmax + cross-entropy (forward and backward in one
// pass over the logits), smooth-L1, and the softmax / NLL entry points of
// include/nn_conflux.h.  Semantics: src/nn/loss.zig:130-215, :259-305.
#include <cfloat>
#include <cstring>

#include "common.cuh"
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

// One warp per row; ITEMS = ceil(C/32) logits per lane held in registers, so
// the logits are read from memory exactly once and dlogits written once.
template <int ITEMS, bool INDEX_LABELS>
__global__ void __launch_bounds__(kLThreads) softmax_ce_kernel(const float* __restrict__ logits, const void* __restrict__ labels,
                                                               size_t rows, int C, float divisor, float* loss_out,
                                                               float* dlogits, int accumulate, float* probs_out,
                                                               float* partial, unsigned* counter) {
  __shared__ float sm32[32];
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  float loss_acc = 0.f;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const float* xr = logits + r * (size_t)C;
    float x[ITEMS];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int j = lane + 32 * i;
      x[i] = (j < C) ? xr[j] : -INFINITY;
      mx = fmaxf(mx, x[i]);
    }
    mx = warp_max(mx);
    float se = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) se += (lane + 32 * i < C) ? expf(x[i] - mx) : 0.f;
    se = warp_sum(se);
    const float lse = mx + logf(se);
    size_t label_idx = 0;
    if (INDEX_LABELS) label_idx = static_cast<const len_t*>(labels)[r];
    const float* tr = INDEX_LABELS ? nullptr : static_cast<const float*>(labels) + r * (size_t)C;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int j = lane + 32 * i;
      if (j < C) {
        const float p = expf(x[i] - lse);
        const float t = INDEX_LABELS ? ((size_t)j == label_idx ? 1.f : 0.f) : tr[j];
        const float safe = fminf(fmaxf(p, 1e-7f), 1.0f - 1e-7f);
        if (t != 0.f) loss_acc -= t * logf(safe);
        const size_t o = r * (size_t)C + j;
        if (probs_out) probs_out[o] = p;
        if (dlogits) {
          const float g = (p - t) / divisor;
          dlogits[o] = accumulate ? dlogits[o] + g : g;
        }
      }
    }
  }
  grid_sum_store(loss_acc, sm32, partial, counter, loss_out, divisor);
}

// Rows wider than 1024: three passes over the row (values come back from L1/L2).
template <bool INDEX_LABELS>
__global__ void __launch_bounds__(kLThreads) softmax_ce_wide_kernel(const float* __restrict__ logits, const void* __restrict__ labels,
                                                                    size_t rows, int C, float divisor, float* loss_out,
                                                                    float* dlogits, int accumulate, float* probs_out,
                                                                    float* partial, unsigned* counter) {
  __shared__ float sm32[32];
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  float loss_acc = 0.f;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const float* xr = logits + r * (size_t)C;
    float mx = -INFINITY;
    for (int j = lane; j < C; j += 32) mx = fmaxf(mx, xr[j]);
    mx = warp_max(mx);
    float se = 0.f;
    for (int j = lane; j < C; j += 32) se += expf(xr[j] - mx);
    se = warp_sum(se);
    const float lse = mx + logf(se);
    size_t label_idx = 0;
    if (INDEX_LABELS) label_idx = static_cast<const len_t*>(labels)[r];
    const float* tr = INDEX_LABELS ? nullptr : static_cast<const float*>(labels) + r * (size_t)C;
    for (int j = lane; j < C; j += 32) {
      const float p = expf(xr[j] - lse);
      const float t = INDEX_LABELS ? ((size_t)j == label_idx ? 1.f : 0.f) : tr[j];
      const float safe = fminf(fmaxf(p, 1e-7f), 1.0f - 1e-7f);
      if (t != 0.f) loss_acc -= t * logf(safe);
      const size_t o = r * (size_t)C + j;
      if (probs_out) probs_out[o] = p;
      if (dlogits) {
        const float g = (p - t) / divisor;
        dlogits[o] = accumulate ? dlogits[o] + g : g;
      }
    }
  }
  grid_sum_store(loss_acc, sm32, partial, counter, loss_out, divisor);
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

template <bool IDX>
static void launch_softmax_ce(cudaStream_t s, const float* logits, const void* labels, size_t rows, int C, float divisor, float* loss_out,
                              float* dlogits, int accumulate, float* probs_out) {
  unsigned g = grid_for(rows, kLThreads / 32, 8);
  if (g > 2048) g = 2048;
  unsigned* counters = nullptr;
  float* partial = static_cast<float*>(workspace(s, sizeof(float) * g, &counters));
  if (!partial) return;
#define ZG_SMCE(ITEMS) softmax_ce_kernel<ITEMS, IDX><<<g, kLThreads, 0, s>>>(logits, labels, rows, C, divisor, loss_out, dlogits, accumulate, probs_out, partial, counters)
  if (C <= 32) ZG_SMCE(1);
  else if (C <= 64) ZG_SMCE(2);
  else if (C <= 128) ZG_SMCE(4);
  else if (C <= 256) ZG_SMCE(8);
  else if (C <= 512) ZG_SMCE(16);
  else if (C <= 1024) ZG_SMCE(32);
  else softmax_ce_wide_kernel<IDX><<<g, kLThreads, 0, s>>>(logits, labels, rows, C, divisor, loss_out, dlogits, accumulate, probs_out, partial, counters);
#undef ZG_SMCE
  ZG_LAUNCH_CHECK();
}

}  // namespace zg

using namespace zg;

extern "C" void zg_softmax_ce_fwd_bwd(dtype id, StreamWrapper w, const void* logits, const void* labels, int label_kind, len_t rows,
                                      len_t C, double loss_div, void* loss_out, void* dlogits, int accumulate, void* probs_out) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_softmax_ce_fwd_bwd: only SINGLE is implemented"); return; }
  if (rows == 0 || C == 0) return;
  if (C > (len_t)0x7fffffff) { set_error(kBadArgument, "zg_softmax_ce_fwd_bwd: C too large"); return; }
  cudaStream_t s = as_stream(w);
  if (label_kind == ZG_LABEL_INDEX)
    launch_softmax_ce<true>(s, (const float*)logits, labels, rows, (int)C, (float)loss_div, (float*)loss_out, (float*)dlogits, accumulate, (float*)probs_out);
  else if (label_kind == ZG_LABEL_ONEHOT)
    launch_softmax_ce<false>(s, (const float*)logits, labels, rows, (int)C, (float)loss_div, (float*)loss_out, (float*)dlogits, accumulate, (float*)probs_out);
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
