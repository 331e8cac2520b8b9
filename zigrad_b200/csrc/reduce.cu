// Reductions: fold_rows / fold_cols / sum_along / max_along / unbroadcast /
// broadcast, the BLAS-1 scalars (dot, nrm2, asum, isamax-style max) and
// clip_nrm2.  Semantics follow src/device/reduce.zig:3-164 and
// src/device/host_device.zig:226-346,573-588,709-874.
//
// Every cross-CTA reduction here is two-stage inside ONE launch: CTAs write
// partials to the stream's workspace, the last CTA to finish (an atomic
// ticket) folds them in a fixed order and applies alpha/beta.  The result is
// therefore deterministic run to run; no float atomics are used.
#include <cfloat>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "../../include/blas_conflux.h"

namespace zg {

constexpr int kRThreads = 256;

// ------------------------------------------------------------ fold_rows
// x: [batch][row][col] -> y: [batch][col];  y = alpha * sum_rows + beta * y.
// Grid: (row_chunks, col_tiles, batch).  A CTA is 8 warps; with VEC a warp
// spans 128 columns (one float4 per lane) and the 8 warps take 8 rows per
// trip, 8 trips unrolled, so a CTA has 64 x 512-byte row segments in flight.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kRThreads) fold_rows_kernel(const T* __restrict__ x, T* y, T* __restrict__ partial,
                                                              unsigned* counters, size_t row, size_t col, T alpha, T beta) {
  constexpr int CW = VEC ? 4 : 1;            // columns per lane
  constexpr int TILE = 32 * CW;              // columns per CTA
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t b = blockIdx.z;
  const size_t c0 = (size_t)blockIdx.y * TILE + lane * CW;
  const size_t chunks = gridDim.x;
  const T* xb = x + b * row * col;
  T acc[CW];
#pragma unroll
  for (int j = 0; j < CW; ++j) acc[j] = T(0);
  const bool active = c0 < col;
  if (active) {
    size_t r = (size_t)blockIdx.x * 8 + warp;
    const size_t rstep = chunks * 8;
    if constexpr (VEC) {
      for (; r + 7 * rstep < row; r += 8 * rstep) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const float4*>(xb + (r + u * rstep) * col + c0);
#pragma unroll
        for (int u = 0; u < 8; ++u) { acc[0] += v[u].x; acc[1] += v[u].y; acc[2] += v[u].z; acc[3] += v[u].w; }
      }
      for (; r + 3 * rstep < row; r += 4 * rstep) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const float4*>(xb + (r + u * rstep) * col + c0);
#pragma unroll
        for (int u = 0; u < 4; ++u) { acc[0] += v[u].x; acc[1] += v[u].y; acc[2] += v[u].z; acc[3] += v[u].w; }
      }
      for (; r < row; r += rstep) {
        const float4 v = *reinterpret_cast<const float4*>(xb + r * col + c0);
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
      }
    } else {
      for (; r < row; r += rstep) acc[0] += xb[r * col + c0];
    }
  }
  __shared__ T sm[8][TILE];
#pragma unroll
  for (int j = 0; j < CW; ++j) sm[warp][lane * CW + j] = acc[j];
  __syncthreads();
  // warp 0 folds the 8 row-lanes and publishes the CTA partial
  const size_t ptile = ((b * gridDim.y + blockIdx.y) * chunks + blockIdx.x) * TILE;
  if (warp == 0) {
#pragma unroll
    for (int j = 0; j < CW; ++j) {
      T s = T(0);
#pragma unroll
      for (int w = 0; w < 8; ++w) s += sm[w][lane * CW + j];
      partial[ptile + lane * CW + j] = s;
    }
  }
  __threadfence();
  __syncthreads();
  __shared__ bool last;
  unsigned* ticket = counters + 0;
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned t = atomicAdd(ticket, 1u);
    last = (t == total - 1);
    if (last) *ticket = 0;  // leave the counter at zero for the next launch
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // final fold by the last CTA: `parts` threads share one output column (each
  // takes every parts-th chunk, four loads in flight), then a shuffle tree
  // combines them -- a fixed order, so the result is reproducible
  const size_t ntile = gridDim.y, nb = gridDim.z;
  const size_t outputs = nb * ntile * TILE;
  const unsigned parts = outputs >= 256 ? 1u : (outputs * 8 <= 256 ? 8u : (outputs * 4 <= 256 ? 4u : (outputs * 2 <= 256 ? 2u : 1u)));
  const unsigned part = threadIdx.x % parts;
  const size_t per_trip = blockDim.x / parts;
  for (size_t base = 0; base < outputs; base += per_trip) {
    const size_t idx = base + threadIdx.x / parts;
    const size_t bb = idx / (ntile * TILE), rem = idx % (ntile * TILE);
    const size_t tile = rem / TILE, cc = rem % TILE;
    const size_t c = tile * TILE + cc;
    const bool ok = idx < outputs && c < col;
    T s0 = T(0), s1 = T(0), s2 = T(0), s3 = T(0);
    if (ok) {
      const T* p = partial + ((bb * ntile + tile) * chunks) * TILE + cc;
      size_t k = part;
      for (; k + 3 * parts < chunks; k += 4 * parts) {
        s0 += __ldcg(p + k * TILE);
        s1 += __ldcg(p + (k + parts) * TILE);
        s2 += __ldcg(p + (k + 2 * parts) * TILE);
        s3 += __ldcg(p + (k + 3 * parts) * TILE);
      }
      for (; k < chunks; k += parts) s0 += __ldcg(p + k * TILE);
    }
    T s = (s0 + s1) + (s2 + s3);
    for (unsigned o = parts >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (ok && part == 0) {
      T* yo = y + bb * col + c;
      *yo = (beta == T(0)) ? alpha * s : alpha * s + beta * (*yo);
    }
  }
}

template <typename T>
void fold_rows_launch(cudaStream_t s, const T* x, T* y, size_t batch, size_t row, size_t col, T alpha, T beta) {
  if (batch == 0 || col == 0) return;
  if (row == 0) return;
  const bool vec = sizeof(T) == 4 && (col % 4 == 0) && host_aligned16(x);
  const size_t tile = vec ? 128 : 32;
  const size_t col_tiles = (col + tile - 1) / tile;
  // row chunks: enough CTAs for ~4 per SM (64 KB of loads in flight on each), at least 64 rows per CTA,
  // and a final fold that stays short (<= 64 chunks)
  size_t want = (size_t)4 * sm_count() / (col_tiles * batch);
  if (want < 1) want = 1;
  size_t by_rows = (row + 63) / 64;
  size_t chunks = want < by_rows ? want : by_rows;
  if (chunks > 64) chunks = 64;
  if (chunks < 1) chunks = 1;
  if (col_tiles > 65535 || batch > 65535) { set_error(kBadArgument, "fold_rows: shape too large (%zu col tiles, batch %zu)", col_tiles, batch); return; }
  unsigned* counters = nullptr;
  T* partial = static_cast<T*>(workspace(s, sizeof(T) * batch * col_tiles * chunks * tile, &counters));
  if (!partial) return;
  dim3 grid((unsigned)chunks, (unsigned)col_tiles, (unsigned)batch);
  if (vec) {
    if constexpr (sizeof(T) == 4) fold_rows_kernel<T, true><<<grid, kRThreads, 0, s>>>(x, y, partial, counters, row, col, alpha, beta);
  } else {
    fold_rows_kernel<T, false><<<grid, kRThreads, 0, s>>>(x, y, partial, counters, row, col, alpha, beta);
  }
  ZG_LAUNCH_CHECK();
}

void fold_rows_f32(cudaStream_t s, const float* x, float* y, size_t row, size_t col) { fold_rows_launch<float>(s, x, y, 1, row, col, 1.f, 0.f); }

// ------------------------------------------------------------ fold_cols
// [row, col] -> [row]: a warp per row (wide rows) or a thread per row.
template <typename T>
__global__ void __launch_bounds__(kRThreads) fold_cols_warp_kernel(const T* __restrict__ x, T* y, size_t row, size_t col, T alpha, T beta) {
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < row; r += warps) {
    const T* xr = x + r * col;
    T s = T(0);
    for (size_t j = lane; j < col; j += 32) s += xr[j];
    s = warp_sum(s);
    if (lane == 0) y[r] = (beta == T(0)) ? alpha * s : alpha * s + beta * y[r];
  }
}
template <typename T>
__global__ void __launch_bounds__(kRThreads) fold_cols_thread_kernel(const T* __restrict__ x, T* y, size_t row, size_t col, T alpha, T beta) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < row; r += nth) {
    const T* xr = x + r * col;
    T s = T(0);
    for (size_t j = 0; j < col; ++j) s += xr[j];
    y[r] = (beta == T(0)) ? alpha * s : alpha * s + beta * y[r];
  }
}
template <typename T>
void fold_cols_launch(cudaStream_t s, const T* x, T* y, size_t row, size_t col, T alpha, T beta) {
  if (row == 0 || col == 0) return;
  if (col <= 16) fold_cols_thread_kernel<T><<<grid_for(row, kRThreads), kRThreads, 0, s>>>(x, y, row, col, alpha, beta);
  else fold_cols_warp_kernel<T><<<grid_for(row, kRThreads / 32), kRThreads, 0, s>>>(x, y, row, col, alpha, beta);
  ZG_LAUNCH_CHECK();
}

// ------------------------------------------------------------ max_along
// x viewed as [outer][d][inner] -> y [outer][inner]; y = max over d, starting
// from -inf, strict '>' comparison (NaNs never win), as the host loop does.
template <typename T>
__global__ void __launch_bounds__(kRThreads) max_along_kernel(const T* __restrict__ x, T* __restrict__ y, size_t ylen, size_t d, size_t inner) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < ylen; i += nth) {
    const size_t base = (i / inner) * (inner * d) + (i % inner);
    T mx = -INFINITY;
    for (size_t j = 0; j < d; ++j) {
      const T v = x[base + j * inner];
      if (v > mx) mx = v;
    }
    y[i] = mx;
  }
}

// inner == 1 (the reduced dimension is the contiguous one), d > 8: a warp per
// output, lanes stride the row with 128-bit loads where the row allows.
template <typename T>
__global__ void __launch_bounds__(kRThreads) max_along_rows_kernel(const T* __restrict__ x, T* __restrict__ y, size_t rows, size_t d) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const bool vec = aligned16(x) && d % V == 0;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const T* xr = x + r * d;
    T mx = -INFINITY;
    if (vec) {
      const uint4* xv = reinterpret_cast<const uint4*>(xr);
      const size_t nv = d / V;
      size_t v = lane;
      for (; v + 96 < nv; v += 128) {
        const uint4 q[4] = {xv[v], xv[v + 32], xv[v + 64], xv[v + 96]};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const T* e = reinterpret_cast<const T*>(&q[u]);
#pragma unroll
          for (int k = 0; k < V; ++k)
            if (e[k] > mx) mx = e[k];
        }
      }
      for (; v < nv; v += 32) {
        const uint4 q = xv[v];
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int k = 0; k < V; ++k)
          if (e[k] > mx) mx = e[k];
      }
    } else {
      for (size_t j = lane; j < d; j += 32) {
        const T v = xr[j];
        if (v > mx) mx = v;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const T other = __shfl_xor_sync(0xffffffffu, mx, o);
      if (other > mx) mx = other;
    }
    if (lane == 0) y[r] = mx;
  }
}

// ------------------------------------------------- full reductions (scalars)
enum ScalarOp { kSum = 0, kAsum = 1, kNrm2 = 2, kDot = 3 };

// One launch: per-thread fp32/fp64 partials, block reduce in double, partials
// to workspace, last CTA folds them in index order.
template <typename T, int OP>
__global__ void __launch_bounds__(kRThreads) scalar_reduce_kernel(const T* __restrict__ a, const T* __restrict__ b, size_t n,
                                                                  double* __restrict__ partial, unsigned* counters, T* out,
                                                                  T alpha, T beta) {
  __shared__ double sm[32];
  const size_t nth = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  auto term = [](T v, T w) -> T {
    if (OP == kSum) return v;
    if (OP == kAsum) return v < T(0) ? -v : v;
    if (OP == kNrm2) return v * v;
    return v * w;
  };
  constexpr int V = 16 / sizeof(T);
  T acc = T(0), a1 = T(0), a2 = T(0), a3 = T(0);
  if (aligned16(a) && (OP != kDot || aligned16(b))) {
    // 128-bit loads, four per operand in flight per thread
    const uint4* av = reinterpret_cast<const uint4*>(a);
    const uint4* bv = reinterpret_cast<const uint4*>(OP == kDot ? b : a);
    const size_t nv = n / V;
    auto fold = [&](const uint4& qa, const uint4& qb, T& dst) {
      const T* ea = reinterpret_cast<const T*>(&qa);
      const T* eb = reinterpret_cast<const T*>(&qb);
#pragma unroll
      for (int e = 0; e < V; ++e) dst += term(ea[e], eb[e]);
    };
    size_t v = tid;
    for (; v + 3 * nth < nv; v += 4 * nth) {
      const uint4 q0 = av[v], q1 = av[v + nth], q2 = av[v + 2 * nth], q3 = av[v + 3 * nth];
      uint4 r0 = q0, r1 = q1, r2 = q2, r3 = q3;
      if (OP == kDot) { r0 = bv[v]; r1 = bv[v + nth]; r2 = bv[v + 2 * nth]; r3 = bv[v + 3 * nth]; }
      fold(q0, r0, acc); fold(q1, r1, a1); fold(q2, r2, a2); fold(q3, r3, a3);
    }
    for (; v < nv; v += nth) {
      const uint4 q0 = av[v];
      uint4 r0 = q0;
      if (OP == kDot) r0 = bv[v];
      fold(q0, r0, acc);
    }
    for (size_t i = nv * V + tid; i < n; i += nth) acc += term(a[i], OP == kDot ? b[i] : a[i]);
    acc = (acc + a1) + (a2 + a3);
  } else {
    for (size_t i = tid; i < n; i += nth) acc += term(a[i], OP == kDot ? b[i] : a[i]);
  }
  const double bs = block_sum<double>((double)acc, sm);
  if (threadIdx.x == 0) partial[blockIdx.x] = bs;
  __threadfence();
  __shared__ bool last;
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(counters, 1u);
    last = (t == gridDim.x - 1);
    if (last) *counters = 0;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  double s = 0.0;
  for (unsigned k = threadIdx.x; k < gridDim.x; k += blockDim.x) s += __ldcg(partial + k);
  s = block_sum<double>(s, sm);
  if (threadIdx.x == 0) {
    T r = (OP == kNrm2) ? (T)sqrt(s) : (T)s;
    *out = (beta == T(0)) ? alpha * r : alpha * r + beta * (*out);
  }
}

template <typename T, int OP>
void scalar_reduce_launch(cudaStream_t s, const T* a, const T* b, size_t n, T* out, T alpha = T(1), T beta = T(0)) {
  unsigned g = grid_for(n ? n : 1, (size_t)kRThreads * 16, 8);
  unsigned* counters = nullptr;
  double* partial = static_cast<double*>(workspace(s, sizeof(double) * g, &counters));
  if (!partial) return;
  scalar_reduce_kernel<T, OP><<<g, kRThreads, 0, s>>>(a, b, n, partial, counters, out, alpha, beta);
  ZG_LAUNCH_CHECK();
}

// isamax-style max: the element of largest magnitude, first index on ties
// (cblas_isamax; src/device/host_device.zig:573-580).
template <typename T>
__global__ void __launch_bounds__(kRThreads) amax_kernel(const T* __restrict__ x, size_t n, T* __restrict__ pval,
                                                         unsigned long long* __restrict__ pidx, unsigned* counters, T* out) {
  __shared__ T sv[kRThreads];
  __shared__ unsigned long long si[kRThreads];
  const size_t nth = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  T best = T(-1);
  unsigned long long bi = ~0ull;
  // a thread visits its elements in increasing index order, so '>' keeps the first index on ties
  auto see = [&](T v, size_t i) {
    const T m = v < T(0) ? -v : v;
    if (m > best) { best = m; bi = i; }
  };
  constexpr int V = 16 / sizeof(T);
  if (aligned16(x)) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    const size_t nv = n / V;
    size_t v = tid;
    for (; v + 3 * nth < nv; v += 4 * nth) {
      const uint4 q[4] = {xv[v], xv[v + nth], xv[v + 2 * nth], xv[v + 3 * nth]};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const T* e = reinterpret_cast<const T*>(&q[u]);
#pragma unroll
        for (int k = 0; k < V; ++k) see(e[k], (v + u * nth) * V + k);
      }
    }
    for (; v < nv; v += nth) {
      const uint4 q = xv[v];
      const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int k = 0; k < V; ++k) see(e[k], v * V + k);
    }
    // the tail holds the largest indices of all: visiting it last keeps the order
    for (size_t i = nv * V + tid; i < n; i += nth) see(x[i], i);
  } else {
    for (size_t i = tid; i < n; i += nth) see(x[i], i);
  }
  sv[threadIdx.x] = best; si[threadIdx.x] = bi;
  __syncthreads();
  for (int o = kRThreads / 2; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      const T ov = sv[threadIdx.x + o];
      const unsigned long long oi = si[threadIdx.x + o];
      if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) { pval[blockIdx.x] = sv[0]; pidx[blockIdx.x] = si[0]; }
  __threadfence();
  __shared__ bool last;
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(counters, 1u);
    last = (t == gridDim.x - 1);
    if (last) *counters = 0;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // fold the CTA partials with the whole CTA: strided pick, then the same tree
  T b = T(-1);
  unsigned long long i0 = ~0ull;
  for (unsigned k = threadIdx.x; k < gridDim.x; k += blockDim.x) {
    const T v = __ldcg(pval + k);
    const unsigned long long ii = __ldcg(pidx + k);
    if (v > b || (v == b && ii < i0)) { b = v; i0 = ii; }
  }
  __syncthreads();
  sv[threadIdx.x] = b; si[threadIdx.x] = i0;
  __syncthreads();
  for (int o = kRThreads / 2; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      const T ov = sv[threadIdx.x + o];
      const unsigned long long oi = si[threadIdx.x + o];
      if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = (si[0] == ~0ull) ? x[0] : x[si[0]];
}

template <typename T>
__global__ void __launch_bounds__(kRThreads) max_bwd_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ yg, T* xg, size_t n) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  const T val = y[0], g = yg[0];
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth)
    if (x[i] == val) xg[i] += g;
}

// x *= max/(norm+delta) when norm > max; norm is read from device memory
template <typename T>
__global__ void __launch_bounds__(kRThreads) clip_scale_kernel(T* x, size_t n, const T* __restrict__ norm, T max_norm, T delta) {
  const T nv = *norm;
  if (!(nv > max_norm)) return;
  const T f = max_norm / (nv + delta);
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth) x[i] *= f;
}

// y[i] = alpha*x[i % xl] + beta*y[i]
template <typename T>
__global__ void __launch_bounds__(kRThreads) broadcast_kernel(const T* __restrict__ x, size_t xl, T* y, size_t yl, T alpha, T beta) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
  size_t col = tid % xl;
  const size_t step = nth % xl;
  for (size_t i = tid; i < yl; i += nth) {
    y[i] = (beta == T(0)) ? alpha * x[col] : alpha * x[col] + beta * y[i];
    col += step;
    if (col >= xl) col -= xl;
  }
}

static size_t prod(const len_t* s, size_t a, size_t b) {
  size_t p = 1;
  for (size_t i = a; i < b; ++i) p *= s[i];
  return p;
}

template <typename T>
void sum_along_impl(cudaStream_t s, const T* x, const len_t* xs, size_t nd, size_t dim, T* y, T alpha, T beta) {
  if (nd == 0 || dim >= nd) { set_error(kBadArgument, "sum_along: dim %zu out of range for rank %zu", dim, nd); return; }
  const size_t total = prod(xs, 0, nd);
  if (total == 0) return;
  const size_t ylen = total / xs[dim];
  if (ylen == 1) return scalar_reduce_launch<T, kSum>(s, x, (const T*)nullptr, total, y, alpha, beta);
  if (dim == 0) return fold_rows_launch<T>(s, x, y, 1, xs[0], prod(xs, 1, nd), alpha, beta);
  if (dim + 1 == nd) return fold_cols_launch<T>(s, x, y, prod(xs, 0, dim), xs[dim], alpha, beta);
  fold_rows_launch<T>(s, x, y, prod(xs, 0, dim), xs[dim], prod(xs, dim + 1, nd), alpha, beta);
}

template <typename T>
void max_along_impl(cudaStream_t s, const T* x, const len_t* xs, size_t nd, size_t dim, T* y) {
  if (nd == 0 || dim >= nd) { set_error(kBadArgument, "max_along: dim %zu out of range for rank %zu", dim, nd); return; }
  const size_t total = prod(xs, 0, nd);
  if (total == 0) return;
  const size_t ylen = total / xs[dim];
  const size_t inner = prod(xs, dim + 1, nd);
  if (inner == 1 && xs[dim] > 8) max_along_rows_kernel<T><<<grid_for(ylen, kRThreads / 32), kRThreads, 0, s>>>(x, y, ylen, xs[dim]);
  else max_along_kernel<T><<<grid_for(ylen, kRThreads), kRThreads, 0, s>>>(x, y, ylen, xs[dim], inner);
  ZG_LAUNCH_CHECK();
}

template <typename T>
__global__ void __launch_bounds__(kRThreads) scaled_copy_kernel(const T* __restrict__ x, T* y, size_t n, T alpha, T beta) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth)
    y[i] = (beta == T(0)) ? alpha * x[i] : alpha * x[i] + beta * y[i];
}

// HostDevice.unbroadcast (src/device/host_device.zig:709-780) restated on the
// host side of the launch: the shape logic picks the same sequence of
// fold_rows / sum_along calls.  Intermediates of a multi-stage reduction live
// in the library's own workspace (two halves used alternately), not in the
// caller's `scratch`: the reference sizes that buffer from the leading dims
// only (src/ndarray.zig:697-715), which is too small when a leading fold is
// followed by an interior reduction, and it reduces scratch into scratch in
// place, which a parallel kernel cannot do.
template <typename T>
void unbroadcast_impl(cudaStream_t s, const T* x, const len_t* x_shape, size_t xnd, T* y, const len_t* y_shape, size_t ynd,
                      T alpha, T beta) {
  const size_t xlen = prod(x_shape, 0, xnd), ylen = prod(y_shape, 0, ynd);
  if (xlen == 0) return;
  if (xlen == ylen) {
    scaled_copy_kernel<T><<<grid_for(xlen, kRThreads * 4), kRThreads, 0, s>>>(x, y, xlen, alpha, beta);
    ZG_LAUNCH_CHECK();
    return;
  }
  if (xnd > 8 || ynd > 8) { set_error(kBadArgument, "unbroadcast: rank above 8"); return; }
  std::vector<len_t> xs(x_shape, x_shape + xnd), ys(y_shape, y_shape + ynd);
  while (!xs.empty() && xs.front() == 1) xs.erase(xs.begin());
  while (!ys.empty() && ys.front() == 1) ys.erase(ys.begin());
  // Trailing ones of y are dropped only together with a trailing one of x.  (The host code drops them
  // unconditionally, host_device.zig:729-731; for x [4,5,6] -> y [5,1] it then folds 20 rows of 6
  // columns into the 5-element y, one element past its end.  Here such a y dimension is reduced
  // like any interior one.)
  while (!ys.empty() && ys.back() == 1 && !xs.empty() && xs.back() == 1) { ys.pop_back(); xs.pop_back(); }
  size_t ones = 0;
  for (len_t v : ys) ones += (v == 1);
  const bool leading = xs.size() > ys.size();
  const size_t stages = (leading ? 1 : 0) + ones;
  T* half[2] = {nullptr, nullptr};
  if (stages > 1) {  // at least one intermediate result
    const size_t cap = ((xlen * sizeof(T) + 255) / 256) * 256;
    char* base = static_cast<char*>(workspace(s, 2 * cap, nullptr, 1));
    if (!base) return;
    half[0] = reinterpret_cast<T*>(base);
    half[1] = reinterpret_cast<T*>(base + cap);
  }
  const T* cur = x;
  int flip = 0;
  if (leading) {
    const size_t dif = xs.size() - ys.size();
    // alpha and beta belong to the LAST stage only: y = alpha * sum + beta * y.
    // (The host code passes them to every stage, which squares alpha and reads
    // unwritten scratch through beta whenever two stages run.)
    T* dst = ones == 0 ? y : half[flip];
    fold_rows_launch<T>(s, cur, dst, 1, prod(xs.data(), 0, dif), prod(xs.data(), dif, xs.size()), ones == 0 ? alpha : T(1),
                        ones == 0 ? beta : T(0));
    if (ones == 0) return;
    cur = dst;
    flip ^= 1;
    xs.erase(xs.begin(), xs.begin() + dif);
  }
  size_t i = 0;
  while (ones > 0 && i < xs.size()) {
    if (ys[i] == 1 && xs[i] != 1) {
      T* dst = (ones == 1) ? y : half[flip];
      sum_along_impl<T>(s, cur, xs.data(), xs.size(), i, dst, ones == 1 ? alpha : T(1), ones == 1 ? beta : T(0));
      cur = dst;
      flip ^= 1;
      xs.erase(xs.begin() + i);
      ys.erase(ys.begin() + i);
      --ones;
      continue;
    }
    ++i;
  }
}

}  // namespace zg

using namespace zg;

#define ZG_FLOAT_SWITCH(NAME, ID, BODY)                                   \
  do {                                                                    \
    if ((ID) == SINGLE) { using T = float; BODY; }                        \
    else if ((ID) == DOUBLE) { using T = double; BODY; }                  \
    else set_error(kUnsupported, NAME ": unsupported dtype %d", (int)(ID)); \
  } while (0)

extern "C" void zg_fold_rows(dtype id, StreamWrapper w, const void* x, void* y, len_t row, len_t col, double alpha, double beta) {
  ZG_FLOAT_SWITCH("zg_fold_rows", id, (fold_rows_launch<T>(as_stream(w), (const T*)x, (T*)y, 1, row, col, (T)alpha, (T)beta)));
}
extern "C" void zg_fold_cols(dtype id, StreamWrapper w, const void* x, void* y, len_t row, len_t col, double alpha, double beta) {
  ZG_FLOAT_SWITCH("zg_fold_cols", id, (fold_cols_launch<T>(as_stream(w), (const T*)x, (T*)y, row, col, (T)alpha, (T)beta)));
}
extern "C" void zg_sum_along(dtype id, StreamWrapper w, const void* x, const len_t* x_shape, len_t ndim, len_t dim, void* y,
                             double alpha, double beta) {
  ZG_FLOAT_SWITCH("zg_sum_along", id, (sum_along_impl<T>(as_stream(w), (const T*)x, x_shape, ndim, dim, (T*)y, (T)alpha, (T)beta)));
}
extern "C" void zg_max_along(dtype id, StreamWrapper w, const void* x, const len_t* x_shape, len_t ndim, len_t dim, void* y) {
  ZG_FLOAT_SWITCH("zg_max_along", id, (max_along_impl<T>(as_stream(w), (const T*)x, x_shape, ndim, dim, (T*)y)));
}
extern "C" void zg_unbroadcast(dtype id, StreamWrapper w, const void* x, const len_t* x_shape, len_t x_ndim, void* y,
                               const len_t* y_shape, len_t y_ndim, void* /*scratch: unused, see unbroadcast_impl*/, double alpha,
                               double beta) {
  ZG_FLOAT_SWITCH("zg_unbroadcast", id,
                  (unbroadcast_impl<T>(as_stream(w), (const T*)x, x_shape, x_ndim, (T*)y, y_shape, y_ndim, (T)alpha, (T)beta)));
}
extern "C" void zg_broadcast(dtype id, StreamWrapper w, const void* x, len_t x_len, void* y, len_t y_len, double alpha, double beta) {
  if (y_len == 0 || x_len == 0) return;
  ZG_FLOAT_SWITCH("zg_broadcast", id,
                  (broadcast_kernel<T><<<grid_for(y_len, kRThreads * 4), kRThreads, 0, as_stream(w)>>>((const T*)x, x_len, (T*)y, y_len, (T)alpha, (T)beta)));
  ZG_LAUNCH_CHECK();
}

extern "C" void dot(dtype id, CublasWrapper w, const void* a, const void* b, void* result, len_t n) {
  ZG_FLOAT_SWITCH("dot", id, (scalar_reduce_launch<T, kDot>(as_stream(w), (const T*)a, (const T*)b, n, (T*)result)));
}
extern "C" void nrm2(dtype id, CublasWrapper w, const void* x, void* y, len_t n) {
  ZG_FLOAT_SWITCH("nrm2", id, (scalar_reduce_launch<T, kNrm2>(as_stream(w), (const T*)x, (const T*)nullptr, n, (T*)y)));
}
extern "C" void reduce_sum(dtype id, CublasWrapper w, const void* a, void* result, len_t n) {
  ZG_FLOAT_SWITCH("reduce_sum", id, (scalar_reduce_launch<T, kAsum>(as_stream(w), (const T*)a, (const T*)nullptr, n, (T*)result)));
}

extern "C" void clip_nrm2(dtype id, CublasWrapper w, void* x, void* cur_nrm2, len_t n, double max_nrm2, double delta) {
  if (n == 0) return;
  nrm2(id, w, x, cur_nrm2, n);
  ZG_FLOAT_SWITCH("clip_nrm2", id,
                  (clip_scale_kernel<T><<<grid_for(n, kRThreads * 4), kRThreads, 0, as_stream(w)>>>((T*)x, n, (const T*)cur_nrm2, (T)max_nrm2, (T)delta)));
  ZG_LAUNCH_CHECK();
}

template <typename T>
static void max_fwd_impl(cudaStream_t s, const T* x, T* y, size_t n) {
  if (n == 0) return;
  unsigned g = grid_for(n, (size_t)kRThreads * 16, 8);
  unsigned* counters = nullptr;
  char* ws = static_cast<char*>(workspace(s, (sizeof(T) + 8) * g + 16, &counters));
  if (!ws) return;
  unsigned long long* pidx = reinterpret_cast<unsigned long long*>(ws);
  T* pval = reinterpret_cast<T*>(ws + 8 * (size_t)g);
  amax_kernel<T><<<g, kRThreads, 0, s>>>(x, n, pval, pidx, counters, y);
  ZG_LAUNCH_CHECK();
}
extern "C" void max_fwd(dtype id, StreamWrapper w, const void* x, void* y, len_t n) {
  ZG_FLOAT_SWITCH("max_fwd", id, (max_fwd_impl<T>(as_stream(w), (const T*)x, (T*)y, n)));
}
extern "C" void max_bwd(dtype id, StreamWrapper w, const void* x_val, void const* y_val, const void* y_grd, void* x_grd, len_t n) {
  if (n == 0) return;
  ZG_FLOAT_SWITCH("max_bwd", id,
                  (max_bwd_kernel<T><<<grid_for(n, kRThreads * 4), kRThreads, 0, as_stream(w)>>>((const T*)x_val, (const T*)y_val, (const T*)y_grd, (T*)x_grd, n)));
  ZG_LAUNCH_CHECK();
}

// ----------------------------------------------------------------- plans
// The reference describes reductions / permutations / contractions to
// cuTENSOR by mode letters; the same description is parsed here into the
// arguments of the kernels above.
namespace zg {
struct Plan {
  int kind;  // 0 reduce, 1 permute, 2 contraction
  dtype id;
  // reduce
  len_t shape[8];
  len_t ndim;
  len_t dim;
  BINARY_OP op;
  // permute (2-D transpose) / contraction
  len_t m, n, k, nA, nB, nC, lda, ldb, ldc;
  bool ta, tb;
};
struct PlanCache { std::vector<Plan*> plans; };
void free_plans(void* p) {
  PlanCache* c = static_cast<PlanCache*>(p);
  if (!c) return;
  for (Plan* q : c->plans) delete q;
  delete c;
}
static Plan* keep(CutensorWrapper w, const Plan& p) {
  OpContext* ctx = static_cast<OpContext*>(w.ptr);
  if (!ctx->plans) ctx->plans = new PlanCache();
  PlanCache* c = static_cast<PlanCache*>(ctx->plans);
  for (Plan* q : c->plans)
    if (memcmp(q, &p, sizeof(Plan)) == 0) return q;
  Plan* q = new Plan(p);
  c->plans.push_back(q);
  return q;
}
void bmm_dispatch(dtype id, dtype c_id, cudaStream_t s, const void* A, const void* B, void* C, len_t nA, len_t nB, len_t nC,
                  len_t m, len_t n, len_t k, bool ta, bool tb, len_t lda, len_t ldb, len_t ldc, double alpha, double beta,
                  int epilogue, const void* bias, const void* mask_src, void* colsum);
}  // namespace zg

extern "C" CutensorPlanWrapper get_reduce_plan(CutensorWrapper w, dtype id, const len_t* src_dims, const unsigned char* src_syms,
                                               len_t src_dims_len, const len_t* /*dst_dims*/, const unsigned char* dst_syms,
                                               len_t dst_dims_len, BINARY_OP op) {
  CutensorPlanWrapper out{nullptr, 0};
  if (src_dims_len == 0 || src_dims_len > 8 || dst_dims_len + 1 != src_dims_len) {
    set_error(kBadArgument, "get_reduce_plan: expected exactly one reduced mode (src rank %lu, dst rank %lu)", src_dims_len, dst_dims_len);
    return out;
  }
  Plan p;
  memset(&p, 0, sizeof(p));
  p.kind = 0; p.id = id; p.ndim = src_dims_len; p.op = op;
  p.dim = src_dims_len - 1;
  for (len_t i = 0; i < src_dims_len; ++i) p.shape[i] = src_dims[i];
  for (len_t i = 0; i < dst_dims_len; ++i)
    if (src_syms[i] != dst_syms[i]) { p.dim = i; break; }
  if (op != ADD && op != MAX) { set_error(kUnsupported, "get_reduce_plan: only ADD and MAX reductions are implemented"); return out; }
  out.plan = keep(w, p);
  return out;
}

extern "C" void reduce(CutensorWrapper w, void* plan, const void* x_vals, void* y_vals, void* /*scratch*/, len_t /*scratch_len*/,
                       const void* alpha, const void* beta) {
  Plan* p = static_cast<Plan*>(plan);
  if (!p || p->kind != 0) { set_error(kBadArgument, "reduce: not a reduce plan"); return; }
  cudaStream_t s = as_stream(w);
  if (p->id == SINGLE) {
    float a, b; memcpy(&a, alpha, 4); memcpy(&b, beta, 4);
    if (p->op == ADD) sum_along_impl<float>(s, (const float*)x_vals, p->shape, p->ndim, p->dim, (float*)y_vals, a, b);
    else max_along_impl<float>(s, (const float*)x_vals, p->shape, p->ndim, p->dim, (float*)y_vals);
  } else if (p->id == DOUBLE) {
    double a, b; memcpy(&a, alpha, 8); memcpy(&b, beta, 8);
    if (p->op == ADD) sum_along_impl<double>(s, (const double*)x_vals, p->shape, p->ndim, p->dim, (double*)y_vals, a, b);
    else max_along_impl<double>(s, (const double*)x_vals, p->shape, p->ndim, p->dim, (double*)y_vals);
  } else set_error(kUnsupported, "reduce: unsupported dtype");
}

extern "C" CutensorPlanWrapper get_permutate_plan(CutensorWrapper w, dtype id, const len_t* src_dims, const unsigned char* src_syms,
                                                  len_t src_dims_len, const len_t* /*dst_dims*/, const unsigned char* dst_syms,
                                                  len_t dst_dims_len) {
  CutensorPlanWrapper out{nullptr, 0};
  if (src_dims_len != 2 || dst_dims_len != 2 || src_syms[0] != dst_syms[1] || src_syms[1] != dst_syms[0]) {
    set_error(kUnsupported, "get_permutate_plan: only the 2-D transpose (ij -> ji) is implemented");
    return out;
  }
  Plan p;
  memset(&p, 0, sizeof(p));
  p.kind = 1; p.id = id; p.m = src_dims[0]; p.n = src_dims[1];
  out.plan = keep(w, p);
  return out;
}

namespace zg {
template <typename T>
__global__ void permute2d_kernel(const T* __restrict__ A, T* __restrict__ B, size_t m, size_t n, T alpha) {
  __shared__ T tile[32][33];
  const size_t bx = (size_t)blockIdx.x * 32, by = (size_t)blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const size_t i = by + r, j = bx + threadIdx.x;
    if (i < m && j < n) tile[r][threadIdx.x] = A[i * n + j];
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const size_t j = bx + r, i = by + threadIdx.x;
    if (i < m && j < n) B[j * m + i] = alpha * tile[threadIdx.x][r];
  }
}
}  // namespace zg

extern "C" void permutate(CutensorWrapper w, void* plan, const void* x_vals, void* y_vals, void* /*scratch*/, len_t /*scratch_len*/,
                          const void* alpha) {
  Plan* p = static_cast<Plan*>(plan);
  if (!p || p->kind != 1) { set_error(kBadArgument, "permutate: not a permutation plan"); return; }
  if (p->m == 0 || p->n == 0) return;
  dim3 grid((unsigned)((p->n + 31) / 32), (unsigned)((p->m + 31) / 32)), block(32, 8);
  if (p->id == SINGLE) {
    float a; memcpy(&a, alpha, 4);
    permute2d_kernel<float><<<grid, block, 0, as_stream(w)>>>((const float*)x_vals, (float*)y_vals, p->m, p->n, a);
  } else if (p->id == DOUBLE) {
    double a; memcpy(&a, alpha, 8);
    permute2d_kernel<double><<<grid, block, 0, as_stream(w)>>>((const double*)x_vals, (double*)y_vals, p->m, p->n, a);
  } else { set_error(kUnsupported, "permutate: unsupported dtype"); return; }
  ZG_LAUNCH_CHECK();
}

// Modes as CudaDevice.bmm_acc builds them (src/device/cuda_device.zig:284-316):
// A "ijk" (or "ikj" when transposed), B "ikm" (or "imk"), C "ijm"; the dims
// arrays hold {batch, M, K}, {batch, K, N}, {batch, M, N} of the op()-ed
// matrices.  Leading dimensions are those of contiguous storage.
extern "C" CutensorPlanWrapper get_contraction_plan(CutensorWrapper w, dtype id, const len_t* x_dims, const unsigned char* x_syms,
                                                    len_t x_dims_len, const len_t* y_dims, const unsigned char* y_syms, len_t y_dims_len,
                                                    const len_t* z_dims, const unsigned char* /*z_syms*/, len_t z_dims_len) {
  CutensorPlanWrapper out{nullptr, 0};
  if (x_dims_len != 3 || y_dims_len != 3 || z_dims_len != 3) {
    set_error(kUnsupported, "get_contraction_plan: expected rank-3 (batch, rows, cols) operands");
    return out;
  }
  Plan p;
  memset(&p, 0, sizeof(p));
  p.kind = 2; p.id = id;
  p.nA = x_dims[0]; p.nB = y_dims[0]; p.nC = z_dims[0];
  p.m = z_dims[1]; p.n = z_dims[2];
  p.ta = !(x_syms[1] == 'j');  // "ikj": contracted mode first => stored [K, M]
  p.tb = !(y_syms[1] == 'k');  // "imk": stored [N, K]
  p.k = x_dims[2];
  p.lda = p.ta ? p.m : p.k;
  p.ldb = p.tb ? p.k : p.n;
  p.ldc = p.n;
  out.plan = keep(w, p);
  return out;
}

extern "C" void contraction(CutensorWrapper w, void* plan, const void* A_vals, const void* x_vals, void* y_vals, void* /*scratch*/,
                            len_t /*scratch_len*/, const void* alpha, const void* gamma) {
  Plan* p = static_cast<Plan*>(plan);
  if (!p || p->kind != 2) { set_error(kBadArgument, "contraction: not a contraction plan"); return; }
  double a, g;
  if (p->id == SINGLE) { float fa, fg; memcpy(&fa, alpha, 4); memcpy(&fg, gamma, 4); a = fa; g = fg; }
  else if (p->id == DOUBLE) { memcpy(&a, alpha, 8); memcpy(&g, gamma, 8); }
  else { set_error(kUnsupported, "contraction: unsupported dtype"); return; }
  bmm_dispatch(p->id, p->id, as_stream(w), A_vals, x_vals, y_vals, p->nA, p->nB, p->nC, p->m, p->n, p->k, p->ta, p->tb, p->lda, p->ldb,
               p->ldc, a, g, ZG_EPI_NONE, nullptr, nullptr, nullptr);
}

// ----------------------------------------------------------------------------
// zg_fold_rows_noalloc: fold_rows for callers that must not allocate.
//
// Some users of this library run where device allocation is off the table:
// a hook that executes while a CUDA graph is being captured or replayed, a
// real-time control loop (the DQN agent acting inside a simulator tick), or a
// host process whose memory budget is fixed up front and audited.  zg_fold_rows
// keeps its cross-CTA partial sums in a workspace that the library grows with
// cudaMalloc the first time a shape needs it; this variant keeps them in a
// fixed array that is part of the library image instead.
//
// The array lives in device memory of every GPU that loads the library until
// the process exits (kNoAllocBytes, about a quarter of a megabyte).  In host
// code its NAME is only a stand-in for the symbol, not a device address; the
// address is obtained once per device with cudaGetSymbolAddress (with that
// device current) and that pointer is what the kernel receives.
//
// Sharing: there is ONE array per device.  Every call uses it and leaves its
// last partial sums behind; two calls that overlap on the GPU (different
// streams, or graphs replayed concurrently) race on it.  The ticket counter at
// its head must be zero when a kernel starts, so each call clears it on the
// caller's stream before launching.
// ----------------------------------------------------------------------------
namespace zg {
constexpr size_t kNoAllocCounterBytes = 256;
constexpr size_t kNoAllocPartialBytes = 256 * 1024;            // partial sums: 65536 floats / 32768 doubles
constexpr size_t kNoAllocBytes = kNoAllocCounterBytes + kNoAllocPartialBytes;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

static std::mutex g_noalloc_mu;
static void* g_noalloc_addr[64] = {nullptr};  // per device ordinal, resolved on first use

// Device address of the static scratch array on the current device (no allocation).
static void* noalloc_scratch_address() {
  int dev = 0;
  if (!ZG_CUDA(cudaGetDevice(&dev))) return nullptr;
  if (dev < 0 || dev >= 64) { set_error(kBadArgument, "zg_fold_rows_noalloc: device ordinal %d out of range", dev); return nullptr; }
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_addr[dev]) {
    void* ptr = nullptr;
    if (!ZG_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch))) return nullptr;
    g_noalloc_addr[dev] = ptr;
  }
  return g_noalloc_addr[dev];
}

template <typename T>
static void fold_rows_noalloc_launch(cudaStream_t s, const T* x, T* y, size_t row, size_t col, T alpha, T beta) {
  if (row == 0 || col == 0) return;
  const bool vec = sizeof(T) == 4 && (col % 4 == 0) && host_aligned16(x);
  const size_t tile = vec ? 128 : 32;
  const size_t col_tiles = (col + tile - 1) / tile;
  const size_t capacity = kNoAllocPartialBytes / sizeof(T);  // partial sums the fixed array can hold
  if (col_tiles > 65535 || col_tiles * tile > capacity) {
    set_error(kBadArgument,
              "zg_fold_rows_noalloc: %zu columns need %zu partial sums per row chunk but the fixed scratch holds %zu "
              "(limit: %zu columns for this element type and alignment); use zg_fold_rows for wider inputs",
              col, col_tiles * tile, capacity, capacity / tile * tile);
    return;
  }
  // same chunking rule as zg_fold_rows, additionally bounded by the fixed capacity
  size_t want = (size_t)2 * sm_count() / col_tiles;
  if (want < 1) want = 1;
  const size_t by_rows = (row + 63) / 64;
  size_t chunks = want < by_rows ? want : by_rows;
  if (chunks > 64) chunks = 64;
  const size_t fit = capacity / (col_tiles * tile);
  if (chunks > fit) chunks = fit;
  if (chunks < 1) chunks = 1;
  unsigned char* base = static_cast<unsigned char*>(noalloc_scratch_address());
  if (!base) return;
  unsigned* counters = reinterpret_cast<unsigned*>(base);
  T* partial = reinterpret_cast<T*>(base + kNoAllocCounterBytes);
  // the ticket counter must start at zero (an earlier call may have been cut short)
  if (!ZG_CUDA(cudaMemsetAsync(counters, 0, kNoAllocCounterBytes, s))) return;
  dim3 grid((unsigned)chunks, (unsigned)col_tiles, 1);
  if (vec) {
    if constexpr (sizeof(T) == 4) fold_rows_kernel<T, true><<<grid, kRThreads, 0, s>>>(x, y, partial, counters, row, col, alpha, beta);
  } else {
    fold_rows_kernel<T, false><<<grid, kRThreads, 0, s>>>(x, y, partial, counters, row, col, alpha, beta);
  }
  ZG_LAUNCH_CHECK();
}
}  // namespace zg

extern "C" void zg_fold_rows_noalloc(dtype id, StreamWrapper w, const void* x, void* y, len_t row, len_t col, double alpha, double beta) {
  ZG_FLOAT_SWITCH("zg_fold_rows_noalloc", id, (fold_rows_noalloc_launch<T>(as_stream(w), (const T*)x, (T*)y, row, col, (T)alpha, (T)beta)));
}
