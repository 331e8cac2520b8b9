// fp32 GEMMs with one very short dimension (the classifier layer of an MLP:
// n = 10 outputs forward, k = 10 backward).  On the tensor-core path such a
// problem is a latency chain (descriptor fetch, first TMA round trip, operand
// split, MMA, TMEM read-back: ~7 us for 2 MB of traffic); here every thread
// issues all of its global loads at once, so a launch costs about one memory
// round trip plus the arithmetic.  Plain FFMA in fp32, sequential accumulation.
//
//   skinny_n_kernel: C[m,n] = epi(alpha A[m,k] op(B) + beta C), n <= 16, k <= 512
//       four threads per row of A, each a quarter of the row's 16-byte words;
//       B (n x k) in shared memory; quad reduction by shuffles
//   skinny_k_kernel: C[m,n] = epi(alpha A[m,k] B[k,n]), k <= 16, n <= 256
//       one thread per (row, 4 consecutive columns); B in shared memory;
//       ReLU mask and column sums (bias gradient) in the same pass
//   skinny_m_kernel: C[m,n] += alpha A[k,m]^T B[k,n], m <= 16, deep k (see below)
#pragma once

#include "common.cuh"
#include "../../include/zg_b200.h"

namespace zg {
namespace skinny {

struct Params {
  const float* A;
  const float* B;
  float* C;
  const float* bias;
  const float* mask;
  float* colsum;
  uint32_t m, n, k;
  uint32_t lda, ldb, ldc;
  float alpha, beta;
  int epilogue;
  int tb;  // B stored [n, k] (1) or [k, n] (0)
};

constexpr int kThreads = 256;

template <int NMAX>
__global__ void __launch_bounds__(kThreads) skinny_n_kernel(const Params p) {
  extern __shared__ __align__(16) float bs[];  // [n][k], k contiguous
  pdl_sync();
  const uint32_t n = p.n, k = p.k;
  const uint32_t q = threadIdx.x & 3;
  const uint32_t row = blockIdx.x * (kThreads / 4) + (threadIdx.x >> 2);
  const bool ok = row < p.m;
  const uint32_t k4 = k >> 2;
  const float4* a4 = reinterpret_cast<const float4*>(p.A + (size_t)(ok ? row : 0) * p.lda);
  // the first four words of this thread's share of the row are requested before B is staged,
  // so that (for k <= 64: all of) A arrives in the same round trip as B
  float4 first[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const uint32_t j = q + 4 * t;
    first[t] = (ok && j < k4) ? __ldg(a4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (uint32_t e = threadIdx.x; e < n * k; e += kThreads) {
    const uint32_t c = e / k, kk = e - c * k;
    bs[e] = p.tb ? p.B[(size_t)c * p.ldb + kk] : p.B[(size_t)kk * p.ldb + c];
  }
  __syncthreads();
  const float4* b4 = reinterpret_cast<const float4*>(bs);
  float acc[NMAX];
#pragma unroll
  for (int c = 0; c < NMAX; ++c) acc[c] = 0.f;
  auto mac = [&](const float4 a, const uint32_t j) {
#pragma unroll
    for (int c = 0; c < NMAX; ++c) {
      if (c < (int)n) {
        const float4 b = b4[c * k4 + j];
        acc[c] = fmaf(a.x, b.x, acc[c]);
        acc[c] = fmaf(a.y, b.y, acc[c]);
        acc[c] = fmaf(a.z, b.z, acc[c]);
        acc[c] = fmaf(a.w, b.w, acc[c]);
      }
    }
  };
#pragma unroll
  for (int t = 0; t < 4; ++t)
    if (q + 4 * t < k4) mac(first[t], q + 4 * t);
#pragma unroll 4
  for (uint32_t j = q + 16; j < k4; j += 4) mac(ok ? __ldg(a4 + j) : make_float4(0.f, 0.f, 0.f, 0.f), j);
#pragma unroll
  for (int c = 0; c < NMAX; ++c) {
    acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
    acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
  }
  if (!ok) return;
  float* crow = p.C + (size_t)row * p.ldc;
#pragma unroll
  for (int c = 0; c < NMAX; ++c) {
    if (c < (int)n && (c & 3) == (int)q) {  // the quad shares the row's stores
      float v = p.alpha * acc[c];
      if (p.beta != 0.f) v = fmaf(p.beta, crow[c], v);
      if (p.epilogue == ZG_EPI_BIAS || p.epilogue == ZG_EPI_BIAS_RELU) v += p.bias[c];
      if (p.epilogue == ZG_EPI_BIAS_RELU) v = v > 0.f ? v : 0.f;
      crow[c] = v;
    }
  }
}

template <int KMAX>
__global__ void __launch_bounds__(kThreads) skinny_k_kernel(const Params p) {
  extern __shared__ __align__(16) float bs[];  // [k][n], n contiguous, then n floats of column sums
  pdl_sync();
  const uint32_t n = p.n, k = p.k, cg = n >> 2;
  float* scol = bs + (size_t)k * n;
  const uint64_t total = (uint64_t)p.m * cg, stride = (uint64_t)gridDim.x * kThreads;
  // the operands of a thread's next output are requested one trip ahead (the first before B is staged)
  float an[KMAX];
  float4 mkn = make_float4(1.f, 1.f, 1.f, 1.f);
  auto request = [&](uint64_t idx) {
    if (idx >= total) return;
    const uint32_t row = (uint32_t)(idx / cg), g = (uint32_t)(idx - (uint64_t)row * cg);
    const float* ar = p.A + (size_t)row * p.lda;
#pragma unroll
    for (int kk = 0; kk < KMAX; ++kk) an[kk] = kk < (int)k ? __ldg(ar + kk) : 0.f;
    if (p.epilogue == ZG_EPI_RELU_MASK) mkn = __ldg(reinterpret_cast<const float4*>(p.mask + (size_t)row * p.ldc + 4 * g));
  };
  request((uint64_t)blockIdx.x * kThreads + threadIdx.x);
  for (uint32_t e = threadIdx.x; e < n * k; e += kThreads) {
    const uint32_t kk = e / n, c = e - kk * n;
    bs[e] = p.tb ? p.B[(size_t)c * p.ldb + kk] : p.B[(size_t)kk * p.ldb + c];
  }
  if (p.colsum)
    for (uint32_t e = threadIdx.x; e < n; e += kThreads) scol[e] = 0.f;
  __syncthreads();
  const float4* b4 = reinterpret_cast<const float4*>(bs);
  float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);
  uint32_t g_last = 0;
  for (uint64_t idx = (uint64_t)blockIdx.x * kThreads + threadIdx.x; idx < total; idx += stride) {
    const uint32_t row = (uint32_t)(idx / cg), g = (uint32_t)(idx - (uint64_t)row * cg);
    g_last = g;  // constant per thread: the launcher makes the stride a multiple of cg when column sums are asked for
    float a[KMAX];
#pragma unroll
    for (int kk = 0; kk < KMAX; ++kk) a[kk] = an[kk];
    const float4 mk = mkn;
    request(idx + stride);
    const size_t o = (size_t)row * p.ldc + 4 * g;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int kk = 0; kk < KMAX; ++kk) {
      if (kk < (int)k) {
        const float4 b = b4[kk * cg + g];
        acc.x = fmaf(a[kk], b.x, acc.x);
        acc.y = fmaf(a[kk], b.y, acc.y);
        acc.z = fmaf(a[kk], b.z, acc.z);
        acc.w = fmaf(a[kk], b.w, acc.w);
      }
    }
    float4 v = make_float4(p.alpha * acc.x, p.alpha * acc.y, p.alpha * acc.z, p.alpha * acc.w);
    if (p.epilogue == ZG_EPI_BIAS || p.epilogue == ZG_EPI_BIAS_RELU) {
      const float4 bb = __ldg(reinterpret_cast<const float4*>(p.bias) + g);
      v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
      if (p.epilogue == ZG_EPI_BIAS_RELU) {
        v.x = v.x > 0.f ? v.x : 0.f; v.y = v.y > 0.f ? v.y : 0.f; v.z = v.z > 0.f ? v.z : 0.f; v.w = v.w > 0.f ? v.w : 0.f;
      }
    } else if (p.epilogue == ZG_EPI_RELU_MASK) {
      if (mk.x <= 0.f) v.x = 0.f;
      if (mk.y <= 0.f) v.y = 0.f;
      if (mk.z <= 0.f) v.z = 0.f;
      if (mk.w <= 0.f) v.w = 0.f;
    }
    *reinterpret_cast<float4*>(p.C + o) = v;
    cs.x += v.x; cs.y += v.y; cs.z += v.z; cs.w += v.w;
  }
  if (p.colsum) {
    // per-CTA column sums in shared memory, then one global atomic per column and CTA
    atomicAdd(&scol[4 * g_last + 0], cs.x);
    atomicAdd(&scol[4 * g_last + 1], cs.y);
    atomicAdd(&scol[4 * g_last + 2], cs.z);
    atomicAdd(&scol[4 * g_last + 3], cs.w);
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < n; e += kThreads) atomicAdd(p.colsum + e, scol[e]);
  }
}

// C[m,n] += alpha A^T B with A stored [k, m] (m <= 16), B stored [k, n] (n a divisor of 256), deep k:
// the weight gradient of a classifier layer.  A CTA takes a block of k rows; a thread owns column
// j = t % n and every (256 / n)-th row of the block, keeps the m sums of its column in registers,
// the row groups are folded in shared memory and the CTA adds its m x n partial into C with
// one atomic per element (C holds beta C already).
template <int MMAX>
__global__ void __launch_bounds__(kThreads) skinny_m_kernel(const Params p, const uint32_t rows_per_cta) {
  extern __shared__ __align__(16) float red[];  // [256 / n][MMAX][n]
  pdl_sync();
  const uint32_t n = p.n, m = p.m, groups = kThreads / n;
  const uint32_t j = threadIdx.x % n, rg = threadIdx.x / n;
  const uint32_t r0 = blockIdx.x * rows_per_cta;
  const uint32_t r1 = (r0 + rows_per_cta < p.k) ? r0 + rows_per_cta : p.k;
  float acc[MMAX];
#pragma unroll
  for (int i = 0; i < MMAX; ++i) acc[i] = 0.f;
#pragma unroll 8
  for (uint32_t r = r0 + rg; r < r1; r += groups) {
    const float b = __ldg(p.B + (size_t)r * p.ldb + j);
    const float* ar = p.A + (size_t)r * p.lda;
#pragma unroll
    for (int i = 0; i < MMAX; ++i)
      if (i < (int)m) acc[i] = fmaf(__ldg(ar + i), b, acc[i]);
  }
#pragma unroll
  for (int i = 0; i < MMAX; ++i) red[(rg * MMAX + i) * n + j] = acc[i];
  __syncthreads();
  // n is a multiple of 16 here; four columns per atomic when C's rows allow 16-byte accesses
  const bool vec = (p.ldc & 3u) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15u) == 0;
  for (uint32_t e = threadIdx.x; e < m * (n >> 2); e += kThreads) {
    const uint32_t i = e / (n >> 2), jj = (e - i * (n >> 2)) << 2;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t g = 0; g < groups; ++g) {
      const float4 t = *reinterpret_cast<const float4*>(&red[(g * MMAX + i) * n + jj]);
      v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
    }
    v.x *= p.alpha; v.y *= p.alpha; v.z *= p.alpha; v.w *= p.alpha;
    float* dst = p.C + (size_t)i * p.ldc + jj;
    if (vec) {
      atomicAdd(reinterpret_cast<float4*>(dst), v);
    } else {
      atomicAdd(dst, v.x); atomicAdd(dst + 1, v.y); atomicAdd(dst + 2, v.z); atomicAdd(dst + 3, v.w);
    }
  }
}

}  // namespace skinny
}  // namespace zg
