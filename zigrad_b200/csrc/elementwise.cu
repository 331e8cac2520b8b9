// Memory-bound elementwise kernels: broadcasting add/sub/mul/div, ReLU and its
// backward forms, clamp, unary maps, axpy, scale, casts, soft update.
//
// All of them stream through HBM once, so they share one skeleton: a
// grid-stride loop over 128-bit vectors (UNROLL independent loads in flight
// per thread) with a scalar tail, falling back to a scalar loop when a
// pointer is not 16-byte aligned.  Grids are sized in multiples of the SM
// count (grid_for).
#include <cstring>

#include "common.cuh"
#include "../../include/blas_conflux.h"
#include "../../include/nn_conflux.h"

namespace zg {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <typename T>
struct VecOf;
template <>
struct VecOf<float> {
  using type = float4;
  static constexpr int N = 4;
};
template <>
struct VecOf<double> {
  using type = double2;
  static constexpr int N = 2;
};

template <typename T, int N>
struct alignas(16) Pack {
  T v[N];
};

template <typename T>
__device__ __forceinline__ Pack<T, VecOf<T>::N> ldv(const T* p) {
  return *reinterpret_cast<const Pack<T, VecOf<T>::N>*>(p);
}
template <typename T>
__device__ __forceinline__ void stv(T* p, const Pack<T, VecOf<T>::N>& v) {
  *reinterpret_cast<Pack<T, VecOf<T>::N>*>(p) = v;
}

// out[i] = f(a[i], b[i], c[i]) for NIN in {1,2,3} same-length inputs.
template <typename T, int NIN, bool VEC, typename F>
__global__ void __launch_bounds__(kThreads) map_kernel(T* out, const T* a, const T* b, const T* c, size_t n, F f) {
  constexpr int N = VecOf<T>::N;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthreads = (size_t)gridDim.x * blockDim.x;
  if constexpr (VEC) {
    const size_t nvec = n / N;
    size_t v = tid;
    // unrolled body: kUnroll vectors per thread per trip, all loads first
    for (; v + (kUnroll - 1) * nthreads < nvec; v += kUnroll * nthreads) {
      Pack<T, N> ra[kUnroll], rb[kUnroll], rc[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const size_t e = (v + u * nthreads) * N;
        ra[u] = ldv(a + e);
        if constexpr (NIN >= 2) rb[u] = ldv(b + e);
        if constexpr (NIN >= 3) rc[u] = ldv(c + e);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        Pack<T, N> r;
#pragma unroll
        for (int j = 0; j < N; ++j)
          r.v[j] = f(ra[u].v[j], NIN >= 2 ? rb[u].v[j] : T(0), NIN >= 3 ? rc[u].v[j] : T(0));
        stv(out + (v + u * nthreads) * N, r);
      }
    }
    for (; v < nvec; v += nthreads) {
      const size_t e = v * N;
      Pack<T, N> ra = ldv(a + e), rb, rc, r;
      if constexpr (NIN >= 2) rb = ldv(b + e);
      if constexpr (NIN >= 3) rc = ldv(c + e);
#pragma unroll
      for (int j = 0; j < N; ++j) r.v[j] = f(ra.v[j], NIN >= 2 ? rb.v[j] : T(0), NIN >= 3 ? rc.v[j] : T(0));
      stv(out + e, r);
    }
    for (size_t i = nvec * N + tid; i < n; i += nthreads)
      out[i] = f(a[i], NIN >= 2 ? b[i] : T(0), NIN >= 3 ? c[i] : T(0));
  } else {
    for (size_t i = tid; i < n; i += nthreads) out[i] = f(a[i], NIN >= 2 ? b[i] : T(0), NIN >= 3 ? c[i] : T(0));
  }
}

template <typename T, int NIN, typename F>
void launch_map(cudaStream_t s, T* out, const T* a, const T* b, const T* c, size_t n, F f) {
  if (n == 0) return;
  bool vec = host_aligned16(out) && host_aligned16(a) && (NIN < 2 || host_aligned16(b)) && (NIN < 3 || host_aligned16(c));
  const unsigned g = grid_for(n, (size_t)kThreads * VecOf<T>::N * kUnroll);
  if (vec) map_kernel<T, NIN, true, F><<<g, kThreads, 0, s>>>(out, a, b, c, n, f);
  else map_kernel<T, NIN, false, F><<<g, kThreads, 0, s>>>(out, a, b, c, n, f);
  ZG_LAUNCH_CHECK();
}

// Broadcast binary op: `lng` has n = R*L elements, `sht` has L (L >= 1); the
// short operand index wraps.  SHORT_IS_X selects the argument order of f.
// The column of each thread's next vector is advanced incrementally (add the
// stride modulo L, subtract L on overflow) so no division runs per element.
template <typename T, bool SHORT_IS_X, bool VEC, typename F>
__global__ void __launch_bounds__(kThreads) bcast_kernel(T* out, const T* lng, const T* sht, size_t n, size_t L, F f) {
  constexpr int N = VecOf<T>::N;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthreads = (size_t)gridDim.x * blockDim.x;
  if constexpr (VEC) {
    const size_t nvec = n / N;
    size_t col = (tid * N) % L;
    const size_t step = (nthreads * N) % L;
    auto apply = [&](const Pack<T, N>& rl, size_t e) {
      Pack<T, N> r;
      size_t cj = col;
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const T sv = sht[cj];
        r.v[j] = SHORT_IS_X ? f(sv, rl.v[j]) : f(rl.v[j], sv);
        cj = (cj + 1 == L) ? 0 : cj + 1;
      }
      stv(out + e, r);
      col += step;
      if (col >= L) col -= L;
    };
    size_t v = tid;
    // four vectors of the long operand in flight per thread before the first store
    for (; v + (kUnroll - 1) * nthreads < nvec; v += kUnroll * nthreads) {
      Pack<T, N> rl[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) rl[u] = ldv(lng + (v + u * nthreads) * N);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) apply(rl[u], (v + u * nthreads) * N);
    }
    for (; v < nvec; v += nthreads) apply(ldv(lng + v * N), v * N);
    for (size_t i = nvec * N + tid; i < n; i += nthreads) {
      const T sv = sht[i % L];
      out[i] = SHORT_IS_X ? f(sv, lng[i]) : f(lng[i], sv);
    }
  } else {
    size_t col = tid % L;
    const size_t step = nthreads % L;
    for (size_t i = tid; i < n; i += nthreads) {
      const T sv = sht[col];
      out[i] = SHORT_IS_X ? f(sv, lng[i]) : f(lng[i], sv);
      col += step;
      if (col >= L) col -= L;
    }
  }
}

struct AddOp { template <typename T> __device__ T operator()(T a, T b) const { return a + b; } };
struct SubOp { template <typename T> __device__ T operator()(T a, T b) const { return a - b; } };
struct MulOp { template <typename T> __device__ T operator()(T a, T b) const { return a * b; } };
struct DivOp { template <typename T> __device__ T operator()(T a, T b) const { return a / b; } };

template <typename F>
struct As3 {  // adapts a binary functor to the 3-input map signature
  F f;
  template <typename T>
  __device__ T operator()(T a, T b, T) const { return f(a, b); }
};

// z[i] = x[i mod xl] op y[i mod yl]  (HostDevice.elwise_binop,
// src/device/host_device.zig:975-1019; CUDA reference blas/addition.cu:17-20)
template <typename T, typename F>
void binary_dispatch(cudaStream_t s, const T* x, const T* y, T* z, size_t xl, size_t yl, size_t zl, F f) {
  if (zl == 0) return;
  if (xl == 0 || yl == 0 || zl != (xl > yl ? xl : yl) || (xl > yl ? xl % yl : yl % xl) != 0) {
    set_error(kBadArgument, "elementwise: lengths %zu,%zu,%zu do not broadcast", xl, yl, zl);
    return;
  }
  if (xl == yl) return launch_map<T, 2>(s, z, x, y, (const T*)nullptr, zl, As3<F>{f});
  const bool short_is_x = xl < yl;
  const T* lng = short_is_x ? y : x;
  const T* sht = short_is_x ? x : y;
  const size_t L = short_is_x ? xl : yl;
  const bool vec = host_aligned16(z) && host_aligned16(lng);
  const unsigned g = grid_for(zl, (size_t)kThreads * VecOf<T>::N * 2);
  if (short_is_x) {
    if (vec) bcast_kernel<T, true, true, F><<<g, kThreads, 0, s>>>(z, lng, sht, zl, L, f);
    else bcast_kernel<T, true, false, F><<<g, kThreads, 0, s>>>(z, lng, sht, zl, L, f);
  } else {
    if (vec) bcast_kernel<T, false, true, F><<<g, kThreads, 0, s>>>(z, lng, sht, zl, L, f);
    else bcast_kernel<T, false, false, F><<<g, kThreads, 0, s>>>(z, lng, sht, zl, L, f);
  }
  ZG_LAUNCH_CHECK();
}

template <typename F>
void binary_entry(const char* name, dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t xl, len_t yl,
                  len_t zl, F f) {
  cudaStream_t s = as_stream(w);
  if (id == SINGLE) binary_dispatch<float>(s, (const float*)x, (const float*)y, (float*)z, xl, yl, zl, f);
  else if (id == DOUBLE) binary_dispatch<double>(s, (const double*)x, (const double*)y, (double*)z, xl, yl, zl, f);
  else set_error(kUnsupported, "%s: unsupported dtype %d", name, (int)id);
}

// ---------------------------------------------------------------- functors
// relu: Zig's @max(0, x) returns 0 for NaN input (the non-NaN operand); `x > 0
// ? x : 0` has the same table, including -0.0 -> +0.0.
struct ReluF { template <typename T> __device__ T operator()(T x, T, T) const { return x > T(0) ? x : T(0); } };
// relu_bwd: x_g += (x > 0) ? y_g : 0     inputs (x, y_g, x_g)
struct ReluBwdF { template <typename T> __device__ T operator()(T x, T yg, T xg) const { return xg + (x > T(0) ? yg : T(0)); } };
// relu_inplace_bwd: if (x <= 0) x_g = 0  inputs (x, x_g)
struct ReluInplaceBwdF { template <typename T> __device__ T operator()(T x, T xg, T) const { return x <= T(0) ? T(0) : xg; } };
template <typename T>
struct ClampF {
  T lo, hi;
  __device__ T operator()(T x, T, T) const {
    // @min(hi, @max(lo, x)) with Zig's NaN rule (NaN operand is dropped)
    T t = (x > lo || lo != lo) ? x : lo;  // max(lo, x)
    if (x != x) t = lo;
    return (t < hi) ? t : hi;
  }
};
template <typename T>
struct ClampBwdF {  // inputs (x, y_g, x_g)
  T lo, hi;
  __device__ T operator()(T x, T yg, T xg) const { return (lo < x && x < hi) ? xg + yg : xg; }
};
template <typename T>
struct AxpyF {  // inputs (x, y): y + a*x, rounded as two operations like a CPU axpy without FMA contraction
  T a;
  __device__ T operator()(T x, T y, T) const { return y + a * x; }
};
template <typename T>
struct AxpyPtrF {  // alpha read from device memory
  const T* a;
  __device__ T operator()(T x, T y, T) const { return y + (*a) * x; }
};
template <typename T>
struct ScaleF {
  T a;
  __device__ T operator()(T x, T, T) const { return x * a; }
};
template <typename T>
struct SoftUpdateF {  // inputs (src, target)
  T tau;
  __device__ T operator()(T s, T t, T) const { return tau * s + (T(1) - tau) * t; }
};

__device__ __forceinline__ float dev_exp(float x) { return expf(x); }
__device__ __forceinline__ double dev_exp(double x) { return exp(x); }
__device__ __forceinline__ float dev_sqrt(float x) { return sqrtf(x); }
__device__ __forceinline__ double dev_sqrt(double x) { return sqrt(x); }
__device__ __forceinline__ float dev_tanh(float x) { return tanhf(x); }
__device__ __forceinline__ double dev_tanh(double x) { return tanh(x); }

__device__ __forceinline__ float dev_pow(float x, float e) { return powf(x, e); }
__device__ __forceinline__ double dev_pow(double x, double e) { return pow(x, e); }

template <typename T>
struct UnaryF {
  int op;
  T p;
  __device__ T operator()(T x, T, T) const {
    switch (op) {
      case ZG_UN_POW: return dev_pow(x, p);  // p = exponent
      case ZG_UN_EXP: return dev_exp(x);
      case ZG_UN_SQRT: return dev_sqrt(x);
      case ZG_UN_RSQRT: return T(1) / dev_sqrt(x > p ? x : p);  // 1/sqrt(max(x, eps))
      case ZG_UN_TANH: return dev_tanh(x);
      default: return T(1) / (T(1) + dev_exp(-x));
    }
  }
};
template <typename T>
struct UnaryBwdF {  // inputs (v, y_g, x_g)
  int op;
  T p;
  __device__ T operator()(T v, T yg, T xg) const {
    switch (op) {
      case ZG_UN_EXP: return xg + v * yg;
      case ZG_UN_SQRT: return (v < p) ? xg : xg + T(0.5) / dev_sqrt(v) * yg;
      case ZG_UN_RSQRT: {
        if (v < p) return xg;
        const T inv = T(1) / (v * dev_sqrt(v));
        return xg + (T(-0.5) * inv) * yg;
      }
      case ZG_UN_TANH: return xg + (T(1) - v * v) * yg;
      default: return xg + v * (T(1) - v) * yg;
    }
  }
};

// pow_bwd (host_device.zig:365-379): x_g += exp * x^(exp-1) * y_g, nothing where x < eps.  inputs (x, y_g, x_g)
template <typename T>
struct PowBwdF {
  T e, em1, eps;
  __device__ T operator()(T x, T yg, T xg) const { return (x < eps) ? xg : xg + e * dev_pow(x, em1) * yg; }
};
// tanh_inplace_bwd / sigm_inplace_bwd (host_device.zig:557-559, 569-571): the gradient is rescaled in
// place by the derivative written in terms of the activation's OUTPUT x.  inputs (x, x_g)
struct TanhInplaceBwdF { template <typename T> __device__ T operator()(T x, T xg, T) const { return xg * (T(1) - (x * x)); } };
struct SigmInplaceBwdF { template <typename T> __device__ T operator()(T x, T xg, T) const { return xg * (x * (T(1) - x)); } };

// ------------------------------------------------------------ byte-mask ops
// One bit per element, eight elements per mask byte, bit b of byte i/8 for
// element i (std.bit_set.IntegerBitSet(8), host_device.zig:16).  A thread owns
// the eight elements of one mask byte: two 128-bit accesses per operand when the
// pointers allow, one byte store (or load) for the mask.
//   MODE 0 relu_mask_fwd  (host_device.zig:652-678): x <= 0 -> x = 0, bit set
//   MODE 1 relu_mask_bwd  (:680-701):                bit set -> x_g = 0
//   MODE 2 clamp_mask_fwd (:600-628): y = x (the reference stores the unclamped value), bit set where
//                                      clamping changes x
//   MODE 3 clamp_mask_bwd (:630-650): bit set -> x_g += y_g
template <typename T, int MODE>
__global__ void __launch_bounds__(kThreads) byte_mask_kernel(T* a, const T* b, unsigned char* mask, size_t n, T lo, T hi) {
  const size_t nbytes = (n + 7) / 8, nth = (size_t)gridDim.x * blockDim.x;
  const bool vec = aligned16(a) && (b == nullptr || aligned16(b));
  ClampF<T> cl{lo, hi};
  for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < nbytes; g += nth) {
    const size_t e0 = g * 8;
    const int cnt = (int)((n - e0) < 8 ? (n - e0) : 8);
    T va[8], vb[8];
    const T* src = (MODE == 2) ? b : a;  // clamp_mask_fwd reads x (b) and writes y (a)
    if (cnt == 8 && vec) {
      constexpr int N = VecOf<T>::N;
#pragma unroll
      for (int q = 0; q < 8 / N; ++q) {
        const Pack<T, N> pk = ldv(src + e0 + q * N);
#pragma unroll
        for (int j = 0; j < N; ++j) va[q * N + j] = pk.v[j];
        if constexpr (MODE == 3) {
          const Pack<T, N> pb = ldv(b + e0 + q * N);
#pragma unroll
          for (int j = 0; j < N; ++j) vb[q * N + j] = pb.v[j];
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        va[j] = j < cnt ? src[e0 + j] : T(0);
        if constexpr (MODE == 3) vb[j] = j < cnt ? b[e0 + j] : T(0);
      }
    }
    unsigned bits = (MODE == 1 || MODE == 3) ? mask[g] : 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if constexpr (MODE == 0) {
        if (j < cnt && va[j] <= T(0)) { va[j] = T(0); bits |= 1u << j; }
      } else if constexpr (MODE == 1) {
        if (bits & (1u << j)) va[j] = T(0);
      } else if constexpr (MODE == 2) {
        if (j < cnt && va[j] != cl(va[j], T(0), T(0))) bits |= 1u << j;
      } else {
        if (bits & (1u << j)) va[j] = va[j] + vb[j];
      }
    }
    if constexpr (MODE == 0 || MODE == 2) mask[g] = (unsigned char)bits;
    if (cnt == 8 && vec) {
      constexpr int N = VecOf<T>::N;
#pragma unroll
      for (int q = 0; q < 8 / N; ++q) {
        Pack<T, N> pk;
#pragma unroll
        for (int j = 0; j < N; ++j) pk.v[j] = va[q * N + j];
        stv(a + e0 + q * N, pk);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < cnt) a[e0 + j] = va[j];
    }
  }
}

template <typename T, int MODE>
void launch_byte_mask(cudaStream_t s, T* a, const T* b, unsigned char* mask, size_t n, T lo, T hi) {
  if (n == 0) return;
  byte_mask_kernel<T, MODE><<<grid_for((n + 7) / 8, kThreads * 2), kThreads, 0, s>>>(a, b, mask, n, lo, hi);
  ZG_LAUNCH_CHECK();
}

// fp32 <-> bf16 casts
__global__ void __launch_bounds__(kThreads) f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
  const bool vec = aligned16(src) && ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0);
  if (vec) {
    const size_t nv = n / 4;
    for (size_t v = tid; v < nv; v += nth) {
      const float4 f = reinterpret_cast<const float4*>(src)[v];
      __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(dst)[v] = o;
    }
    for (size_t i = nv * 4 + tid; i < n; i += nth) dst[i] = __float2bfloat16_rn(src[i]);
  } else {
    for (size_t i = tid; i < n; i += nth) dst[i] = __float2bfloat16_rn(src[i]);
  }
}
__global__ void __launch_bounds__(kThreads) bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, size_t n) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
  if (((reinterpret_cast<uintptr_t>(src) & 7u) == 0) && aligned16(dst)) {
    // 4 elements per thread and trip: one 64-bit load, ONE 128-bit store, so that a warp's store covers
    // 512 contiguous bytes (with 8 elements per thread its two stores each touched every other 16 bytes);
    // eight trips in flight per thread
    const size_t nv = n / 4;
    auto put = [&](const uint2& q, size_t v) {  // a bfloat16 is the upper half of the fp32 with the same value
      float4 o;
      o.x = __uint_as_float(q.x << 16); o.y = __uint_as_float(q.x & 0xffff0000u);
      o.z = __uint_as_float(q.y << 16); o.w = __uint_as_float(q.y & 0xffff0000u);
      reinterpret_cast<float4*>(dst)[v] = o;
    };
    const uint2* sv = reinterpret_cast<const uint2*>(src);
    size_t v = tid;
    for (; v + 7 * nth < nv; v += 8 * nth) {
      uint2 q[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) q[u] = sv[v + u * nth];
#pragma unroll
      for (int u = 0; u < 8; ++u) put(q[u], v + u * nth);
    }
    for (; v < nv; v += nth) put(sv[v], v);
    for (size_t i = nv * 4 + tid; i < n; i += nth) dst[i] = __bfloat162float(src[i]);
  } else {
    for (size_t i = tid; i < n; i += nth) dst[i] = __bfloat162float(src[i]);
  }
}

// B[n, m] = A[m, n]^T + alpha * B through a 64x64 shared tile: 128-bit loads
// along A's rows, 128-bit stores along B's rows (needs m % 4 == n % 4 == 0
// and 16-byte aligned bases; fp32 only).
__global__ void __launch_bounds__(256) transpose64_kernel(const float* __restrict__ A, float* __restrict__ B, size_t m, size_t n, float alpha) {
  __shared__ float tile[64][65];
  const size_t bx = (size_t)blockIdx.x * 64, by = (size_t)blockIdx.y * 64;
  const int q = threadIdx.x & 15, r0 = threadIdx.x >> 4;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = r0 + 16 * k;
    const size_t i = by + r, j = bx + 4 * q;
    if (i < m && j < n) {
      const float4 v = *reinterpret_cast<const float4*>(A + i * n + j);
      tile[r][4 * q] = v.x; tile[r][4 * q + 1] = v.y; tile[r][4 * q + 2] = v.z; tile[r][4 * q + 3] = v.w;
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = r0 + 16 * k;                       // row of B inside the tile = column of A
    const size_t j = bx + r, i = by + 4 * q;
    if (j < n && i < m) {
      float4 v;
      v.x = tile[4 * q][r]; v.y = tile[4 * q + 1][r]; v.z = tile[4 * q + 2][r]; v.w = tile[4 * q + 3][r];
      float4* dst = reinterpret_cast<float4*>(B + j * m + i);
      if (alpha != 0.f) {
        const float4 o = *dst;
        v.x += alpha * o.x; v.y += alpha * o.y; v.z += alpha * o.z; v.w += alpha * o.w;
      }
      *dst = v;
    }
  }
}

template <typename T>
__global__ void transpose_kernel(const T* __restrict__ A, T* __restrict__ B, size_t m, size_t n, T alpha) {
  __shared__ T tile[32][33];
  const size_t bx = (size_t)blockIdx.x * 32, by = (size_t)blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const size_t i = by + r, j = bx + threadIdx.x;
    if (i < m && j < n) tile[r][threadIdx.x] = A[i * n + j];
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const size_t j = bx + r, i = by + threadIdx.x;  // B is [n, m]
    if (i < m && j < n) {
      const T prev = (alpha == T(0)) ? T(0) : alpha * B[j * m + i];
      B[j * m + i] = tile[threadIdx.x][r] + prev;
    }
  }
}

static bool is_device_pointer(const void* p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

}  // namespace zg

using namespace zg;

#define ZG_FLOAT_SWITCH(NAME, ID, BODY)                                   \
  do {                                                                    \
    if ((ID) == SINGLE) { using T = float; BODY; }                        \
    else if ((ID) == DOUBLE) { using T = double; BODY; }                  \
    else set_error(kUnsupported, NAME ": unsupported dtype %d", (int)(ID)); \
  } while (0)

extern "C" void addition(dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t xl, len_t yl, len_t zl) {
  binary_entry("addition", id, w, x, y, z, xl, yl, zl, AddOp{});
}
extern "C" void subtraction(dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t xl, len_t yl, len_t zl) {
  binary_entry("subtraction", id, w, x, y, z, xl, yl, zl, SubOp{});
}
extern "C" void multiplication(dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t xl, len_t yl, len_t zl) {
  binary_entry("multiplication", id, w, x, y, z, xl, yl, zl, MulOp{});
}
extern "C" void division(dtype id, StreamWrapper w, const void* x, const void* y, void* z, len_t xl, len_t yl, len_t zl) {
  binary_entry("division", id, w, x, y, z, xl, yl, zl, DivOp{});
}

extern "C" void relu_fwd(dtype id, StreamWrapper w, const void* x, void* y, len_t n) {
  ZG_FLOAT_SWITCH("relu_fwd", id, (launch_map<T, 1>(as_stream(w), (T*)y, (const T*)x, (const T*)nullptr, (const T*)nullptr, n, ReluF{})));
}
extern "C" void relu_bwd(dtype id, StreamWrapper w, const void* x, const void* y_grd, void* x_grd, len_t n) {
  ZG_FLOAT_SWITCH("relu_bwd", id, (launch_map<T, 3>(as_stream(w), (T*)x_grd, (const T*)x, (const T*)y_grd, (const T*)x_grd, n, ReluBwdF{})));
}
extern "C" void zg_relu_inplace_bwd(dtype id, StreamWrapper w, const void* x, void* x_g, len_t n) {
  ZG_FLOAT_SWITCH("zg_relu_inplace_bwd", id, (launch_map<T, 2>(as_stream(w), (T*)x_g, (const T*)x, (const T*)x_g, (const T*)nullptr, n, ReluInplaceBwdF{})));
}
extern "C" void clamp(dtype id, StreamWrapper w, const void* x, void* y, len_t n, double lower, double upper) {
  ZG_FLOAT_SWITCH("clamp", id, (launch_map<T, 1>(as_stream(w), (T*)y, (const T*)x, (const T*)nullptr, (const T*)nullptr, n, ClampF<T>{(T)lower, (T)upper})));
}
extern "C" void zg_clamp_bwd(dtype id, StreamWrapper w, const void* x, const void* y_g, void* x_g, len_t n, double lo, double hi) {
  ZG_FLOAT_SWITCH("zg_clamp_bwd", id, (launch_map<T, 3>(as_stream(w), (T*)x_g, (const T*)x, (const T*)y_g, (const T*)x_g, n, ClampBwdF<T>{(T)lo, (T)hi})));
}
extern "C" void pow_exp(dtype id, StreamWrapper w, const void* x, void* y, len_t n) {
  zg_unary_fwd(id, w, ZG_UN_EXP, x, y, n, 0.0);
}
extern "C" void zg_unary_fwd(dtype id, StreamWrapper w, int op, const void* x, void* y, len_t n, double p) {
  if (op < ZG_UN_EXP || op > ZG_UN_POW) { set_error(kBadArgument, "zg_unary_fwd: unknown op %d", op); return; }
  ZG_FLOAT_SWITCH("zg_unary_fwd", id, (launch_map<T, 1>(as_stream(w), (T*)y, (const T*)x, (const T*)nullptr, (const T*)nullptr, n, UnaryF<T>{op, (T)p})));
}
extern "C" void zg_unary_bwd(dtype id, StreamWrapper w, int op, const void* v, const void* y_g, void* x_g, len_t n, double p) {
  if (op < ZG_UN_EXP || op > ZG_UN_SIGM) { set_error(kBadArgument, "zg_unary_bwd: unknown op %d", op); return; }
  ZG_FLOAT_SWITCH("zg_unary_bwd", id, (launch_map<T, 3>(as_stream(w), (T*)x_g, (const T*)v, (const T*)y_g, (const T*)x_g, n, UnaryBwdF<T>{op, (T)p})));
}

extern "C" void zg_pow_bwd(dtype id, StreamWrapper w, const void* x, const void* y_g, void* x_g, len_t n, double exponent, double eps) {
  ZG_FLOAT_SWITCH("zg_pow_bwd", id, (launch_map<T, 3>(as_stream(w), (T*)x_g, (const T*)x, (const T*)y_g, (const T*)x_g, n,
                                                      PowBwdF<T>{(T)exponent, (T)exponent - T(1), (T)(float)eps})));
}
extern "C" void zg_unary_inplace_bwd(dtype id, StreamWrapper w, int op, const void* x, void* x_g, len_t n) {
  if (op == ZG_UN_TANH) {
    ZG_FLOAT_SWITCH("zg_unary_inplace_bwd", id, (launch_map<T, 2>(as_stream(w), (T*)x_g, (const T*)x, (const T*)x_g, (const T*)nullptr, n, TanhInplaceBwdF{})));
  } else if (op == ZG_UN_SIGM) {
    ZG_FLOAT_SWITCH("zg_unary_inplace_bwd", id, (launch_map<T, 2>(as_stream(w), (T*)x_g, (const T*)x, (const T*)x_g, (const T*)nullptr, n, SigmInplaceBwdF{})));
  } else {
    set_error(kBadArgument, "zg_unary_inplace_bwd: op %d has no in-place backward (tanh and sigmoid do)", op);
  }
}
extern "C" void zg_relu_mask_fwd(dtype id, StreamWrapper w, void* x, unsigned char* mask, len_t n) {
  ZG_FLOAT_SWITCH("zg_relu_mask_fwd", id, (launch_byte_mask<T, 0>(as_stream(w), (T*)x, (const T*)nullptr, mask, n, T(0), T(0))));
}
extern "C" void zg_relu_mask_bwd(dtype id, StreamWrapper w, void* x_g, const unsigned char* mask, len_t n) {
  ZG_FLOAT_SWITCH("zg_relu_mask_bwd", id, (launch_byte_mask<T, 1>(as_stream(w), (T*)x_g, (const T*)nullptr, const_cast<unsigned char*>(mask), n, T(0), T(0))));
}
extern "C" void zg_clamp_mask_fwd(dtype id, StreamWrapper w, const void* x, void* y, unsigned char* mask, len_t n, double lo, double hi) {
  ZG_FLOAT_SWITCH("zg_clamp_mask_fwd", id, (launch_byte_mask<T, 2>(as_stream(w), (T*)y, (const T*)x, mask, n, (T)lo, (T)hi)));
}
extern "C" void zg_clamp_mask_bwd(dtype id, StreamWrapper w, void* x_g, const void* y_g, const unsigned char* mask, len_t n) {
  ZG_FLOAT_SWITCH("zg_clamp_mask_bwd", id, (launch_byte_mask<T, 3>(as_stream(w), (T*)x_g, (const T*)y_g, const_cast<unsigned char*>(mask), n, T(0), T(0))));
}

extern "C" void scale(dtype id, CublasWrapper w, void* a_data, len_t n, double alpha) {
  ZG_FLOAT_SWITCH("scale", id, (launch_map<T, 1>(as_stream(w), (T*)a_data, (const T*)a_data, (const T*)nullptr, (const T*)nullptr, n, ScaleF<T>{(T)alpha})));
}

extern "C" void axpy(dtype id, CublasWrapper w, const void* x, void* y, len_t n, const void* alpha) {
  const bool dev = is_device_pointer(alpha);
  if (id == SINGLE) {
    if (dev) launch_map<float, 2>(as_stream(w), (float*)y, (const float*)x, (const float*)y, (const float*)nullptr, n, AxpyPtrF<float>{(const float*)alpha});
    else { float a; memcpy(&a, alpha, 4); launch_map<float, 2>(as_stream(w), (float*)y, (const float*)x, (const float*)y, (const float*)nullptr, n, AxpyF<float>{a}); }
  } else if (id == DOUBLE) {
    if (dev) launch_map<double, 2>(as_stream(w), (double*)y, (const double*)x, (const double*)y, (const double*)nullptr, n, AxpyPtrF<double>{(const double*)alpha});
    else { double a; memcpy(&a, alpha, 8); launch_map<double, 2>(as_stream(w), (double*)y, (const double*)x, (const double*)y, (const double*)nullptr, n, AxpyF<double>{a}); }
  } else {
    set_error(kUnsupported, "axpy: unsupported dtype %d", (int)id);
  }
}

extern "C" void zg_soft_update(dtype id, StreamWrapper w, const void* src, void* target, len_t n, double tau) {
  ZG_FLOAT_SWITCH("zg_soft_update", id, (launch_map<T, 2>(as_stream(w), (T*)target, (const T*)src, (const T*)target, (const T*)nullptr, n, SoftUpdateF<T>{(T)tau})));
}

extern "C" void zg_cast(dtype src_id, dtype dst_id, StreamWrapper w, const void* src, void* dst, len_t n) {
  if (n == 0) return;
  cudaStream_t s = as_stream(w);
  if (src_id == SINGLE && dst_id == BF16)
    f32_to_bf16_kernel<<<grid_for(n, kThreads * 8), kThreads, 0, s>>>((const float*)src, (__nv_bfloat16*)dst, n);
  else if (src_id == BF16 && dst_id == SINGLE)
    bf16_to_f32_kernel<<<grid_for(n, kThreads * 8), kThreads, 0, s>>>((const __nv_bfloat16*)src, (float*)dst, n);
  else { set_error(kUnsupported, "zg_cast: %d -> %d not supported", (int)src_id, (int)dst_id); return; }
  ZG_LAUNCH_CHECK();
}

extern "C" void zg_transpose(dtype id, StreamWrapper w, const void* A, void* B, len_t m, len_t n, double alpha) {
  if (m == 0 || n == 0) return;
  if (id == SINGLE && m % 4 == 0 && n % 4 == 0 && host_aligned16(A) && host_aligned16(B) && (m + 63) / 64 <= 65535) {
    dim3 grid64((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64));
    transpose64_kernel<<<grid64, 256, 0, as_stream(w)>>>((const float*)A, (float*)B, m, n, (float)alpha);
    ZG_LAUNCH_CHECK();
    return;
  }
  dim3 grid((unsigned)((n + 31) / 32), (unsigned)((m + 31) / 32)), block(32, 8);
  ZG_FLOAT_SWITCH("zg_transpose", id, (transpose_kernel<T><<<grid, block, 0, as_stream(w)>>>((const T*)A, (T*)B, m, n, (T)alpha)));
  ZG_LAUNCH_CHECK();
}
