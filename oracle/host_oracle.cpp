// CPU oracle: a restatement of zigrad's HostDevice (BLAS) backend for the
// training hot path.  TEST INFRASTRUCTURE ONLY -- nothing shipped in the
// product library includes, links or calls this file; it exists so that the
// CUDA backend's results can be compared against the reference algorithm on
// identical inputs, and so that the CPU path can be timed next to the GPU.
//
// Every function cites the reference file:line it follows (paths relative to
// the zigrad source tree).  The GEMM / axpy / nrm2 arithmetic of the reference
// lives in the system BLAS it links (build.zig:40-49: OpenBLAS by default on
// Linux, unpinned); the stand-in here is the OpenBLAS copy bundled with SciPy,
// resolved at run time with dlopen (orc_blas_init).  When no BLAS has been
// loaded the wrappers fall back to plain loops with the textbook definition
// of each routine, which is enough for the small golden vectors.
//
// Build: make -C oracle   (g++ only; no CUDA, no reference sources copied)

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <limits>
#include <dlfcn.h>

typedef unsigned long len_t;

namespace {

// ---------------------------------------------------------------------------
// BLAS binding (cblas interface, LP64).  host_device.zig:226-347 call sites.
// ---------------------------------------------------------------------------
enum { kRowMajor = 101, kNoTrans = 111, kTrans = 112 };

typedef void (*sgemm_fn)(int, int, int, int, int, int, float, const float*, int,
                         const float*, int, float, float*, int);
typedef void (*saxpy_fn)(int, float, const float*, int, float*, int);
typedef float (*snrm2_fn)(int, const float*, int);
typedef float (*sasum_fn)(int, const float*, int);
typedef float (*sdot_fn)(int, const float*, int, const float*, int);
typedef void (*sscal_fn)(int, float, float*, int);
typedef size_t (*isamax_fn)(int, const float*, int);
typedef void (*sgemv_fn)(int, int, int, int, float, const float*, int,
                         const float*, int, float, float*, int);
typedef void (*setthreads_fn)(int);

struct Blas {
  void* handle = nullptr;
  sgemm_fn sgemm = nullptr;
  saxpy_fn saxpy = nullptr;
  snrm2_fn snrm2 = nullptr;
  sasum_fn sasum = nullptr;
  sdot_fn sdot = nullptr;
  sscal_fn sscal = nullptr;
  isamax_fn isamax = nullptr;
  sgemv_fn sgemv = nullptr;
  setthreads_fn set_threads = nullptr;
} g_blas;

void* sym2(void* h, const char* a, const char* b) {
  void* p = dlsym(h, a);
  if (!p) p = dlsym(h, b);
  return p;
}

// Textbook fallbacks (used only when no BLAS was loaded).
void naive_sgemm(bool ta, bool tb, len_t m, len_t n, len_t k, float alpha,
                 const float* A, len_t lda, const float* B, len_t ldb,
                 float beta, float* C, len_t ldc) {
  for (len_t i = 0; i < m; ++i)
    for (len_t j = 0; j < n; ++j) {
      float acc = 0.f;
      for (len_t p = 0; p < k; ++p) {
        float a = ta ? A[p * lda + i] : A[i * lda + p];
        float b = tb ? B[j * ldb + p] : B[p * ldb + j];
        acc += a * b;
      }
      float prev = (beta == 0.f) ? 0.f : beta * C[i * ldc + j];
      C[i * ldc + j] = alpha * acc + prev;
    }
}

}  // namespace

extern "C" {

// Loads a CBLAS provider.  Returns 0 on success, 1 if the library or a
// required symbol is missing.  Symbols are looked up under both the plain
// `cblas_*` names and SciPy's `scipy_cblas_*` prefix.
int orc_blas_init(const char* path) {
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) return 1;
  Blas b;
  b.handle = h;
  b.sgemm = (sgemm_fn)sym2(h, "cblas_sgemm", "scipy_cblas_sgemm");
  b.saxpy = (saxpy_fn)sym2(h, "cblas_saxpy", "scipy_cblas_saxpy");
  b.snrm2 = (snrm2_fn)sym2(h, "cblas_snrm2", "scipy_cblas_snrm2");
  b.sasum = (sasum_fn)sym2(h, "cblas_sasum", "scipy_cblas_sasum");
  b.sdot = (sdot_fn)sym2(h, "cblas_sdot", "scipy_cblas_sdot");
  b.sscal = (sscal_fn)sym2(h, "cblas_sscal", "scipy_cblas_sscal");
  b.isamax = (isamax_fn)sym2(h, "cblas_isamax", "scipy_cblas_isamax");
  b.sgemv = (sgemv_fn)sym2(h, "cblas_sgemv", "scipy_cblas_sgemv");
  b.set_threads = (setthreads_fn)sym2(h, "openblas_set_num_threads",
                                      "scipy_openblas_set_num_threads");
  if (!b.sgemm || !b.saxpy || !b.snrm2 || !b.sasum || !b.sdot || !b.sscal ||
      !b.isamax || !b.sgemv)
    return 1;
  g_blas = b;
  return 0;
}

int orc_blas_loaded() { return g_blas.sgemm != nullptr; }

void orc_blas_set_threads(int n) {
  if (g_blas.set_threads) g_blas.set_threads(n);
}

// ---------------------------------------------------------------------------
// Element-wise binary ops with "wrapping" broadcast.
// host_device.zig:975-1019 (elwise_binop and helpers); opspec.zig:1-57.
// op: 0 add, 1 sub, 2 mul, 3 div.
// ---------------------------------------------------------------------------
static inline float apply_op(int op, float a, float b) {
  switch (op) {
    case 0: return a + b;
    case 1: return a - b;
    case 2: return a * b;
    default: return a / b;
  }
}

void orc_elwise(int op, const float* x, len_t xl, const float* y, len_t yl,
                float* z, len_t zl) {
  if (xl == 1 || yl == 1) {  // _elwise_binop_scalar_dispatch :994-1003
    if (zl == 1) {
      z[0] = apply_op(op, x[0], y[0]);
    } else if (xl == 1) {
      const float s = x[0];
      for (len_t j = 0; j < zl; ++j) z[j] = apply_op(op, s, y[j]);
    } else {
      const float s = y[0];
      for (len_t j = 0; j < zl; ++j) z[j] = apply_op(op, x[j], s);
    }
    return;
  }
  if (xl == yl) {  // :978-979
    for (len_t j = 0; j < zl; ++j) z[j] = apply_op(op, x[j], y[j]);
    return;
  }
  // general path: chunks of min(xl, yl); the shorter operand is re-read for
  // every chunk, the longer one advances (:981-992)
  const len_t mn = std::min(xl, yl);
  const len_t xs = (xl == zl) ? mn : 0;
  const len_t ys = (yl == zl) ? mn : 0;
  len_t xo = 0, yo = 0;
  for (len_t zo = 0; zo < zl; zo += mn, xo += xs, yo += ys)
    for (len_t j = 0; j < mn; ++j) z[zo + j] = apply_op(op, x[xo + j], y[yo + j]);
}

// ---------------------------------------------------------------------------
// BLAS wrappers.  host_device.zig:226-347.
// ---------------------------------------------------------------------------

// matmul: cblas_sgemm(RowMajor, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta,
// C, ldc) (host_device.zig:242-250).
void orc_matmul(const float* A, const float* B, float* C, len_t m, len_t n,
                len_t k, int ta, int tb, len_t lda, len_t ldb, len_t ldc,
                float alpha, float beta) {
  if (g_blas.sgemm) {
    g_blas.sgemm(kRowMajor, ta ? kTrans : kNoTrans, tb ? kTrans : kNoTrans,
                 (int)m, (int)n, (int)k, alpha, A, (int)lda, B, (int)ldb, beta,
                 C, (int)ldc);
  } else {
    naive_sgemm(ta != 0, tb != 0, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
  }
}

// bmm_acc: loop over the C batches; operand batch index wraps with
// `i % n_batches` (host_device.zig:277-313).  Shapes are {batch, rows, cols}
// as produced by NDArray.bmm_acc_impl (ndarray.zig:881-895): A_shape =
// {nA, M, K}, B_shape = {nB, K, N}, C_shape = {nC, M, N} (already "op"-ed
// dims), lda/ldb = stored column counts.
void orc_bmm_acc(const float* A, const float* B, float* C, const len_t* As,
                 const len_t* Bs, const len_t* Cs, int ta, int tb, len_t lda,
                 len_t ldb, len_t ldc, float alpha, float beta) {
  const len_t a_chunk = As[1] * As[2], b_chunk = Bs[1] * Bs[2],
              c_chunk = Cs[1] * Cs[2];
  for (len_t i = 0; i < Cs[0]; ++i) {
    const float* a = A + (i % As[0]) * a_chunk;
    const float* b = B + (i % Bs[0]) * b_chunk;
    float* c = C + i * c_chunk;
    orc_matmul(a, b, c, Cs[1], Cs[2], As[2], ta, tb, lda, ldb, ldc, alpha, beta);
  }
}

// matvec: cblas_sgemv(RowMajor, ta, m, n, ..., lda = n) (:232-240)
void orc_matvec(const float* A, const float* x, float* y, len_t m, len_t n,
                int ta, float alpha, float beta) {
  if (g_blas.sgemv) {
    g_blas.sgemv(kRowMajor, ta ? kTrans : kNoTrans, (int)m, (int)n, alpha, A,
                 (int)n, x, 1, beta, y, 1);
    return;
  }
  const len_t rows = ta ? n : m, cols = ta ? m : n;
  for (len_t i = 0; i < rows; ++i) {
    float acc = 0.f;
    for (len_t j = 0; j < cols; ++j) acc += (ta ? A[j * n + i] : A[i * n + j]) * x[j];
    y[i] = alpha * acc + (beta == 0.f ? 0.f : beta * y[i]);
  }
}

// axpy: y += alpha * x  (:269-275)
void orc_axpy(const float* x, float* y, len_t n, float alpha) {
  if (g_blas.saxpy) {
    g_blas.saxpy((int)n, alpha, x, 1, y, 1);
  } else {
    for (len_t i = 0; i < n; ++i) y[i] += alpha * x[i];
  }
}

// dot (:226-232)
float orc_dot(const float* x, const float* y, len_t n) {
  if (g_blas.sdot) return g_blas.sdot((int)n, x, 1, y, 1);
  float s = 0.f;
  for (len_t i = 0; i < n; ++i) s += x[i] * y[i];
  return s;
}

// "sum" is cblas_sasum, i.e. the sum of ABSOLUTE values (:315-321).
float orc_sum(const float* x, len_t n) {
  if (g_blas.sasum) return g_blas.sasum((int)n, x, 1);
  float s = 0.f;
  for (len_t i = 0; i < n; ++i) s += std::fabs(x[i]);
  return s;
}

// scale: cblas_sscal (:323-329)
void orc_scale(float* x, len_t n, float alpha) {
  if (g_blas.sscal) {
    g_blas.sscal((int)n, alpha, x, 1);
  } else {
    for (len_t i = 0; i < n; ++i) x[i] *= alpha;
  }
}

// nrm2: cblas_snrm2 (:331-337)
float orc_nrm2(const float* x, len_t n) {
  if (g_blas.snrm2) return g_blas.snrm2((int)n, x, 1);
  double s = 0.0;
  for (len_t i = 0; i < n; ++i) s += (double)x[i] * x[i];
  return (float)std::sqrt(s);
}

// clip_nrm2: if ||x|| > max_norm: x *= max_norm / (||x|| + delta) (:339-346)
void orc_clip_nrm2(float* x, len_t n, float max_norm, float delta) {
  const float norm = orc_nrm2(x, n);
  if (norm > max_norm) orc_scale(x, n, max_norm / (norm + delta));
}

// outer: cblas_sger, A += alpha x y^T, lda = |y| (:252-258)
void orc_outer(const float* x, len_t xl, const float* y, len_t yl, float* A,
               float alpha) {
  for (len_t i = 0; i < xl; ++i)
    for (len_t j = 0; j < yl; ++j) A[i * yl + j] += alpha * x[i] * y[j];
}

// transpose: B[j,i] = A[i,j] + alpha * B[j,i]  (:261-267)
void orc_transpose(const float* A, float* B, len_t m, len_t n, float alpha) {
  for (len_t i = 0; i < m; ++i)
    for (len_t j = 0; j < n; ++j) B[j * m + i] = A[i * n + j] + alpha * B[j * m + i];
}

// ---------------------------------------------------------------------------
// Non-linear ops.  host_device.zig:352-598.
// ---------------------------------------------------------------------------

// relu_fwd: y = @max(0, x) (:524-537).  Zig's @max on floats returns the
// non-NaN operand when exactly one operand is NaN, so relu(NaN) = 0; and
// max(0, -0.0) may return either zero -- compare with == (not bit-wise) there.
void orc_relu_fwd(const float* x, float* y, len_t n) {
  for (len_t i = 0; i < n; ++i) y[i] = (x[i] > 0.f) ? x[i] : 0.f;
}

// relu_bwd: x_g += (x > 0) ? y_g : 0  (:539-541)
void orc_relu_bwd(const float* x, float* x_g, const float* y_g, len_t n) {
  for (len_t i = 0; i < n; ++i) x_g[i] += (x[i] > 0.f) ? y_g[i] : 0.f;
}

// relu_inplace_bwd: if (x <= 0) x_g = 0  (:543-547); x is the POST-activation
// value (nn.zig:39-62)
void orc_relu_inplace_bwd(const float* x, float* x_g, len_t n) {
  for (len_t i = 0; i < n; ++i)
    if (x[i] <= 0.f) x_g[i] = 0.f;
}

// clamp_fwd: y = min(max_, max(min_, x)) (:590-592)
void orc_clamp_fwd(const float* x, float* y, len_t n, float lo, float hi) {
  for (len_t i = 0; i < n; ++i) y[i] = std::fmin(hi, std::fmax(lo, x[i]));
}

// clamp_bwd: if (min < x && x < max) x_g += y_g  (:594-598)
void orc_clamp_bwd(const float* x, float* x_g, const float* y_g, len_t n,
                   float lo, float hi) {
  for (len_t i = 0; i < n; ++i)
    if (lo < x[i] && x[i] < hi) x_g[i] += y_g[i];
}

// exp_fwd (:497-510), exp_bwd: x_g += y * y_g (:512-515)
void orc_exp_fwd(const float* x, float* y, len_t n) {
  for (len_t i = 0; i < n; ++i) y[i] = std::exp(x[i]);
}
void orc_exp_bwd(float* x_g, const float* y, const float* y_g, len_t n) {
  for (len_t i = 0; i < n; ++i) x_g[i] += y[i] * y_g[i];
}

// rsqrt_fwd native path: r = 1 / sqrt(max(a, eps)) (:463-482)
void orc_rsqrt_fwd(const float* x, float* y, len_t n, float eps) {
  for (len_t i = 0; i < n; ++i) y[i] = 1.f / std::sqrt(std::fmax(x[i], eps));
}

// rsqrt_bwd: x < eps -> +0 ; else x_g += -0.5 / (x*sqrt(x)) * y_g (:485-503)
void orc_rsqrt_bwd(const float* x, float* x_g, const float* y_g, len_t n, float eps) {
  for (len_t i = 0; i < n; ++i) {
    if (x[i] < eps) continue;
    const float s = std::sqrt(x[i]);
    const float inv = 1.0f / (x[i] * s);
    x_g[i] += (-0.5f * inv) * y_g[i];
  }
}

// sqrt_fwd (:383-387); sqrt_bwd: x<eps -> 0 else x_g += 0.5/sqrt(x)*y_g (:396-408)
void orc_sqrt_fwd(const float* x, float* y, len_t n) {
  for (len_t i = 0; i < n; ++i) y[i] = std::sqrt(x[i]);
}
void orc_sqrt_bwd(const float* x, float* x_g, const float* y_g, len_t n, float eps) {
  for (len_t i = 0; i < n; ++i)
    if (!(x[i] < eps)) x_g[i] += 0.5f / std::sqrt(x[i]) * y_g[i];
}

// tanh / sigmoid families (:549-571)
void orc_tanh_fwd(const float* x, float* y, len_t n) {
  for (len_t i = 0; i < n; ++i) y[i] = std::tanh(x[i]);
}
void orc_tanh_bwd(float* x_g, const float* y, const float* y_g, len_t n) {
  for (len_t i = 0; i < n; ++i) x_g[i] += (1.f - y[i] * y[i]) * y_g[i];
}
void orc_sigm_fwd(const float* x, float* y, len_t n) {
  for (len_t i = 0; i < n; ++i) y[i] = 1.f / (1.f + std::exp(-x[i]));
}
void orc_sigm_bwd(float* x_g, const float* y, const float* y_g, len_t n) {
  for (len_t i = 0; i < n; ++i) x_g[i] += y[i] * (1.f - y[i]) * y_g[i];
}

// tanh_inplace_bwd: x_g *= 1 - x*x (:557-559); sigm_inplace_bwd: x_g *= x*(1-x) (:569-571)
void orc_tanh_inplace_bwd(const float* x, float* x_g, len_t n) {
  for (len_t i = 0; i < n; ++i) x_g[i] *= (1.f - (x[i] * x[i]));
}
void orc_sigm_inplace_bwd(const float* x, float* x_g, len_t n) {
  for (len_t i = 0; i < n; ++i) x_g[i] *= (x[i] * (1.f - x[i]));
}

// pow_fwd / pow_fwd_ : y = pow(x, exp) (:353-361; y may alias x);
// pow_bwd: x < eps -> +0, else x_g += exp * pow(x, exp-1) * y_g (:365-379)
void orc_pow_fwd(const float* x, float* y, len_t n, float e) {
  for (len_t i = 0; i < n; ++i) y[i] = std::pow(x[i], e);
}
void orc_pow_bwd(const float* x, float* x_g, const float* y_g, len_t n, float e, float eps) {
  const float em1 = e - 1.f;
  for (len_t i = 0; i < n; ++i)
    if (!(x[i] < eps)) x_g[i] += e * std::pow(x[i], em1) * y_g[i];
}

// Byte-mask activations (:600-701): bit (i % 8) of mask[i / 8] per element
// (std.bit_set.IntegerBitSet(8), :16).  The loops below state the per-element
// rule of the reference's full-byte loops and apply it to the last n % 8
// elements as well (the reference's tail code of the two clamp forms names
// fields that its op structs do not have, :621 and :633).
// relu_mask_fwd (:652-678): x <= 0 -> x = 0, bit set.
void orc_relu_mask_fwd(float* x, unsigned char* mask, len_t n) {
  for (len_t b = 0; b < (n + 7) / 8; ++b) mask[b] = 0;
  for (len_t i = 0; i < n; ++i)
    if (x[i] <= 0.f) {
      x[i] = 0.f;
      mask[i / 8] |= (unsigned char)(1u << (i % 8));
    }
}
// relu_mask_bwd (:680-701): bit set -> x_g = 0
void orc_relu_mask_bwd(float* x_g, const unsigned char* mask, len_t n) {
  for (len_t i = 0; i < n; ++i)
    if (mask[i / 8] & (1u << (i % 8))) x_g[i] = 0.f;
}
// clamp_mask_fwd (:600-628): bit = (x != min(hi, max(lo, x))); y receives x itself (:611)
void orc_clamp_mask_fwd(const float* x, float* y, unsigned char* mask, len_t n, float lo, float hi) {
  for (len_t b = 0; b < (n + 7) / 8; ++b) mask[b] = 0;
  for (len_t i = 0; i < n; ++i) {
    const float clamped = std::fmin(hi, std::fmax(lo, x[i]));
    if (x[i] != clamped) mask[i / 8] |= (unsigned char)(1u << (i % 8));
    y[i] = x[i];
  }
}
// clamp_mask_bwd (:630-650): bit set -> x_g += y_g
void orc_clamp_mask_bwd(float* x_g, const float* y_g, const unsigned char* mask, len_t n) {
  for (len_t i = 0; i < n; ++i)
    if (mask[i / 8] & (1u << (i % 8))) x_g[i] += y_g[i];
}

// max_fwd: y = x[isamax(x)] -- the element of largest MAGNITUDE (:573-580);
// max_bwd: every position equal to y receives the gradient (:582-588)
void orc_max_fwd(const float* x, float* y, len_t n) {
  len_t idx = 0;
  if (g_blas.isamax) {
    idx = g_blas.isamax((int)n, x, 1);
  } else {
    float best = -1.f;
    for (len_t i = 0; i < n; ++i)
      if (std::fabs(x[i]) > best) { best = std::fabs(x[i]); idx = i; }
  }
  y[0] = x[idx];
}
void orc_max_bwd(const float* x, float* x_g, const float* y, const float* y_g, len_t n) {
  for (len_t i = 0; i < n; ++i)
    if (y[0] == x[i]) x_g[i] += y_g[0];
}

// ---------------------------------------------------------------------------
// Reductions.  reduce.zig:3-164 and host_device.zig:709-874.
// ---------------------------------------------------------------------------
static const len_t kLanes = 8;  // std.simd.suggestVectorLength(f32) on AVX2

// scaled_copy: y = alpha*x + beta*y (reduce.zig:3-11)
void orc_scaled_copy(const float* x, float* y, len_t n, float alpha, float beta) {
  for (len_t i = 0; i < n; ++i) y[i] = alpha * x[i] + beta * y[i];
}

// flat_reduce: lane-wise partial sums over whole vectors, a horizontal add,
// then the scalar tail (reduce.zig:13-46)
void orc_flat_reduce(const float* x, len_t n, float* y, float alpha, float beta) {
  float lanes[kLanes] = {0};
  len_t i = 0;
  for (; i + kLanes <= n; i += kLanes)
    for (len_t l = 0; l < kLanes; ++l) lanes[l] += x[i + l];
  // @reduce(.Add) -- pairwise tree, the shape LLVM emits for a vector reduce
  float t[kLanes];
  std::memcpy(t, lanes, sizeof(t));
  for (len_t w = kLanes / 2; w >= 1; w /= 2)
    for (len_t l = 0; l < w; ++l) t[l] += t[l + w];
  float s = t[0];
  for (; i < n; ++i) s += x[i];
  y[0] = alpha * s + beta * y[0];
}

// fold_rows (M,N)->(N): every column is summed in plain row order, starting
// from row 0's value; then y = alpha*s + beta*y (reduce.zig:49-128).  The
// reference's 32-vector blocking only changes which columns are processed
// together, never the per-column order, so it is not restated.
void orc_fold_rows(const float* x, float* y, len_t row, len_t col, float alpha, float beta) {
  for (len_t c = 0; c < col; ++c) {
    float s = x[c];
    for (len_t r = 1; r < row; ++r) s += x[r * col + c];
    y[c] = alpha * s + beta * y[c];
  }
}

// fold_cols (M,N)->(M): per row, lane partials + horizontal add + tail
// (reduce.zig:131-164)
void orc_fold_cols(const float* x, float* y, len_t row, len_t col, float alpha, float beta) {
  for (len_t r = 0; r < row; ++r) {
    const float* xr = x + r * col;
    float lanes[kLanes] = {0};
    len_t j = 0;
    for (; j + kLanes <= col; j += kLanes)
      for (len_t l = 0; l < kLanes; ++l) lanes[l] += xr[j + l];
    for (len_t w = kLanes / 2; w >= 1; w /= 2)
      for (len_t l = 0; l < w; ++l) lanes[l] += lanes[l + w];
    float s = 0.f;
    s += lanes[0];
    for (; j < col; ++j) s += xr[j];
    y[r] = alpha * s + beta * y[r];
  }
}

static len_t prod(const len_t* s, len_t a, len_t b) {
  len_t p = 1;
  for (len_t i = a; i < b; ++i) p *= s[i];
  return p;
}

// sum_along (host_device.zig:798-848): flat / head / tail base cases, else a
// fold_rows per leading chunk.
void orc_sum_along(const float* x, const len_t* xs, len_t nd, float* y, len_t ylen,
                   len_t dim, float alpha, float beta) {
  if (ylen == 1) return orc_flat_reduce(x, prod(xs, 0, nd), y, alpha, beta);
  if (dim == 0) return orc_fold_rows(x, y, xs[0], prod(xs, 1, nd), alpha, beta);
  if (dim + 1 == nd) return orc_fold_cols(x, y, prod(xs, 0, dim), xs[dim], alpha, beta);
  const len_t n_chunks = prod(xs, 0, dim);
  const len_t ychunk = prod(xs, dim + 1, nd);
  const len_t xchunk = xs[dim] * ychunk;
  for (len_t c = 0; c < n_chunks; ++c)
    orc_fold_rows(x + xchunk * c, y + ychunk * c, xs[dim], ychunk, alpha, beta);
}

// max_along (host_device.zig:853-874): alpha/beta are ignored by the host.
void orc_max_along(const float* x, const len_t* xs, len_t nd, float* y, len_t ylen, len_t dim) {
  const len_t dsz = xs[dim];
  const len_t slice = prod(xs, dim + 1, nd);
  for (len_t i = 0; i < ylen; ++i) {
    float mx = -std::numeric_limits<float>::infinity();
    const len_t base = (i / slice) * (slice * dsz) + (i % slice);
    for (len_t j = 0; j < dsz; ++j) {
      const float v = x[base + j * slice];
      if (v > mx) mx = v;
    }
    y[i] = mx;
  }
}

// unbroadcast (host_device.zig:709-780).  `scratch` must hold what
// NDArray.unbroadcast_ sizes (ndarray.zig:697-715).  Returns 0, or 1 if the
// shapes exceed 8 dims.
int orc_unbroadcast(const float* x, const len_t* x_shape, len_t xnd, float* y,
                    const len_t* y_shape, len_t ynd, float* scratch, float alpha, float beta) {
  const len_t xlen = prod(x_shape, 0, xnd), ylen = prod(y_shape, 0, ynd);
  if (xlen == ylen) { orc_scaled_copy(x, y, xlen, alpha, beta); return 0; }
  if (xnd > 8 || ynd > 8) return 1;
  // trim leading ones of x; leading AND trailing ones of y (:723-731)
  std::vector<len_t> xsv(x_shape, x_shape + xnd), ysv(y_shape, y_shape + ynd);
  while (!xsv.empty() && xsv.front() == 1) xsv.erase(xsv.begin());
  while (!ysv.empty() && ysv.front() == 1) ysv.erase(ysv.begin());
  bool trimmed_back = false;
  while (!ysv.empty() && ysv.back() == 1) { ysv.pop_back(); trimmed_back = true; }
  // With trailing ones trimmed off y the reference lines y's dimensions up against the wrong
  // dimensions of x: for x [4,5,6] -> y [5,1] it folds 6 columns into the 5-element y (one past
  // its end), for x [4,5,1] -> y [5,1] it writes y[0] only.  The restatement reports these
  // shapes instead of reproducing an out-of-bounds write.
  if (trimmed_back) return 2;
  len_t ones = (len_t)std::count(ysv.begin(), ysv.end(), (len_t)1);
  const len_t orig_x_rank = xnd;
  if (xsv.size() > ysv.size()) {
    const len_t dif = xsv.size() - ysv.size();
    orc_fold_rows(x, ones == 0 ? y : scratch, prod(xsv.data(), 0, dif),
                  prod(xsv.data(), dif, xsv.size()), alpha, beta);
    if (ones == 0) return 0;
    xsv.erase(xsv.begin(), xsv.begin() + dif);
  }
  len_t i = 0;
  while (ones > 0 && i < xsv.size()) {
    if (ysv[i] == 1 && xsv[i] != 1) {
      const float* xd = (xsv.size() == orig_x_rank) ? x : scratch;
      float* yd = (ones == 1) ? y : scratch;
      std::vector<len_t> yshape_now(ysv);
      const len_t yl = prod(yshape_now.data(), 0, yshape_now.size());
      orc_sum_along(xd, xsv.data(), xsv.size(), yd, yl, i, alpha, beta);
      xsv.erase(xsv.begin() + i);
      ysv.erase(ysv.begin() + i);
      --ones;
      continue;
    }
    ++i;
  }
  return 0;
}

// broadcast (host_device.zig:782-795): the equal-length branch does NOT
// return, so the generic loop runs afterwards as well (kept as is).
void orc_broadcast(const float* x, len_t xl, float* y, len_t yl, float alpha, float beta) {
  if (xl == yl) orc_scaled_copy(x, y, xl, alpha, beta);
  for (len_t i = 0; i < yl; ++i) y[i] = alpha * x[i % xl] + beta * y[i % yl];
}

// ---------------------------------------------------------------------------
// Index ops.  host_device.zig:950-953 (mem_take), :1039-1086 (scatter_add),
// :1356-1403 (GCN propagate).
// ---------------------------------------------------------------------------
void orc_take(const float* src, const len_t* idx, len_t n, float* dst) {
  for (len_t j = 0; j < n; ++j) dst[j] = src[idx[j]];
}

// scatter_add: dst[offs[i]] += src[i] in index order (the vectorised branch
// of the reference handles runs of consecutive offsets and adds the same
// values to the same places)
void orc_scatter_add(const float* src, const len_t* offs, len_t n, float* dst) {
  for (len_t i = 0; i < n; ++i) dst[offs[i]] += src[i];
}

// scatter_add_2d (:1137-1160): dst[indices[i], :] += src[i, :], blocks of `stride`
void orc_scatter_add_2d(const float* src, const len_t* indices, len_t n_blocks, len_t stride, float* dst) {
  for (len_t b = 0; b < n_blocks; ++b)
    for (len_t j = 0; j < stride; ++j) dst[indices[b] * stride + j] += src[b * stride + j];
}
// scatter_add_csr (:1325-1335): dst[j] += src[i] for j in [row_ptr[i], row_ptr[i+1])
void orc_scatter_add_csr(const float* src, const len_t* row_ptr, len_t n_seg, float* dst) {
  for (len_t i = 0; i < n_seg; ++i)
    for (len_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j) dst[j] += src[i];
}
// segment_sum_csr (:1337-1351) with the native left-to-right vsum_contig (:1318-1322)
void orc_segment_sum_csr(const float* src, const len_t* row_ptr, len_t n_seg, float* dst) {
  for (len_t i = 0; i < n_seg; ++i) {
    float s = 0.f;
    for (len_t j = row_ptr[i]; j < row_ptr[i + 1]; ++j) s += src[j];
    dst[i] = s;
  }
}

void orc_scatter_gcn_deg_scaled(float* dst, const float* h, const float* deg,
                                const len_t* src_idx, const len_t* tgt_idx,
                                len_t stride, len_t n_edge) {
  for (len_t e = 0; e < n_edge; ++e) {
    const len_t s = src_idx[e], t = tgt_idx[e];
    const float w = deg[s] * deg[t];
    for (len_t j = 0; j < stride; ++j) dst[t * stride + j] += w * h[s * stride + j];
  }
}

void orc_scatter_gcn_deg_scaled_bwd(const float* grad_out, const float* h, const float* deg,
                                    const len_t* src_idx, const len_t* tgt_idx,
                                    float* grad_h, float* grad_deg, len_t stride, len_t n_edge) {
  for (len_t e = 0; e < n_edge; ++e) {
    const len_t s = src_idx[e], t = tgt_idx[e];
    const float ds = deg[s], dt = deg[t];
    float gs = 0.f, gt = 0.f;
    for (len_t j = 0; j < stride; ++j) {
      const float go = grad_out[t * stride + j];
      const float hv = h[s * stride + j];
      grad_h[s * stride + j] += go * ds * dt;
      gs += go * dt * hv;
      gt += go * ds * hv;
    }
    grad_deg[s] += gs;
    grad_deg[t] += gt;
  }
}

// ---------------------------------------------------------------------------
// Losses.  nn/loss.zig:130-215 (softmax cross-entropy), :259-305 (smooth L1).
// ---------------------------------------------------------------------------

// _softmax_fwd over the last dim of [rows, C] (loss.zig:175-215):
// p = exp(x - (max + log(sum exp(x - max))))
void orc_softmax_rows(const float* x, float* p, len_t rows, len_t C) {
  for (len_t r = 0; r < rows; ++r) {
    const float* xr = x + r * C;
    float* pr = p + r * C;
    float mx = xr[0];
    for (len_t j = 1; j < C; ++j) mx = std::fmax(mx, xr[j]);
    float se = 0.f;
    for (len_t j = 0; j < C; ++j) se += std::exp(xr[j] - mx);
    const float lse = mx + std::log(se);
    for (len_t j = 0; j < C; ++j) pr[j] = std::exp(xr[j] - lse);
  }
}

// forward: returns mean loss; writes softmax probabilities to sm (kept for the
// backward, as CceBwd keeps sm_preds).  Targets are one-hot/probability rows.
// The running sum is sequential in fp32 over all rows*C entries
// (loss.zig:141-146).  `batch` is the divisor (shape[0], or 1 for 1-D input).
float orc_softmax_ce_fwd(const float* logits, const float* target, float* sm,
                         len_t rows, len_t C, len_t batch) {
  orc_softmax_rows(logits, sm, rows, C);
  const float eps = 1e-7f;
  float sum_loss = 0.f;
  for (len_t i = 0; i < rows * C; ++i) {
    const float safe = std::fmin(std::fmax(sm[i], eps), 1.0f - eps);
    sum_loss -= target[i] * std::log(safe);
  }
  return sum_loss / (float)batch;
}

// backward: grad += (sm - target) / batch   (loss.zig:148-160)
void orc_softmax_ce_bwd(const float* sm, const float* target, float* grad,
                        len_t n, len_t batch) {
  const float b = (float)batch;
  for (len_t i = 0; i < n; ++i) grad[i] += (sm[i] - target[i]) / b;
}

// smooth L1 (Huber) forward, mean over n (loss.zig:259-275)
float orc_smooth_l1_fwd(const float* pred, const float* target, len_t n, float beta) {
  float sum_loss = 0.f;
  for (len_t i = 0; i < n; ++i) {
    const float d = pred[i] - target[i];
    const float ad = std::fabs(d);
    if (ad < beta) sum_loss += 0.5f * (d * d) / beta;
    else sum_loss += ad - (0.5f * beta);
  }
  return sum_loss / (float)n;
}

// smooth L1 backward: |d|<beta -> d/(beta*n) else sign(d)/n (loss.zig:277-295)
void orc_smooth_l1_bwd(const float* pred, const float* target, float* grad, len_t n, float beta) {
  const float fn = (float)n;
  for (len_t i = 0; i < n; ++i) {
    const float d = pred[i] - target[i];
    if (std::fabs(d) < beta) grad[i] += d / (beta * fn);
    else grad[i] += (float)((d > 0.f) - (d < 0.f)) / fn;
  }
}

// ---------------------------------------------------------------------------
// Optimizers.  nn/optim.zig:100-122 (SGD), :177-234 (Adam).
// ---------------------------------------------------------------------------

// SGD.update for one tensor: optional clip of the gradient, then
// p += (-lr) * g with lr cast f64 -> f32 (optim.zig:103)
void orc_sgd_update(float* p, float* g, len_t n, double lr, int clip, float max_norm, float delta) {
  const float nlr = -(float)lr;
  if (clip) orc_clip_nrm2(g, n, max_norm, delta);
  orc_axpy(g, p, n, nlr);
}

// Adam.update for one tensor.  `t` is the optimizer-wide counter AFTER the
// increment that happens inside update, i.e. it advances once per parameter
// tensor, not once per step (optim.zig:189).  All arithmetic in f32.
void orc_adam_update(float* p, float* g, float* m, float* v, len_t n, double lr_, double b1_,
                     double b2_, double eps_, len_t t, int clip, float max_norm, float delta) {
  const float lr = (float)lr_, beta1 = (float)b1_, beta2 = (float)b2_, epsilon = (float)eps_;
  const float t_f = (float)t;
  const float lr_t = lr * std::sqrt(1.f - std::pow(beta2, t_f)) / (1.f - std::pow(beta1, t_f));
  if (clip) orc_clip_nrm2(g, n, max_norm, delta);
  for (len_t i = 0; i < n; ++i) {
    const float gi = g[i];
    m[i] = beta1 * m[i] + (1.f - beta1) * gi;
    v[i] = beta2 * v[i] + (1.f - beta2) * gi * gi;
    p[i] -= lr_t * m[i] / (std::sqrt(v[i]) + epsilon);
  }
}

// ---------------------------------------------------------------------------
// bf16 helpers for the mixed-precision configuration (no counterpart in the
// reference, which is fp32/fp64 only): round-to-nearest-even fp32 -> bf16,
// returned as fp32 so the BLAS path can consume it.
// ---------------------------------------------------------------------------
void orc_round_bf16(const float* x, float* y, len_t n) {
  for (len_t i = 0; i < n; ++i) {
    uint32_t u;
    std::memcpy(&u, &x[i], 4);
    if ((u & 0x7f800000u) == 0x7f800000u) {  // inf / nan: keep, quiet the nan
      if (u & 0x007fffffu) u |= 0x00400000u;
      u &= 0xffff0000u;
    } else {
      u += 0x7fffu + ((u >> 16) & 1u);
      u &= 0xffff0000u;
    }
    std::memcpy(&y[i], &u, 4);
  }
}

}  // extern "C"

#include "steps.inc"
