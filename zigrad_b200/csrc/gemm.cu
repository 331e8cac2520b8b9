// GEMM entry points: zg_bmm (include/zg_b200.h), gemm / gemv / ger
// (include/blas_conflux.h).  Large, TMA-addressable problems go to the
// tcgen05 kernel (gemm_tc.cuh); everything else (tiny shapes, rows whose byte
// stride is not a multiple of 16, fp64) runs on a register-tiled FFMA kernel.
#include <cmath>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "driver_api.h"
#include "gemm_tc.cuh"
#include "gemm_tc_persistent.cuh"
#include "gemm_skinny.cuh"
#include "mlp_tail.cuh"
#include "../../include/blas_conflux.h"

namespace zg {

static int g_math_mode = ZG_MATH_FP32X3;

// =====================================================================
// FFMA kernel: 64x64 tile, 16-deep k-slabs, 256 threads x (4x4) outputs.
// Generic in element type (double / float / bf16 inputs with float math),
// operand transposes and leading dimensions.  gridDim.z = batches * splits.
// =====================================================================
template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v) { return (typename Acc<T>::type)v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename TC, typename A> __device__ __forceinline__ TC from_acc(A v) { return (TC)v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

struct SimtParams {
  size_t nA, nB, m, n, k, lda, ldb, ldc, a_stride, b_stride, c_stride;
  bool ta, tb;
  double alpha, beta;
  int epilogue;
  const float* bias;
  const void* mask;
  float* colsum;
  unsigned splits;
  size_t k_per_split;
};

template <typename TI, typename TC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TI* __restrict__ A, const TI* __restrict__ B, TC* C, const SimtParams p) {
  using AT = typename Acc<TI>::type;
  constexpr int TM = 64, TN = 64, TK = 16;
  pdl_sync();
  __shared__ AT As[TK][TM + 1];
  __shared__ AT Bs[TK][TN + 1];
  const unsigned batch = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
  const TI* a = A + (batch % p.nA) * p.a_stride;
  const TI* b = B + (batch % p.nB) * p.b_stride;
  TC* c = C + (size_t)batch * p.c_stride;
  const size_t m0 = (size_t)blockIdx.y * TM, n0 = (size_t)blockIdx.x * TN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  AT acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = AT(0);
  const size_t kb = split * p.k_per_split;
  size_t ke = kb + p.k_per_split;
  if (ke > p.k) ke = p.k;
  // Cooperative loads: 1024 elements per operand slab, 4 per thread; the
  // fastest-varying thread index follows the contiguous dimension in memory.
  // The next slab is fetched into registers while the current one is being
  // multiplied, so a trip costs the arithmetic, not a round trip to memory.
  AT ar[4], br[4];
  auto fetch = [&](size_t k0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = threadIdx.x + q * 256;
      int mm, kk;
      if (p.ta) { mm = e % TM; kk = e / TM; } else { kk = e % TK; mm = e / TK; }
      const size_t gm = m0 + mm, gk = k0 + kk;
      ar[q] = (gm < p.m && gk < ke) ? to_acc<TI>(p.ta ? a[gk * p.lda + gm] : a[gm * p.lda + gk]) : AT(0);
      int nn;
      if (p.tb) { kk = e % TK; nn = e / TK; } else { nn = e % TN; kk = e / TN; }
      const size_t gn = n0 + nn, gk2 = k0 + kk;
      br[q] = (gn < p.n && gk2 < ke) ? to_acc<TI>(p.tb ? b[gn * p.ldb + gk2] : b[gk2 * p.ldb + gn]) : AT(0);
    }
  };
  if (kb < ke) fetch(kb);
  for (size_t k0 = kb; k0 < ke; k0 += TK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = threadIdx.x + q * 256;
      int mm, kk, nn;
      if (p.ta) { mm = e % TM; kk = e / TM; } else { kk = e % TK; mm = e / TK; }
      As[kk][mm] = ar[q];
      if (p.tb) { kk = e % TK; nn = e / TK; } else { nn = e % TN; kk = e / TN; }
      Bs[kk][nn] = br[q];
    }
    __syncthreads();
    if (k0 + TK < ke) fetch(k0 + TK);
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      AT av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
  const AT alpha = (AT)p.alpha, beta = (AT)p.beta;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t gm = m0 + ty * 4 + i;
    if (gm >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t gn = n0 + tx + 16 * j;
      if (gn >= p.n) continue;
      const size_t o = gm * p.ldc + gn;
      AT v = alpha * acc[i][j];
      if (p.splits > 1) {
        if constexpr (sizeof(TC) == 4 || sizeof(TC) == 8) atomicAdd(reinterpret_cast<AT*>(c) + o, v);
        continue;
      }
      if (beta != AT(0)) v += beta * to_acc<TC>(c[o]);
      if (p.epilogue == ZG_EPI_BIAS) v += (AT)p.bias[gn];
      else if (p.epilogue == ZG_EPI_BIAS_RELU) { v += (AT)p.bias[gn]; v = v > AT(0) ? v : AT(0); }
      else if (p.epilogue == ZG_EPI_RELU_MASK) {
        const TC* mk = static_cast<const TC*>(p.mask) + (size_t)batch * p.c_stride;
        if (to_acc<TC>(mk[o]) <= AT(0)) v = AT(0);
      }
      c[o] = from_acc<TC, AT>(v);
      if (p.colsum) atomicAdd(p.colsum + gn, (float)v);
    }
  }
}

// C[b][i][j] *= beta over an [m, n] window with leading dimension ldc
template <typename T>
__global__ void scale_c_kernel(T* C, size_t batches, size_t m, size_t n, size_t ldc, size_t c_stride, T beta) {
  pdl_sync();
  const size_t total = batches * m * n, nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nth) {
    const size_t b = i / (m * n), r = (i % (m * n)) / n, cidx = i % n;
    T* p = C + b * c_stride + r * ldc + cidx;
    *p = (beta == T(0)) ? T(0) : beta * (*p);
  }
}

template <typename T>
static void prescale_c(cudaStream_t s, T* C, size_t batches, size_t m, size_t n, size_t ldc, size_t c_stride, double beta) {
  if (beta == 1.0) return;
  launch_pdl(scale_c_kernel<T>, dim3(grid_for(batches * m * n, 1024)), dim3(256), 0, s, C, batches, m, n, ldc, c_stride, (T)beta);
}

template <typename TI, typename TC>
static void launch_simt(cudaStream_t s, const void* A, const void* B, void* C, len_t nA, len_t nB, len_t nC, len_t m, len_t n, len_t k,
                        bool ta, bool tb, len_t lda, len_t ldb, len_t ldc, double alpha, double beta, int epilogue, const void* bias,
                        const void* mask, void* colsum) {
  SimtParams p;
  p.colsum = static_cast<float*>(colsum);
  p.nA = nA; p.nB = nB; p.m = m; p.n = n; p.k = k; p.lda = lda; p.ldb = ldb; p.ldc = ldc;
  p.a_stride = (ta ? k : m) * lda; p.b_stride = (tb ? n : k) * ldb; p.c_stride = m * ldc;
  p.ta = ta; p.tb = tb; p.alpha = alpha; p.beta = beta; p.epilogue = epilogue;
  p.bias = static_cast<const float*>(bias); p.mask = mask;
  const size_t tiles = ((m + 63) / 64) * ((n + 63) / 64) * nC;
  unsigned splits = 1;
  // deep-k, few-tile problems (weight gradients): split K over more CTAs
  if (epilogue == ZG_EPI_NONE && !colsum && sizeof(TC) >= 4 && k >= 128 && tiles * 2 <= (size_t)sm_count()) {
    size_t want = (size_t)sm_count() * 2 / tiles;
    size_t maxs = k / 32;  // at least two 16-deep slabs per split
    splits = (unsigned)(want < maxs ? want : maxs);
    if (splits < 1) splits = 1;
  }
  p.splits = splits;
  p.k_per_split = splits > 1 ? ((k + splits - 1) / splits + 15) / 16 * 16 : k;
  if (splits > 1) {
    if constexpr (sizeof(TC) >= 4) prescale_c<TC>(s, static_cast<TC*>(C), nC, m, n, ldc, p.c_stride, beta);
  }
  dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64), (unsigned)(nC * splits));
  if (grid.y > 65535 || grid.z > 65535) { set_error(kBadArgument, "gemm: grid too large (m=%lu, batches=%lu)", m, nC); return; }
  launch_pdl(gemm_simt_kernel<TI, TC>, grid, dim3(256), 0, s, static_cast<const TI*>(A), static_cast<const TI*>(B), static_cast<TC*>(C), p);
}

// =====================================================================
// tcgen05 path: host side
// =====================================================================
static int* tc_error_flag() {
  // one device-visible flag per device, read back by zg_last_error callers via check_tc_errors()
  static int* flags[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!flags[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    // the legacy stream does not order against the library's non-blocking streams: finish the clear here
    cudaMemset(p, 0, sizeof(int));
    cudaDeviceSynchronize();
    flags[dev] = p;
  }
  return flags[dev];
}

static bool make_tmap(CUtensorMap* map, bool bf16, const void* base, uint64_t inner, uint64_t rows, uint64_t batches, uint64_t ld,
                      uint32_t box_inner, uint32_t box_rows, bool atom32) {
  static auto encode = ZG_DRV(cuTensorMapEncodeTiled);
  if (!encode) return false;
  const uint64_t es = bf16 ? 2 : 4;
  cuuint64_t dims[3] = {inner, rows, batches};
  cuuint64_t strides[2] = {ld * es, rows * ld * es};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims,
                      strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return ZG_CU(r);
}

template <int BN, bool AK, bool BK_, int MODE, bool ATM = false>
static bool launch_tc_inst(cudaStream_t s, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tcm, const tc::Params& p, dim3 grid) {
  using SL = tc::SmemLayout<BN, MODE, ATM>;
  auto kern = tc::gemm_tc_kernel<BN, AK, BK_, MODE, ATM>;
  static bool attr_set = false;
  if (!attr_set) {
    if (!ZG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SL::kTotal))) return false;
    attr_set = true;
  }
  return launch_pdl(kern, grid, dim3(tc::tc_threads(MODE)), (size_t)SL::kTotal, s, ta, tb, tcm, p);
}

// FP32X3: the hi/lo parts of A live in tensor memory (ZG_X3_TMEM_A=0 keeps them in shared memory)
static bool x3_tmem_a() {
  static const bool on = [] { const char* e = getenv("ZG_X3_TMEM_A"); return !(e && e[0] == '0'); }();
  return on;
}

template <int MODE>
static bool launch_tc_mode(cudaStream_t s, int bn, bool a_kmajor, bool b_kmajor, const CUtensorMap& ta, const CUtensorMap& tb,
                           const CUtensorMap& tcm, const tc::Params& p, dim3 grid) {
#define ZG_TC_CASE(BNV)                                                                       \
  if (bn == BNV) {                                                                            \
    if constexpr (MODE == tc::kFP32X3) {                                                      \
      if (x3_tmem_a()) {                                                                      \
        if (a_kmajor && b_kmajor) return launch_tc_inst<BNV, true, true, MODE, true>(s, ta, tb, tcm, p, grid);   \
        if (a_kmajor) return launch_tc_inst<BNV, true, false, MODE, true>(s, ta, tb, tcm, p, grid);              \
        if (b_kmajor) return launch_tc_inst<BNV, false, true, MODE, true>(s, ta, tb, tcm, p, grid);              \
        return launch_tc_inst<BNV, false, false, MODE, true>(s, ta, tb, tcm, p, grid);                           \
      }                                                                                       \
    }                                                                                         \
    if (a_kmajor && b_kmajor) return launch_tc_inst<BNV, true, true, MODE>(s, ta, tb, tcm, p, grid);   \
    if (a_kmajor && !b_kmajor) return launch_tc_inst<BNV, true, false, MODE>(s, ta, tb, tcm, p, grid); \
    if (!a_kmajor && b_kmajor) return launch_tc_inst<BNV, false, true, MODE>(s, ta, tb, tcm, p, grid); \
    return launch_tc_inst<BNV, false, false, MODE>(s, ta, tb, tcm, p, grid);                       \
  }
  if constexpr (MODE != tc::kBF16) { ZG_TC_CASE(32) }
  ZG_TC_CASE(64)
  ZG_TC_CASE(128)
#undef ZG_TC_CASE
  set_error(kBadArgument, "gemm: no tensor-core instance for BN=%d", bn);
  return false;
}

template <bool AK, bool BK_, int MODE>
static bool launch_persistent_inst(cudaStream_t s, const CUtensorMap& ta, const CUtensorMap& tb, const tc::Params& p, uint32_t tiles_m,
                                   uint32_t tiles_n, uint32_t n_tiles) {
  using SL = tc::PersistentSmem<MODE>;
  auto kern = tc::gemm_tc_persistent_kernel<AK, BK_, MODE>;
  static bool attr_set = false;
  if (!attr_set) {
    if (!ZG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SL::kTotal))) return false;
    attr_set = true;
  }
  const unsigned grid = n_tiles < (uint32_t)sm_count() ? n_tiles : (unsigned)sm_count();
  // work-item counter: zero between launches (slot 2 of the stream's workspace)
  unsigned* unused = nullptr;
  unsigned* counter = static_cast<unsigned*>(workspace(s, 256, &unused, 2));
  if (!counter) return false;
  return launch_pdl(kern, dim3(grid), dim3(tc::kThreadsPersistent), (size_t)SL::kTotal, s, ta, tb, p, tiles_m, tiles_n, n_tiles, counter);
}

template <int MODE>
static bool launch_persistent(cudaStream_t s, bool a_kmajor, bool b_kmajor, const CUtensorMap& ta, const CUtensorMap& tb,
                              const tc::Params& p, uint32_t tiles_m, uint32_t tiles_n, uint32_t n_tiles) {
  if (a_kmajor && b_kmajor) return launch_persistent_inst<true, true, MODE>(s, ta, tb, p, tiles_m, tiles_n, n_tiles);
  if (a_kmajor && !b_kmajor) return launch_persistent_inst<true, false, MODE>(s, ta, tb, p, tiles_m, tiles_n, n_tiles);
  if (!a_kmajor && b_kmajor) return launch_persistent_inst<false, true, MODE>(s, ta, tb, p, tiles_m, tiles_n, n_tiles);
  return launch_persistent_inst<false, false, MODE>(s, ta, tb, p, tiles_m, tiles_n, n_tiles);
}

// fp32 problems with n <= 16 or k <= 16 (see gemm_skinny.cuh).  Returns true when taken.
static bool try_skinny(dtype id, dtype c_id, cudaStream_t s, const void* A, const void* B, void* C, len_t nA, len_t nB, len_t nC, len_t m,
                       len_t n, len_t k, bool ta, bool tb, len_t lda, len_t ldb, len_t ldc, double alpha, double beta, int epilogue,
                       const void* bias, const void* mask, void* colsum) {
  static const bool off = [] { const char* e = getenv("ZG_GEMM_NO_SKINNY"); return e && e[0] == '1'; }();
  if (off || id != SINGLE || c_id != SINGLE || nA != 1 || nB != 1 || nC != 1) return false;
  if (m > 0x7fffffffu || k == 0 || k > 0x7fffffffu || lda > 0xffffffffu || ldb > 0xffffffffu || ldc > 0xffffffffu) return false;
  skinny::Params p;
  p.A = static_cast<const float*>(A); p.B = static_cast<const float*>(B); p.C = static_cast<float*>(C);
  p.bias = static_cast<const float*>(bias); p.mask = static_cast<const float*>(mask); p.colsum = static_cast<float*>(colsum);
  p.m = (uint32_t)m; p.n = (uint32_t)n; p.k = (uint32_t)k;
  p.lda = (uint32_t)lda; p.ldb = (uint32_t)ldb; p.ldc = (uint32_t)ldc;
  p.alpha = (float)alpha; p.beta = (float)beta; p.epilogue = epilogue; p.tb = tb ? 1 : 0;
  if (ta) {
    // weight gradient of a narrow layer: A [k, m], B [k, n]
    if (tb || m > 16 || n < 16 || n > 256 || 256 % n != 0 || k < 1024 || epilogue != ZG_EPI_NONE || colsum) return false;
    prescale_c<float>(s, static_cast<float*>(C), 1, m, n, ldc, m * ldc, beta);
    const size_t ctas = std::min<size_t>((k + 31) / 32, (size_t)sm_count() * 2);
    const uint32_t rows_per_cta = (uint32_t)((k + ctas - 1) / ctas);
    const unsigned grid = (unsigned)((k + rows_per_cta - 1) / rows_per_cta);
    const int mmax = m <= 4 ? 4 : (m <= 8 ? 8 : (m <= 12 ? 12 : 16));
    const size_t smem = (size_t)(skinny::kThreads / n) * mmax * n * sizeof(float);
    if (mmax == 4) return launch_pdl(skinny::skinny_m_kernel<4>, dim3(grid), dim3(skinny::kThreads), smem, s, p, rows_per_cta);
    if (mmax == 8) return launch_pdl(skinny::skinny_m_kernel<8>, dim3(grid), dim3(skinny::kThreads), smem, s, p, rows_per_cta);
    if (mmax == 12) return launch_pdl(skinny::skinny_m_kernel<12>, dim3(grid), dim3(skinny::kThreads), smem, s, p, rows_per_cta);
    return launch_pdl(skinny::skinny_m_kernel<16>, dim3(grid), dim3(skinny::kThreads), smem, s, p, rows_per_cta);
  }
  if (m < 256) return false;
  if (n <= 16 && k >= 16 && k <= 512 && k % 4 == 0 && lda % 4 == 0 && host_aligned16(A) && epilogue != ZG_EPI_RELU_MASK && !colsum) {
    const unsigned grid = (unsigned)((m + skinny::kThreads / 4 - 1) / (skinny::kThreads / 4));
    const size_t smem = (size_t)n * k * sizeof(float);
    if (n <= 4) return launch_pdl(skinny::skinny_n_kernel<4>, dim3(grid), dim3(skinny::kThreads), smem, s, p);
    if (n <= 8) return launch_pdl(skinny::skinny_n_kernel<8>, dim3(grid), dim3(skinny::kThreads), smem, s, p);
    if (n <= 12) return launch_pdl(skinny::skinny_n_kernel<12>, dim3(grid), dim3(skinny::kThreads), smem, s, p);
    return launch_pdl(skinny::skinny_n_kernel<16>, dim3(grid), dim3(skinny::kThreads), smem, s, p);
  }
  if (k <= 16 && n >= 16 && n <= 256 && n % 4 == 0 && ldc % 4 == 0 && host_aligned16(C) && beta == 0.0 &&
      (epilogue != ZG_EPI_RELU_MASK || host_aligned16(mask)) && (!bias || host_aligned16(bias))) {
    const size_t cg = n / 4;
    if (colsum && (cg & (cg - 1)) != 0) return false;  // a thread keeps one column group only when cg divides the stride
    const size_t want = (m * cg + skinny::kThreads - 1) / skinny::kThreads;
    const unsigned grid = (unsigned)std::min<size_t>(want, (size_t)sm_count() * 8);
    const size_t smem = ((size_t)n * k + n) * sizeof(float);
    if (k <= 4) return launch_pdl(skinny::skinny_k_kernel<4>, dim3(grid), dim3(skinny::kThreads), smem, s, p);
    if (k <= 8) return launch_pdl(skinny::skinny_k_kernel<8>, dim3(grid), dim3(skinny::kThreads), smem, s, p);
    if (k <= 12) return launch_pdl(skinny::skinny_k_kernel<12>, dim3(grid), dim3(skinny::kThreads), smem, s, p);
    return launch_pdl(skinny::skinny_k_kernel<16>, dim3(grid), dim3(skinny::kThreads), smem, s, p);
  }
  return false;
}

// SM budget of the zg_bmm call in progress (zg_bmm_sm_budget): GEMMs that run side by side on parallel
// streams size their split-K grids for a share of the SMs, so that together they fit in one wave
// (a CTA of these kernels takes a whole SM's shared memory; an oversubscribed launch runs its
// surplus CTAs in a second wave after the first has drained).
static thread_local int g_next_sm_budget = 0, g_sm_budget = 0;
static size_t sm_share() {
  const size_t all = (size_t)sm_count();
  return (g_sm_budget > 0 && (size_t)g_sm_budget < all) ? (size_t)g_sm_budget : all;
}
extern "C" void zg_bmm_sm_budget(int sms) { g_next_sm_budget = sms > 0 ? sms : 0; }

// Returns true when the tensor-core path took the problem.
static bool try_tensor_core(dtype id, dtype c_id, cudaStream_t s, const void* A, const void* B, void* C, len_t nA, len_t nB, len_t nC,
                            len_t m, len_t n, len_t k, bool ta, bool tb, len_t lda, len_t ldb, len_t ldc, double alpha, double beta,
                            int epilogue, const void* bias, const void* mask, void* colsum) {
  const bool bf16 = (id == BF16);
  if (!(id == SINGLE || bf16)) return false;
  if (id == SINGLE && (g_math_mode == ZG_MATH_FFMA || c_id != SINGLE)) return false;
  if (bf16 && !(c_id == SINGLE || c_id == BF16)) return false;
  const size_t es = bf16 ? 2 : 4;
  if (!host_aligned16(A) || !host_aligned16(B) || (lda * es) % 16 || (ldb * es) % 16) return false;
  if (m == 0 || n == 0 || nC == 0) return false;
  if (m > 0x7fffffffu || n > 0x7fffffffu || k > 0x7fffffffu || ldc > 0xffffffffu) return false;
  // tiny problems are launch-bound either way; keep them on the FFMA kernel
  const char* force = getenv("ZG_GEMM_FORCE_TC");
  if (!(force && force[0] == '1') && (double)m * (double)n * (double)k < 64.0 * 64.0 * 64.0) return false;

  const int mode = bf16 ? tc::kBF16 : (g_math_mode == ZG_MATH_TF32 ? tc::kTF32 : tc::kFP32X3);
  const int atom = bf16 ? 64 : 32;        // M/N elements per 128-byte column block
  const int bk = bf16 ? 64 : 32;
  const bool a_kmajor = !ta;              // A stored [m,k] -> K contiguous
  const bool b_kmajor = tb;               // B stored [n,k] -> K contiguous
  // Large single-pass problems: persistent kernel over 128 x 256 tiles
  // (at least one tile per SM, k deep enough to amortise the tile hand-over).
  const char* no_persist = getenv("ZG_GEMM_NO_PERSISTENT");
  const size_t ptiles = ((m + 127) / 128) * ((n + 255) / 256) * nC;
  const bool persistent = mode != tc::kFP32X3 && n > 128 && k >= 8 * (size_t)bk && ptiles * 2 >= (size_t)sm_count() &&
                          ptiles <= 0x3fffffffu && !(no_persist && no_persist[0] == '1');
  int bn = persistent ? 256 : (n <= 32 ? 32 : (n <= 64 ? 64 : 128));
  if (bn < atom) bn = atom;               // MN-major B needs whole column blocks; bf16 has no BN=32 instance
  size_t tiles = ((m + 127) / 128) * ((n + bn - 1) / bn) * nC;
  // Deep-k problems with a plain epilogue (weight gradients) get their
  // parallelism from K splits, so they keep the wide tile (fewer operand bytes
  // per flop through shared memory); everything else halves BN when there are
  // too few tiles to occupy the SMs.
  // (with a fused epilogue or column sums the last CTA of a tile applies them to the finished sums)
  // and that costs a second pass over the tile, so it is kept for problems with very few tiles)
  const bool deferred = epilogue != ZG_EPI_NONE || colsum;
  const bool can_split = !persistent && c_id == SINGLE && k >= 512 && (!deferred || tiles * 4 <= sm_share());
  if (!can_split && bn == 128 && tiles * 2 <= sm_share() && n > 64) {
    bn = 64;
    tiles = ((m + 127) / 128) * ((n + bn - 1) / bn) * nC;
  }

  unsigned splits = 1;
  if (persistent && epilogue == ZG_EPI_NONE && !colsum && c_id == SINGLE) {
    // K ranges as work items when that fills the last wave better (>= 16 k-slabs per range)
    const double sms = (double)sm_count();
    double best = 0.0;
    for (unsigned sp = 1; sp <= 4; sp *= 2) {
      if (sp > 1 && k / sp < 16 * (size_t)bk) break;
      const double items = (double)ptiles * sp;
      const double eff = items / (std::ceil(items / sms) * sms);
      if (eff > best + 0.03) { best = eff; splits = sp; }
    }
  }
  if (can_split && tiles * 2 <= sm_share()) {
    size_t want = sm_share() / tiles;
    size_t maxs = k / (4 * (size_t)bk);  // at least four k-slabs per split
    splits = (unsigned)(want < maxs ? want : maxs);
    if (splits < 1) splits = 1;
  }
  const size_t k_per_split = splits > 1 ? ((k + splits - 1) / splits + bk - 1) / bk * bk : ((k + bk - 1) / bk * bk);
  if (splits > 1) splits = (unsigned)((k + k_per_split - 1) / k_per_split);

  CUtensorMap tmA, tmB;
  bool ok;
  // MN-major fp32 operands travel in the 128-byte swizzle with 32-byte atoms
  if (a_kmajor) ok = make_tmap(&tmA, bf16, A, k, m, nA, lda, bk, 128, false);
  else ok = make_tmap(&tmA, bf16, A, m, k, nA, lda, atom, bk, !bf16);
  if (!ok) return true;  // error recorded
  if (b_kmajor) ok = make_tmap(&tmB, bf16, B, k, n, nB, ldb, bk, bn, false);
  else ok = make_tmap(&tmB, bf16, B, n, k, nB, ldb, atom, bk, !bf16);
  if (!ok) return true;

  tc::Params p;
  memset(&p, 0, sizeof(p));
  if (c_id == SINGLE) { p.C = static_cast<float*>(C); p.mask = static_cast<const float*>(mask); }
  else { p.Cb = static_cast<__nv_bfloat16*>(C); p.maskb = static_cast<const __nv_bfloat16*>(mask); }
  p.bias = static_cast<const float*>(bias);
  p.colsum = static_cast<float*>(colsum);
  p.c_batch_stride = (uint64_t)m * ldc;
  p.m = (uint32_t)m; p.n = (uint32_t)n; p.k = (uint32_t)k; p.ldc = (uint32_t)ldc;
  p.nA = (uint32_t)nA; p.nB = (uint32_t)nB;
  p.splits = splits; p.k_per_split = (uint32_t)k_per_split;
  p.alpha = (float)alpha; p.beta = (float)beta; p.epilogue = epilogue;
  {
    const size_t ce = (c_id == SINGLE) ? 4 : 2;
    bool ok = host_aligned16(C) && (ldc * ce) % 16 == 0 && ((uint64_t)m * ldc * ce) % 16 == 0;
    if (mask) ok = ok && host_aligned16(mask);
    if (bias) ok = ok && host_aligned16(bias);
    p.vec_ok = ok ? 1 : 0;
  }
  p.error_flag = tc_error_flag();
  if (persistent) {
    const uint32_t tiles_m = (uint32_t)((m + 127) / 128), tiles_n = (uint32_t)((n + 255) / 256);
    const uint32_t items = (uint32_t)(ptiles * splits);
    if (splits > 1) prescale_c<float>(s, static_cast<float*>(C), nC, m, n, ldc, m * ldc, beta);
    if (mode == tc::kBF16) launch_persistent<tc::kBF16>(s, a_kmajor, b_kmajor, tmA, tmB, p, tiles_m, tiles_n, items);
    else launch_persistent<tc::kTF32>(s, a_kmajor, b_kmajor, tmA, tmB, p, tiles_m, tiles_n, items);
    return true;
  }
  if (splits > 1) prescale_c<float>(s, static_cast<float*>(C), nC, m, n, ldc, m * ldc, beta);
  if (splits > 1 && deferred) {
    unsigned* unused = nullptr;
    p.tile_tickets = static_cast<unsigned*>(workspace(s, sizeof(unsigned) * tiles, &unused, 2));
    if (!p.tile_tickets) return true;
    p.deferred_epilogue = epilogue;
    p.deferred_colsum = p.colsum;
    p.epilogue = ZG_EPI_NONE;
    p.colsum = nullptr;
  }
  dim3 grid((unsigned)((n + bn - 1) / bn), (unsigned)((m + 127) / 128), (unsigned)(nC * splits));
  if (grid.y > 65535 || grid.z > 65535) return false;
  // Output through the C tensor map where the epilogue needs nothing from global memory but the bias
  // (ZG_GEMM_TMA_EPILOGUE=0 keeps the register path)
  CUtensorMap tmC;
  memset(&tmC, 0, sizeof(tmC));
  static const bool tma_epi_on = [] { const char* e = getenv("ZG_GEMM_TMA_EPILOGUE"); return !(e && e[0] == '0'); }();
  if (tma_epi_on && c_id == SINGLE && p.vec_ok && !p.tile_tickets && !p.colsum && nC <= 0x7fffffffu &&
      (splits > 1 ? epilogue == ZG_EPI_NONE : (beta == 0.0 && epilogue != ZG_EPI_RELU_MASK))) {
    if (!make_tmap(&tmC, false, C, n, m, nC, ldc, 32, 32, false)) return true;
    p.tma_epilogue = splits > 1 ? 2 : 1;
  }
  if (mode == tc::kBF16) launch_tc_mode<tc::kBF16>(s, bn, a_kmajor, b_kmajor, tmA, tmB, tmC, p, grid);
  else if (mode == tc::kTF32) launch_tc_mode<tc::kTF32>(s, bn, a_kmajor, b_kmajor, tmA, tmB, tmC, p, grid);
  else launch_tc_mode<tc::kFP32X3>(s, bn, a_kmajor, b_kmajor, tmA, tmB, tmC, p, grid);
  return true;
}

void bmm_dispatch(dtype id, dtype c_id, cudaStream_t s, const void* A, const void* B, void* C, len_t nA, len_t nB, len_t nC, len_t m,
                  len_t n, len_t k, bool ta, bool tb, len_t lda, len_t ldb, len_t ldc, double alpha, double beta, int epilogue,
                  const void* bias, const void* mask, void* colsum) {
  g_sm_budget = g_next_sm_budget;
  g_next_sm_budget = 0;
  if (m == 0 || n == 0 || nC == 0) return;
  if (nA == 0 || nB == 0) { set_error(kBadArgument, "bmm: empty operand batch"); return; }
  if (epilogue < ZG_EPI_NONE || epilogue > ZG_EPI_RELU_MASK) { set_error(kBadArgument, "bmm: unknown epilogue %d", epilogue); return; }
  if ((epilogue == ZG_EPI_BIAS || epilogue == ZG_EPI_BIAS_RELU) && !bias) { set_error(kBadArgument, "bmm: bias epilogue without bias"); return; }
  if (epilogue == ZG_EPI_RELU_MASK && !mask) { set_error(kBadArgument, "bmm: mask epilogue without mask source"); return; }
  if (colsum && id == DOUBLE) { set_error(kUnsupported, "bmm: column sums are fp32 only"); return; }
  if (try_skinny(id, c_id, s, A, B, C, nA, nB, nC, m, n, k, ta, tb, lda, ldb, ldc, alpha, beta, epilogue, bias, mask, colsum)) return;
  if (try_tensor_core(id, c_id, s, A, B, C, nA, nB, nC, m, n, k, ta, tb, lda, ldb, ldc, alpha, beta, epilogue, bias, mask, colsum)) return;
  if (id == SINGLE && c_id == SINGLE) launch_simt<float, float>(s, A, B, C, nA, nB, nC, m, n, k, ta, tb, lda, ldb, ldc, alpha, beta, epilogue, bias, mask, colsum);
  else if (id == DOUBLE && c_id == DOUBLE) launch_simt<double, double>(s, A, B, C, nA, nB, nC, m, n, k, ta, tb, lda, ldb, ldc, alpha, beta, epilogue, bias, mask, colsum);
  else if (id == BF16 && c_id == SINGLE) launch_simt<__nv_bfloat16, float>(s, A, B, C, nA, nB, nC, m, n, k, ta, tb, lda, ldb, ldc, alpha, beta, epilogue, bias, mask, colsum);
  else if (id == BF16 && c_id == BF16) launch_simt<__nv_bfloat16, __nv_bfloat16>(s, A, B, C, nA, nB, nC, m, n, k, ta, tb, lda, ldb, ldc, alpha, beta, epilogue, bias, mask, colsum);
  else set_error(kUnsupported, "bmm: unsupported dtype combination %d -> %d", (int)id, (int)c_id);
}

// ---- fused middle of the MLP step (mlp_tail.cuh)
template <int CP>
static bool launch_tail_inst(cudaStream_t s, const CUtensorMap& ta, const CUtensorMap& tk, const CUtensorMap& tn, const CUtensorMap& t1,
                             const CUtensorMap& td1, const CUtensorMap& td0, const tail::Params& p, unsigned grid) {
  auto kern = tail::mlp_tail_kernel<CP>;
  static bool attr_set = false;
  if (!attr_set) {
    if (!ZG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tail::kSmemBytes))) return false;
    attr_set = true;
  }
  return launch_pdl(kern, dim3(grid), dim3(tail::kThreads), (size_t)tail::kSmemBytes, s, ta, tk, tn, t1, td1, td0, p);
}

void mlp_tail_launch(cudaStream_t s, len_t rows, len_t h1, len_t h2, len_t C, const void* act0, const void* W1, const void* b1, const void* W2,
                     const void* b2, const void* labels, int label_kind, len_t ld_out, double loss_div, void* act1, void* logits, void* loss_out,
                     void* dlogits, void* dact1, void* dact0, void* db2, void* db1, void* db0, int weights_ready) {
  if (rows == 0) return;
  if (h1 != (len_t)tail::kH1 || h2 != (len_t)tail::kH2 || C == 0 || C > (len_t)tail::kCMax) {
    set_error(kUnsupported, "zg_mlp_tail_fwd_bwd: widths %lu -> %lu -> %lu (built for %d -> %d -> at most %d)", h1, h2, C, tail::kH1, tail::kH2, tail::kCMax);
    return;
  }
  if (rows > 0x7fffffffu || ld_out < C || ld_out > 0xffffffffu) { set_error(kBadArgument, "zg_mlp_tail_fwd_bwd: rows %lu, ld_out %lu", rows, ld_out); return; }
  if (label_kind != ZG_LABEL_ONEHOT && label_kind != ZG_LABEL_INDEX) { set_error(kBadArgument, "zg_mlp_tail_fwd_bwd: unknown label kind %d", label_kind); return; }
  const void* ptrs[] = {act0, W1, b1, W2, b2, labels, act1, logits, loss_out, dlogits, dact1, dact0, db2, db1, db0};
  for (const void* q : ptrs)
    if (!q) { set_error(kBadArgument, "zg_mlp_tail_fwd_bwd: NULL argument"); return; }
  if (!host_aligned16(act0) || !host_aligned16(W1) || !host_aligned16(act1) || !host_aligned16(dact1) || !host_aligned16(dact0)) {
    set_error(kBadArgument, "zg_mlp_tail_fwd_bwd: act0, W1, act1, dact1 and dact0 must be 16-byte aligned");
    return;
  }
  if (ld_out > (len_t)tail::kCMax) { set_error(kBadArgument, "zg_mlp_tail_fwd_bwd: ld_out %lu above %d", ld_out, tail::kCMax); return; }
  CUtensorMap tmA, tmK, tmN, tm1, tmD1, tmD0;
  // outputs leave through TMA stores of [128 rows x 32 floats] slabs (rows past the end are clipped)
  if (!make_tmap(&tm1, false, act1, tail::kH2, rows, 1, tail::kH2, 32, tail::kRows, false)) return;
  if (!make_tmap(&tmD1, false, dact1, tail::kH2, rows, 1, tail::kH2, 32, tail::kRows, false)) return;
  if (!make_tmap(&tmD0, false, dact0, tail::kH1, rows, 1, tail::kH1, 32, tail::kRows, false)) return;
  if (!make_tmap(&tmA, false, act0, tail::kH1, rows, 1, tail::kH1, 32, tail::kRows, false)) return;
  if (!make_tmap(&tmK, false, W1, tail::kH1, tail::kH2, 1, tail::kH1, 32, tail::kH2, false)) return;   // B of act0 W1^T: [n = 64 rows][k contiguous]
  if (!make_tmap(&tmN, false, W1, tail::kH1, tail::kH2, 1, tail::kH1, 32, 32, true)) return;           // B of dact1 W1: [k = 64 rows][n contiguous]
  const unsigned grid = (unsigned)((rows + tail::kRows - 1) / tail::kRows);
  unsigned* counters = nullptr;
  float* partial = static_cast<float*>(workspace(s, sizeof(float) * grid, &counters));
  if (!partial) return;
  tail::Params p;
  memset(&p, 0, sizeof(p));
  p.W2 = static_cast<const float*>(W2); p.b1 = static_cast<const float*>(b1); p.b2 = static_cast<const float*>(b2);
  p.labels = labels; p.label_index = label_kind == ZG_LABEL_INDEX ? 1 : 0;
  p.logits = static_cast<float*>(logits); p.dlogits = static_cast<float*>(dlogits);
  p.db2 = static_cast<float*>(db2); p.db1 = static_cast<float*>(db1); p.db0 = static_cast<float*>(db0);
  p.loss_out = static_cast<float*>(loss_out); p.loss_partial = partial; p.counter = counters;
  p.rows = (uint32_t)rows; p.C = (uint32_t)C; p.ld_out = (uint32_t)ld_out;
  p.divisor = (float)loss_div; p.inv_divisor = 1.f / p.divisor;
  int e = 0;
  p.exact_inv = (std::frexp(p.divisor, &e) == 0.5f && std::isnormal(p.inv_divisor)) ? 1 : 0;
  p.early_weights = weights_ready ? 1 : 0;
  p.error_flag = tc_error_flag();
  if (C <= 4) launch_tail_inst<4>(s, tmA, tmK, tmN, tm1, tmD1, tmD0, p, grid);
  else if (C <= 8) launch_tail_inst<8>(s, tmA, tmK, tmN, tm1, tmD1, tmD0, p, grid);
  else if (C <= 12) launch_tail_inst<12>(s, tmA, tmK, tmN, tm1, tmD1, tmD0, p, grid);
  else launch_tail_inst<16>(s, tmA, tmK, tmN, tm1, tmD1, tmD0, p, grid);
}

int* kernel_timeout_flag() { return tc_error_flag(); }

// Reads (and clears) the device flag that a kernel raises when one of its bounded waits runs out.
void check_tc_errors() {
  int* f = tc_error_flag();
  if (!f) return;
  int v = 0;
  if (cudaMemcpy(&v, f, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess && v) {
    cudaMemset(f, 0, sizeof(int));
    cudaDeviceSynchronize();
    set_error(kKernelTimeout, "a kernel gave up waiting on a pipeline barrier");
  }
}

// y = alpha*op(A)x + beta*y : one warp per output element of the no-trans
// case, one thread per output element (coalesced over columns) when transposed
template <typename T>
__global__ void __launch_bounds__(256) gemv_n_kernel(const T* __restrict__ A, const T* __restrict__ x, T* y, size_t m, size_t n, T alpha, T beta) {
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < m; r += warps) {
    T s = T(0);
    for (size_t j = lane; j < n; j += 32) s += A[r * n + j] * x[j];
    s = warp_sum(s);
    if (lane == 0) y[r] = (beta == T(0)) ? alpha * s : alpha * s + beta * y[r];
  }
}
template <typename T>
__global__ void __launch_bounds__(256) gemv_t_kernel(const T* __restrict__ A, const T* __restrict__ x, T* y, size_t m, size_t n, T alpha, T beta) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < n; c += nth) {
    T s = T(0);
    for (size_t i = 0; i < m; ++i) s += A[i * n + c] * x[i];
    y[c] = (beta == T(0)) ? alpha * s : alpha * s + beta * y[c];
  }
}
template <typename T>
__global__ void __launch_bounds__(256) ger_kernel(const T* __restrict__ a, const T* __restrict__ b, T* C, size_t m, size_t n, size_t ldc, T alpha) {
  const size_t total = m * n, nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nth) {
    const size_t r = i / n, c = i % n;
    C[r * ldc + c] += alpha * a[r] * b[c];
  }
}

}  // namespace zg

using namespace zg;

namespace zg {
void mlp_tail_launch(cudaStream_t s, len_t rows, len_t h1, len_t h2, len_t C, const void* act0, const void* W1, const void* b1, const void* W2,
                     const void* b2, const void* labels, int label_kind, len_t ld_out, double loss_div, void* act1, void* logits, void* loss_out,
                     void* dlogits, void* dact1, void* dact0, void* db2, void* db1, void* db0, int weights_ready);
}
extern "C" int zg_mlp_tail_supported(dtype id, len_t h1, len_t h2, len_t C) {
  return (id == SINGLE && g_math_mode != ZG_MATH_FFMA && h1 == (len_t)tail::kH1 && h2 == (len_t)tail::kH2 && C >= 1 && C <= (len_t)tail::kCMax) ? 1 : 0;
}
extern "C" void zg_mlp_tail_fwd_bwd(dtype id, StreamWrapper stream, len_t rows, len_t h1, len_t h2, len_t C, const void* act0, const void* W1,
                                    const void* b1, const void* W2, const void* b2, const void* labels, int label_kind, len_t ld_out,
                                    double loss_div, void* act1, void* logits, void* loss_out, void* dlogits, void* dact1, void* dact0,
                                    void* db2, void* db1, void* db0, int weights_ready) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_mlp_tail_fwd_bwd: only SINGLE is implemented"); return; }
  mlp_tail_launch(as_stream(stream), rows, h1, h2, C, act0, W1, b1, W2, b2, labels, label_kind, ld_out, loss_div, act1, logits, loss_out,
                  dlogits, dact1, dact0, db2, db1, db0, weights_ready);
}

extern "C" void zg_set_math_mode(int mode) {
  if (mode < ZG_MATH_FP32X3 || mode > ZG_MATH_FFMA) { set_error(kBadArgument, "zg_set_math_mode: unknown mode %d", mode); return; }
  g_math_mode = mode;
}
extern "C" int zg_get_math_mode(void) { return g_math_mode; }

extern "C" void zg_bmm(dtype id, dtype c_id, StreamWrapper stream, const void* A, const void* B, void* C, len_t nA, len_t nB, len_t nC,
                       len_t m, len_t n, len_t k, bool trans_a, bool trans_b, len_t lda, len_t ldb, len_t ldc, double alpha, double beta,
                       int epilogue, const void* bias, const void* mask_src, void* colsum) {
  bmm_dispatch(id, c_id, as_stream(stream), A, B, C, nA, nB, nC, m, n, k, trans_a, trans_b, lda, ldb, ldc, alpha, beta, epilogue, bias, mask_src, colsum);
}

extern "C" void gemm(dtype id, CublasWrapper w, const void* a, const void* b, void* c, len_t m, len_t n, len_t k, bool trans_a,
                     bool trans_b, len_t lda, len_t ldb, len_t ldc, double alpha, double beta) {
  bmm_dispatch(id, id, as_stream(w), a, b, c, 1, 1, 1, m, n, k, trans_a, trans_b, lda, ldb, ldc, alpha, beta, ZG_EPI_NONE, nullptr, nullptr, nullptr);
}

extern "C" void gemv(dtype id, CublasWrapper w, const void* a, const void* x, void* y, len_t m, len_t n, bool trans_a, double alpha,
                     double beta) {
  if (m == 0 || n == 0) return;
  cudaStream_t s = as_stream(w);
  if (id == SINGLE) {
    if (trans_a) gemv_t_kernel<float><<<grid_for(n, 256), 256, 0, s>>>((const float*)a, (const float*)x, (float*)y, m, n, (float)alpha, (float)beta);
    else gemv_n_kernel<float><<<grid_for(m, 8), 256, 0, s>>>((const float*)a, (const float*)x, (float*)y, m, n, (float)alpha, (float)beta);
  } else if (id == DOUBLE) {
    if (trans_a) gemv_t_kernel<double><<<grid_for(n, 256), 256, 0, s>>>((const double*)a, (const double*)x, (double*)y, m, n, alpha, beta);
    else gemv_n_kernel<double><<<grid_for(m, 8), 256, 0, s>>>((const double*)a, (const double*)x, (double*)y, m, n, alpha, beta);
  } else { set_error(kUnsupported, "gemv: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}

extern "C" void ger(dtype id, CublasWrapper w, const void* a, const void* b, void* c, len_t m, len_t n, len_t ldc, double alpha) {
  if (m == 0 || n == 0) return;
  cudaStream_t s = as_stream(w);
  if (id == SINGLE) ger_kernel<float><<<grid_for(m * n, 1024), 256, 0, s>>>((const float*)a, (const float*)b, (float*)c, m, n, ldc, (float)alpha);
  else if (id == DOUBLE) ger_kernel<double><<<grid_for(m * n, 1024), 256, 0, s>>>((const double*)a, (const double*)b, (double*)c, m, n, ldc, alpha);
  else { set_error(kUnsupported, "ger: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}
