// Shared helpers of the device library: status handling, stream casts,
// vector access and warp/block reductions.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/decls.h"
#include "../../include/zg_b200.h"

namespace zg {

// ---------------------------------------------------------------- status
// The first error since the last zg_clear_error() is kept (sticky); later
// ones are dropped so that the root cause is what the caller sees.
enum Status : int {
  kOk = 0,
  kCudaError = 1,       // a CUDA runtime/driver call failed
  kBadArgument = 2,     // shapes / dtype / alignment not supported
  kOutOfMemory = 3,
  kKernelTimeout = 4,   // a bounded device-side wait ran out
  kUnsupported = 5,
};

void set_error(int code, const char* fmt, ...);
bool check_cuda(cudaError_t e, const char* what, const char* file, int line);

#define ZG_CUDA(expr) ::zg::check_cuda((expr), #expr, __FILE__, __LINE__)
#define ZG_LAUNCH_CHECK() ::zg::check_cuda(cudaPeekAtLastError(), "kernel launch", __FILE__, __LINE__)

// A stream-bound op context: what CublasWrapper / CudnnWrapper /
// CutensorWrapper point to.
struct OpContext {
  cudaStream_t stream;
  void* plans;  // plan cache (owned; see reduce_plan.cu)
};

static inline cudaStream_t as_stream(StreamWrapper w) { return static_cast<cudaStream_t>(w.ptr); }
static inline cudaStream_t as_stream(CublasWrapper w) { return static_cast<OpContext*>(w.ptr)->stream; }
static inline cudaStream_t as_stream(CudnnWrapper w) { return static_cast<OpContext*>(w.ptr)->stream; }
static inline cudaStream_t as_stream(CutensorWrapper w) { return static_cast<OpContext*>(w.ptr)->stream; }

int sm_count();  // SMs of the current device (cached)

// Per-stream scratch owned by the library (runtime.cu).  Returns a 256-byte
// aligned buffer of at least `bytes`; *counters points at 64 zero-initialised
// unsigned counters that a kernel must leave at zero when it finishes.
// Slots 0 and 1 are scratch; slot 2 is zero when handed out and every kernel
// that uses it leaves it zero (arrival counters of multi-CTA reductions).
void* workspace(cudaStream_t s, size_t bytes, unsigned** counters, int slot = 0);

// y[col] = column sums of x[row, col] (fp32, two-stage, deterministic; uses workspace slot 0)
void fold_rows_f32(cudaStream_t s, const float* x, float* y, size_t row, size_t col);

// gemm.cu: reads (and clears) the per-device flag that a tensor-core kernel
// raises when one of its bounded waits runs out; allocates the flag on first use.
void check_tc_errors();
// The same per-device flag (device memory, int): any kernel with bounded waits raises it when one runs out.
int* kernel_timeout_flag();

// Grid size for a grid-stride kernel: enough CTAs for `work_items` at
// `per_cta` items each, capped at `waves` resident waves of the device.
static inline unsigned grid_for(size_t work_items, size_t per_cta, int ctas_per_sm = 8) {
  size_t want = (work_items + per_cta - 1) / per_cta;
  size_t cap = (size_t)sm_count() * ctas_per_sm;
  if (want < 1) want = 1;
  return (unsigned)(want < cap ? want : cap);
}

// ------------------------------------------- programmatic dependent launch
// Kernels launched through launch_pdl() may begin (block scheduling, their
// prologue up to pdl_wait()) while the previous kernel of the stream is still
// draining; pdl_wait() returns once that kernel has completed and its writes
// are visible.  A kernel launched this way must call pdl_wait() before its
// first global-memory access of data another kernel produces or still reads,
// and pdl_trigger() after it, so that at most one successor is resident early.
// Inside a captured graph the edge becomes a programmatic dependency.
bool pdl_enabled();  // runtime.cu; off with ZG_PDL=0 in the environment

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
static inline bool launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr;
  memset(&attr, 0, sizeof(attr));
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return check_cuda(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), "kernel launch", __FILE__, __LINE__);
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_sync() { pdl_wait(); pdl_trigger(); }

// ------------------------------------------------------------- device side
template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T>
__device__ __forceinline__ T warp_max(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    T u = __shfl_xor_sync(0xffffffffu, v, o);
    v = u > v ? u : v;
  }
  return v;
}

// Block-wide sum; every thread receives the result.  `smem` needs 32 slots.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  T r = (threadIdx.x < nw) ? smem[threadIdx.x] : T(0);
  if (warp == 0) {
    r = warp_sum(r);
    if (lane == 0) smem[0] = r;
  }
  __syncthreads();
  return smem[0];
}

template <typename T>
struct Vec4 {};
template <>
struct Vec4<float> {
  using type = float4;
};
template <>
struct Vec4<double> {
  using type = double4;  // 32 bytes; split into two 16-byte accesses by the compiler
};

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
#endif

static inline bool host_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace zg
