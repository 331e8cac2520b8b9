// Device / stream / memory / graph-capture / virtual-memory entry points
// (include/cuda_utils.h) and the sticky error status (include/zg_b200.h).
#include <cmath>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include <cuda.h>

#include "common.cuh"
#include "driver_api.h"
#include "../../include/cuda_utils.h"

namespace zg {

// ------------------------------------------------------------------ status
static std::mutex g_err_mu;
static int g_err_code = 0;
static char g_err_msg[512] = "";

void set_error(int code, const char* fmt, ...) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  if (g_err_code != 0) return;  // keep the first
  g_err_code = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err_msg, sizeof(g_err_msg), fmt, ap);
  va_end(ap);
  if (getenv("ZG_CUDA_VERBOSE")) fprintf(stderr, "[zigrad-b200] error %d: %s\n", code, g_err_msg);
}

bool check_cuda(cudaError_t e, const char* what, const char* file, int line) {
  if (e == cudaSuccess) return true;
  set_error(e == cudaErrorMemoryAllocation ? kOutOfMemory : kCudaError, "%s failed: %s (%s) at %s:%d", what,
            cudaGetErrorName(e), cudaGetErrorString(e), file, line);
  return false;
}

bool check_cu(CUresult r, const char* what, const char* file, int line) {
  if (r == CUDA_SUCCESS) return true;
  set_error(r == CUDA_ERROR_OUT_OF_MEMORY ? kOutOfMemory : kCudaError, "%s failed: CUresult %d at %s:%d", what, (int)r,
            file, line);
  return false;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Driver entry points are resolved through the runtime so that the library
// does not link libcuda directly (it must load on machines without a driver).
void* driver_symbol(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
    set_error(kCudaError, "driver entry point %s unavailable", name);
    (void)cudaGetLastError();
    return nullptr;
  }
  return fn;
}

// --------------------------------------------------------- fill / sequence
template <typename T>
__global__ void fill_kernel(T* __restrict__ p, size_t n, T v) {
  pdl_sync();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if constexpr (sizeof(T) == 4) {
    // 128-bit stores over the aligned body, scalar head/tail
    const uintptr_t addr = reinterpret_cast<uintptr_t>(p);
    size_t head = ((16 - (addr & 15)) & 15) / sizeof(T);
    if (head > n) head = n;
    const size_t nvec = (n - head) / 4;
    float4 vv;
    vv.x = vv.y = vv.z = vv.w = __int_as_float(*reinterpret_cast<int*>(&v));
    float4* pv = reinterpret_cast<float4*>(p + head);
    for (size_t j = i; j < nvec; j += stride) pv[j] = vv;
    const size_t tail0 = head + nvec * 4;
    for (size_t j = i; j < head; j += stride) p[j] = v;
    for (size_t j = tail0 + i; j < n; j += stride) p[j] = v;
  } else {
    for (; i < n; i += stride) p[i] = v;
  }
}

template <typename T>
__global__ void sequence_kernel(T* __restrict__ p, size_t n, T init, T step) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = init + step * (T)i;
}

template <typename T, typename I>
__global__ void take_kernel(const T* __restrict__ src, const I* __restrict__ idx, size_t n, T* __restrict__ dst) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = src[idx[i]];
}

// Philox-4x32-10 counter-based generator (Salmon et al., SC'11): element i
// of a buffer uses counter (i/4) and lane i%4, so results do not depend on the
// launch geometry.
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
__device__ __forceinline__ void philox4x32(uint64_t ctr, uint32_t seed, uint32_t (&out)[4]) {
  uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u};
  uint32_t k0 = seed, k1 = 0x5EEDu;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

template <typename T>
__global__ void random_kernel(T* __restrict__ p, size_t n, int normal, uint32_t seed) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t ngroups = (n + 3) / 4;
  for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < ngroups; g += stride) {
    uint32_t r[4];
    philox4x32(g, seed, r);
    float u[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) u[j] = (float)(r[j] >> 8) * (1.0f / 16777216.0f);  // [0,1)
    float o[4];
    if (normal) {  // Box-Muller on pairs
      const float a0 = sqrtf(-2.f * logf(1.f - u[0])), a1 = sqrtf(-2.f * logf(1.f - u[2]));
      o[0] = a0 * cospif(2.f * u[1]); o[1] = a0 * sinpif(2.f * u[1]);
      o[2] = a1 * cospif(2.f * u[3]); o[3] = a1 * sinpif(2.f * u[3]);
    } else {
      o[0] = u[0]; o[1] = u[1]; o[2] = u[2]; o[3] = u[3];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (g * 4 + j < n) p[g * 4 + j] = (T)o[j];
  }
}


// Library-owned scratch ("workspace") per stream: partial results of the
// two-stage reductions and split-K GEMMs live here.  Grown with cudaMalloc on
// demand (so the first call of a given size must happen outside a stream
// capture); never shrinks, and an outgrown buffer stays allocated, so a graph
// captured while it was current remains valid to replay.  The first 256 bytes hold counters that kernels
// leave at zero when they finish.  Slot 0 holds kernel partials; slot 1 holds
// intermediates of multi-stage host-sequenced reductions (which themselves
// launch kernels that use slot 0).
struct Workspace {
  void* base = nullptr;
  size_t bytes = 0;
};
static std::mutex g_ws_mu;
static std::map<std::pair<std::pair<int, int>, cudaStream_t>, Workspace> g_ws;
static std::vector<void*> g_ws_retired;

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("ZG_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

void* workspace(cudaStream_t s, size_t bytes, unsigned** counters, int slot) {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(g_ws_mu);
  Workspace& w = g_ws[{{dev, slot}, s}];
  const size_t need = bytes + 256;
  if (w.bytes < need) {
    size_t cap = w.bytes ? w.bytes : (size_t)1 << 20;
    while (cap < need) cap *= 2;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(s, &st);
    if (st != cudaStreamCaptureStatusNone) {
      set_error(kBadArgument, "workspace of %zu bytes must be grown before stream capture (run the op once eagerly first)", need);
      return nullptr;
    }
    void* p = nullptr;
    if (!ZG_CUDA(cudaMalloc(&p, cap))) return nullptr;
    // counters (and slot 2, which its users keep at zero) start cleared; the clear is enqueued on the
    // stream that will use the buffer, so the kernel launched next is ordered after it
    if (!ZG_CUDA(cudaMemsetAsync(p, 0, cap, s))) return nullptr;
    // The outgrown buffer is retired, not freed: graphs captured earlier on this stream hold its
    // address in their kernel nodes and may be replayed after this call.  Capacities double, so all
    // retired buffers together are smaller than the live one; they go back with the process.
    if (w.base) g_ws_retired.push_back(w.base);
    w.base = p;
    w.bytes = cap;
  }
  if (counters) *counters = static_cast<unsigned*>(w.base);
  return static_cast<char*>(w.base) + 256;
}

struct GraphBackend {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
};

// Physical allocations mapped into a caller-reserved virtual range.
struct Memmap {
  int device;
  struct Entry { CUdeviceptr dptr; size_t size; CUmemGenericAllocationHandle handle; };
  std::vector<Entry> entries;
};

}  // namespace zg

using namespace zg;

// ======================================================================
// status
// ======================================================================
extern "C" int zg_last_error(void) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  return g_err_code;
}
extern "C" const char* zg_last_error_message(void) { return g_err_msg; }
extern "C" void zg_clear_error(void) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  g_err_code = 0;
  g_err_msg[0] = 0;
  (void)cudaGetLastError();
}
extern "C" int zg_device_available(void) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  (void)cudaGetLastError();
  return (e == cudaSuccess && n > 0) ? 1 : 0;
}
extern "C" int zg_sm_count(void) { return sm_count(); }
extern "C" void zg_set_device(unsigned device_number) { ZG_CUDA(cudaSetDevice((int)device_number)); }

// ======================================================================
// device
// ======================================================================
extern "C" unsigned device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return (unsigned)n;
}

extern "C" DevicePropertiesWrapper init_device(unsigned device_number) {
  DevicePropertiesWrapper w{nullptr};
  int n = 0;
  if (!ZG_CUDA(cudaGetDeviceCount(&n))) return w;
  if ((int)device_number >= n) {
    set_error(kBadArgument, "init_device: device %u requested but only %d present", device_number, n);
    return w;
  }
  // primary context (shared with any other runtime user in the process)
  if (!ZG_CUDA(cudaSetDevice((int)device_number))) return w;
  if (!ZG_CUDA(cudaFree(0))) return w;
  cudaDeviceProp* prop = new cudaDeviceProp();
  if (!ZG_CUDA(cudaGetDeviceProperties(prop, (int)device_number))) {
    delete prop;
    return w;
  }
  check_tc_errors();  // also allocates the per-device flag, outside any capture
  w.ptr = prop;
  return w;
}

extern "C" void check_last_error(void) {
  ZG_CUDA(cudaDeviceSynchronize());
  ZG_CUDA(cudaGetLastError());
}

extern "C" void device_synchronize(void) {
  if (ZG_CUDA(cudaDeviceSynchronize())) check_tc_errors();
}

extern "C" len_t device_total_memory(unsigned device_number) {
  cudaDeviceProp prop;
  if (!ZG_CUDA(cudaGetDeviceProperties(&prop, (int)device_number))) return 0;
  return (len_t)prop.totalGlobalMem;
}

// ======================================================================
// streams and op contexts
// ======================================================================
extern "C" StreamWrapper init_stream(void) {
  cudaStream_t s = nullptr;
  ZG_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  return StreamWrapper{s};
}
extern "C" void deinit_stream(StreamWrapper stream) {
  if (stream.ptr) ZG_CUDA(cudaStreamDestroy(as_stream(stream)));
}
extern "C" void* zg_host_alloc_pinned(len_t nbytes) {
  void* p = nullptr;
  if (!ZG_CUDA(cudaHostAlloc(&p, nbytes ? nbytes : 1, cudaHostAllocDefault))) return nullptr;
  return p;
}

extern "C" void zg_host_free_pinned(void* hptr) {
  if (hptr) ZG_CUDA(cudaFreeHost(hptr));
}

extern "C" void zg_stream_wait(StreamWrapper waiter, StreamWrapper signaller) {
  // events come from a ring that lives as long as the process: a wait only
  // needs its event until the wait has been enqueued (or captured)
  static std::mutex mu;
  static cudaEvent_t ring[64][32];
  static bool made[64] = {false};
  static unsigned next[64] = {0};
  int dev = 0;
  if (!ZG_CUDA(cudaGetDevice(&dev))) return;
  if (dev < 0 || dev >= 64) { set_error(kBadArgument, "zg_stream_wait: device ordinal %d out of range", dev); return; }
  cudaEvent_t ev;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!made[dev]) {
      for (int i = 0; i < 32; ++i)
        if (!ZG_CUDA(cudaEventCreateWithFlags(&ring[dev][i], cudaEventDisableTiming))) return;
      made[dev] = true;
    }
    ev = ring[dev][next[dev]++ % 32];
  }
  if (!ZG_CUDA(cudaEventRecord(ev, as_stream(signaller)))) return;
  ZG_CUDA(cudaStreamWaitEvent(as_stream(waiter), ev, 0));
}

// Explicit events: a point of one stream that another stream (or the same one later) waits for.
extern "C" void* zg_event_create(void) {
  cudaEvent_t ev = nullptr;
  if (!ZG_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming))) return nullptr;
  return ev;
}
extern "C" void zg_event_destroy(void* event) {
  if (event) ZG_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
}
extern "C" void zg_event_record(void* event, StreamWrapper stream) {
  if (!event) { set_error(kBadArgument, "zg_event_record: NULL event"); return; }
  ZG_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), as_stream(stream)));
}
extern "C" void zg_stream_wait_event(StreamWrapper stream, void* event) {
  if (!event) { set_error(kBadArgument, "zg_stream_wait_event: NULL event"); return; }
  ZG_CUDA(cudaStreamWaitEvent(as_stream(stream), static_cast<cudaEvent_t>(event), 0));
}

extern "C" void stream_synchronize(StreamWrapper stream) {
  if (ZG_CUDA(cudaStreamSynchronize(as_stream(stream)))) check_tc_errors();
}

namespace zg {
void free_plans(void* plans);
}

static OpContext* new_ctx(StreamWrapper s) { return new OpContext{as_stream(s), nullptr}; }
static void del_ctx(void* p) {
  OpContext* c = static_cast<OpContext*>(p);
  if (!c) return;
  free_plans(c->plans);
  delete c;
}
extern "C" CublasWrapper init_cublas_handle(StreamWrapper stream) { return CublasWrapper{new_ctx(stream)}; }
extern "C" void deinit_cublas_handle(CublasWrapper h) { del_ctx(h.ptr); }
extern "C" CudnnWrapper init_cudnn_handle(StreamWrapper stream) { return CudnnWrapper{new_ctx(stream)}; }
extern "C" void deinit_cudnn_handle(CudnnWrapper h) { del_ctx(h.ptr); }
extern "C" CutensorWrapper init_cutensor_handle(StreamWrapper stream) { return CutensorWrapper{new_ctx(stream)}; }
extern "C" void deinit_cutensor_handle(CutensorWrapper h) { del_ctx(h.ptr); }

// ======================================================================
// memory
// ======================================================================
extern "C" void* mem_alloc(len_t nbytes, StreamWrapper stream) {
  void* p = nullptr;
  if (nbytes == 0) return nullptr;
  cudaError_t e = cudaMallocAsync(&p, nbytes, as_stream(stream));
  if (e != cudaSuccess) {
    (void)cudaGetLastError();  // OOM is reported through the NULL return, as the Zig side expects
    if (e != cudaErrorMemoryAllocation) ZG_CUDA(e);
    return nullptr;
  }
  return p;
}
extern "C" void mem_free(void* dptr, StreamWrapper stream) {
  if (dptr) ZG_CUDA(cudaFreeAsync(dptr, as_stream(stream)));
}
extern "C" void memcpy_HtoD(void* dptr, void const* hptr, len_t nbytes, StreamWrapper stream) {
  if (nbytes) ZG_CUDA(cudaMemcpyAsync(dptr, hptr, nbytes, cudaMemcpyHostToDevice, as_stream(stream)));
}
extern "C" void memcpy_DtoH(void* hptr, void const* dptr, len_t nbytes, StreamWrapper stream) {
  if (nbytes) ZG_CUDA(cudaMemcpyAsync(hptr, dptr, nbytes, cudaMemcpyDeviceToHost, as_stream(stream)));
}
// 128-bit copy, four loads in flight per thread (large same-device copies: a
// kernel reaches the HBM copy rate, the driver's device-to-device copy does not)
__global__ void __launch_bounds__(256) copy16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nv) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; v + 3 * nth < nv; v += 4 * nth) {
    const uint4 a = src[v], b = src[v + nth], c = src[v + 2 * nth], d = src[v + 3 * nth];
    dst[v] = a; dst[v + nth] = b; dst[v + 2 * nth] = c; dst[v + 3 * nth] = d;
  }
  for (; v < nv; v += nth) dst[v] = src[v];
}

static bool on_current_device(const void* p) {
  cudaPointerAttributes at;
  int dev = -1;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { (void)cudaGetLastError(); return false; }
  cudaGetDevice(&dev);
  return at.type == cudaMemoryTypeDevice && at.device == dev;
}

extern "C" void memcpy_DtoD(void* dst, void const* src, len_t nbytes, StreamWrapper stream) {
  if (!nbytes) return;
  cudaStream_t s = as_stream(stream);
  if (nbytes >= ((len_t)1 << 20) && nbytes % 16 == 0 && host_aligned16(dst) && host_aligned16(src) && on_current_device(dst) &&
      on_current_device(src)) {
    const size_t nv = nbytes / 16;
    copy16_kernel<<<grid_for(nv, 256 * 4), 256, 0, s>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), nv);
    ZG_LAUNCH_CHECK();
    return;
  }
  ZG_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, s));
}

extern "C" void mem_fill(dtype id, void* data, len_t n, const void* value, StreamWrapper stream) {
  if (n == 0) return;
  cudaStream_t s = as_stream(stream);
  if (id == SINGLE) {
    float v;
    memcpy(&v, value, 4);
    // zero fill of a large buffer: the memset path; small ones stay kernels so
    // that a captured step is an unbroken chain of kernel nodes
    if (v == 0.f && !std::signbit(v) && n > ((size_t)1 << 22)) {
      ZG_CUDA(cudaMemsetAsync(data, 0, n * 4, s));
      return;
    }
    launch_pdl(fill_kernel<float>, dim3(grid_for(n, 256 * 4)), dim3(256), 0, s, static_cast<float*>(data), (size_t)n, v);
  } else if (id == DOUBLE) {
    double v;
    memcpy(&v, value, 8);
    launch_pdl(fill_kernel<double>, dim3(grid_for(n, 256 * 8)), dim3(256), 0, s, static_cast<double*>(data), (size_t)n, v);
  } else {
    set_error(kUnsupported, "mem_fill: unsupported dtype %d", (int)id);
    return;
  }
  ZG_LAUNCH_CHECK();
}

extern "C" void mem_sequence(dtype id, void* data, len_t n, const void* init, const void* step, StreamWrapper stream) {
  if (n == 0) return;
  cudaStream_t s = as_stream(stream);
  if (id == SINGLE) {
    float a, b;
    memcpy(&a, init, 4);
    memcpy(&b, step, 4);
    sequence_kernel<float><<<grid_for(n, 256 * 8), 256, 0, s>>>(static_cast<float*>(data), n, a, b);
  } else if (id == DOUBLE) {
    double a, b;
    memcpy(&a, init, 8);
    memcpy(&b, step, 8);
    sequence_kernel<double><<<grid_for(n, 256 * 8), 256, 0, s>>>(static_cast<double*>(data), n, a, b);
  } else {
    set_error(kUnsupported, "mem_sequence: unsupported dtype %d", (int)id);
    return;
  }
  ZG_LAUNCH_CHECK();
}

extern "C" void mem_random(dtype id, void* x, len_t n, randtype op, unsigned seed, StreamWrapper stream) {
  if (n == 0) return;
  cudaStream_t s = as_stream(stream);
  const unsigned g = grid_for((n + 3) / 4, 256 * 4);
  if (id == SINGLE) random_kernel<float><<<g, 256, 0, s>>>(static_cast<float*>(x), n, op == NORMAL, seed);
  else if (id == DOUBLE) random_kernel<double><<<g, 256, 0, s>>>(static_cast<double*>(x), n, op == NORMAL, seed);
  else { set_error(kUnsupported, "mem_random: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}

extern "C" void mem_take(dtype id, const void* src, len_t /*src_len*/, const len_t* idxs, len_t idxs_len, void* dst,
                         StreamWrapper stream) {
  if (idxs_len == 0) return;
  cudaStream_t s = as_stream(stream);
  const unsigned g = grid_for(idxs_len, 256 * 4);
  if (id == SINGLE)
    take_kernel<float, len_t><<<g, 256, 0, s>>>(static_cast<const float*>(src), idxs, idxs_len, static_cast<float*>(dst));
  else if (id == DOUBLE)
    take_kernel<double, len_t><<<g, 256, 0, s>>>(static_cast<const double*>(src), idxs, idxs_len, static_cast<double*>(dst));
  else { set_error(kUnsupported, "mem_take: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}

// ======================================================================
// stream capture
// ======================================================================
extern "C" GraphWrapper open_capture(StreamWrapper stream) {
  // thread-local mode: other threads of the process (e.g. a communication
  // library's watchdog) may keep making unrelated CUDA calls while we capture
  if (!ZG_CUDA(cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeThreadLocal))) return GraphWrapper{nullptr};
  return GraphWrapper{new GraphBackend()};
}
extern "C" void save_capture(GraphWrapper graph, StreamWrapper stream) {
  GraphBackend* b = static_cast<GraphBackend*>(graph.ptr);
  if (!b) return;
  if (!ZG_CUDA(cudaStreamEndCapture(as_stream(stream), &b->graph))) return;
  ZG_CUDA(cudaGraphInstantiate(&b->exec, b->graph, 0));
}
extern "C" void free_capture(GraphWrapper graph, StreamWrapper /*stream*/) {
  GraphBackend* b = static_cast<GraphBackend*>(graph.ptr);
  if (!b) return;
  if (b->exec) ZG_CUDA(cudaGraphExecDestroy(b->exec));
  if (b->graph) ZG_CUDA(cudaGraphDestroy(b->graph));
  delete b;
}
extern "C" void run_capture(GraphWrapper graph, StreamWrapper stream) {
  GraphBackend* b = static_cast<GraphBackend*>(graph.ptr);
  if (!b || !b->exec) {
    set_error(kBadArgument, "run_capture: graph was not saved");
    return;
  }
  ZG_CUDA(cudaGraphLaunch(b->exec, as_stream(stream)));
}

extern "C" len_t zg_capture_kernel_count(GraphWrapper graph) {
  GraphBackend* b = static_cast<GraphBackend*>(graph.ptr);
  if (!b || !b->graph) return 0;
  size_t n = 0;
  if (!ZG_CUDA(cudaGraphGetNodes(b->graph, nullptr, &n)) || n == 0) return 0;
  std::vector<cudaGraphNode_t> nodes(n);
  if (!ZG_CUDA(cudaGraphGetNodes(b->graph, nodes.data(), &n))) return 0;
  len_t kernels = 0;
  for (size_t i = 0; i < n; ++i) {
    cudaGraphNodeType t;
    if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++kernels;
  }
  return kernels;
}

// ======================================================================
// virtual-memory arena (DataHandler of the Zig CachingAllocator)
// ======================================================================
static bool vmm_prop(unsigned device_id, CUmemAllocationProp* prop) {
  memset(prop, 0, sizeof(*prop));
  prop->type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop->location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop->location.id = (int)device_id;
  return true;
}

extern "C" len_t mem_page_size(unsigned device_id) {
  auto fn = ZG_DRV(cuMemGetAllocationGranularity);
  if (!fn) return 0;
  CUmemAllocationProp prop;
  vmm_prop(device_id, &prop);
  size_t g = 0;
  if (!ZG_CU(fn(&g, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM))) return 0;
  return (len_t)g;
}

extern "C" void* mem_map(unsigned device_id, size_t virtual_buffer_size) {
  // Address reservation is per process, not per context; binding the primary
  // context of the device on this thread is enough (no helper thread needed).
  int prev = 0;
  cudaGetDevice(&prev);
  if (!ZG_CUDA(cudaSetDevice((int)device_id)) || !ZG_CUDA(cudaFree(0))) return nullptr;
  auto fn = ZG_DRV(cuMemAddressReserve);
  CUdeviceptr base = 0;
  const len_t page = mem_page_size(device_id);
  bool ok = fn && page && ZG_CU(fn(&base, virtual_buffer_size, page, 0, 0));
  cudaSetDevice(prev);
  return ok ? reinterpret_cast<void*>(base) : nullptr;
}

extern "C" void mem_unmap(unsigned /*device_id*/, void* base_address, size_t virtual_buffer_size) {
  auto fn = ZG_DRV(cuMemAddressFree);
  if (fn && base_address) ZG_CU(fn(reinterpret_cast<CUdeviceptr>(base_address), virtual_buffer_size));
}

extern "C" MemmapWrapper init_memmap(unsigned device_id) {
  Memmap* m = new Memmap();
  m->device = (int)device_id;
  return MemmapWrapper{m};
}

extern "C" void mem_map_alloc(MemmapWrapper map, void* address, len_t size) {
  Memmap* m = static_cast<Memmap*>(map.ptr);
  auto create = ZG_DRV(cuMemCreate);
  auto mapfn = ZG_DRV(cuMemMap);
  auto access = ZG_DRV(cuMemSetAccess);
  auto release = ZG_DRV(cuMemRelease);
  if (!m || !create || !mapfn || !access || !release) return;
  CUmemAllocationProp prop;
  vmm_prop((unsigned)m->device, &prop);
  CUmemGenericAllocationHandle h;
  if (!ZG_CU(create(&h, size, &prop, 0))) return;
  const CUdeviceptr dptr = reinterpret_cast<CUdeviceptr>(address);
  if (!ZG_CU(mapfn(dptr, size, 0, h, 0))) {
    release(h);
    return;
  }
  CUmemAccessDesc desc;
  memset(&desc, 0, sizeof(desc));
  desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  desc.location.id = m->device;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (!ZG_CU(access(dptr, size, &desc, 1))) return;
  m->entries.push_back({dptr, (size_t)size, h});
}

extern "C" void reset_memmap(MemmapWrapper map) {
  Memmap* m = static_cast<Memmap*>(map.ptr);
  if (!m) return;
  auto unmap = ZG_DRV(cuMemUnmap);
  auto release = ZG_DRV(cuMemRelease);
  if (!unmap || !release) return;
  for (auto& e : m->entries) {
    ZG_CU(unmap(e.dptr, e.size));
    ZG_CU(release(e.handle));
  }
  m->entries.clear();
}

extern "C" void deinit_memmap(MemmapWrapper map) {
  reset_memmap(map);
  delete static_cast<Memmap*>(map.ptr);
}
