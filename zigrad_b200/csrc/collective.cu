// One-shot sum all-reduce of a small fp32 buffer over peer memory
// (NVLink / NVSwitch stores between the GPUs of one box), for the
// data-parallel step's flat gradient buffer when it is latency-bound (a few
// hundred KB): one kernel per rank per step, no library collective.
//
// Low-latency protocol: a value travels together with its validity flag in
// one 8-byte word {fp32 bits, epoch}, two such words per 16-byte store.  Every
// rank PUSHES its gradients into a receive slot of every peer (posted remote
// stores: one-way latency, no fence, no separate flag write) and then sums, in
// rank order, what the peers pushed into its own slots, polling each word
// until it carries the epoch of this launch.  An 8-byte word is written
// atomically, so a word with the right epoch holds the right value.
//
// Every rank owns a "comm region" in plain device memory that the other ranks
// map through CUDA IPC:
//   [0, 512)   control: [0] epoch of the last finished launch, [1] finish tickets,
//              [2] error (a wait ran out)
//   [512, ..)  receive slots [2 epoch parities][world][cap/2] of 16 bytes
// Slots alternate with the epoch's parity: a peer can be at most one epoch ahead
// (it needs this rank's words of the current epoch to finish), so it never
// overwrites words that are still being read.  The epoch lives in device memory
// and advances by one per launch, which keeps the kernel replayable from a
// captured graph.  The sum is formed in rank order on every rank: bit-identical
// replicas.  Polls are bounded; a rank that gives up sets the error word and
// leaves its buffer partly reduced.
#include <cstring>

#include "common.cuh"

namespace zg {

constexpr int kArThreads = 256;
constexpr int kArMaxWorld = 8;
constexpr unsigned kArSpinLimit = 1u << 24;  // polls (with back-off) before a wait gives up: seconds
constexpr size_t kArHeader = 512;

struct ArArgs {
  float* params;  // optional fused SGD: params += nlr * (reduced gradient)
  float nlr;
  float* grads;
  size_t n, cap_pairs;
  unsigned rank, world;
  char* comm[kArMaxWorld];
};

__device__ __forceinline__ void st_word_pair(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_word_pair(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const ArArgs a) {
  pdl_sync();
  unsigned* ctl = reinterpret_cast<unsigned*>(a.comm[a.rank]);
  const unsigned e = *reinterpret_cast<volatile unsigned*>(ctl) + 1u;
  const size_t nth = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t npairs = (a.n + 1) / 2;
  // slot of source rank `src` inside the region of rank `dst`, for this epoch's parity
  auto slot = [&](unsigned dst, unsigned src) -> uint4* {
    return reinterpret_cast<uint4*>(a.comm[dst] + kArHeader) + ((size_t)(e & 1u) * a.world + src) * a.cap_pairs;
  };
  // ---- 1. push my values to every peer
  for (size_t i = tid; i < npairs; i += nth) {
    uint4 w;
    w.x = __float_as_uint(a.grads[2 * i]);
    w.z = (2 * i + 1 < a.n) ? __float_as_uint(a.grads[2 * i + 1]) : 0u;
    w.y = w.w = e;
#pragma unroll
    for (unsigned p = 0; p < kArMaxWorld; ++p)
      if (p < a.world && p != a.rank) st_word_pair(slot(p, a.rank) + i, w);
  }
  // ---- 2. sum, in rank order, my own values and what the peers pushed to me
  bool gave_up = false;
  for (size_t i = tid; i < npairs && !gave_up; i += nth) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (unsigned p = 0; p < kArMaxWorld; ++p) {
      if (p >= a.world) continue;
      if (p == a.rank) {
        s0 += a.grads[2 * i];
        if (2 * i + 1 < a.n) s1 += a.grads[2 * i + 1];
        continue;
      }
      const uint4* src = slot(a.rank, p) + i;
      uint4 w = ld_word_pair(src);
      for (unsigned it = 0; (w.y != e || w.w != e) && it < kArSpinLimit; ++it) {
        if (it > 64) __nanosleep(it > 4096 ? 200 : 20);
        w = ld_word_pair(src);
      }
      if (w.y != e || w.w != e) { gave_up = true; break; }
      s0 += __uint_as_float(w.x);
      s1 += __uint_as_float(w.z);
    }
    if (gave_up) break;
    a.grads[2 * i] = s0;
    if (2 * i + 1 < a.n) a.grads[2 * i + 1] = s1;
    if (a.params) {  // the SGD update of src/nn/optim.zig:100-122 (no clipping) on the reduced gradient
      a.params[2 * i] = fmaf(a.nlr, s0, a.params[2 * i]);
      if (2 * i + 1 < a.n) a.params[2 * i + 1] = fmaf(a.nlr, s1, a.params[2 * i + 1]);
    }
  }
  if (gave_up) ctl[2] = 1;
  // ---- the last CTA to finish advances the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(&ctl[1], 1u);
    if (t == gridDim.x - 1) {
      ctl[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned*>(ctl) = e;
    }
  }
}

}  // namespace zg

using namespace zg;

static size_t comm_bytes(len_t cap_elems, unsigned world) { return kArHeader + 2 * (size_t)world * ((size_t)cap_elems / 2) * 16; }

extern "C" void* zg_comm_alloc(len_t cap_elems, unsigned world) {
  if (world < 1 || world > (unsigned)kArMaxWorld || cap_elems % 2 != 0) { set_error(kBadArgument, "zg_comm_alloc: world %u, capacity %lu", world, cap_elems); return nullptr; }
  void* p = nullptr;
  const size_t bytes = comm_bytes(cap_elems, world);
  if (!ZG_CUDA(cudaMalloc(&p, bytes))) return nullptr;
  if (!ZG_CUDA(cudaMemset(p, 0, bytes))) return nullptr;
  if (!ZG_CUDA(cudaDeviceSynchronize())) return nullptr;
  return p;
}

extern "C" void zg_comm_free(void* region) {
  if (region) ZG_CUDA(cudaFree(region));
}

extern "C" void zg_ipc_export(void* dptr, unsigned char* handle_out64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  if (!ZG_CUDA(cudaIpcGetMemHandle(&h, dptr))) return;
  memcpy(handle_out64, &h, 64);
}

extern "C" void* zg_ipc_open(const unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (!ZG_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess))) return nullptr;
  return p;
}

extern "C" void zg_ipc_close(void* dptr) {
  if (dptr) ZG_CUDA(cudaIpcCloseMemHandle(dptr));
}

extern "C" int zg_comm_error(void* region, StreamWrapper stream) {
  unsigned v = 0;
  if (!ZG_CUDA(cudaMemcpyAsync(&v, static_cast<char*>(region) + 8, 4, cudaMemcpyDeviceToHost, as_stream(stream)))) return -1;
  if (!ZG_CUDA(cudaStreamSynchronize(as_stream(stream)))) return -1;
  return (int)v;
}

static void allreduce_launch(StreamWrapper stream, void* grads, len_t n, unsigned rank, unsigned world, void* const* comm, len_t cap_elems,
                             void* params, double lr);

extern "C" void zg_allreduce_oneshot(StreamWrapper stream, void* grads, len_t n, unsigned rank, unsigned world, void* const* comm,
                                     len_t cap_elems) {
  allreduce_launch(stream, grads, n, rank, world, comm, cap_elems, nullptr, 0.0);
}

extern "C" void zg_allreduce_sgd_oneshot(StreamWrapper stream, void* grads, void* params, len_t n, double lr, unsigned rank, unsigned world,
                                         void* const* comm, len_t cap_elems) {
  if (!params) { set_error(kBadArgument, "zg_allreduce_sgd_oneshot: params is NULL"); return; }
  allreduce_launch(stream, grads, n, rank, world, comm, cap_elems, params, lr);
}

static void allreduce_launch(StreamWrapper stream, void* grads, len_t n, unsigned rank, unsigned world, void* const* comm, len_t cap_elems,
                             void* params, double lr) {
  if (n == 0) return;
  if (world < 1 || world > (unsigned)kArMaxWorld || rank >= world) { set_error(kBadArgument, "zg_allreduce_oneshot: rank %u / world %u", rank, world); return; }
  if (n > cap_elems) { set_error(kBadArgument, "zg_allreduce_oneshot: %lu elements exceed the comm region's %lu", n, cap_elems); return; }
  if (cap_elems % 2 != 0) { set_error(kBadArgument, "zg_allreduce_oneshot: capacity must be even"); return; }
  ArArgs a;
  memset(&a, 0, sizeof(a));
  a.grads = static_cast<float*>(grads);
  a.params = static_cast<float*>(params);
  a.nlr = -(float)lr;
  a.n = n; a.cap_pairs = cap_elems / 2; a.rank = rank; a.world = world;
  for (unsigned p = 0; p < world; ++p) {
    if (!comm[p]) { set_error(kBadArgument, "zg_allreduce_oneshot: comm region of rank %u is NULL", p); return; }
    a.comm[p] = static_cast<char*>(comm[p]);
  }
  // one pair of values per thread and trip; the CTAs of a rank do not wait for one another
  unsigned g = (unsigned)(((n + 1) / 2 + kArThreads - 1) / kArThreads);
  if (g < 1) g = 1;
  const unsigned cap = (unsigned)sm_count() * 2;
  if (g > cap) g = cap;
  launch_pdl(allreduce_oneshot_kernel, dim3(g), dim3(kArThreads), 0, as_stream(stream), a);
}
