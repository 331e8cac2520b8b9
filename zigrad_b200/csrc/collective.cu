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
// replicas.  Polls are bounded (zg_comm_set_spin_limit / ZG_SPIN_LIMIT); a rank
// that gives up sets the error word and the library's time-out flag and leaves
// its buffer partly reduced.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace zg {

constexpr int kArThreads = 256;
constexpr int kArMaxWorld = 8;
constexpr unsigned kArSpinLimit = 1u << 24;  // default polls (with back-off) before a wait gives up: seconds
constexpr size_t kArHeader = 512;

struct ArArgs {
  float* params;  // optional fused SGD: params += nlr * (reduced gradient)
  float nlr;
  float* grads;
  int zero_grads;  // with params: leave zeros instead of the sum in grads
  size_t n, cap_pairs;
  unsigned rank, world;
  unsigned spin_limit;  // polls before a wait on a peer's word gives up
  int* timeout_flag;    // the per-device flag that stream_synchronize turns into kKernelTimeout
  char* comm[kArMaxWorld];
};

// A wait ran out: the comm region's error word (zg_comm_error reads and clears it) and the
// library-wide time-out flag are raised; the kernel goes on to its epilogue and returns.
__device__ __forceinline__ void ar_report_gave_up(unsigned* ctl, const ArArgs& a) {
  ctl[2] = 1;
  if (a.timeout_flag) *a.timeout_flag = 1;
}

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
  // ---- 2. sum, in rank order, my own values and what the peers pushed to me.  The words of all
  // peers are requested before the first is looked at (one memory round trip when they have
  // all arrived, instead of one per peer); only a word that is not there yet is polled.
  bool gave_up = false;
  for (size_t i = tid; i < npairs && !gave_up; i += nth) {
    uint4 w[kArMaxWorld];
#pragma unroll
    for (unsigned p = 0; p < kArMaxWorld; ++p)
      if (p < a.world && p != a.rank) w[p] = ld_word_pair(slot(a.rank, p) + i);
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
      for (unsigned it = 0; (w[p].y != e || w[p].w != e) && it < a.spin_limit; ++it) {
        if (it > 64) __nanosleep(it > 4096 ? 200 : 20);
        w[p] = ld_word_pair(src);
      }
      if (w[p].y != e || w[p].w != e) { gave_up = true; break; }
      s0 += __uint_as_float(w[p].x);
      s1 += __uint_as_float(w[p].z);
    }
    if (gave_up) break;
    a.grads[2 * i] = a.zero_grads ? 0.f : s0;
    if (2 * i + 1 < a.n) a.grads[2 * i + 1] = a.zero_grads ? 0.f : s1;
    if (a.params) {  // the SGD update of src/nn/optim.zig:100-122 (no clipping) on the reduced gradient
      a.params[2 * i] = fmaf(a.nlr, s0, a.params[2 * i]);
      if (2 * i + 1 < a.n) a.params[2 * i + 1] = fmaf(a.nlr, s1, a.params[2 * i + 1]);
    }
  }
  if (gave_up) ar_report_gave_up(ctl, a);
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

// Two-shot variant for larger worlds (same protocol words, a quarter of the
// bytes at 8 ranks): the buffer is cut into `world` slices; (1) every rank pushes,
// for each peer, its values of THAT PEER's slice; (2) the owner of a slice sums
// the `world` contributions in rank order and pushes the result to every peer;
// (3) every rank collects the other slices.  The reduced value of an element is
// computed once, by its owner, so the replicas are bit-identical by
// construction.  Slots in the comm region: [2 parities]{ scatter [world][S],
// gather [world][S] } of 16-byte word pairs, S = pairs per slice.
// Step (2) of a slice element depends on step (1) of the peers, and step (3)
// on step (2) of the peers: no cycle as long as the CTAs that own step (2)
// (the lowest-numbered ones) are resident, which the small grid guarantees.
__global__ void __launch_bounds__(kArThreads) allreduce_twoshot_kernel(const ArArgs a, const size_t S) {
  pdl_sync();
  unsigned* ctl = reinterpret_cast<unsigned*>(a.comm[a.rank]);
  const unsigned e = *reinterpret_cast<volatile unsigned*>(ctl) + 1u;
  const size_t nth = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t npairs = (a.n + 1) / 2;
  const unsigned W = a.world;
  auto scatter_slot = [&](unsigned dst, unsigned src) -> uint4* {
    return reinterpret_cast<uint4*>(a.comm[dst] + kArHeader) + ((size_t)(e & 1u) * 2 * W + src) * S;
  };
  auto gather_slot = [&](unsigned dst, unsigned src) -> uint4* {
    return reinterpret_cast<uint4*>(a.comm[dst] + kArHeader) + ((size_t)(e & 1u) * 2 * W + W + src) * S;
  };
  auto poll = [&](const uint4* src, uint4& w) -> bool {
    w = ld_word_pair(src);
    for (unsigned it = 0; (w.y != e || w.w != e) && it < a.spin_limit; ++it) {
      if (it > 64) __nanosleep(it > 4096 ? 200 : 20);
      w = ld_word_pair(src);
    }
    return w.y == e && w.w == e;
  };
  auto local_pair = [&](size_t i, float& v0, float& v1) {
    v0 = a.grads[2 * i];
    v1 = (2 * i + 1 < a.n) ? a.grads[2 * i + 1] : 0.f;
  };
  auto store_result = [&](size_t i, float s0, float s1) {
    a.grads[2 * i] = a.zero_grads ? 0.f : s0;
    if (2 * i + 1 < a.n) a.grads[2 * i + 1] = a.zero_grads ? 0.f : s1;
    if (a.params) {
      a.params[2 * i] = fmaf(a.nlr, s0, a.params[2 * i]);
      if (2 * i + 1 < a.n) a.params[2 * i + 1] = fmaf(a.nlr, s1, a.params[2 * i + 1]);
    }
  };
  bool gave_up = false;
  // ---- (2) first in program order for the threads that own slice elements, but it needs the
  // peers' step (1): so every thread does its share of step (1) before anything that waits
  for (size_t i = tid; i < npairs; i += nth) {
    const unsigned owner = (unsigned)(i / S);
    if (owner == a.rank) continue;
    float v0, v1;
    local_pair(i, v0, v1);
    uint4 w;
    w.x = __float_as_uint(v0); w.z = __float_as_uint(v1); w.y = w.w = e;
    st_word_pair(scatter_slot(owner, a.rank) + (i - (size_t)owner * S), w);
  }
  // ---- (2) reduce my slice in rank order, push the result to every peer
  const size_t my0 = (size_t)a.rank * S;
  const size_t my_n = my0 < npairs ? ((npairs - my0) < S ? (npairs - my0) : S) : 0;
  for (size_t j = tid; j < my_n && !gave_up; j += nth) {
    // the contributions of all peers are requested before the first is looked at
    uint4 c[kArMaxWorld];
#pragma unroll
    for (unsigned p = 0; p < kArMaxWorld; ++p)
      if (p < W && p != a.rank) c[p] = ld_word_pair(scatter_slot(a.rank, p) + j);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (unsigned p = 0; p < kArMaxWorld; ++p) {
      if (p >= W) continue;
      if (p == a.rank) {
        float v0, v1;
        local_pair(my0 + j, v0, v1);
        s0 += v0; s1 += v1;
      } else {
        if ((c[p].y != e || c[p].w != e) && !poll(scatter_slot(a.rank, p) + j, c[p])) { gave_up = true; break; }
        s0 += __uint_as_float(c[p].x); s1 += __uint_as_float(c[p].z);
      }
    }
    if (gave_up) break;
    uint4 w;
    w.x = __float_as_uint(s0); w.z = __float_as_uint(s1); w.y = w.w = e;
    for (unsigned p = 0; p < W; ++p)
      if (p != a.rank) st_word_pair(gather_slot(p, a.rank) + j, w);
    store_result(my0 + j, s0, s1);
  }
  // ---- (3) collect the slices the peers reduced
  for (size_t i = tid; i < npairs && !gave_up; i += nth) {
    const unsigned owner = (unsigned)(i / S);
    if (owner == a.rank) continue;
    uint4 w;
    if (!poll(gather_slot(a.rank, owner) + (i - (size_t)owner * S), w)) { gave_up = true; break; }
    store_result(i, __uint_as_float(w.x), __uint_as_float(w.z));
  }
  if (gave_up) ar_report_gave_up(ctl, a);
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
  // read-and-clear: one failed launch is reported once, later launches start clean
  if (v && !ZG_CUDA(cudaMemsetAsync(static_cast<char*>(region) + 8, 0, 4, as_stream(stream)))) return -1;
  if (v && !ZG_CUDA(cudaStreamSynchronize(as_stream(stream)))) return -1;
  return (int)v;
}

static unsigned g_spin_limit = 0;  // 0 = not set yet
extern "C" void zg_comm_set_spin_limit(unsigned polls) { g_spin_limit = polls ? polls : kArSpinLimit; }
static unsigned spin_limit() {
  if (g_spin_limit == 0) {
    const char* v = getenv("ZG_SPIN_LIMIT");
    const long n = v ? atol(v) : 0;
    g_spin_limit = n > 0 ? (unsigned)n : kArSpinLimit;
  }
  return g_spin_limit;
}

static void allreduce_launch(StreamWrapper stream, void* grads, len_t n, unsigned rank, unsigned world, void* const* comm, len_t cap_elems,
                             void* params, double lr, int zero_grads);

extern "C" void zg_allreduce_oneshot(StreamWrapper stream, void* grads, len_t n, unsigned rank, unsigned world, void* const* comm,
                                     len_t cap_elems) {
  allreduce_launch(stream, grads, n, rank, world, comm, cap_elems, nullptr, 0.0, 0);
}

extern "C" void zg_allreduce_sgd_oneshot(StreamWrapper stream, void* grads, void* params, len_t n, double lr, unsigned rank, unsigned world,
                                         void* const* comm, len_t cap_elems, int zero_grads) {
  if (!params) { set_error(kBadArgument, "zg_allreduce_sgd_oneshot: params is NULL"); return; }
  allreduce_launch(stream, grads, n, rank, world, comm, cap_elems, params, lr, zero_grads);
}

static void allreduce_launch(StreamWrapper stream, void* grads, len_t n, unsigned rank, unsigned world, void* const* comm, len_t cap_elems,
                             void* params, double lr, int zero_grads) {
  if (n == 0) return;
  if (world < 1 || world > (unsigned)kArMaxWorld || rank >= world) { set_error(kBadArgument, "zg_allreduce_oneshot: rank %u / world %u", rank, world); return; }
  if (n > cap_elems) { set_error(kBadArgument, "zg_allreduce_oneshot: %lu elements exceed the comm region's %lu", n, cap_elems); return; }
  if (cap_elems % 2 != 0) { set_error(kBadArgument, "zg_allreduce_oneshot: capacity must be even"); return; }
  ArArgs a;
  memset(&a, 0, sizeof(a));
  a.grads = static_cast<float*>(grads);
  a.params = static_cast<float*>(params);
  a.nlr = -(float)lr;
  a.zero_grads = (params && zero_grads) ? 1 : 0;
  a.n = n; a.cap_pairs = cap_elems / 2; a.rank = rank; a.world = world;
  a.spin_limit = spin_limit();
  a.timeout_flag = kernel_timeout_flag();
  for (unsigned p = 0; p < world; ++p) {
    if (!comm[p]) { set_error(kBadArgument, "zg_allreduce_oneshot: comm region of rank %u is NULL", p); return; }
    a.comm[p] = static_cast<char*>(comm[p]);
  }
  // one pair of values per thread and trip; the CTAs of a rank do not wait for one another
  unsigned g = (unsigned)(((n + 1) / 2 + kArThreads - 1) / kArThreads);
  if (g < 1) g = 1;
  const unsigned cap = (unsigned)sm_count() * 2;
  if (g > cap) g = cap;
  const size_t npairs = ((size_t)n + 1) / 2;
  const size_t S = (npairs + world - 1) / world;
  // two-shot from 4 ranks up when the buffer is not tiny (its slots fit: 2 S <= capacity in pairs; measured on the
  // 437 KB MLP buffer at 4 ranks: 61.1 us per step against 62.9 with the one-shot kernel);
  // ZG_ALLREDUCE=1 / 2 in the environment forces the one-shot / two-shot kernel
  static const int force = [] { const char* v = getenv("ZG_ALLREDUCE"); return !v ? 0 : (v[0] == '1' ? 1 : (v[0] == '2' ? 2 : 0)); }();
  const bool two_shot = force == 2 ? world >= 2 : (force == 1 ? false : world >= 4);
  if (two_shot && n >= 16384 && 2 * S <= a.cap_pairs) {
    launch_pdl(allreduce_twoshot_kernel, dim3(g), dim3(kArThreads), 0, as_stream(stream), a, S);
    return;
  }
  launch_pdl(allreduce_oneshot_kernel, dim3(g), dim3(kArThreads), 0, as_stream(stream), a);
}
