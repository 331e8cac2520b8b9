// Library collectives behind the C ABI (include/zg_b200.h: zg_nccl_*, zg_comm_init_rank,
// zg_allreduce, zg_reduce_scatter, zg_all_gather, zg_comm_peer_regions): the data plane of a
// data-parallel step for hosts that are not Python -- the bandwidth-bound gradient buffers of
// the wide model go through NCCL (NVLink / NVSwitch), the latency-bound ones through the
// peer-memory kernel of collective.cu, whose regions this file can also exchange.
//
// NCCL is bound at run time (dlopen), so the library loads, and everything else in it works,
// on a machine without NCCL; only these entry points then report kUnsupported.  Only the public
// C API of NCCL is used: the handful of prototypes below restate nccl.h.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace zg {

typedef struct { char internal[128]; } NcclUniqueId;  // ncclUniqueId (NCCL_UNIQUE_ID_BYTES = 128)
typedef void* NcclComm;
enum { kNcclSuccess = 0 };
enum { kNcclSum = 0 };
enum { kNcclUint8 = 1, kNcclFloat32 = 7, kNcclFloat64 = 8, kNcclBfloat16 = 9 };

struct NcclApi {
  void* handle = nullptr;
  int version = 0;
  int (*GetVersion)(int*) = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
};
static NcclApi g_nccl;
static std::mutex g_nccl_mu;

struct Comm {
  NcclComm nccl;
  unsigned rank, world;
  int device;
};

static bool bind_nccl(const char* path) {
  std::lock_guard<std::mutex> lk(g_nccl_mu);
  if (g_nccl.handle) return true;
  void* h = nullptr;
  const char* env = getenv("ZG_NCCL_LIB");
  if (path && path[0]) h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h && env && env[0]) h = dlopen(env, RTLD_NOW | RTLD_LOCAL);
  // a copy that the process has loaded already (e.g. the one bundled with its tensor library)
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL | RTLD_NOLOAD);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
  if (!h) return false;
  NcclApi a;
  a.handle = h;
  a.GetVersion = reinterpret_cast<decltype(a.GetVersion)>(dlsym(h, "ncclGetVersion"));
  a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
  a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
  a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
  a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
  a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
  a.ReduceScatter = reinterpret_cast<decltype(a.ReduceScatter)>(dlsym(h, "ncclReduceScatter"));
  a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
  if (!a.GetVersion || !a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.GetErrorString || !a.AllReduce || !a.ReduceScatter ||
      !a.AllGather) {
    dlclose(h);
    return false;
  }
  if (a.GetVersion(&a.version) != kNcclSuccess) a.version = 0;
  g_nccl = a;
  return true;
}

static bool nccl_ready(const char* who) {
  if (g_nccl.handle || bind_nccl(nullptr)) return true;
  set_error(kUnsupported, "%s: no NCCL library could be loaded (set ZG_NCCL_LIB or call zg_nccl_load with its path)", who);
  return false;
}

static bool nccl_ok(int r, const char* what) {
  if (r == kNcclSuccess) return true;
  set_error(kCudaError, "%s failed: NCCL error %d (%s)", what, r, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?");
  return false;
}

static int nccl_type(dtype id, size_t* size) {
  switch (id) {
    case SINGLE: *size = 4; return kNcclFloat32;
    case DOUBLE: *size = 8; return kNcclFloat64;
    case BF16: *size = 2; return kNcclBfloat16;
    default: return -1;
  }
}

}  // namespace zg

using namespace zg;

extern "C" int zg_nccl_load(const char* path) {
  if (!bind_nccl(path)) return 0;
  return g_nccl.version;
}

extern "C" void zg_nccl_unique_id(unsigned char* id_out128) {
  if (!id_out128 || !nccl_ready("zg_nccl_unique_id")) return;
  NcclUniqueId id;
  memset(&id, 0, sizeof(id));
  if (!nccl_ok(g_nccl.GetUniqueId(&id), "ncclGetUniqueId")) return;
  memcpy(id_out128, &id, sizeof(id));
}

extern "C" CommWrapper zg_comm_init_rank(const unsigned char* id128, unsigned rank, unsigned world) {
  CommWrapper out{nullptr};
  if (!id128 || world == 0 || rank >= world) { set_error(kBadArgument, "zg_comm_init_rank: rank %u / world %u", rank, world); return out; }
  if (!nccl_ready("zg_comm_init_rank")) return out;
  NcclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  int dev = 0;
  if (!ZG_CUDA(cudaGetDevice(&dev))) return out;
  NcclComm c = nullptr;
  if (!nccl_ok(g_nccl.CommInitRank(&c, (int)world, id, (int)rank), "ncclCommInitRank")) return out;
  out.ptr = new Comm{c, rank, world, dev};
  return out;
}

extern "C" void zg_comm_destroy(CommWrapper comm) {
  Comm* c = static_cast<Comm*>(comm.ptr);
  if (!c) return;
  if (g_nccl.CommDestroy) nccl_ok(g_nccl.CommDestroy(c->nccl), "ncclCommDestroy");
  delete c;
}

extern "C" unsigned zg_comm_rank(CommWrapper comm) { return comm.ptr ? static_cast<Comm*>(comm.ptr)->rank : 0; }
extern "C" unsigned zg_comm_world(CommWrapper comm) { return comm.ptr ? static_cast<Comm*>(comm.ptr)->world : 0; }

extern "C" void zg_allreduce(CommWrapper comm, void* buf, len_t n, dtype id, StreamWrapper stream) {
  Comm* c = static_cast<Comm*>(comm.ptr);
  if (!c) { set_error(kBadArgument, "zg_allreduce: NULL communicator"); return; }
  if (n == 0) return;
  size_t es = 0;
  const int t = nccl_type(id, &es);
  if (t < 0) { set_error(kUnsupported, "zg_allreduce: unsupported dtype %d", (int)id); return; }
  nccl_ok(g_nccl.AllReduce(buf, buf, n, t, kNcclSum, c->nccl, as_stream(stream)), "ncclAllReduce");
}

extern "C" void zg_reduce_scatter(CommWrapper comm, const void* send, void* recv, len_t recv_n, dtype id, StreamWrapper stream) {
  Comm* c = static_cast<Comm*>(comm.ptr);
  if (!c) { set_error(kBadArgument, "zg_reduce_scatter: NULL communicator"); return; }
  if (recv_n == 0) return;
  size_t es = 0;
  const int t = nccl_type(id, &es);
  if (t < 0) { set_error(kUnsupported, "zg_reduce_scatter: unsupported dtype %d", (int)id); return; }
  nccl_ok(g_nccl.ReduceScatter(send, recv, recv_n, t, kNcclSum, c->nccl, as_stream(stream)), "ncclReduceScatter");
}

extern "C" void zg_all_gather(CommWrapper comm, const void* send, void* recv, len_t send_n, dtype id, StreamWrapper stream) {
  Comm* c = static_cast<Comm*>(comm.ptr);
  if (!c) { set_error(kBadArgument, "zg_all_gather: NULL communicator"); return; }
  if (send_n == 0) return;
  size_t es = 0;
  const int t = nccl_type(id, &es);
  if (t < 0) { set_error(kUnsupported, "zg_all_gather: unsupported dtype %d", (int)id); return; }
  nccl_ok(g_nccl.AllGather(send, recv, send_n, t, c->nccl, as_stream(stream)), "ncclAllGather");
}

// Rendezvous of the peer-memory all-reduce: every rank's comm region (zg_comm_alloc) is exported
// as a CUDA IPC handle, the 64-byte handles are all-gathered over the communicator, and the
// peers' regions are mapped into this process.  regions_out[r] is rank r's region as seen here
// (regions_out[rank] = my_region).  Blocks the host until the exchange is done.
extern "C" int zg_comm_peer_regions(CommWrapper comm, void* my_region, void** regions_out, StreamWrapper stream) {
  Comm* c = static_cast<Comm*>(comm.ptr);
  if (!c || !my_region || !regions_out) { set_error(kBadArgument, "zg_comm_peer_regions: NULL argument"); return -1; }
  if (c->world > 8) { set_error(kBadArgument, "zg_comm_peer_regions: at most 8 ranks"); return -1; }
  unsigned char mine[64];
  zg_ipc_export(my_region, mine);
  if (zg_last_error()) return -1;
  unsigned char* d = nullptr;
  std::vector<unsigned char> all((size_t)64 * c->world);
  cudaStream_t s = as_stream(stream);
  if (!ZG_CUDA(cudaMalloc(&d, (size_t)64 * (c->world + 1)))) return -1;
  bool ok = ZG_CUDA(cudaMemcpyAsync(d, mine, 64, cudaMemcpyHostToDevice, s)) &&
            nccl_ok(g_nccl.AllGather(d, d + 64, 64, kNcclUint8, c->nccl, s), "ncclAllGather") &&
            ZG_CUDA(cudaMemcpyAsync(all.data(), d + 64, all.size(), cudaMemcpyDeviceToHost, s)) && ZG_CUDA(cudaStreamSynchronize(s));
  cudaFree(d);
  if (!ok) return -1;
  for (unsigned r = 0; r < c->world; ++r) {
    if (r == c->rank) { regions_out[r] = my_region; continue; }
    regions_out[r] = zg_ipc_open(all.data() + (size_t)64 * r);
    if (!regions_out[r]) return -1;
  }
  return 0;
}
