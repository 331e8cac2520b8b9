// Stream-ordered caching allocator for device memory (include/zg_b200.h,
// zg_cache_*): the device-side replacement of zigrad's CachingAllocator +
// BlockPool (src/allocators/caching_allocator.zig:15-162,
// src/allocators/block_pool.zig:103-412).
//
// Like the reference it has a small pool and a large pool split at 1 MiB
// (caching_allocator.zig:20,158-160), carves blocks out of larger segments,
// splits on allocation and fuses free neighbours on release, and hands the
// block pointer back to the caller as an opaque `ctx` (device_data.zig:32-40).
// Unlike the reference it is stream-aware: a block remembers the stream that
// used it last.  Reuse on the same stream needs no synchronisation (stream
// order already separates the old and new use); reuse from another stream
// makes the new stream wait on an event recorded on the old one.  Segments come
// from cudaMalloc, which is the only synchronising call and only runs when the
// cache has to grow; once warmed up, alloc/free are pure host bookkeeping and
// are therefore legal while a stream capture is in progress.
#include <map>
#include <mutex>
#include <set>
#include <vector>

#include "common.cuh"

namespace zg {

constexpr size_t kSmallLimit = (size_t)1 << 20;       // requests below this use the small pool
constexpr size_t kSmallRound = 512;
constexpr size_t kSmallSegment = (size_t)2 << 20;
constexpr size_t kLargeRound = (size_t)2 << 20;
constexpr size_t kLargeSegmentMin = (size_t)20 << 20;
constexpr size_t kLargeSplitMin = (size_t)1 << 20;    // do not leave large-pool remainders below this

struct Block {
  char* ptr;
  size_t size;
  bool small;
  bool in_use;
  cudaStream_t stream;  // last stream that used the block
  Block* prev;          // address-adjacent neighbours inside the segment
  Block* next;
};

struct BlockLess {
  bool operator()(const Block* a, const Block* b) const {
    if (a->size != b->size) return a->size < b->size;
    return a->ptr < b->ptr;
  }
};

struct Cache {
  int device;
  size_t max_bytes;
  size_t reserved = 0, live = 0, hits = 0, grows = 0;
  std::mutex mu;
  std::set<Block*, BlockLess> free_small, free_large;
  std::vector<void*> segments;
  cudaEvent_t xstream_event = nullptr;
  Block* scratch = nullptr;

  std::set<Block*, BlockLess>& pool(bool small) { return small ? free_small : free_large; }
};

static size_t round_size(size_t n, bool* small) {
  if (n < kSmallLimit) {
    *small = true;
    return ((n ? n : 1) + kSmallRound - 1) / kSmallRound * kSmallRound;
  }
  *small = false;
  return (n + kLargeRound - 1) / kLargeRound * kLargeRound;
}

static Block* find_free(Cache* c, size_t size, bool small, cudaStream_t stream) {
  auto& pool = c->pool(small);
  Block key{nullptr, size, small, false, nullptr, nullptr, nullptr};
  // best fit on the requesting stream first, then any stream
  Block* other = nullptr;
  for (auto it = pool.lower_bound(&key); it != pool.end(); ++it) {
    Block* b = *it;
    if (!small && b->size > size * 2 && b->size - size >= kLargeSegmentMin) break;  // do not shred huge blocks
    if (b->stream == stream) return b;
    if (!other) other = b;
  }
  return other;
}

static Block* grow(Cache* c, size_t size, bool small, cudaStream_t stream) {
  size_t seg = small ? kSmallSegment : (size < kLargeSegmentMin ? kLargeSegmentMin : size);
  if (c->max_bytes && c->reserved + seg > c->max_bytes) {
    if (!small && c->reserved + size <= c->max_bytes) seg = size;  // exact fit still allowed under the budget
    else return nullptr;
  }
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (stream) cudaStreamIsCapturing(stream, &st);
  if (st != cudaStreamCaptureStatusNone) {
    set_error(kBadArgument, "zg_cache_alloc: the cache must grow by %zu bytes during a stream capture; run the step once eagerly first", seg);
    return nullptr;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, seg);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  c->segments.push_back(p);
  c->reserved += seg;
  c->grows++;
  return new Block{static_cast<char*>(p), seg, small, false, stream, nullptr, nullptr};
}

static void release_cached(Cache* c) {
  // free whole segments whose single block is unused
  for (int pass = 0; pass < 2; ++pass) {
    auto& pool = c->pool(pass == 0);
    for (auto it = pool.begin(); it != pool.end();) {
      Block* b = *it;
      if (b->prev == nullptr && b->next == nullptr) {
        cudaFree(b->ptr);
        for (auto s = c->segments.begin(); s != c->segments.end(); ++s)
          if (*s == b->ptr) { c->segments.erase(s); break; }
        c->reserved -= b->size;
        it = pool.erase(it);
        delete b;
      } else {
        ++it;
      }
    }
  }
}

static Block* alloc_locked(Cache* c, size_t nbytes, cudaStream_t stream) {
  bool small = false;
  const size_t size = round_size(nbytes, &small);
  Block* b = find_free(c, size, small, stream);
  if (b) {
    c->pool(small).erase(b);
    c->hits++;
  } else {
    b = grow(c, size, small, stream);
    if (!b) {  // give cached segments back to the driver and retry once
      cudaDeviceSynchronize();
      release_cached(c);
      b = grow(c, size, small, stream);
    }
    if (!b) return nullptr;
  }
  // split off the tail when it is worth keeping
  const size_t rem = b->size - size;
  if ((small && rem >= kSmallRound) || (!small && rem >= kLargeSplitMin)) {
    Block* tail = new Block{b->ptr + size, rem, small, false, b->stream, b, b->next};
    if (b->next) b->next->prev = tail;
    b->next = tail;
    b->size = size;
    c->pool(small).insert(tail);
  }
  if (b->stream != stream) {
    // cross-stream reuse: everything queued so far on the old stream (which
    // includes the block's last use) must finish before the new stream touches it
    if (!c->xstream_event) ZG_CUDA(cudaEventCreateWithFlags(&c->xstream_event, cudaEventDisableTiming));
    if (c->xstream_event) {
      ZG_CUDA(cudaEventRecord(c->xstream_event, b->stream));
      ZG_CUDA(cudaStreamWaitEvent(stream, c->xstream_event, 0));
    }
    b->stream = stream;
  }
  b->in_use = true;
  c->live += b->size;
  return b;
}

static void free_locked(Cache* c, Block* b, cudaStream_t stream) {
  b->in_use = false;
  b->stream = stream;
  c->live -= b->size;
  auto& pool = c->pool(b->small);
  // fuse with free neighbours that were last used on the same stream
  if (b->prev && !b->prev->in_use && b->prev->stream == stream) {
    Block* p = b->prev;
    pool.erase(p);
    p->size += b->size;
    p->next = b->next;
    if (b->next) b->next->prev = p;
    delete b;
    b = p;
  }
  if (b->next && !b->next->in_use && b->next->stream == stream) {
    Block* n = b->next;
    pool.erase(n);
    b->size += n->size;
    b->next = n->next;
    if (n->next) n->next->prev = b;
    delete n;
  }
  pool.insert(b);
}

}  // namespace zg

using namespace zg;

extern "C" CacheWrapper zg_cache_create(unsigned device_id, len_t max_bytes) {
  Cache* c = new Cache();
  c->device = (int)device_id;
  c->max_bytes = max_bytes;
  return CacheWrapper{c};
}

extern "C" void zg_cache_destroy(CacheWrapper cache) {
  Cache* c = static_cast<Cache*>(cache.ptr);
  if (!c) return;
  cudaDeviceSynchronize();
  for (void* p : c->segments) cudaFree(p);
  (void)cudaGetLastError();
  // blocks: walk every segment chain via the pools and in-use lists is not
  // needed for correctness of teardown; free the bookkeeping we can reach
  for (int pass = 0; pass < 2; ++pass)
    for (Block* b : c->pool(pass == 0)) delete b;
  if (c->xstream_event) cudaEventDestroy(c->xstream_event);
  delete c;
}

extern "C" zg_block zg_cache_alloc(CacheWrapper cache, len_t nbytes, StreamWrapper stream) {
  Cache* c = static_cast<Cache*>(cache.ptr);
  zg_block out{nullptr, 0};
  if (!c) return out;
  std::lock_guard<std::mutex> lk(c->mu);
  Block* b = alloc_locked(c, nbytes, as_stream(stream));
  if (!b) return out;  // caller maps NULL to error.DeviceOOM
  out.ptr = b->ptr;
  out.ctx = reinterpret_cast<len_t>(b);
  return out;
}

extern "C" void zg_cache_free(CacheWrapper cache, zg_block block, StreamWrapper stream) {
  Cache* c = static_cast<Cache*>(cache.ptr);
  Block* b = reinterpret_cast<Block*>(block.ctx);
  if (!c || !b) return;
  std::lock_guard<std::mutex> lk(c->mu);
  if (!b->in_use || b->ptr != block.ptr) {
    set_error(kBadArgument, "zg_cache_free: block %p is not a live allocation of this cache", block.ptr);
    return;
  }
  free_locked(c, b, as_stream(stream));
}

extern "C" void* zg_cache_scratch(CacheWrapper cache, len_t nbytes, StreamWrapper stream) {
  Cache* c = static_cast<Cache*>(cache.ptr);
  if (!c) return nullptr;
  if (nbytes == 0) return nullptr;
  std::lock_guard<std::mutex> lk(c->mu);
  // one grow-only buffer, as CachingAllocator.alloc_scratch keeps
  // (caching_allocator.zig:133-156); contents are valid until the next call
  if (c->scratch && c->scratch->size >= nbytes) return c->scratch->ptr;
  if (c->scratch) free_locked(c, c->scratch, as_stream(stream));
  c->scratch = alloc_locked(c, nbytes, as_stream(stream));
  return c->scratch ? c->scratch->ptr : nullptr;
}

extern "C" void zg_cache_clear(CacheWrapper cache) {
  Cache* c = static_cast<Cache*>(cache.ptr);
  if (!c) return;
  cudaDeviceSynchronize();
  std::lock_guard<std::mutex> lk(c->mu);
  release_cached(c);
}

extern "C" void zg_cache_stats(CacheWrapper cache, len_t* out4) {
  Cache* c = static_cast<Cache*>(cache.ptr);
  if (!c || !out4) return;
  std::lock_guard<std::mutex> lk(c->mu);
  out4[0] = c->reserved;
  out4[1] = c->live;
  out4[2] = c->hits;
  out4[3] = c->grows;
}
