"""The stream-ordered cache (zg_cache_*) tested as an allocator, through the C ABI.

Behaviours to match: zigrad's CachingAllocator (alloc / free / scratch lifetime /
OOM -> error.DeviceOOM, src/allocators/caching_allocator.zig:80-156) and BlockPool
(split on alloc, fuse with free neighbours on free, src/allocators/block_pool.zig:185-324);
added here: reuse across streams is ordered by an event.
"""
import ctypes as C

import numpy as np
import pytest

from zigrad_b200 import abi
from zigrad_b200.abi import SINGLE
from zigrad_b200.device import CudaDevice, DeviceOOM

pytestmark = pytest.mark.gpu

MiB = 1 << 20


def stats(L, cache):
    out = (abi.len_t * 4)()
    L.zg_cache_stats(cache, out)
    return dict(reserved=out[0], live=out[1], hits=out[2], grows=out[3])


def fill(L, ptr, n, value, stream):
    v = C.c_float(value)
    L.mem_fill(SINGLE, ptr, n, C.byref(v), stream)


def read_f32(L, ptr, n, stream):
    host = np.empty(n, np.float32)
    L.memcpy_DtoH(host.ctypes.data, ptr, 4 * n, stream)
    L.stream_synchronize(stream)
    return host


@pytest.fixture()
def cache(gpu):
    L = gpu.L
    c = L.zg_cache_create(gpu.device_number, 0)
    yield c
    L.zg_cache_destroy(c)


def test_same_stream_reuse_returns_the_same_block_without_growing(gpu, cache):
    L, s = gpu.L, gpu.stream
    a = L.zg_cache_alloc(cache, 4096, s)
    g0 = stats(L, cache)["grows"]
    fill(L, a.ptr, 1024, 3.0, s)
    L.zg_cache_free(cache, a, s)
    b = L.zg_cache_alloc(cache, 4096, s)          # no synchronisation in between: stream order is enough
    assert b.ptr == a.ptr
    st = stats(L, cache)
    assert st["grows"] == g0 and st["hits"] >= 1 and st["live"] == 4096
    fill(L, b.ptr, 1024, 4.0, s)
    assert (read_f32(L, b.ptr, 1024, s) == 4.0).all()
    L.zg_cache_free(cache, b, s)
    assert stats(L, cache)["live"] == 0


def test_block_freed_on_one_stream_and_taken_on_another_waits_for_the_first(gpu, cache):
    """Stream A still has a queue of fills over the block when it frees it; stream B takes the
    block at once and reads it: it must see A's LAST fill, i.e. B waited for A."""
    L, sa = gpu.L, gpu.stream
    sb = L.init_stream()
    n = 64 * MiB  # floats: 256 MiB, each fill takes tens of microseconds
    a = L.zg_cache_alloc(cache, 4 * n, sa)
    assert a.ptr
    for i in range(24):
        fill(L, a.ptr, n, float(i), sa)
    L.zg_cache_free(cache, a, sa)
    b = L.zg_cache_alloc(cache, 4 * n, sb)        # same memory, other stream
    assert b.ptr == a.ptr
    tail = read_f32(L, b.ptr + 4 * (n - 256), 256, sb)   # enqueued on B, synchronises B only
    assert (tail == 23.0).all(), tail[:8]
    # and the other way round: B writes, frees; A must not overtake B's writes
    for i in range(12):
        fill(L, b.ptr, n, 100.0 + i, sb)
    L.zg_cache_free(cache, b, sb)
    c = L.zg_cache_alloc(cache, 4 * n, sa)
    assert c.ptr == a.ptr
    assert (read_f32(L, c.ptr, 256, sa) == 111.0).all()
    L.zg_cache_free(cache, c, sa)
    L.stream_synchronize(sa)
    L.stream_synchronize(sb)
    L.deinit_stream(sb)


@pytest.mark.parametrize("order", [(0, 1, 2), (2, 1, 0), (1, 0, 2), (1, 2, 0), (0, 2, 1)])
def test_split_blocks_fuse_back_into_one_segment_in_any_free_order(gpu, cache, order):
    L, s = gpu.L, gpu.stream
    blocks = [L.zg_cache_alloc(cache, nb, s) for nb in (1000, 2000, 3000)]
    st = stats(L, cache)
    assert st["grows"] == 1 and st["reserved"] == 2 * MiB          # one small-pool segment, split three times
    assert blocks[1].ptr == blocks[0].ptr + 1024 and blocks[2].ptr == blocks[1].ptr + 2048   # 512-byte granules
    assert st["live"] == 1024 + 2048 + 3072
    L.zg_cache_free(cache, blocks[order[0]], s)
    L.zg_cache_free(cache, blocks[order[1]], s)
    L.zg_cache_clear(cache)
    assert stats(L, cache)["reserved"] == 2 * MiB                  # a live block pins the segment
    L.zg_cache_free(cache, blocks[order[2]], s)
    whole = L.zg_cache_alloc(cache, MiB - 512, s)                  # the largest small-pool request: served from the
    assert whole.ptr == blocks[0].ptr and stats(L, cache)["grows"] == 1   # segment's START only if everything fused
    L.zg_cache_free(cache, whole, s)
    L.zg_cache_clear(cache)
    st = stats(L, cache)
    assert st["reserved"] == 0 and st["live"] == 0                 # fused into one block, returned to the driver


def test_large_pool_split_and_fuse(gpu, cache):
    L, s = gpu.L, gpu.stream
    a = L.zg_cache_alloc(cache, 4 * MiB, s)       # 20 MiB segment, 4 MiB head, 16 MiB tail stays cached
    b = L.zg_cache_alloc(cache, 6 * MiB, s)
    st = stats(L, cache)
    assert st["reserved"] == 20 * MiB and st["grows"] == 1 and b.ptr == a.ptr + 4 * MiB
    L.zg_cache_free(cache, a, s)
    L.zg_cache_free(cache, b, s)
    c = L.zg_cache_alloc(cache, 20 * MiB, s)
    assert c.ptr == a.ptr and stats(L, cache)["grows"] == 1
    L.zg_cache_free(cache, c, s)


def test_budget_exhaustion_returns_null_and_maps_to_device_oom(gpu):
    L = gpu.L
    L.zg_clear_error()
    c = L.zg_cache_create(gpu.device_number, 64 * MiB)
    s = gpu.stream
    a = L.zg_cache_alloc(c, 30 * MiB, s)
    b = L.zg_cache_alloc(c, 30 * MiB, s)
    assert a.ptr and b.ptr
    z = L.zg_cache_alloc(c, 30 * MiB, s)          # 90 MiB > 64 MiB
    assert not z.ptr and z.ctx == 0
    assert L.zg_last_error() == 0                 # out of memory is reported by the NULL block alone
    assert not L.zg_cache_scratch(c, 30 * MiB, s)
    L.zg_cache_free(c, a, s)
    again = L.zg_cache_alloc(c, 30 * MiB, s)      # the freed block serves the same request
    assert again.ptr == a.ptr
    L.zg_cache_free(c, again, s)
    L.zg_cache_free(c, b, s)
    L.zg_cache_destroy(c)
    # the host-side device object turns the NULL block into DeviceOOM (error.DeviceOOM of the reference)
    d = CudaDevice(gpu.device_number, cache_max_bytes=8 * MiB)
    keep = d.mem_cache_alloc(SINGLE, MiB)         # 4 MiB
    with pytest.raises(DeviceOOM):
        d.mem_cache_alloc(SINGLE, 4 * MiB)        # 16 MiB
    d.mem_cache_free(keep)
    d.deinit()


def test_scratch_is_one_buffer_valid_until_the_next_scratch_call(gpu, cache):
    L, s = gpu.L, gpu.stream
    p1 = L.zg_cache_scratch(cache, 4000, s)
    fill(L, p1, 1000, 7.0, s)
    other = L.zg_cache_alloc(cache, 4000, s)      # ordinary allocations do not disturb it
    assert other.ptr != p1
    fill(L, other.ptr, 1000, 1.0, s)
    p2 = L.zg_cache_scratch(cache, 2000, s)       # smaller request: the same buffer, contents kept
    assert p2 == p1
    assert (read_f32(L, p2, 1000, s) == 7.0).all()
    p3 = L.zg_cache_scratch(cache, 3 * MiB, s)    # larger: the old one goes back to the cache
    assert p3 and p3 != p1
    fill(L, p3, 3 * MiB // 4, 9.0, s)
    assert (read_f32(L, p3, 16, s) == 9.0).all()
    st = stats(L, cache)
    assert st["live"] == 4096 + 4 * MiB           # `other` + the current scratch (2 MiB granules)
    L.zg_cache_free(cache, other, s)
    assert L.zg_cache_scratch(cache, 0, s) is None


def test_freeing_a_foreign_or_stale_block_is_refused(gpu, cache):
    L, s = gpu.L, gpu.stream
    L.zg_clear_error()
    a = L.zg_cache_alloc(cache, 512, s)
    L.zg_cache_free(cache, a, s)
    L.zg_cache_free(cache, a, s)                  # double free
    assert L.zg_last_error() == 2
    L.zg_clear_error()


def test_random_alloc_free_with_guard_words_and_no_overlap(gpu, cache):
    """10 000 requests of 40 B .. 134 MB (log-uniform: the sizes a training step asks for), each
    block's first and last 32 bytes stamped with its serial number, checked when it is freed;
    live blocks are checked for overlap on the host."""
    L, s = gpu.L, gpu.stream
    g = np.random.Generator(np.random.PCG64(2024))
    live = {}                                     # serial -> (block, nbytes)
    live_bytes, cap = 0, 3 << 30
    G = 8                                         # guard floats at either end

    def stamp(blk, nbytes, serial):
        fill(L, blk.ptr, G, float(serial), s)
        fill(L, blk.ptr + nbytes - 4 * G, G, float(-serial), s)

    def check(blk, nbytes, serial):
        lo = read_f32(L, blk.ptr, G, s)
        hi = read_f32(L, blk.ptr + nbytes - 4 * G, G, s)
        assert (lo == float(serial)).all() and (hi == float(-serial)).all(), (serial, nbytes, lo[:4], hi[:4])

    for serial in range(1, 10001):
        want_free = live and (live_bytes > cap or g.random() < 0.48)
        if want_free:
            k = list(live)[int(g.integers(0, len(live)))]
            blk, nb = live.pop(k)
            if k % 16 == 0 or nb > MiB:           # reading back every small block would dominate the run time
                check(blk, nb, k)
            L.zg_cache_free(cache, blk, s)
            live_bytes -= nb
            continue
        nb = int(np.exp(g.uniform(np.log(40), np.log(134e6))))
        nb = max(nb, 8 * G) // 4 * 4              # room for both guard regions, whole floats
        blk = L.zg_cache_alloc(cache, nb, s)
        assert blk.ptr, (serial, nb)
        assert blk.ptr % 512 == 0
        stamp(blk, nb, serial)
        live[serial] = (blk, nb)
        live_bytes += nb
        if serial % 500 == 0:                     # no two live blocks overlap
            spans = sorted((b.ptr, b.ptr + n) for b, n in live.values())
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 <= b0, (a0, a1, b0, b1)
            st = stats(L, cache)
            assert st["live"] >= live_bytes and st["reserved"] >= st["live"]
    for k, (blk, nb) in live.items():
        check(blk, nb, k)
        L.zg_cache_free(cache, blk, s)
    assert stats(L, cache)["live"] == 0
    assert L.zg_last_error() == 0


# ------------------------------------------------------------------ bounded waits
def test_a_peer_that_never_arrives_makes_the_allreduce_give_up_and_report(gpu):
    """One GPU, two comm regions, only "rank 0" of a world of two launches: nothing ever writes
    rank 1's words, so rank 0's polls run out (a short limit), the kernel returns, the region's
    error word and the library's time-out status are raised, and the stream still answers."""
    L, s = gpu.L, gpu.stream
    L.zg_clear_error()
    n = 4096
    regions = [L.zg_comm_alloc(n, 2), L.zg_comm_alloc(n, 2)]
    assert all(regions)
    comm = (C.c_void_p * 2)(*regions)
    buf = gpu.from_numpy(np.arange(n, dtype=np.float32))
    L.zg_comm_set_spin_limit(3000)
    try:
        L.zg_allreduce_oneshot(s, buf.ptr, n, 0, 2, comm, n)
        assert L.zg_comm_error(regions[0], s) == 1
        assert L.zg_comm_error(regions[0], s) == 0          # read-and-clear
        L.stream_synchronize(s)                             # picks up the device-side time-out flag
        assert L.zg_last_error() == 4                       # kKernelTimeout
        L.zg_clear_error()
        # the context is intact: later work on the same stream runs and is correct
        fill(L, buf.ptr, n, 2.5, s)
        assert (read_f32(L, buf.ptr, n, s) == 2.5).all()
        # and a complete world (both "ranks" launched back to back is NOT possible on one GPU, so a
        # world of one) still reduces correctly through the same region afterwards
        one = (C.c_void_p * 1)(regions[0])
        L.zg_allreduce_oneshot(s, buf.ptr, n, 0, 1, one, n)
        assert L.zg_comm_error(regions[0], s) == 0
        assert (read_f32(L, buf.ptr, n, s) == 2.5).all()
        L.stream_synchronize(s)
        assert L.zg_last_error() == 0
    finally:
        L.zg_comm_set_spin_limit(0)
        gpu.mem_cache_free(buf)
        for r in regions:
            L.zg_comm_free(r)
        L.zg_clear_error()
