// Index ops: scatter_add (flat, blocked and CSR forms), CSR segment sums, row
// gather, and the GCN degree-scaled edge scatter with its backward.  Semantics:
// src/device/host_device.zig:1039-1086, :1137-1160, :1325-1351, :1356-1403 and
// src/ndarray.zig:593-633.
//
// Accumulation into shared destinations uses red.global.add.f32; the values
// added are the reference's, the order in which duplicates land is not.
#include "common.cuh"

namespace zg {

constexpr int kIThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kIThreads) scatter_add_kernel(const T* __restrict__ src, const len_t* __restrict__ offs, size_t n, T* dst) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth) atomicAdd(dst + offs[i], src[i]);
}

template <typename T>
__global__ void __launch_bounds__(kIThreads) gather_rows_kernel(const T* __restrict__ src, const len_t* __restrict__ idx, size_t rows, size_t cols,
                                                                T* __restrict__ dst, len_t* __restrict__ offsets_out, int* bad) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += nth) {
    const size_t c = idx[r];
    if (c >= cols) {  // the reference returns error.IndexOutOfBounds; never read out of range
      if (bad) *bad = 1;
      dst[r] = T(0);
      if (offsets_out) offsets_out[r] = r * cols;
      continue;
    }
    const size_t o = r * cols + c;
    dst[r] = src[o];
    if (offsets_out) offsets_out[r] = o;
  }
}

// dst[tgt,:] += deg[src]*deg[tgt] * h[src,:]   -- one thread per (edge, feature)
__global__ void __launch_bounds__(kIThreads) gcn_scatter_kernel(float* dst, const float* __restrict__ h, const float* __restrict__ deg,
                                                                const len_t* __restrict__ src_idx, const len_t* __restrict__ tgt_idx,
                                                                size_t stride, size_t n_edge) {
  const size_t total = n_edge * stride, nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nth) {
    const size_t e = i / stride, j = i % stride;
    const size_t s = src_idx[e], t = tgt_idx[e];
    const float w = deg[s] * deg[t];
    atomicAdd(dst + t * stride + j, w * h[s * stride + j]);
  }
}

// one thread per edge: the per-edge sums over the feature dim are formed in
// the reference's order, then added to grad_deg with one atomic each
__global__ void __launch_bounds__(kIThreads) gcn_scatter_bwd_kernel(const float* __restrict__ go, const float* __restrict__ h,
                                                                    const float* __restrict__ deg, const len_t* __restrict__ src_idx,
                                                                    const len_t* __restrict__ tgt_idx, float* grad_h, float* grad_deg,
                                                                    size_t stride, size_t n_edge) {
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n_edge; e += nth) {
    const size_t s = src_idx[e], t = tgt_idx[e];
    const float ds = deg[s], dt = deg[t];
    float gs = 0.f, gt = 0.f;
    for (size_t j = 0; j < stride; ++j) {
      const float g = go[t * stride + j];
      const float hv = h[s * stride + j];
      atomicAdd(grad_h + s * stride + j, g * ds * dt);
      gs += g * dt * hv;
      gt += g * ds * hv;
    }
    atomicAdd(grad_deg + s, gs);
    atomicAdd(grad_deg + t, gt);
  }
}

// GCN propagation over a CSR adjacency, no atomics.  A warp owns a row: its
// lanes fetch up to 32 neighbours at once (index, degree scale and feature
// row: the loads of a hub node's many neighbours are in flight together) and
// park the products in shared memory, then lane j adds column j up IN EDGE
// ORDER.  mode 0 = forward of scatter_gcn_deg_scaled with the edges grouped by
// TARGET (row = target t, col = source s):
//     out[t, j] = sum_e (deg[s] * deg[t]) * x[s, j]            (+ bias[j], ReLU)
// mode 1 = its gradient w.r.t. h with the edges grouped by SOURCE (row = s,
// col = t):  out[s, j] = sum_e (x[t, j] * deg[s]) * deg[t]
// -- the products in the order of host_device.zig:1356-1403, the sums in edge
// order when the CSR was built by a stable sort of the edge list, which makes
// the result bit-identical to the host loops.
constexpr int kCsrWarps = kIThreads / 32;

__global__ void __launch_bounds__(kIThreads) csr_gcn_propagate_kernel(float* out, const float* __restrict__ x, const float* __restrict__ deg,
                                                                      const len_t* __restrict__ row_ptr, const len_t* __restrict__ col,
                                                                      size_t n_rows, size_t F, size_t ld_x, size_t ld_out, int mode,
                                                                      int epilogue, const float* __restrict__ bias) {
  __shared__ float prod[kCsrWarps][32][33];  // [neighbour of the chunk][feature of the tile], padded: both access patterns conflict-free
  pdl_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n_rows; r += warps) {
    const len_t k0 = row_ptr[r], k1 = row_ptr[r + 1];
    const float dr = deg[r];
    for (size_t j0 = 0; j0 < F; j0 += 32) {
      const int fw = (int)((F - j0) < 32 ? (F - j0) : 32);
      float acc = 0.f;  // lane j < fw: feature j0 + j
      for (len_t kc = k0; kc < k1; kc += 32) {
        const int nk = (int)((k1 - kc) < 32 ? (k1 - kc) : 32);
        if (lane < nk) {
          const size_t c = col[kc + lane];
          const float dc = deg[c];
          const float* xr = x + c * ld_x + j0;
          for (int j = 0; j < fw; ++j) {
            const float v = xr[j];
            prod[warp][lane][j] = mode == 0 ? (dc * dr) * v : (v * dr) * dc;
          }
        }
        __syncwarp();
        if (lane < fw)
          for (int l = 0; l < nk; ++l) acc += prod[warp][l][lane];
        __syncwarp();
      }
      if (lane < fw) {
        if (epilogue == ZG_EPI_BIAS || epilogue == ZG_EPI_BIAS_RELU) acc += bias[j0 + lane];
        if (epilogue == ZG_EPI_BIAS_RELU) acc = acc > 0.f ? acc : 0.f;
        out[r * ld_out + j0 + lane] = acc;
      }
    }
  }
}

// scatter_add_2d (host_device.zig:1137-1160): dst[indices[i], :] += src[i, :] for blocks of `stride`
// contiguous elements; one thread per (block, element), consecutive threads on consecutive
// elements of a block so both sides are coalesced.
template <typename T>
__global__ void __launch_bounds__(kIThreads) scatter_add_2d_kernel(const T* __restrict__ src, const len_t* __restrict__ indices, size_t n_blocks,
                                                                   size_t stride, T* dst) {
  const size_t total = n_blocks * stride, nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nth) {
    const size_t blk = i / stride, j = i - blk * stride;
    atomicAdd(dst + indices[blk] * stride + j, src[i]);
  }
}

// scatter_add_csr (host_device.zig:1325-1335): dst[j] += src[i] for j in [row_ptr[i], row_ptr[i+1]).
// A warp walks a segment; segments do not overlap, so no atomics and the result is exact.
template <typename T>
__global__ void __launch_bounds__(kIThreads) scatter_add_csr_kernel(const T* __restrict__ src, const len_t* __restrict__ row_ptr, size_t n_seg, T* dst) {
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n_seg; r += warps) {
    const len_t k0 = row_ptr[r], k1 = row_ptr[r + 1];
    const T v = src[r];
    for (len_t j = k0 + lane; j < k1; j += 32) dst[j] += v;
  }
}

// segment_sum_csr (host_device.zig:1337-1351): dst[i] = sum of src[row_offsets[i] .. row_offsets[i+1]).
// A warp per segment: lane l adds elements l, l+32, ... in order, then the 32 partial sums are
// folded by a shuffle tree (fixed order, so repeatable; not the host's left-to-right order).
template <typename T>
__global__ void __launch_bounds__(kIThreads) segment_sum_csr_kernel(const T* __restrict__ src, const len_t* __restrict__ row_ptr, size_t n_seg, T* __restrict__ dst) {
  const int lane = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n_seg; r += warps) {
    const len_t k0 = row_ptr[r], k1 = row_ptr[r + 1];
    T acc = T(0);
    if (k1 - k0 <= 32) {  // short segment: lane 0 adds left to right, the host's order exactly
      const T v = (k0 + lane < k1) ? src[k0 + lane] : T(0);
      for (int l = 0; l < 32; ++l) {
        const T u = __shfl_sync(0xffffffffu, v, l);
        if ((len_t)l < k1 - k0) acc += u;
      }
    } else {
      for (len_t j = k0 + lane; j < k1; j += 32) acc += src[j];
      acc = warp_sum(acc);
    }
    if (lane == 0) dst[r] = acc;
  }
}

}  // namespace zg

using namespace zg;

extern "C" void zg_scatter_add_2d(dtype id, StreamWrapper w, const void* src, const len_t* indices, len_t n_blocks, len_t stride, void* dst) {
  if (n_blocks == 0 || stride == 0) return;
  cudaStream_t s = as_stream(w);
  const unsigned g = grid_for((size_t)n_blocks * stride, kIThreads * 2);
  if (id == SINGLE) scatter_add_2d_kernel<float><<<g, kIThreads, 0, s>>>((const float*)src, indices, n_blocks, stride, (float*)dst);
  else if (id == DOUBLE) scatter_add_2d_kernel<double><<<g, kIThreads, 0, s>>>((const double*)src, indices, n_blocks, stride, (double*)dst);
  else { set_error(kUnsupported, "zg_scatter_add_2d: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}

extern "C" void zg_scatter_add_csr(dtype id, StreamWrapper w, const void* src, const len_t* row_ptr, len_t n_segments, void* dst) {
  if (n_segments == 0) return;
  cudaStream_t s = as_stream(w);
  const unsigned g = grid_for(n_segments, kIThreads / 32);
  if (id == SINGLE) scatter_add_csr_kernel<float><<<g, kIThreads, 0, s>>>((const float*)src, row_ptr, n_segments, (float*)dst);
  else if (id == DOUBLE) scatter_add_csr_kernel<double><<<g, kIThreads, 0, s>>>((const double*)src, row_ptr, n_segments, (double*)dst);
  else { set_error(kUnsupported, "zg_scatter_add_csr: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}

extern "C" void zg_segment_sum_csr(dtype id, StreamWrapper w, const void* src, const len_t* row_offsets, len_t n_segments, void* dst) {
  if (n_segments == 0) return;
  cudaStream_t s = as_stream(w);
  const unsigned g = grid_for(n_segments, kIThreads / 32);
  if (id == SINGLE) segment_sum_csr_kernel<float><<<g, kIThreads, 0, s>>>((const float*)src, row_offsets, n_segments, (float*)dst);
  else if (id == DOUBLE) segment_sum_csr_kernel<double><<<g, kIThreads, 0, s>>>((const double*)src, row_offsets, n_segments, (double*)dst);
  else { set_error(kUnsupported, "zg_segment_sum_csr: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}

extern "C" void zg_scatter_add(dtype id, StreamWrapper w, const void* src, const len_t* offsets, len_t n, void* dst) {
  if (n == 0) return;
  cudaStream_t s = as_stream(w);
  if (id == SINGLE) scatter_add_kernel<float><<<grid_for(n, kIThreads * 2), kIThreads, 0, s>>>((const float*)src, offsets, n, (float*)dst);
  else if (id == DOUBLE) scatter_add_kernel<double><<<grid_for(n, kIThreads * 2), kIThreads, 0, s>>>((const double*)src, offsets, n, (double*)dst);
  else { set_error(kUnsupported, "zg_scatter_add: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}

extern "C" void zg_gather_rows(dtype id, StreamWrapper w, const void* src, const len_t* idx, len_t rows, len_t cols, void* dst,
                               len_t* offsets_out) {
  if (rows == 0) return;
  cudaStream_t s = as_stream(w);
  if (id == SINGLE) gather_rows_kernel<float><<<grid_for(rows, kIThreads), kIThreads, 0, s>>>((const float*)src, idx, rows, cols, (float*)dst, offsets_out, nullptr);
  else if (id == DOUBLE) gather_rows_kernel<double><<<grid_for(rows, kIThreads), kIThreads, 0, s>>>((const double*)src, idx, rows, cols, (double*)dst, offsets_out, nullptr);
  else { set_error(kUnsupported, "zg_gather_rows: unsupported dtype %d", (int)id); return; }
  ZG_LAUNCH_CHECK();
}

extern "C" void zg_scatter_gcn_deg_scaled(dtype id, StreamWrapper w, void* dst, const void* h, const void* deg, const len_t* src_idx,
                                          const len_t* tgt_idx, len_t stride, len_t n_edge) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_scatter_gcn_deg_scaled: only SINGLE is implemented"); return; }
  if (n_edge == 0 || stride == 0) return;
  gcn_scatter_kernel<<<grid_for(n_edge * stride, kIThreads * 2), kIThreads, 0, as_stream(w)>>>((float*)dst, (const float*)h, (const float*)deg, src_idx, tgt_idx, stride, n_edge);
  ZG_LAUNCH_CHECK();
}

extern "C" void zg_scatter_gcn_deg_scaled_bwd(dtype id, StreamWrapper w, const void* grad_out, const void* h, const void* deg,
                                              const len_t* src_idx, const len_t* tgt_idx, void* grad_h, void* grad_deg, len_t stride,
                                              len_t n_edge) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_scatter_gcn_deg_scaled_bwd: only SINGLE is implemented"); return; }
  if (n_edge == 0 || stride == 0) return;
  gcn_scatter_bwd_kernel<<<grid_for(n_edge, kIThreads), kIThreads, 0, as_stream(w)>>>((const float*)grad_out, (const float*)h, (const float*)deg, src_idx, tgt_idx, (float*)grad_h, (float*)grad_deg, stride, n_edge);
  ZG_LAUNCH_CHECK();
}

extern "C" void zg_csr_gcn_propagate(dtype id, StreamWrapper w, void* out, const void* x, const void* deg, const len_t* row_ptr,
                                     const len_t* col_idx, len_t n_rows, len_t n_feat, len_t ld_x, len_t ld_out, int transpose_form,
                                     int epilogue, const void* bias) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_csr_gcn_propagate: only SINGLE is implemented"); return; }
  if (n_rows == 0 || n_feat == 0) return;
  if (epilogue != ZG_EPI_NONE && epilogue != ZG_EPI_BIAS && epilogue != ZG_EPI_BIAS_RELU) { set_error(kBadArgument, "zg_csr_gcn_propagate: epilogue %d", epilogue); return; }
  if (epilogue != ZG_EPI_NONE && !bias) { set_error(kBadArgument, "zg_csr_gcn_propagate: bias epilogue without bias"); return; }
  launch_pdl(csr_gcn_propagate_kernel, dim3(grid_for(n_rows, kCsrWarps)), dim3(kIThreads), 0, as_stream(w), (float*)out, (const float*)x,
             (const float*)deg, row_ptr, col_idx, (size_t)n_rows, (size_t)n_feat, (size_t)ld_x, (size_t)ld_out, transpose_form ? 1 : 0, epilogue,
             (const float*)bias);
}
