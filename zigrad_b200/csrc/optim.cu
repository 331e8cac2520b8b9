// Multi-tensor optimizer updates over one flat parameter buffer and one flat
// gradient buffer.  Semantics: src/nn/optim.zig:100-122 (SGD), :177-234 (Adam),
// gradient clipping src/device/host_device.zig:339-346.
#include <cmath>
#include <cstring>

#include "common.cuh"

namespace zg {

constexpr int kOThreads = 256;
constexpr int kMaxSeg = 48;  // segments per launch (table travels in kernel parameters)

struct SegTable {
  unsigned long long offset[kMaxSeg];
  unsigned long long len[kMaxSeg];
  float lr_t[kMaxSeg];  // Adam: bias-corrected step size of the segment
  int n;
  int first;  // index of the first segment of this launch in the caller's list
};

// fp32 elements from p up to the next 16-byte boundary
__device__ __forceinline__ size_t misalign_elems(const void* p) { return ((16u - (unsigned)(reinterpret_cast<uintptr_t>(p) & 15u)) & 15u) >> 2; }
__device__ __forceinline__ bool same_phase(const void* a, const void* b) {
  return ((reinterpret_cast<uintptr_t>(a) ^ reinterpret_cast<uintptr_t>(b)) & 15u) == 0;
}

// norms[first + j] = ||g_j||_2 for every segment of the table.  grid = (chunks, n);
// chunk partials are folded by the last CTA of each segment in index order.
__global__ void __launch_bounds__(kOThreads) seg_nrm2_kernel(const float* __restrict__ g, const __grid_constant__ SegTable tab,
                                                             float* norms, double* partial, unsigned* counters, int squares) {
  __shared__ double sm[32];
  pdl_sync();
  const int seg = blockIdx.y;
  const float* p = g + tab.offset[seg];
  const size_t n = tab.len[seg];
  const size_t nth = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // scalar head up to the first 16-byte boundary, 128-bit body (4 loads in flight per thread), scalar tail
  size_t head = misalign_elems(p);
  if (head > n) head = n;
  float acc = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  for (size_t i = tid; i < head; i += nth) acc += p[i] * p[i];
  const float4* pv = reinterpret_cast<const float4*>(p + head);
  const size_t nv = (n - head) / 4;
  size_t v = tid;
  for (; v + 3 * nth < nv; v += 4 * nth) {
    const float4 q0 = pv[v], q1 = pv[v + nth], q2 = pv[v + 2 * nth], q3 = pv[v + 3 * nth];
    acc += q0.x * q0.x + q0.y * q0.y + q0.z * q0.z + q0.w * q0.w;
    a1 += q1.x * q1.x + q1.y * q1.y + q1.z * q1.z + q1.w * q1.w;
    a2 += q2.x * q2.x + q2.y * q2.y + q2.z * q2.z + q2.w * q2.w;
    a3 += q3.x * q3.x + q3.y * q3.y + q3.z * q3.z + q3.w * q3.w;
  }
  for (; v < nv; v += nth) {
    const float4 q0 = pv[v];
    acc += q0.x * q0.x + q0.y * q0.y + q0.z * q0.z + q0.w * q0.w;
  }
  for (size_t i = head + nv * 4 + tid; i < n; i += nth) acc += p[i] * p[i];
  acc = (acc + a1) + (a2 + a3);
  const double bs = block_sum<double>((double)acc, sm);
  double* mine = partial + (size_t)seg * gridDim.x;
  if (threadIdx.x == 0) mine[blockIdx.x] = bs;
  __threadfence();
  __shared__ bool last;
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(counters + 1 + seg, 1u);
    last = (t == gridDim.x - 1);
    if (last) counters[1 + seg] = 0;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  double s = 0.0;
  for (unsigned k = threadIdx.x; k < gridDim.x; k += blockDim.x) s += __ldcg(mine + k);
  s = block_sum<double>(s, sm);
  if (threadIdx.x == 0) norms[tab.first + seg] = squares ? (float)s : (float)sqrt(s);  // squares: the caller sums them over shards first
}

__device__ __forceinline__ float clip_factor(const float* norms, int idx, float max_norm, float delta, bool* on) {
  const float nv = norms[idx];
  *on = nv > max_norm;
  return *on ? max_norm / (nv + delta) : 1.f;
}

// p += (-lr) * g, with the gradient scaled (and written back) first when its
// norm exceeds max_norm.
template <bool CLIP>
__global__ void __launch_bounds__(kOThreads) sgd_kernel(float* params, float* grads, const __grid_constant__ SegTable tab, float nlr,
                                                        const float* __restrict__ norms, float max_norm, float delta, const int zero) {
  pdl_sync();
  const int seg = blockIdx.y;
  float* p = params + tab.offset[seg];
  float* g = grads + tab.offset[seg];
  const size_t n = tab.len[seg];
  bool on = false;
  float f = 1.f;
  if (CLIP) f = clip_factor(norms, tab.first + seg, max_norm, delta, &on);
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (same_phase(p, g) && (reinterpret_cast<uintptr_t>(p) & 3u) == 0) {
    size_t head = misalign_elems(p);
    if (head > n) head = n;
    const size_t nv = (n - head) / 4;
    for (size_t i = tid; i < head; i += nth) {
      float gi = g[i];
      if (CLIP && on) { gi *= f; g[i] = gi; }
      if (zero) g[i] = 0.f;
      p[i] = fmaf(nlr, gi, p[i]);
    }
    float4* gq = reinterpret_cast<float4*>(g + head);
    float4* pq = reinterpret_cast<float4*>(p + head);
    for (size_t v = tid; v < nv; v += nth) {
      float4 gv = gq[v];
      float4 pv = pq[v];
      if (CLIP && on) {
        gv.x *= f; gv.y *= f; gv.z *= f; gv.w *= f;
        gq[v] = gv;
      }
      if (zero) gq[v] = make_float4(0.f, 0.f, 0.f, 0.f);
      pv.x = fmaf(nlr, gv.x, pv.x); pv.y = fmaf(nlr, gv.y, pv.y); pv.z = fmaf(nlr, gv.z, pv.z); pv.w = fmaf(nlr, gv.w, pv.w);
      pq[v] = pv;
    }
    for (size_t i = head + nv * 4 + tid; i < n; i += nth) {
      float gi = g[i];
      if (CLIP && on) { gi *= f; g[i] = gi; }
      if (zero) g[i] = 0.f;
      p[i] = fmaf(nlr, gi, p[i]);
    }
  } else {
    for (size_t i = tid; i < n; i += nth) {
      float gi = g[i];
      if (CLIP && on) { gi *= f; g[i] = gi; }
      if (zero) g[i] = 0.f;
      p[i] = fmaf(nlr, gi, p[i]);
    }
  }
}

// Adam in fp32, operation for operation as the reference loop:
//   m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*g*g ; p -= lr_t * m / (sqrt(v) + eps)
template <bool CLIP, bool BF16COPY>
__global__ void __launch_bounds__(kOThreads) adam_kernel(float* params, float* grads, float* ms, float* vs, const __grid_constant__ SegTable tab,
                                                         float b1, float b2, float eps, const float* __restrict__ norms, float max_norm,
                                                         float delta, __nv_bfloat16* copy, const unsigned long long* t_dev, float lr) {
  pdl_sync();
  const int seg = blockIdx.y;
  const size_t off = tab.offset[seg];
  float* p = params + off;
  float* g = grads + off;
  float* m = ms + off;
  float* v = vs + off;
  const size_t n = tab.len[seg];
  float lr_t = tab.lr_t[seg];
  if (t_dev) {  // step counter kept on the device (graph replay): t = counter + position of this tensor
    const float t_f = (float)(*t_dev + (unsigned long long)(tab.first + seg + 1));
    lr_t = lr * sqrtf(1.f - powf(b2, t_f)) / (1.f - powf(b1, t_f));
  }
  const float omb1 = 1.f - b1, omb2 = 1.f - b2;
  bool on = false;
  float f = 1.f;
  if (CLIP) f = clip_factor(norms, tab.first + seg, max_norm, delta, &on);
  const size_t nth = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  // one element, operation for operation as the host loop (no contraction: the file is built with --fmad=false)
  auto one = [&](float& gi, float& mi, float& vi, float& pi) {
    if (CLIP && on) gi *= f;
    mi = b1 * mi + omb1 * gi;
    vi = b2 * vi + omb2 * gi * gi;
    pi = pi - lr_t * mi / (sqrtf(vi) + eps);
  };
  auto scalar = [&](size_t i) {
    float gi = g[i], mi = m[i], vi = v[i], pi = p[i];
    one(gi, mi, vi, pi);
    if (CLIP && on) g[i] = gi;
    m[i] = mi; v[i] = vi; p[i] = pi;
    if (BF16COPY) copy[off + i] = __float2bfloat16_rn(pi);
  };
  size_t head = misalign_elems(p);
  if (head > n) head = n;
  bool vec = same_phase(p, g) && same_phase(p, m) && same_phase(p, v) && (reinterpret_cast<uintptr_t>(p) & 3u) == 0;
  if (BF16COPY) vec = vec && (reinterpret_cast<uintptr_t>(copy + off + head) & 7u) == 0;
  if (!vec) {
    for (size_t i = tid; i < n; i += nth) scalar(i);
    return;
  }
  const size_t nv = (n - head) / 4;
  for (size_t i = tid; i < head; i += nth) scalar(i);
  float4* gq = reinterpret_cast<float4*>(g + head);
  float4* mq = reinterpret_cast<float4*>(m + head);
  float4* vq = reinterpret_cast<float4*>(v + head);
  float4* pq = reinterpret_cast<float4*>(p + head);
  for (size_t k = tid; k < nv; k += nth) {
    float4 gv = gq[k], mv = mq[k], vv = vq[k], pv = pq[k];
    one(gv.x, mv.x, vv.x, pv.x);
    one(gv.y, mv.y, vv.y, pv.y);
    one(gv.z, mv.z, vv.z, pv.z);
    one(gv.w, mv.w, vv.w, pv.w);
    if (CLIP && on) gq[k] = gv;
    mq[k] = mv; vq[k] = vv; pq[k] = pv;
    if (BF16COPY) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(pv.x, pv.y), hi = __floats2bfloat162_rn(pv.z, pv.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo);
      o.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(copy + off + head + 4 * k) = o;
    }
  }
  for (size_t i = head + nv * 4 + tid; i < n; i += nth) scalar(i);
}

__global__ void counter_add_kernel(unsigned long long* c, unsigned long long inc) {
  pdl_sync();
  *c += inc;
}

static unsigned chunks_for(const zg_segment* seg, size_t n_seg) {
  size_t mx = 0;
  for (size_t j = 0; j < n_seg; ++j) mx = seg[j].len > mx ? seg[j].len : mx;
  size_t c = (mx + (size_t)kOThreads * 4 - 1) / ((size_t)kOThreads * 4);
  size_t cap = (size_t)sm_count() * 8 / (n_seg ? n_seg : 1);
  if (cap < 8) cap = 8;
  if (c > cap) c = cap;
  return (unsigned)(c < 1 ? 1 : c);
}

static bool compute_norms(cudaStream_t s, const float* grads, const zg_segment* seg, size_t n_seg, float* norms, int squares = 0) {
  if (!norms) { set_error(kBadArgument, "optimizer: clip requested but norms scratch is NULL"); return false; }
  for (size_t first = 0; first < n_seg; first += kMaxSeg) {
    SegTable tab;
    memset(&tab, 0, sizeof(tab));
    tab.n = (int)((n_seg - first) < (size_t)kMaxSeg ? (n_seg - first) : kMaxSeg);
    tab.first = (int)first;
    for (int j = 0; j < tab.n; ++j) { tab.offset[j] = seg[first + j].offset; tab.len[j] = seg[first + j].len; }
    unsigned chunks = chunks_for(seg + first, tab.n);
    if (chunks > 256) chunks = 256;
    unsigned* counters = nullptr;
    double* partial = static_cast<double*>(workspace(s, sizeof(double) * chunks * tab.n, &counters));
    if (!partial) return false;
    if (!launch_pdl(seg_nrm2_kernel, dim3(chunks, tab.n), dim3(kOThreads), 0, s, grads, tab, norms, partial, counters, squares)) return false;
  }
  return true;
}

}  // namespace zg

using namespace zg;

extern "C" void zg_sgd_step(dtype id, StreamWrapper w, void* params, void* grads, const zg_segment* seg, len_t n_seg, double lr,
                            int clip, double max_norm, double delta, void* norms, int zero_grads) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_sgd_step: only SINGLE is implemented"); return; }
  if (n_seg == 0) return;
  cudaStream_t s = as_stream(w);
  const float nlr = -(float)lr;  // lr cast f64 -> f32, then negated (optim.zig:103)
  if (clip == 1 && !compute_norms(s, (const float*)grads, seg, n_seg, (float*)norms)) return;
  if (clip == 2 && !norms) { set_error(kBadArgument, "optimizer: clip with given norms but norms is NULL"); return; }
  for (size_t first = 0; first < n_seg; first += kMaxSeg) {
    SegTable tab;
    memset(&tab, 0, sizeof(tab));
    tab.n = (int)((n_seg - first) < (size_t)kMaxSeg ? (n_seg - first) : kMaxSeg);
    tab.first = (int)first;
    for (int j = 0; j < tab.n; ++j) { tab.offset[j] = seg[first + j].offset; tab.len[j] = seg[first + j].len; }
    const dim3 grid(chunks_for(seg + first, tab.n), tab.n);
    if (clip) launch_pdl(sgd_kernel<true>, grid, dim3(kOThreads), 0, s, (float*)params, (float*)grads, tab, nlr, (const float*)norms, (float)max_norm, (float)delta, zero_grads);
    else launch_pdl(sgd_kernel<false>, grid, dim3(kOThreads), 0, s, (float*)params, (float*)grads, tab, nlr, (const float*)nullptr, 0.f, 0.f, zero_grads);
  }
}

extern "C" void zg_adam_step_part(dtype id, StreamWrapper w, void* params, void* grads, void* m, void* v, const zg_segment* seg, len_t n_seg,
                                  len_t t_first, double lr_, double beta1_, double beta2_, double eps_, int clip, double max_norm, double delta,
                                  void* norms, void* bf16_copy, void* step_counter, int advance_counter) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_adam_step: only SINGLE is implemented"); return; }
  const unsigned long long* TD = static_cast<const unsigned long long*>(step_counter);
  if (n_seg == 0) return;
  cudaStream_t s = as_stream(w);
  const float lr = (float)lr_, beta1 = (float)beta1_, beta2 = (float)beta2_, eps = (float)eps_;
  if (clip == 1 && !compute_norms(s, (const float*)grads, seg, n_seg, (float*)norms)) return;
  if (clip == 2 && !norms) { set_error(kBadArgument, "optimizer: clip with given norms but norms is NULL"); return; }
  for (size_t first = 0; first < n_seg; first += kMaxSeg) {
    SegTable tab;
    memset(&tab, 0, sizeof(tab));
    tab.n = (int)((n_seg - first) < (size_t)kMaxSeg ? (n_seg - first) : kMaxSeg);
    tab.first = (int)first;
    for (int j = 0; j < tab.n; ++j) {
      tab.offset[j] = seg[first + j].offset;
      tab.len[j] = seg[first + j].len;
      const float t_f = (float)(t_first + first + j);  // counter advances once per tensor (optim.zig:189)
      tab.lr_t[j] = lr * std::sqrt(1.f - std::pow(beta2, t_f)) / (1.f - std::pow(beta1, t_f));
    }
    const dim3 grid(chunks_for(seg + first, tab.n), tab.n);
    float* P = (float*)params; float* G = (float*)grads; float* M = (float*)m; float* V = (float*)v;
    __nv_bfloat16* cp = (__nv_bfloat16*)bf16_copy;
    const float* NR = (const float*)norms;
    __nv_bfloat16* no_copy = nullptr;
    const dim3 blk(kOThreads);
    if (clip && cp) launch_pdl(adam_kernel<true, true>, grid, blk, 0, s, P, G, M, V, tab, beta1, beta2, eps, NR, (float)max_norm, (float)delta, cp, TD, lr);
    else if (clip) launch_pdl(adam_kernel<true, false>, grid, blk, 0, s, P, G, M, V, tab, beta1, beta2, eps, NR, (float)max_norm, (float)delta, no_copy, TD, lr);
    else if (cp) launch_pdl(adam_kernel<false, true>, grid, blk, 0, s, P, G, M, V, tab, beta1, beta2, eps, (const float*)nullptr, 0.f, 0.f, cp, TD, lr);
    else launch_pdl(adam_kernel<false, false>, grid, blk, 0, s, P, G, M, V, tab, beta1, beta2, eps, (const float*)nullptr, 0.f, 0.f, no_copy, TD, lr);
  }
  if (step_counter && advance_counter) {  // advance the device counter once per tensor, after every update kernel has read it
    launch_pdl(counter_add_kernel, dim3(1), dim3(1), 0, s, static_cast<unsigned long long*>(step_counter), (unsigned long long)n_seg);
  }
}

extern "C" void zg_adam_step(dtype id, StreamWrapper w, void* params, void* grads, void* m, void* v, const zg_segment* seg, len_t n_seg,
                             len_t t_first, double lr, double beta1, double beta2, double eps, int clip, double max_norm, double delta,
                             void* norms, void* bf16_copy, void* step_counter) {
  zg_adam_step_part(id, w, params, grads, m, v, seg, n_seg, t_first, lr, beta1, beta2, eps, clip, max_norm, delta, norms, bf16_copy, step_counter, 1);
}

extern "C" void zg_segment_sumsq(dtype id, StreamWrapper w, const void* x, const zg_segment* seg, len_t n_seg, void* out) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_segment_sumsq: only SINGLE is implemented"); return; }
  if (n_seg == 0) return;
  compute_norms(as_stream(w), (const float*)x, seg, n_seg, (float*)out, 1);
}
