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

// norms[first + j] = ||g_j||_2 for every segment of the table.  grid = (chunks, n);
// chunk partials are folded by the last CTA of each segment in index order.
__global__ void __launch_bounds__(kOThreads) seg_nrm2_kernel(const float* __restrict__ g, const __grid_constant__ SegTable tab,
                                                             float* norms, double* partial, unsigned* counters) {
  __shared__ double sm[32];
  const int seg = blockIdx.y;
  const float* p = g + tab.offset[seg];
  const size_t n = tab.len[seg];
  float acc = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) acc += p[i] * p[i];
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
  if (threadIdx.x == 0) norms[tab.first + seg] = (float)sqrt(s);
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
                                                        const float* __restrict__ norms, float max_norm, float delta) {
  const int seg = blockIdx.y;
  float* p = params + tab.offset[seg];
  float* g = grads + tab.offset[seg];
  const size_t n = tab.len[seg];
  bool on = false;
  float f = 1.f;
  if (CLIP) f = clip_factor(norms, tab.first + seg, max_norm, delta, &on);
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool vec = aligned16(p) && aligned16(g);
  if (vec) {
    const size_t nv = n / 4;
    for (size_t v = tid; v < nv; v += nth) {
      float4 gv = reinterpret_cast<float4*>(g)[v];
      float4 pv = reinterpret_cast<float4*>(p)[v];
      if (CLIP && on) {
        gv.x *= f; gv.y *= f; gv.z *= f; gv.w *= f;
        reinterpret_cast<float4*>(g)[v] = gv;
      }
      pv.x = fmaf(nlr, gv.x, pv.x); pv.y = fmaf(nlr, gv.y, pv.y); pv.z = fmaf(nlr, gv.z, pv.z); pv.w = fmaf(nlr, gv.w, pv.w);
      reinterpret_cast<float4*>(p)[v] = pv;
    }
    for (size_t i = nv * 4 + tid; i < n; i += nth) {
      float gi = g[i];
      if (CLIP && on) { gi *= f; g[i] = gi; }
      p[i] = fmaf(nlr, gi, p[i]);
    }
  } else {
    for (size_t i = tid; i < n; i += nth) {
      float gi = g[i];
      if (CLIP && on) { gi *= f; g[i] = gi; }
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
  const size_t nth = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth) {
    float gi = g[i];
    if (CLIP && on) { gi *= f; g[i] = gi; }
    const float mi = b1 * m[i] + omb1 * gi;
    const float vi = b2 * v[i] + omb2 * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float pi = p[i] - lr_t * mi / (sqrtf(vi) + eps);
    p[i] = pi;
    if (BF16COPY) copy[off + i] = __float2bfloat16_rn(pi);
  }
}

__global__ void counter_add_kernel(unsigned long long* c, unsigned long long inc) { *c += inc; }

static unsigned chunks_for(const zg_segment* seg, size_t n_seg) {
  size_t mx = 0;
  for (size_t j = 0; j < n_seg; ++j) mx = seg[j].len > mx ? seg[j].len : mx;
  size_t c = (mx + (size_t)kOThreads * 8 - 1) / ((size_t)kOThreads * 8);
  const size_t cap = (size_t)sm_count() * 4;
  if (c > cap) c = cap;
  return (unsigned)(c < 1 ? 1 : c);
}

static bool compute_norms(cudaStream_t s, const float* grads, const zg_segment* seg, size_t n_seg, float* norms) {
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
    seg_nrm2_kernel<<<dim3(chunks, tab.n), kOThreads, 0, s>>>(grads, tab, norms, partial, counters);
    if (!ZG_LAUNCH_CHECK()) return false;
  }
  return true;
}

}  // namespace zg

using namespace zg;

extern "C" void zg_sgd_step(dtype id, StreamWrapper w, void* params, void* grads, const zg_segment* seg, len_t n_seg, double lr,
                            int clip, double max_norm, double delta, void* norms) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_sgd_step: only SINGLE is implemented"); return; }
  if (n_seg == 0) return;
  cudaStream_t s = as_stream(w);
  const float nlr = -(float)lr;  // lr cast f64 -> f32, then negated (optim.zig:103)
  if (clip && !compute_norms(s, (const float*)grads, seg, n_seg, (float*)norms)) return;
  for (size_t first = 0; first < n_seg; first += kMaxSeg) {
    SegTable tab;
    memset(&tab, 0, sizeof(tab));
    tab.n = (int)((n_seg - first) < (size_t)kMaxSeg ? (n_seg - first) : kMaxSeg);
    tab.first = (int)first;
    for (int j = 0; j < tab.n; ++j) { tab.offset[j] = seg[first + j].offset; tab.len[j] = seg[first + j].len; }
    const dim3 grid(chunks_for(seg + first, tab.n), tab.n);
    if (clip) sgd_kernel<true><<<grid, kOThreads, 0, s>>>((float*)params, (float*)grads, tab, nlr, (const float*)norms, (float)max_norm, (float)delta);
    else sgd_kernel<false><<<grid, kOThreads, 0, s>>>((float*)params, (float*)grads, tab, nlr, nullptr, 0.f, 0.f);
    ZG_LAUNCH_CHECK();
  }
}

extern "C" void zg_adam_step(dtype id, StreamWrapper w, void* params, void* grads, void* m, void* v, const zg_segment* seg, len_t n_seg,
                             len_t t_first, double lr_, double beta1_, double beta2_, double eps_, int clip, double max_norm, double delta,
                             void* norms, void* bf16_copy, void* step_counter) {
  if (id != SINGLE) { set_error(kUnsupported, "zg_adam_step: only SINGLE is implemented"); return; }
  const unsigned long long* TD = static_cast<const unsigned long long*>(step_counter);
  if (n_seg == 0) return;
  cudaStream_t s = as_stream(w);
  const float lr = (float)lr_, beta1 = (float)beta1_, beta2 = (float)beta2_, eps = (float)eps_;
  if (clip && !compute_norms(s, (const float*)grads, seg, n_seg, (float*)norms)) return;
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
    if (clip && cp) adam_kernel<true, true><<<grid, kOThreads, 0, s>>>(P, G, M, V, tab, beta1, beta2, eps, (const float*)norms, (float)max_norm, (float)delta, cp, TD, lr);
    else if (clip) adam_kernel<true, false><<<grid, kOThreads, 0, s>>>(P, G, M, V, tab, beta1, beta2, eps, (const float*)norms, (float)max_norm, (float)delta, nullptr, TD, lr);
    else if (cp) adam_kernel<false, true><<<grid, kOThreads, 0, s>>>(P, G, M, V, tab, beta1, beta2, eps, nullptr, 0.f, 0.f, cp, TD, lr);
    else adam_kernel<false, false><<<grid, kOThreads, 0, s>>>(P, G, M, V, tab, beta1, beta2, eps, nullptr, 0.f, 0.f, nullptr, TD, lr);
    ZG_LAUNCH_CHECK();
  }
  if (step_counter) {  // advance the device counter once per tensor, after every update kernel has read it
    counter_add_kernel<<<1, 1, 0, s>>>(static_cast<unsigned long long*>(step_counter), (unsigned long long)n_seg);
    ZG_LAUNCH_CHECK();
  }
}
