// C++ host side of the device backend: the counterpart of the reference's
// CudaDevice (src/device/cuda_device.zig) above the C ABI of libamalgamate.so.
// One method per opspec struct, selected by overload through dispatch()
// (DeviceReference.dispatch, src/device/device_reference.zig:15-27); memory
// calls as in device_reference.zig:29-131; CUDA-graph capture as
// cuda_device.zig:558-611.  Every op is asynchronous on the device stream.
// There is no CPU fallback: the constructor throws without a usable GPU.
// Errors: the library records a sticky status instead of exiting; check()
// turns it into a DeviceError (the Zig shim panics with the same message).
#pragma once

#include <array>
#include <cstring>
#include <stdexcept>
#include <string>
#include <type_traits>

#include "../../include/blas_conflux.h"
#include "../../include/cuda_utils.h"
#include "../../include/nn_conflux.h"
#include "../../include/zg_b200.h"
#include "opspec.hpp"

namespace zg {

struct DeviceError : std::runtime_error {
  int code;
  DeviceError(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};
struct DeviceOOM : std::bad_alloc {};

template <typename T>
constexpr dtype dtype_of() {
  static_assert(std::is_same<T, float>::value || std::is_same<T, double>::value, "f32 or f64");
  return std::is_same<T, float>::value ? SINGLE : DOUBLE;
}

// A cached device allocation: the slice plus the block handle that must go
// back to mem_cache_free (DeviceData, src/allocators/device_data.zig:27-40).
template <typename T>
struct DeviceData {
  Slice<T> raw;
  len_t ctx = 0;
};

class CudaDevice;

class ExecutionGraph {
 public:
  explicit ExecutionGraph(CudaDevice* d) : dev_(d) {}
  void open();
  void save();
  void run();
  void free();
  bool empty() const { return wrapper_.ptr == nullptr; }
  std::size_t kernel_count() const { return wrapper_.ptr ? zg_capture_kernel_count(wrapper_) : 0; }

 private:
  CudaDevice* dev_;
  GraphWrapper wrapper_{nullptr};
  bool saved_ = false;
};

class CudaDevice {
 public:
  explicit CudaDevice(unsigned device_number = 0) : capture(this), device_number_(device_number) {
    if (!zg_device_available()) throw DeviceError(1, "CudaDevice: no CUDA device is available (this backend has no CPU fallback)");
    properties_ = init_device(device_number);
    check();
    stream_ = init_stream();
    cublas_ = init_cublas_handle(stream_);
    cache_ = zg_cache_create(device_number, 0);
    check();
  }
  ~CudaDevice() {
    stream_synchronize(stream_);
    capture.free();
    zg_cache_destroy(cache_);
    deinit_cublas_handle(cublas_);
    if (side_.ptr) deinit_stream(side_);
    deinit_stream(stream_);
  }
  CudaDevice(const CudaDevice&) = delete;
  CudaDevice& operator=(const CudaDevice&) = delete;

  static void check() {
    const int code = zg_last_error();
    if (code != 0) {
      const std::string msg = zg_last_error_message();
      zg_clear_error();
      throw DeviceError(code, msg);
    }
  }
  void sync() {
    stream_synchronize(stream_);
    check();
  }
  StreamWrapper stream() const { return stream_; }
  int sm_count() const { return zg_sm_count(); }

  // ------------------------------------------------------------- memory
  template <typename T>
  DeviceData<T> mem_cache_alloc(std::size_t n) {
    const zg_block b = zg_cache_alloc(cache_, (n ? n : 1) * sizeof(T), stream_);
    if (!b.ptr) throw DeviceOOM();
    DeviceData<T> d;
    d.raw = Slice<T>(static_cast<T*>(b.ptr), n);
    d.ctx = b.ctx;
    return d;
  }
  template <typename T>
  void mem_cache_free(DeviceData<T>& d) {
    if (d.raw.ptr) zg_cache_free(cache_, zg_block{d.raw.ptr, d.ctx}, stream_);
    d = DeviceData<T>();
  }
  template <typename T>
  void mem_fill(Slice<T> s, T value) { ::mem_fill(dtype_of<T>(), s.ptr, s.len, &value, cur()); }
  template <typename T>
  void mem_copy(Slice<const T> src, Slice<T> dst) { memcpy_DtoD(dst.ptr, src.ptr, src.len * sizeof(T), stream_); }
  template <typename T>
  void mem_transfer(const T* host_src, Slice<T> dst) { memcpy_HtoD(dst.ptr, host_src, dst.len * sizeof(T), stream_); }
  template <typename T>
  void mem_transfer(Slice<const T> src, T* host_dst) {
    memcpy_DtoH(host_dst, src.ptr, src.len * sizeof(T), stream_);
    sync();
  }
  template <typename T>
  void mem_take(Slice<const T> src, Slice<const std::size_t> idxs, Slice<T> dst) {
    ::mem_take(dtype_of<T>(), src.ptr, src.len, reinterpret_cast<const len_t*>(idxs.ptr), idxs.len, dst.ptr, stream_);
  }

  // --------------------------------------------------- side stream (branches)
  // Ops issued between branch() and end_branch() go to the side stream, ordered
  // after everything issued so far on the main stream; join() makes the main
  // stream wait for them.
  void branch() {
    if (!side_.ptr) side_ = init_stream();
    zg_stream_wait(side_, main());
    in_branch_ = true;
  }
  void end_branch() { in_branch_ = false; }
  void join() {
    if (side_.ptr) zg_stream_wait(main(), side_);
  }

  // ------------------------------------------------------------ dispatch
  template <typename P>
  void dispatch(const P& p) { op(p); }

  template <typename T> void op(const opspec::add<T>& p) { addition(dtype_of<T>(), cur(), p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len); }
  template <typename T> void op(const opspec::sub<T>& p) { subtraction(dtype_of<T>(), cur(), p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len); }
  template <typename T> void op(const opspec::mul<T>& p) { multiplication(dtype_of<T>(), cur(), p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len); }
  template <typename T> void op(const opspec::div<T>& p) { division(dtype_of<T>(), cur(), p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len); }
  template <typename T> void op(const opspec::dot<T>& p) { ::dot(dtype_of<T>(), cublas_, p.x.ptr, p.y.ptr, p.z.ptr, p.x.len); }
  template <typename T> void op(const opspec::axpy<T>& p) { ::axpy(dtype_of<T>(), cublas_, p.x.ptr, p.y.ptr, p.x.len, p.alpha); }
  template <typename T> void op(const opspec::matvec<T>& p) { gemv(dtype_of<T>(), cublas_, p.A.ptr, p.x.ptr, p.y.ptr, p.m, p.n, p.trans_a, p.alpha, p.beta); }
  template <typename T> void op(const opspec::matmul<T>& p) {
    gemm(dtype_of<T>(), cublas_, p.A.ptr, p.B.ptr, p.C.ptr, p.m, p.n, p.k, p.trans_a, p.trans_b, p.lda, p.ldb, p.ldc, p.alpha, p.beta);
  }
  template <typename T> void op(const opspec::bmm_acc<T>& p) {
    zg_bmm(dtype_of<T>(), dtype_of<T>(), cur(), p.A.ptr, p.B.ptr, p.C.ptr, p.A_shape[0], p.B_shape[0], p.C_shape[0], p.C_shape[1],
           p.C_shape[2], p.A_shape[2], p.trans_a, p.trans_b, p.lda, p.ldb, p.ldc, p.alpha, p.beta, ZG_EPI_NONE, nullptr, nullptr, nullptr);
  }
  template <typename T> void op(const opspec::linear<T>& p) {
    if (p.sm_budget > 0) zg_bmm_sm_budget(p.sm_budget);
    zg_bmm(dtype_of<T>(), dtype_of<T>(), cur(), p.A.ptr, p.B.ptr, p.C.ptr, 1, 1, 1, p.m, p.n, p.k, p.trans_a, p.trans_b, p.lda, p.ldb, p.ldc,
           p.alpha, p.beta, static_cast<int>(p.epilogue), p.bias.ptr, p.mask_src.ptr, p.colsum.ptr);
  }
  bool mlp_tail_supported(dtype id, std::size_t h1, std::size_t h2, std::size_t classes) const { return zg_mlp_tail_supported(id, h1, h2, classes) != 0; }
  template <typename T> void op(const opspec::mlp_tail<T>& p) {
    const bool idx = p.label_index.ptr != nullptr;
    zg_mlp_tail_fwd_bwd(dtype_of<T>(), cur(), p.rows, p.h1, p.h2, p.classes, p.act0.ptr, p.W1.ptr, p.b1.ptr, p.W2.ptr, p.b2.ptr,
                        idx ? static_cast<const void*>(p.label_index.ptr) : p.onehot.ptr, idx ? ZG_LABEL_INDEX : ZG_LABEL_ONEHOT, p.ld_out,
                        p.loss_div, p.act1.ptr, p.logits.ptr, p.loss.ptr, p.dlogits.ptr, p.dact1.ptr, p.dact0.ptr, p.db2.ptr, p.db1.ptr,
                        p.db0.ptr, p.weights_ready ? 1 : 0);
  }
  template <typename T> void op(const opspec::sum<T>& p) { reduce_sum(dtype_of<T>(), cublas_, p.x.ptr, p.y.ptr, p.x.len); }
  template <typename T> void op(const opspec::scale<T>& p) { ::scale(dtype_of<T>(), cublas_, p.x.ptr, p.x.len, p.alpha); }
  template <typename T> void op(const opspec::nrm2<T>& p) { ::nrm2(dtype_of<T>(), cublas_, p.x.ptr, p.y.ptr, p.x.len); }
  template <typename T> void op(const opspec::relu_fwd<T>& p) { ::relu_fwd(dtype_of<T>(), cur(), p.x.ptr, p.y.ptr, p.x.len); }
  template <typename T> void op(const opspec::relu_bwd<T>& p) { ::relu_bwd(dtype_of<T>(), cur(), p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len); }
  template <typename T> void op(const opspec::relu_inplace_bwd<T>& p) { zg_relu_inplace_bwd(dtype_of<T>(), cur(), p.x.ptr, p.x_g.ptr, p.x.len); }
  template <typename T> void op(const opspec::clamp_fwd<T>& p) { clamp(dtype_of<T>(), cur(), p.x.ptr, p.y.ptr, p.x.len, p.min, p.max); }
  template <typename T> void op(const opspec::clamp_bwd<T>& p) { zg_clamp_bwd(dtype_of<T>(), cur(), p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.min, p.max); }
  template <typename T> void op(const opspec::exp_fwd<T>& p) { zg_unary_fwd(dtype_of<T>(), cur(), ZG_UN_EXP, p.x.ptr, p.y.ptr, p.x.len, 0.0); }
  template <typename T> void op(const opspec::sqrt_fwd<T>& p) { zg_unary_fwd(dtype_of<T>(), cur(), ZG_UN_SQRT, p.x.ptr, p.y.ptr, p.x.len, 0.0); }
  template <typename T> void op(const opspec::sqrt_fwd_<T>& p) { zg_unary_fwd(dtype_of<T>(), cur(), ZG_UN_SQRT, p.x.ptr, p.x.ptr, p.x.len, 0.0); }
  template <typename T> void op(const opspec::rsqrt_fwd<T>& p) { zg_unary_fwd(dtype_of<T>(), cur(), ZG_UN_RSQRT, p.x.ptr, p.y.ptr, p.x.len, p.eps); }
  template <typename T> void op(const opspec::tanh_fwd<T>& p) { zg_unary_fwd(dtype_of<T>(), cur(), ZG_UN_TANH, p.x.ptr, p.y.ptr, p.x.len, 0.0); }
  template <typename T> void op(const opspec::sigm_fwd<T>& p) { zg_unary_fwd(dtype_of<T>(), cur(), ZG_UN_SIGM, p.x.ptr, p.y.ptr, p.x.len, 0.0); }
  template <typename T> void op(const opspec::pow_fwd<T>& p) { zg_unary_fwd(dtype_of<T>(), cur(), ZG_UN_POW, p.x.ptr, p.y.ptr, p.x.len, p.exp); }
  template <typename T> void op(const opspec::pow_fwd_<T>& p) { zg_unary_fwd(dtype_of<T>(), cur(), ZG_UN_POW, p.x.ptr, p.x.ptr, p.x.len, p.exp); }
  template <typename T> void op(const opspec::exp_bwd<T>& p) { zg_unary_bwd(dtype_of<T>(), cur(), ZG_UN_EXP, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0.0); }
  template <typename T> void op(const opspec::tanh_bwd<T>& p) { zg_unary_bwd(dtype_of<T>(), cur(), ZG_UN_TANH, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0.0); }
  template <typename T> void op(const opspec::sigm_bwd<T>& p) { zg_unary_bwd(dtype_of<T>(), cur(), ZG_UN_SIGM, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0.0); }
  template <typename T> void op(const opspec::sqrt_bwd<T>& p) { zg_unary_bwd(dtype_of<T>(), cur(), ZG_UN_SQRT, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.eps); }
  template <typename T> void op(const opspec::rsqrt_bwd<T>& p) { zg_unary_bwd(dtype_of<T>(), cur(), ZG_UN_RSQRT, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.eps); }
  template <typename T> void op(const opspec::pow_bwd<T>& p) { zg_pow_bwd(dtype_of<T>(), cur(), p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.exp, p.eps); }
  template <typename T> void op(const opspec::tanh_inplace_bwd<T>& p) { zg_unary_inplace_bwd(dtype_of<T>(), cur(), ZG_UN_TANH, p.x.ptr, p.x_g.ptr, p.x.len); }
  template <typename T> void op(const opspec::sigm_inplace_bwd<T>& p) { zg_unary_inplace_bwd(dtype_of<T>(), cur(), ZG_UN_SIGM, p.x.ptr, p.x_g.ptr, p.x.len); }
  template <typename T> void op(const opspec::relu_mask_fwd<T>& p) { zg_relu_mask_fwd(dtype_of<T>(), cur(), p.x.ptr, p.mask.ptr, p.x.len); }
  template <typename T> void op(const opspec::relu_mask_bwd<T>& p) { zg_relu_mask_bwd(dtype_of<T>(), cur(), p.x_g.ptr, p.mask.ptr, p.x_g.len); }
  template <typename T> void op(const opspec::clamp_mask_fwd<T>& p) { zg_clamp_mask_fwd(dtype_of<T>(), cur(), p.x.ptr, p.y.ptr, p.mask.ptr, p.x.len, p.min, p.max); }
  template <typename T> void op(const opspec::clamp_mask_bwd<T>& p) { zg_clamp_mask_bwd(dtype_of<T>(), cur(), p.x_g.ptr, p.y_g.ptr, p.mask.ptr, p.x_g.len); }
  template <typename T> void op(const opspec::scatter_add_2d<T>& p) {
    zg_scatter_add_2d(dtype_of<T>(), cur(), p.src.ptr, reinterpret_cast<const len_t*>(p.indices.ptr), p.indices.len, p.stride, p.dst.ptr);
  }
  template <typename T> void op(const opspec::scatter_add_csr<T>& p) {
    zg_scatter_add_csr(dtype_of<T>(), cur(), p.src.ptr, reinterpret_cast<const len_t*>(p.row_ptr.ptr), p.src.len, p.dst.ptr);
  }
  template <typename T> void op(const opspec::segment_sum_csr<T>& p) {
    zg_segment_sum_csr(dtype_of<T>(), cur(), p.src.ptr, reinterpret_cast<const len_t*>(p.row_offsets.ptr), p.dst.len, p.dst.ptr);
  }
  template <typename T> void op(const opspec::max_fwd<T>& p) { ::max_fwd(dtype_of<T>(), cur(), p.x.ptr, p.y.ptr, p.x.len); }
  template <typename T> void op(const opspec::unbroadcast<T>& p) {
    std::vector<len_t> xs(p.x_shape.begin(), p.x_shape.end()), ys(p.y_shape.begin(), p.y_shape.end());
    zg_unbroadcast(dtype_of<T>(), cur(), p.x.ptr, xs.data(), xs.size(), p.y.ptr, ys.data(), ys.size(), nullptr, p.alpha, p.beta);
  }
  template <typename T> void op(const opspec::sum_along<T>& p) {
    std::vector<len_t> xs(p.x_shape.begin(), p.x_shape.end());
    zg_sum_along(dtype_of<T>(), cur(), p.x.ptr, xs.data(), xs.size(), p.dim, p.y.ptr, p.alpha, p.beta);
  }
  template <typename T> void op(const opspec::max_along<T>& p) {
    std::vector<len_t> xs(p.x_shape.begin(), p.x_shape.end());
    zg_max_along(dtype_of<T>(), cur(), p.x.ptr, xs.data(), xs.size(), p.dim, p.y.ptr);
  }
  template <typename T> void op(const opspec::scatter_add<T>& p) {
    zg_scatter_add(dtype_of<T>(), cur(), p.src.ptr, reinterpret_cast<const len_t*>(p.offsets.ptr), p.src.len, p.dst.ptr);
  }
  template <typename T> void op(const opspec::softmax_ce<T>& p) {
    const bool idx = p.label_index.ptr != nullptr;
    zg_softmax_ce_fwd_bwd(dtype_of<T>(), cur(), p.logits.ptr, idx ? static_cast<const void*>(p.label_index.ptr) : p.onehot.ptr,
                          idx ? ZG_LABEL_INDEX : ZG_LABEL_ONEHOT, p.rows, p.classes, p.ld, p.loss_div > 0 ? p.loss_div : (double)p.rows,
                          p.loss.ptr, p.grad.ptr, p.accumulate ? 1 : 0, nullptr, p.bias_grad.ptr);
  }
  template <typename T> void op(const opspec::smooth_l1<T>& p) {
    zg_smooth_l1_fwd_bwd(dtype_of<T>(), cur(), p.pred.ptr, p.target.ptr, p.pred.len, p.beta, p.loss.ptr, p.grad.ptr);
  }
  template <typename T> void op(const opspec::sgd<T>& p) {
    const std::vector<zg_segment> seg = segments(p.segments);
    zg_sgd_step(dtype_of<T>(), cur(), p.params.ptr, p.grads.ptr, seg.data(), seg.size(), p.lr, p.clip ? 1 : 0, p.max_norm, p.delta, p.norms.ptr,
                p.zero_grads ? 1 : 0);
  }
  template <typename T> void op(const opspec::adam<T>& p) {
    const std::vector<zg_segment> seg = segments(p.segments);
    zg_adam_step_part(dtype_of<T>(), cur(), p.params.ptr, p.grads.ptr, p.m.ptr, p.v.ptr, seg.data(), seg.size(), p.t_first, p.lr, p.beta1,
                      p.beta2, p.eps, p.clip ? 1 : 0, p.max_norm, p.delta, p.norms.ptr, nullptr, p.step_counter.ptr, p.advance_counter ? 1 : 0);
  }

  ExecutionGraph capture;

 private:
  friend class ExecutionGraph;
  StreamWrapper main() const { return stream_; }
  StreamWrapper cur() const { return in_branch_ ? side_ : stream_; }
  static std::vector<zg_segment> segments(const opspec::Segments& s) {
    std::vector<zg_segment> out;
    out.reserve(s.size());
    for (const auto& p : s) out.push_back(zg_segment{p.first, p.second});
    return out;
  }
  unsigned device_number_;
  DevicePropertiesWrapper properties_{nullptr};
  StreamWrapper stream_{nullptr}, side_{nullptr};
  CublasWrapper cublas_{nullptr};
  CacheWrapper cache_{nullptr};
  bool in_branch_ = false;
};

// Library collectives over one communicator per rank (NCCL bound at run time).  Rank 0 makes the
// 128-byte id (Communicator::unique_id) and hands it to the other ranks over any host channel;
// every rank then constructs its Communicator with it.
class Communicator {
 public:
  static std::array<unsigned char, 128> unique_id() {
    std::array<unsigned char, 128> id{};
    zg_nccl_unique_id(id.data());
    CudaDevice::check();
    return id;
  }
  Communicator(const std::array<unsigned char, 128>& id, unsigned rank, unsigned world) : comm_(zg_comm_init_rank(id.data(), rank, world)) {
    CudaDevice::check();
  }
  ~Communicator() { if (comm_.ptr) zg_comm_destroy(comm_); }
  Communicator(const Communicator&) = delete;
  Communicator& operator=(const Communicator&) = delete;
  unsigned rank() const { return zg_comm_rank(comm_); }
  unsigned world() const { return zg_comm_world(comm_); }
  // buf[i] = sum over the ranks of buf[i]
  template <typename T> void allreduce(Slice<T> buf, StreamWrapper s) { zg_allreduce(comm_, buf.ptr, buf.len, dtype_of<T>(), s); }
  // recv[i] = sum over the ranks of send[rank * recv.len + i]
  template <typename T> void reduce_scatter(Slice<const T> send, Slice<T> recv, StreamWrapper s) {
    zg_reduce_scatter(comm_, send.ptr, recv.ptr, recv.len, dtype_of<T>(), s);
  }
  // recv[r * send.len + i] = rank r's send[i]
  template <typename T> void all_gather(Slice<const T> send, Slice<T> recv, StreamWrapper s) {
    zg_all_gather(comm_, send.ptr, recv.ptr, send.len, dtype_of<T>(), s);
  }
  CommWrapper handle() const { return comm_; }

 private:
  CommWrapper comm_{nullptr};
};

inline void ExecutionGraph::open() {
  free();
  dev_->sync();
  wrapper_ = open_capture(dev_->main());
  CudaDevice::check();
  saved_ = false;
}
inline void ExecutionGraph::save() {
  if (wrapper_.ptr && !saved_) {
    save_capture(wrapper_, dev_->main());
    CudaDevice::check();
    saved_ = true;
  }
}
inline void ExecutionGraph::run() {
  if (!wrapper_.ptr) throw DeviceError(2, "UndefinedCapture");
  if (!saved_) throw DeviceError(2, "CaptureInProgress");
  run_capture(wrapper_, dev_->main());
}
inline void ExecutionGraph::free() {
  save();
  if (wrapper_.ptr) {
    stream_synchronize(dev_->main());
    free_capture(wrapper_, dev_->main());
    wrapper_.ptr = nullptr;
  }
}

}  // namespace zg
