// Operation parameter structs of the device interface, C++ mirror of
// src/device/opspec.zig: one struct per op with the same field names; the
// struct's `name` is the method DeviceReference.dispatch selects
// (src/device/device_reference.zig:15-27).  Slices are (pointer, length)
// pairs over device memory.  The last section holds the ops this backend adds
// (the reference runs them as host loops): softmax_ce, smooth_l1, sgd, adam,
// linear.
#pragma once

#include <cstddef>
#include <cstdint>
#include <utility>
#include <vector>

namespace zg {

template <typename T>
struct Slice {
  T* ptr = nullptr;
  std::size_t len = 0;
  Slice() = default;
  Slice(T* p, std::size_t n) : ptr(p), len(n) {}
  Slice view(std::size_t offset, std::size_t n) const { return Slice(ptr + offset, n); }
  operator Slice<const T>() const { return Slice<const T>(ptr, len); }
};

using Shape = std::vector<std::size_t>;

namespace opspec {

// ---- binary element-wise (opspec.zig:19-57)
#define ZG_BINARY_OP(NAME)                              \
  template <typename T>                                 \
  struct NAME {                                         \
    static constexpr const char* name = #NAME;          \
    Slice<const T> x, y;                                \
    Slice<T> z;                                         \
  };
ZG_BINARY_OP(add)
ZG_BINARY_OP(sub)
ZG_BINARY_OP(mul)
ZG_BINARY_OP(div)
#undef ZG_BINARY_OP

// ---- linear algebra (opspec.zig:66-203)
template <typename T>
struct dot {
  static constexpr const char* name = "dot";
  Slice<const T> x, y;
  Slice<T> z;
};
template <typename T>
struct axpy {
  static constexpr const char* name = "axpy";
  Slice<const T> x;
  Slice<T> y;
  const T* alpha;  // host scalar, as SGD passes it (src/nn/optim.zig:114-118)
};
template <typename T>
struct matvec {
  static constexpr const char* name = "matvec";
  Slice<const T> A, x;
  Slice<T> y;
  std::size_t m, n;
  bool trans_a;
  T alpha, beta;
};
template <typename T>
struct matmul {
  static constexpr const char* name = "matmul";
  Slice<const T> A, B;
  Slice<T> C;
  std::size_t m, n, k;
  bool trans_a, trans_b;
  std::size_t lda, ldb, ldc;
  T alpha, beta;
};
template <typename T>
struct bmm_acc {
  static constexpr const char* name = "bmm_acc";
  Slice<const T> A, B;
  Slice<T> C;
  Shape A_shape, B_shape, C_shape;  // (batch, rows, cols) of op(A), op(B), C
  bool trans_a, trans_b;
  std::size_t lda, ldb, ldc;
  T alpha, beta;
};
template <typename T>
struct sum {
  static constexpr const char* name = "sum";
  Slice<const T> x;
  Slice<T> y;
};
template <typename T>
struct scale {
  static constexpr const char* name = "scale";
  Slice<T> x;
  T alpha;
};
template <typename T>
struct nrm2 {
  static constexpr const char* name = "nrm2";
  Slice<const T> x;
  Slice<T> y;
};
template <typename T>
struct clip_nrm2 {
  static constexpr const char* name = "clip_nrm2";
  Slice<T> x;
  T max_norm, delta;
};

// ---- non-linear (opspec.zig:205-455)
template <typename T>
struct relu_fwd {
  static constexpr const char* name = "relu_fwd";
  Slice<const T> x;
  Slice<T> y;
};
template <typename T>
struct relu_bwd {
  static constexpr const char* name = "relu_bwd";
  Slice<const T> x;
  Slice<T> x_g;
  Slice<const T> y_g;
};
template <typename T>
struct relu_inplace_bwd {
  static constexpr const char* name = "relu_inplace_bwd";
  Slice<const T> x;
  Slice<T> x_g;
};
template <typename T>
struct clamp_fwd {
  static constexpr const char* name = "clamp_fwd";
  Slice<const T> x;
  Slice<T> y;
  T min, max;
};
template <typename T>
struct clamp_bwd {
  static constexpr const char* name = "clamp_bwd";
  Slice<const T> x;
  Slice<T> x_g;
  Slice<const T> y_g;
  T min, max;
};
template <typename T>
struct max_fwd {
  static constexpr const char* name = "max_fwd";
  Slice<const T> x;
  Slice<T> y;
};

// unary maps and their backward passes (opspec.zig:205-393)
#define ZG_UNARY_FWD(NAME)                     \
  template <typename T>                        \
  struct NAME {                                \
    static constexpr const char* name = #NAME; \
    Slice<const T> x;                          \
    Slice<T> y;                                \
  };
ZG_UNARY_FWD(exp_fwd)
ZG_UNARY_FWD(sqrt_fwd)
ZG_UNARY_FWD(tanh_fwd)
ZG_UNARY_FWD(sigm_fwd)
#undef ZG_UNARY_FWD
#define ZG_UNARY_BWD_Y(NAME)                   \
  template <typename T>                        \
  struct NAME {                                \
    static constexpr const char* name = #NAME; \
    Slice<T> x_g;                              \
    Slice<const T> y, y_g;                     \
  };
ZG_UNARY_BWD_Y(exp_bwd)
ZG_UNARY_BWD_Y(tanh_bwd)
ZG_UNARY_BWD_Y(sigm_bwd)
#undef ZG_UNARY_BWD_Y
#define ZG_INPLACE_BWD(NAME)                   \
  template <typename T>                        \
  struct NAME {                                \
    static constexpr const char* name = #NAME; \
    Slice<const T> x;                          \
    Slice<T> x_g;                              \
  };
ZG_INPLACE_BWD(tanh_inplace_bwd)
ZG_INPLACE_BWD(sigm_inplace_bwd)
#undef ZG_INPLACE_BWD
template <typename T>
struct rsqrt_fwd {
  static constexpr const char* name = "rsqrt_fwd";
  Slice<const T> x;
  Slice<T> y;
  float eps;
};
template <typename T>
struct sqrt_bwd {
  static constexpr const char* name = "sqrt_bwd";
  Slice<const T> x;
  Slice<T> x_g;
  Slice<const T> y_g;
  float eps;
};
template <typename T>
struct rsqrt_bwd {
  static constexpr const char* name = "rsqrt_bwd";
  Slice<const T> x;
  Slice<T> x_g;
  Slice<const T> y_g;
  float eps;
};
template <typename T>
struct sqrt_fwd_ {
  static constexpr const char* name = "sqrt_fwd_";
  Slice<T> x;
};
template <typename T>
struct pow_fwd {
  static constexpr const char* name = "pow_fwd";
  Slice<const T> x;
  T exp;
  Slice<T> y;
};
template <typename T>
struct pow_fwd_ {
  static constexpr const char* name = "pow_fwd_";
  Slice<T> x;
  T exp;
};
template <typename T>
struct pow_bwd {
  static constexpr const char* name = "pow_bwd";
  Slice<const T> x;
  Slice<T> x_g;
  T exp;
  Slice<const T> y_g;
  float eps;
};
// byte-mask activations (opspec.zig:438-475): one bit per element, ceil(n/8) mask bytes
template <typename T>
struct clamp_mask_fwd {
  static constexpr const char* name = "clamp_mask_fwd";
  Slice<const T> x;
  Slice<T> y;
  T min, max;
  Slice<unsigned char> mask;
};
template <typename T>
struct clamp_mask_bwd {
  static constexpr const char* name = "clamp_mask_bwd";
  Slice<T> x_g;
  Slice<const T> y_g;
  Slice<unsigned char> mask;
};
template <typename T>
struct relu_mask_fwd {
  static constexpr const char* name = "relu_mask_fwd";
  Slice<T> x;
  Slice<unsigned char> mask;
};
template <typename T>
struct relu_mask_bwd {
  static constexpr const char* name = "relu_mask_bwd";
  Slice<T> x_g;
  Slice<unsigned char> mask;
};

// ---- shape-aware reductions (opspec.zig:477-531)
template <typename T>
struct unbroadcast {
  static constexpr const char* name = "unbroadcast";
  Slice<const T> x;
  Shape x_shape;
  Slice<T> y;
  Shape y_shape;
  Slice<T> scratch;  // kept for interface compatibility; the device uses its own workspace
  T alpha = T(1), beta = T(0);
};
template <typename T>
struct sum_along {
  static constexpr const char* name = "sum_along";
  Slice<const T> x;
  Shape x_shape;
  Slice<T> y;
  std::size_t dim;
  T alpha = T(1), beta = T(0);
};
template <typename T>
struct max_along {
  static constexpr const char* name = "max_along";
  Slice<const T> x;
  Shape x_shape;
  Slice<T> y;
  std::size_t dim;
};

// ---- index ops (opspec.zig:533-659)
template <typename T>
struct scatter_add {
  static constexpr const char* name = "scatter_add";
  Slice<const T> src;
  Slice<const std::size_t> offsets;
  Slice<T> dst;
};

template <typename T>
struct scatter_add_2d {
  static constexpr const char* name = "scatter_add_2d";
  Slice<const T> src;                  // [n_blocks, stride]
  Slice<const std::size_t> indices;    // [n_blocks]
  Slice<T> dst;                        // [n_segments, stride]
  std::size_t stride;
};
template <typename T>
struct scatter_add_csr {
  static constexpr const char* name = "scatter_add_csr";
  Slice<const T> src;                  // [n_segments]
  Slice<const std::size_t> row_ptr;    // [n_segments + 1]
  Slice<T> dst;                        // [total_elements]
};
template <typename T>
struct segment_sum_csr {
  static constexpr const char* name = "segment_sum_csr";
  Slice<const T> src;                    // [total_elems]
  Slice<const std::size_t> row_offsets;  // [n_segments + 1]
  Slice<T> dst;                          // [n_segments]
};

// ---------------------------------------------------------------------------
// ops added by this backend (host loops in the reference)
// ---------------------------------------------------------------------------
enum class Epilogue { none = 0, bias = 1, bias_relu = 2, relu_mask = 3 };

// Linear layer GEMM with a fused epilogue: C = epi(alpha op(A) op(B) + beta C)
// (bmm_acc followed by bias.add_ / relu_ / relu_inplace_bwd in the reference).
template <typename T>
struct linear {
  static constexpr const char* name = "linear";
  Slice<const T> A, B;
  Slice<T> C;
  std::size_t m, n, k;
  bool trans_a, trans_b;
  std::size_t lda, ldb, ldc;
  T alpha = T(1), beta = T(0);
  Epilogue epilogue = Epilogue::none;
  Slice<const float> bias;      // [n]
  Slice<const T> mask_src;      // C's shape
  Slice<float> colsum;          // [n], optional: column sums of the stored values are added
  int sm_budget = 0;            // > 0: size the split-K grid for this many SMs (GEMMs side by side on parallel streams share them)
};

// The last two Linear layers of an MLP, their softmax cross-entropy and the backward pass down to the
// gradient of the layer in front of them, as one device op (zg_mlp_tail_fwd_bwd): the op sequence of
// examples/mnist/src/model.zig:34-55 + src/nn/loss.zig:130-171 + the BmmAccBwd / relu backward calls of
// src/ndtensor.zig:1092-1136 for those two layers.  The three bias gradients are ADDED into db2/db1/db0.
template <typename T>
struct mlp_tail {
  static constexpr const char* name = "mlp_tail";
  Slice<const T> act0;                      // [rows, h1]
  Slice<const T> W1, b1;                    // [h2, h1], [h2]
  Slice<const T> W2, b2;                    // [classes, h2], [classes]
  Slice<const T> onehot;                    // [rows, classes] probability rows, or
  Slice<const std::size_t> label_index;     // [rows] class indices (exactly one of the two is set)
  std::size_t rows, h1, h2, classes;
  std::size_t ld_out;                       // row stride of logits / dlogits
  double loss_div;
  Slice<T> act1, logits, loss, dlogits, dact1, dact0;
  Slice<float> db2, db1, db0;
  bool weights_ready = false;               // the kernel launched just before does not write W1/b1/W2/b2
};

// src/nn/loss.zig:130-215 as one device op
template <typename T>
struct softmax_ce {
  static constexpr const char* name = "softmax_ce";
  Slice<const T> logits;
  Slice<const T> onehot;                    // [rows, C] probability rows, or
  Slice<const std::size_t> label_index;     // [rows] class indices (exactly one of the two is set)
  std::size_t rows, classes;
  Slice<T> loss;                            // one element
  Slice<T> grad;                            // optional
  double loss_div = 0;                      // 0 = rows
  bool accumulate = true;
  std::size_t ld = 0;                       // row stride of logits / grad (0 = classes)
  Slice<float> bias_grad;                   // optional [classes]
};

// src/nn/loss.zig:259-305
template <typename T>
struct smooth_l1 {
  static constexpr const char* name = "smooth_l1";
  Slice<const T> pred, target;
  T beta;
  Slice<T> loss;
  Slice<T> grad;
};

using Segments = std::vector<std::pair<std::size_t, std::size_t>>;  // (offset, length) per tensor, attach order

// SGD.update over a flat parameter set (src/nn/optim.zig:100-122)
template <typename T>
struct sgd {
  static constexpr const char* name = "sgd";
  Slice<T> params, grads;
  Segments segments;
  double lr;
  bool clip = false;
  double max_norm = 10.0, delta = 1e-6;
  Slice<float> norms;  // scratch, one per tensor (clip only)
  bool zero_grads = false;  // also clear the applied gradients (the next step's zero_grad)
};

// Adam.update over a flat parameter set (src/nn/optim.zig:177-234)
template <typename T>
struct adam {
  static constexpr const char* name = "adam";
  Slice<T> params, grads, m, v;
  Segments segments;
  std::size_t t_first;
  double lr, beta1 = 0.9, beta2 = 0.999, eps = 1e-8;
  bool clip = false;
  double max_norm = 10.0, delta = 1e-6;
  Slice<float> norms;
  Slice<std::uint64_t> step_counter;  // optional device counter (graph replay)
  bool advance_counter = true;        // false: read step_counter without advancing it (one step as several calls over parts of the model)
};

}  // namespace opspec
}  // namespace zg
