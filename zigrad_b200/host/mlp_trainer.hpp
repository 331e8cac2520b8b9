// MLP training step above the device interface: the reference's MNIST example
// (examples/mnist/src/model.zig:57-112 model and zero_grad, main-simple.zig
// train loop, src/nn/loss.zig softmax cross-entropy, src/nn/optim.zig SGD) as
// the fixed sequence of device ops its autograd issues, with the fusions this
// backend adds: Linear = GEMM + bias (+ReLU) epilogue, dX GEMM + ReLU mask +
// bias-gradient column sums, loss forward+backward (+ last bias gradient) in one
// op, one multi-tensor SGD.  Same layout and op order as zigrad_b200/mlp.py.
#pragma once

#include <vector>

#include "cuda_device.hpp"

namespace zg {

class MlpTrainer {
 public:
  // weights[l]: [dims[l+1], dims[l]] row-major, biases[l]: [dims[l+1]]
  MlpTrainer(CudaDevice& dev, const std::vector<std::size_t>& dims, std::size_t batch, const std::vector<std::vector<float>>& weights,
             const std::vector<std::vector<float>>& biases, double lr, std::size_t loss_div = 0)
      : d_(dev), dims_(dims), B_(batch), L_(dims.size() - 1), lr_(lr), loss_div_(loss_div ? loss_div : batch) {
    std::size_t off = 0;
    for (std::size_t l = 0; l < L_; ++l) {
      segments_.push_back({off, dims_[l + 1] * dims_[l]});
      off += dims_[l + 1] * dims_[l];
      segments_.push_back({off, dims_[l + 1]});
      off += dims_[l + 1];
    }
    n_params_ = off;
    params_ = d_.mem_cache_alloc<float>(off);
    grads_ = d_.mem_cache_alloc<float>(off);
    std::vector<float> flat;
    flat.reserve(off);
    for (std::size_t l = 0; l < L_; ++l) {
      flat.insert(flat.end(), weights[l].begin(), weights[l].end());
      flat.insert(flat.end(), biases[l].begin(), biases[l].end());
    }
    d_.mem_transfer(flat.data(), params_.raw);
    d_.mem_fill(grads_.raw, 0.f);
    // logits rows padded to a multiple of 4 floats: the skinny last-layer GEMMs then meet the 16-byte stride rule of TMA
    const std::size_t C = dims_[L_];
    ld_out_ = (C + 3) / 4 * 4;
    for (std::size_t l = 0; l < L_; ++l) {
      const std::size_t ld = l + 1 < L_ ? dims_[l + 1] : ld_out_;
      ld_.push_back(ld);
      act_.push_back(d_.mem_cache_alloc<float>(B_ * ld));
      dact_.push_back(d_.mem_cache_alloc<float>(B_ * ld));
    }
    d_.mem_fill(act_.back().raw, 0.f);
    d_.mem_fill(dact_.back().raw, 0.f);
    loss_ = d_.mem_cache_alloc<float>(1);
    d_.sync();
  }
  ~MlpTrainer() {
    d_.sync();
    for (auto& a : act_) d_.mem_cache_free(a);
    for (auto& a : dact_) d_.mem_cache_free(a);
    d_.mem_cache_free(params_);
    d_.mem_cache_free(grads_);
    d_.mem_cache_free(loss_);
  }

  Slice<float> W(std::size_t l) { return params_.raw.view(segments_[2 * l].first, segments_[2 * l].second); }
  Slice<float> b(std::size_t l) { return params_.raw.view(segments_[2 * l + 1].first, segments_[2 * l + 1].second); }
  Slice<float> dW(std::size_t l) { return grads_.raw.view(segments_[2 * l].first, segments_[2 * l].second); }
  Slice<float> db(std::size_t l) { return grads_.raw.view(segments_[2 * l + 1].first, segments_[2 * l + 1].second); }

  void forward(Slice<const float> X) {
    d_.mem_fill(grads_.raw, 0.f);  // zero_grad (model.zig:57-62) as one fill of the flat buffer
    Slice<const float> in = X;
    for (std::size_t l = 0; l < L_; ++l) {
      opspec::linear<float> p;
      p.A = in; p.B = W(l); p.C = act_[l].raw;
      p.m = B_; p.n = dims_[l + 1]; p.k = dims_[l];
      p.trans_a = false; p.trans_b = true;
      p.lda = dims_[l]; p.ldb = dims_[l]; p.ldc = ld_[l];
      p.epilogue = l + 1 == L_ ? opspec::Epilogue::bias : opspec::Epilogue::bias_relu;
      p.bias = b(l);
      d_.dispatch(p);
      in = act_[l].raw;
    }
  }
  void loss_and_grad(Slice<const float> onehot) {
    opspec::softmax_ce<float> p;
    p.logits = act_[L_ - 1].raw; p.onehot = onehot;
    p.rows = B_; p.classes = dims_[L_];
    p.loss = loss_.raw; p.grad = dact_[L_ - 1].raw;
    p.loss_div = (double)loss_div_; p.accumulate = false; p.ld = ld_out_;
    p.bias_grad = db(L_ - 1);  // the last layer's bias gradient comes out of the same pass
    d_.dispatch(p);
  }
  void backward(Slice<const float> X) {
    for (std::size_t l = L_; l-- > 0;) {
      const std::size_t K = dims_[l], N = dims_[l + 1];
      Slice<const float> a_in = l == 0 ? X : Slice<const float>(act_[l - 1].raw);
      Slice<const float> dy = dact_[l].raw;
      // dW += dY^T . a_in on the side stream (nothing later in the backward pass reads it)
      d_.branch();
      {
        opspec::linear<float> p;
        p.A = dy; p.B = a_in; p.C = dW(l);
        p.m = N; p.n = K; p.k = B_;
        p.trans_a = true; p.trans_b = false;
        p.lda = ld_[l]; p.ldb = K; p.ldc = K;
        p.beta = 1.f;
        d_.dispatch(p);
      }
      d_.end_branch();
      if (l > 0) {  // dX = dY . W, zero where the previous activation is <= 0; its column sums are db[l-1]
        opspec::linear<float> p;
        p.A = dy; p.B = W(l); p.C = dact_[l - 1].raw;
        p.m = B_; p.n = K; p.k = N;
        p.trans_a = false; p.trans_b = false;
        p.lda = ld_[l]; p.ldb = K; p.ldc = K;
        p.epilogue = opspec::Epilogue::relu_mask;
        p.mask_src = act_[l - 1].raw;
        p.colsum = db(l - 1);
        d_.dispatch(p);
      }
    }
    d_.join();
  }
  void update() {
    opspec::sgd<float> p;
    p.params = params_.raw; p.grads = grads_.raw; p.segments = segments_; p.lr = lr_;
    d_.dispatch(p);
  }
  // True when the last two layers, the loss and their backward pass can run as the one fused op
  bool has_tail() const { return L_ >= 3 && d_.mlp_tail_supported(SINGLE, dims_[L_ - 2], dims_[L_ - 1], dims_[L_]); }
  // forward + loss + backward with opspec::mlp_tail in the middle (same results as forward / loss_and_grad / backward)
  void forward_backward_tail(Slice<const float> X, Slice<const float> onehot) {
    d_.mem_fill(grads_.raw, 0.f);
    Slice<const float> in = X;
    for (std::size_t l = 0; l + 2 < L_; ++l) {
      opspec::linear<float> p;
      p.A = in; p.B = W(l); p.C = act_[l].raw;
      p.m = B_; p.n = dims_[l + 1]; p.k = dims_[l];
      p.trans_a = false; p.trans_b = true;
      p.lda = dims_[l]; p.ldb = dims_[l]; p.ldc = ld_[l];
      p.epilogue = opspec::Epilogue::bias_relu;
      p.bias = b(l);
      d_.dispatch(p);
      in = act_[l].raw;
    }
    {
      opspec::mlp_tail<float> p;
      p.act0 = act_[L_ - 3].raw; p.W1 = W(L_ - 2); p.b1 = b(L_ - 2); p.W2 = W(L_ - 1); p.b2 = b(L_ - 1);
      p.onehot = onehot;
      p.rows = B_; p.h1 = dims_[L_ - 2]; p.h2 = dims_[L_ - 1]; p.classes = dims_[L_];
      p.ld_out = ld_out_; p.loss_div = (double)loss_div_;
      p.act1 = act_[L_ - 2].raw; p.logits = act_[L_ - 1].raw; p.loss = loss_.raw;
      p.dlogits = dact_[L_ - 1].raw; p.dact1 = dact_[L_ - 2].raw; p.dact0 = dact_[L_ - 3].raw;
      p.db2 = db(L_ - 1); p.db1 = db(L_ - 2); p.db0 = db(L_ - 3);
      p.weights_ready = true;  // the kernel in front is the preceding layer's forward GEMM
      d_.dispatch(p);
    }
    auto weight_grad = [&](std::size_t l, int sm_budget) {
      opspec::linear<float> p;
      p.A = dact_[l].raw; p.B = l == 0 ? X : Slice<const float>(act_[l - 1].raw); p.C = dW(l);
      p.m = dims_[l + 1]; p.n = dims_[l]; p.k = B_;
      p.trans_a = true; p.trans_b = false;
      p.lda = ld_[l]; p.ldb = dims_[l]; p.ldc = dims_[l];
      p.beta = 1.f;
      p.sm_budget = sm_budget;
      d_.dispatch(p);
    };
    // three layers: dW0 (main stream) runs beside the two weight gradients of the tail layers (side stream),
    // the SMs shared out by 128 x 128 output tiles
    int first = 0, second = 0;
    if (L_ == 3) {
      const std::size_t t0 = ((dims_[1] + 127) / 128) * ((dims_[0] + 127) / 128), t1 = ((dims_[2] + 127) / 128) * ((dims_[1] + 127) / 128);
      const std::size_t sms = (std::size_t)d_.sm_count();
      const std::size_t f = sms * t0 / (t0 + t1) / t0 * t0;
      if (f > 0 && f < sms) { first = (int)f; second = (int)(sms - f); }
    }
    d_.branch();
    weight_grad(L_ - 2, second);
    weight_grad(L_ - 1, 0);
    d_.end_branch();
    for (std::size_t l = L_ - 2; l-- > 0;) {
      if (l == 0) {
        weight_grad(0, first);
      } else {
        d_.branch();
        weight_grad(l, 0);
        d_.end_branch();
        opspec::linear<float> p;
        p.A = dact_[l].raw; p.B = W(l); p.C = dact_[l - 1].raw;
        p.m = B_; p.n = dims_[l]; p.k = dims_[l + 1];
        p.trans_a = false; p.trans_b = false;
        p.lda = ld_[l]; p.ldb = dims_[l]; p.ldc = dims_[l];
        p.epilogue = opspec::Epilogue::relu_mask;
        p.mask_src = act_[l - 1].raw;
        p.colsum = db(l - 1);
        d_.dispatch(p);
      }
    }
    d_.join();
  }
  void step(Slice<const float> X, Slice<const float> onehot) {
    if (has_tail()) {
      forward_backward_tail(X, onehot);
    } else {
      forward(X);
      loss_and_grad(onehot);
      backward(X);
    }
    update();
  }
  float read_loss() {
    float v = 0.f;
    d_.mem_transfer(Slice<const float>(loss_.raw), &v);
    return v;
  }
  std::vector<float> read_params() {
    std::vector<float> out(n_params_);
    d_.mem_transfer(Slice<const float>(params_.raw), out.data());
    return out;
  }
  std::size_t n_params() const { return n_params_; }

 private:
  CudaDevice& d_;
  std::vector<std::size_t> dims_;
  std::size_t B_, L_;
  double lr_;
  std::size_t loss_div_, n_params_ = 0, ld_out_ = 0;
  opspec::Segments segments_;
  std::vector<std::size_t> ld_;
  DeviceData<float> params_, grads_, loss_;
  std::vector<DeviceData<float>> act_, dact_;
};

}  // namespace zg
