// Runs MLP training steps through the C++ host side (zigrad_b200/host) and
// writes the losses and the final parameters, for comparison with the oracle
// by tests/test_gpu_cpp_host.py.
//
//   mlp_step_main <in.bin> <out.bin>
// in.bin : u64 n_layers+1, u64 dims[], u64 batch, u64 steps, u64 use_graph, f64 lr,
//          then per layer W (f32 [out,in]) and b (f32 [out]), then X (f32 [batch,in]), T (f32 one-hot [batch,classes])
// out.bin: f32 loss per step, then f32 params (flat, attach order)
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../zigrad_b200/host/mlp_trainer.hpp"

template <typename T>
static void rd(FILE* f, T* p, size_t n) {
  if (fread(p, sizeof(T), n, f) != n) { fprintf(stderr, "short read\n"); exit(2); }
}

int main(int argc, char** argv) {
  if (argc != 3) { fprintf(stderr, "usage: %s in.bin out.bin\n", argv[0]); return 2; }
  FILE* f = fopen(argv[1], "rb");
  if (!f) { perror("open input"); return 2; }
  uint64_t nd = 0;
  rd(f, &nd, 1);
  std::vector<uint64_t> d64(nd);
  rd(f, d64.data(), nd);
  uint64_t batch = 0, steps = 0, use_graph = 0;
  double lr = 0;
  rd(f, &batch, 1); rd(f, &steps, 1); rd(f, &use_graph, 1); rd(f, &lr, 1);
  std::vector<size_t> dims(d64.begin(), d64.end());
  std::vector<std::vector<float>> Ws, bs;
  for (size_t l = 0; l + 1 < dims.size(); ++l) {
    Ws.emplace_back(dims[l + 1] * dims[l]);
    rd(f, Ws.back().data(), Ws.back().size());
    bs.emplace_back(dims[l + 1]);
    rd(f, bs.back().data(), bs.back().size());
  }
  std::vector<float> X(batch * dims.front()), T(batch * dims.back());
  rd(f, X.data(), X.size());
  rd(f, T.data(), T.size());
  fclose(f);
  try {
    zg::CudaDevice dev(0);
    zg::MlpTrainer tr(dev, dims, batch, Ws, bs, lr);
    auto Xd = dev.mem_cache_alloc<float>(X.size());
    auto Td = dev.mem_cache_alloc<float>(T.size());
    dev.mem_transfer(X.data(), Xd.raw);
    dev.mem_transfer(T.data(), Td.raw);
    std::vector<float> losses;
    if (use_graph) {
      tr.step(Xd.raw, Td.raw);  // eager first step: library workspaces grow here
      losses.push_back(tr.read_loss());
      dev.capture.open();
      tr.step(Xd.raw, Td.raw);
      dev.capture.save();
      for (uint64_t s = 1; s < steps; ++s) {
        dev.capture.run();
        losses.push_back(tr.read_loss());
      }
      fprintf(stderr, "graph: %zu kernels per step\n", dev.capture.kernel_count());
      dev.capture.free();
    } else {
      for (uint64_t s = 0; s < steps; ++s) {
        tr.step(Xd.raw, Td.raw);
        losses.push_back(tr.read_loss());
      }
    }
    dev.sync();
    const std::vector<float> params = tr.read_params();
    FILE* o = fopen(argv[2], "wb");
    if (!o) { perror("open output"); return 2; }
    fwrite(losses.data(), sizeof(float), losses.size(), o);
    fwrite(params.data(), sizeof(float), params.size(), o);
    fclose(o);
    dev.mem_cache_free(Xd);
    dev.mem_cache_free(Td);
  } catch (const zg::DeviceError& e) {
    fprintf(stderr, "DeviceError %d: %s\n", e.code, e.what());
    return 1;
  }
  return 0;
}
