// Numerics of the C++ frontend's fused sm_100a path against its own libtorch formulation: every op of
// itb/ops.h runs once on cuda:0 under bf16 autocast and once on the CPU in fp32 on the same values;
// outputs and gradients are compared with a bf16-sized tolerance.  Needs the CUDA build
// (python examples/cpp/build.py --cuda --src examples/cpp/check_fused.cc --out <exe>) and a B200.
// Prints one line per op and exits 0 when all agree and no bounded wait gave up.
#include <cstdio>

#include "itb/itb.h"

using itb::Tensor;

static int g_bad = 0;
static void report(const char* what, const Tensor& got, const Tensor& want, double tol) {
  Tensor g = got.detach().to(torch::kCPU, torch::kFloat32), w = want.detach().to(torch::kCPU, torch::kFloat32);
  double err = (g - w).abs().max().item<double>(), scale = std::max(1e-6, w.abs().max().item<double>());
  bool ok = g.sizes() == w.sizes() && err <= tol * scale && !torch::isnan(g).any().item<bool>();
  std::printf("%-28s max|diff| %.3e of scale %.3e  %s\n", what, err, scale, ok ? "ok" : "MISMATCH");
  if (!ok) ++g_bad;
}
static Tensor leaf(const Tensor& t, torch::Device d) { return t.detach().to(d).clone().set_requires_grad(true); }

int main() {
#ifndef ITB_WITH_CUDA
  std::printf("built without ITB_WITH_CUDA: nothing to check\n");
  return 2;
#else
  torch::manual_seed(0);
  torch::Device gpu(torch::kCUDA, 0), cpu(torch::kCPU);
  const double tol = 3e-2;   // bf16 operands, fp32 accumulation
  auto both = [&](auto&& fn, const std::vector<Tensor>& inputs, const char* name) {
    std::vector<Tensor> a, b;
    for (auto& t : inputs) {
      bool fl = t.is_floating_point();
      a.push_back(fl ? leaf(t, gpu) : t.to(gpu));
      b.push_back(fl ? leaf(t, cpu) : t);
    }
    Tensor ya, yb;
    {
      itb::AutocastGuard ac(torch::kBFloat16);
      ya = fn(a);
    }
    yb = fn(b);
    report(name, ya, yb, tol);
    Tensor go = torch::randn(yb.sizes());
    ya.backward(go.to(gpu).to(ya.scalar_type()));
    yb.backward(go);
    for (size_t i = 0; i < inputs.size(); ++i)
      if (a[i].requires_grad() && b[i].grad().defined()) {
        std::string n = std::string(name) + " grad " + std::to_string(i);
        TORCH_CHECK(a[i].grad().defined(), n, " is missing on the GPU");
        report(n.c_str(), a[i].grad(), b[i].grad(), tol);
      }
  };
  const int64_t M = 512, K = 256, N = 384;
  Tensor x = torch::randn({2, M / 2, K}) * 0.5, w = torch::randn({N, K}) * 0.05, bias = torch::randn({N}) * 0.1;
  Tensor res = torch::randn({2, M / 2, N}) * 0.5;
  both([](auto& v) { return itb::ops::linear(v[0], v[1], v[2]); }, {x, w, bias}, "linear");
  both([](auto& v) { return itb::ops::linear(v[0], v[1], v[2], c10::nullopt, true); }, {x, w, bias}, "linear+gelu");
  both([](auto& v) { return itb::ops::linear(v[0], v[1], v[2], v[3]); }, {x, w, bias, res}, "linear+residual");
  Tensor g1 = torch::rand({K}) + 0.5, b1 = torch::randn({K}) * 0.1;
  both([](auto& v) { return itb::ops::layernorm(v[0], v[1], v[2], 1e-5); }, {x, g1, b1}, "layernorm");
  both([](auto& v) { return itb::ops::rmsnorm(v[0], v[1], 1e-5); }, {x, g1}, "rmsnorm");
  both([](auto& v) { return itb::ops::gelu(v[0]); }, {x}, "gelu");
  both([](auto& v) { return itb::ops::swiglu(v[0], v[1]); }, {x, x * 0.7 + 0.1}, "swiglu");
  for (int64_t D : {64, 128}) {
    const int64_t B = 2, T = 256, H = 4, KV = 2;
    Tensor qkv = torch::randn({B, T, (H + 2 * KV) * D}) * 0.5;
    Tensor freqs = itb::ops::precompute_freqs_cis(D, 2 * T, 500000.0);
    std::string n = "attention D=" + std::to_string(D);
    both([&](auto& v) { return itb::ops::attention_packed(v[0], H, KV, D, c10::nullopt, 0, true); }, {qkv}, n.c_str());
    n += " rope";
    both([&](auto& v) { return itb::ops::attention_packed(v[0], H, KV, D, freqs.to(v[0].device()), 0, true); }, {qkv}, n.c_str());
  }
  Tensor idx = torch::randint(0, 1000, {4, 64}, torch::kInt64), wte = torch::randn({1000, K}) * 0.1, wpe = torch::randn({128, K}) * 0.1;
  both([](auto& v) { return itb::ops::embedding(v[0], v[1], v[2], 0); }, {idx, wte, wpe}, "embedding");
  Tensor logits = torch::randn({256, 1000}), tgt = torch::randint(0, 1000, {256}, torch::kInt64);
  both([](auto& v) { return itb::ops::cross_entropy(v[0] * 1.0, v[1]); }, {logits, tgt}, "cross_entropy");
  int64_t status = itb::ops::fused::kernel_status();
  std::printf("kernel status word: %lld\n", (long long)status);
  return g_bad == 0 && status == 0 ? 0 : 1;
#endif
}
