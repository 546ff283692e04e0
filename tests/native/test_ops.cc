// Device-parameterised numerics of the C++ frontend's functional ops (itb/ops.h): every case runs on
// the CPU (libtorch formulation, the oracle) and, in the CUDA pass, on cuda:0 where the fused sm_100a
// kernels take over under bf16 autocast.  Values are compared with closed forms or with a float64
// restatement of the op; gradients with autograd through that restatement.  The reference's
// per-op suites (tests/autograd/test_autograd_*_forward.cc / _backward.cc) mostly assert shapes; these
// assert numbers.
#define ITB_TEST_WITH_TORCH
#include "itb_test.h"

#include "itb/itb.h"

using itb::Tensor;
using itbtest::device;

namespace {

double rel_err(const Tensor& got, const Tensor& want) {
  Tensor g = got.detach().to(torch::kCPU, torch::kFloat64), w = want.detach().to(torch::kCPU, torch::kFloat64);
  return ((g - w).norm() / (w.norm() + 1e-12)).item<double>();
}
// bf16 autocast on the GPU, plain fp32 on the CPU: the tolerance that goes with it
double tol() { return itbtest::current_device() == itbtest::Dev::kCUDA ? 2e-2 : 1e-5; }
Tensor leaf(const Tensor& t) { return t.detach().to(device()).clone().set_requires_grad(true); }
Tensor leaf64(const Tensor& t) { return t.detach().to(torch::kFloat64).clone().set_requires_grad(true); }

struct MaybeAutocast {
  std::unique_ptr<itb::AutocastGuard> g;
  MaybeAutocast() {
    if (itbtest::current_device() == itbtest::Dev::kCUDA) g = std::make_unique<itb::AutocastGuard>(torch::kBFloat16);
  }
};

}  // namespace

ITB_TEST_P(Ops, LinearForwardBackward) {
  torch::manual_seed(1);
  Tensor x = torch::randn({2, 64, 128}) * 0.5, w = torch::randn({192, 128}) * 0.05, b = torch::randn({192}) * 0.1;
  Tensor xd = leaf(x), wd = leaf(w), bd = leaf(b);
  Tensor y;
  {
    MaybeAutocast ac;
    y = itb::ops::linear(xd, wd, bd);
  }
  Tensor x6 = leaf64(x), w6 = leaf64(w), b6 = leaf64(b);
  Tensor y6 = torch::matmul(x6, w6.t()) + b6;
  EXPECT(y.sizes() == torch::IntArrayRef({2, 64, 192}));
  EXPECT(rel_err(y, y6) < tol());
  Tensor go = torch::randn({2, 64, 192});
  y.backward(go.to(device()).to(y.scalar_type()));
  y6.backward(go.to(torch::kFloat64));
  EXPECT(rel_err(xd.grad(), x6.grad()) < tol());
  EXPECT(rel_err(wd.grad(), w6.grad()) < tol());
  EXPECT(rel_err(bd.grad(), b6.grad()) < tol());
}

ITB_TEST_P(Ops, LinearGeluAndResidualEpilogues) {
  torch::manual_seed(2);
  Tensor x = torch::randn({128, 64}) * 0.5, w = torch::randn({64, 64}) * 0.1, r = torch::randn({128, 64});
  Tensor x6 = x.to(torch::kFloat64), w6 = w.to(torch::kFloat64);
  Tensor h = torch::matmul(x6, w6.t());
  Tensor gelu6 = 0.5 * h * (1.0 + torch::tanh(0.7978845608028654 * (h + 0.044715 * h.pow(3))));
  MaybeAutocast ac;
  Tensor yg = itb::ops::linear(x.to(device()), w.to(device()), c10::nullopt, c10::nullopt, true);
  EXPECT(rel_err(yg, gelu6) < tol());
  Tensor rd = itbtest::current_device() == itbtest::Dev::kCUDA ? r.to(device()).to(torch::kBFloat16) : r;
  Tensor yr = itb::ops::linear(x.to(device()), w.to(device()), c10::nullopt, rd);
  EXPECT(rel_err(yr, h + r.to(torch::kFloat64)) < tol());
}

ITB_TEST_P(Ops, LayerNormMatchesTwoPassVariance) {
  torch::manual_seed(3);
  Tensor x = torch::randn({4, 33, 256}) * 2 + 0.5, g = torch::rand({256}) + 0.5, b = torch::randn({256}) * 0.1;
  Tensor xd = leaf(x), gd = leaf(g), bd = leaf(b);
  Tensor y = itb::ops::layernorm(xd, gd, bd, 1e-5);
  Tensor x6 = leaf64(x), g6 = leaf64(g), b6 = leaf64(b);
  Tensor mu = x6.mean(-1, true), var = (x6 - mu).pow(2).mean(-1, true);   // E[(x - mean)^2], not E[x^2] - mean^2
  Tensor y6 = (x6 - mu) * torch::rsqrt(var + 1e-5) * g6 + b6;
  EXPECT(rel_err(y, y6) < 1e-4);
  Tensor go = torch::randn(x.sizes());
  y.backward(go.to(device()));
  y6.backward(go.to(torch::kFloat64));
  EXPECT(rel_err(xd.grad(), x6.grad()) < 1e-4);
  EXPECT(rel_err(gd.grad(), g6.grad()) < 1e-4 && rel_err(bd.grad(), b6.grad()) < 1e-4);
}

ITB_TEST_P(Ops, RMSNormAndWideRows) {
  torch::manual_seed(4);
  for (int64_t C : {64, 2048, 4096}) {
    Tensor x = torch::randn({17, C}), g = torch::rand({C}) + 0.5;
    Tensor xd = leaf(x), gd = leaf(g);
    Tensor y = itb::ops::rmsnorm(xd, gd, 1e-6);
    Tensor x6 = leaf64(x), g6 = leaf64(g);
    Tensor y6 = x6 * torch::rsqrt(x6.pow(2).mean(-1, true) + 1e-6) * g6;
    EXPECT(rel_err(y, y6) < 1e-4);
    Tensor go = torch::randn(x.sizes());
    y.backward(go.to(device()));
    y6.backward(go.to(torch::kFloat64));
    EXPECT(rel_err(xd.grad(), x6.grad()) < 1e-4 && rel_err(gd.grad(), g6.grad()) < 1e-4);
  }
}

ITB_TEST_P(Ops, ActivationsGateOrder) {
  // NewGELU is the tanh approximation; "SwiGLU" multiplies the FIRST projection by silu of the SECOND
  // (reference mlp.cc:84-90), which fixes the llm.c weight mapping.
  torch::manual_seed(5);
  Tensor a = torch::randn({9, 64}), b = torch::randn({9, 64});
  Tensor s = itb::ops::swiglu(a.to(device()), b.to(device()));
  EXPECT(rel_err(s, a.to(torch::kFloat64) * (b.to(torch::kFloat64) * torch::sigmoid(b.to(torch::kFloat64)))) < 1e-5);
  Tensor ge = itb::ops::gelu(a.to(device()));
  EXPECT(rel_err(ge, torch::gelu(a.to(torch::kFloat64), "tanh")) < 1e-3);
}

ITB_TEST_P(Ops, RotaryTableAndRotation) {
  Tensor f = itb::ops::precompute_freqs_cis(64, 128, 500000.0);
  EXPECT(f.sizes() == torch::IntArrayRef({128, 32, 2}));             // [T, D/2, (cos, sin)]
  EXPECT_NEAR(f[0][0][0].item<double>(), 1.0, 1e-6);
  EXPECT_NEAR(f[0][0][1].item<double>(), 0.0, 1e-6);
  EXPECT_NEAR(f[3][0][1].item<double>(), std::sin(3.0), 1e-5);        // pair 0 turns by one radian per position
  // interleaved (even, odd) pairs rotate; norms are preserved
  Tensor x = torch::randn({1, 8, 2, 64});
  Tensor y = itb::ops::apply_rope(x.to(device()), f.to(device()));
  EXPECT(rel_err(y.pow(2).sum(-1), x.pow(2).sum(-1)) < 1e-5);
  EXPECT(rel_err(y.select(1, 0), x.select(1, 0)) < 1e-6);             // position 0 is the identity
}

ITB_TEST_P(Ops, CausalAttentionWithGroupedHeads) {
  torch::manual_seed(6);
  const int64_t B = 2, T = 128, H = 4, KV = 2, D = 64;
  Tensor qkv = torch::randn({B, T, (H + 2 * KV) * D}) * 0.5;
  Tensor out;
  {
    MaybeAutocast ac;
    Tensor in = itbtest::current_device() == itbtest::Dev::kCUDA ? qkv.to(device()).to(torch::kBFloat16) : qkv;
    out = itb::ops::attention_packed(in, H, KV, D, c10::nullopt, 0, true);
  }
  // float64 restatement: head h reads key/value head h / (H / KV); position t sees positions <= t
  Tensor q = qkv.slice(2, 0, H * D).reshape({B, T, H, D}).to(torch::kFloat64);
  Tensor k = qkv.slice(2, H * D, (H + KV) * D).reshape({B, T, KV, D}).to(torch::kFloat64);
  Tensor v = qkv.slice(2, (H + KV) * D).reshape({B, T, KV, D}).to(torch::kFloat64);
  k = k.repeat_interleave(H / KV, 2);
  v = v.repeat_interleave(H / KV, 2);
  Tensor sc = torch::einsum("bthd,bshd->bhts", {q, k}) / std::sqrt(static_cast<double>(D));
  Tensor mask = torch::ones({T, T}, torch::kBool).tril();
  sc = sc.masked_fill(~mask, -1e30);
  Tensor want = torch::einsum("bhts,bshd->bthd", {torch::softmax(sc, -1), v}).reshape({B, T, H * D});
  EXPECT(out.sizes() == torch::IntArrayRef({B, T, H * D}));
  EXPECT(rel_err(out, want) < tol());
}

ITB_TEST_P(Ops, EmbeddingWithPositionsAndItsGradient) {
  torch::manual_seed(7);
  Tensor idx = torch::randint(0, 50, {2, 16}, torch::kInt64);
  idx[0][3] = idx[0][5];                                              // a repeated id accumulates
  Tensor wte = torch::randn({50, 64}), wpe = torch::randn({32, 64});
  Tensor wd = leaf(wte), pd = leaf(wpe);
  Tensor out = itb::ops::embedding(idx.to(device()), wd, pd, 0);
  Tensor want = wte.index_select(0, idx.reshape({-1})).reshape({2, 16, 64}) + wpe.slice(0, 0, 16);
  EXPECT(rel_err(out, want) < 1e-6);
  out.sum().backward();
  Tensor counts = torch::bincount(idx.reshape({-1}), {}, 50).to(torch::kFloat32);
  EXPECT(rel_err(wd.grad().sum(1), counts * 64) < 1e-6);
  EXPECT(rel_err(pd.grad().slice(0, 0, 16), torch::full({16, 64}, 2.0)) < 1e-6);
  EXPECT(pd.grad().slice(0, 16).abs().max().item<double>() == 0.0);
}

ITB_TEST_P(Ops, CrossEntropyIsTheMeanOverRows) {
  torch::manual_seed(8);
  Tensor logits = torch::randn({48, 1000}), tgt = torch::randint(0, 1000, {48}, torch::kInt64);
  Tensor ld = leaf(logits);
  Tensor loss = itb::ops::cross_entropy(ld * 1.0, tgt.to(device()));
  Tensor l6 = leaf64(logits);
  Tensor want = torch::nll_loss(torch::log_softmax(l6, -1), tgt);
  EXPECT_NEAR(loss.item<double>(), want.item<double>(), 1e-4);
  loss.backward();
  want.backward();
  EXPECT(rel_err(ld.grad(), l6.grad()) < 1e-4);
  // uniform logits: loss = log(V)
  Tensor flat = itb::ops::cross_entropy(torch::zeros({4, 1000}, torch::TensorOptions().device(device())), tgt.slice(0, 0, 4).to(device()));
  EXPECT_NEAR(flat.item<double>(), std::log(1000.0), 1e-4);
}

ITB_TEST_P(Ops, FusedKernelsReportNoTimeout) {
  ITB_ONLY_CUDA();
#ifdef ITB_WITH_CUDA
  EXPECT(itb::ops::fused::kernel_status() == 0);
#else
  throw itbtest::Skip("built without the sm_100a kernels");
#endif
}

ITB_TEST_MAIN()
