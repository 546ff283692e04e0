// Unit checks of the C++ frontend's API on CPU: the behaviours the reference's gtest suites assert
// (tests/transformer/test_transformer_architecture.cc, tests/optimizer, tests/checkpoint, tests/hook).
// Prints "ok <n>" and exits 0, or names the failed check and exits 1.
#include <cstdio>
#include <cstdlib>

#include "itb/itb.h"

static int g_checks = 0;
#define EXPECT(cond)                                                         \
  do {                                                                       \
    ++g_checks;                                                              \
    if (!(cond)) {                                                           \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      std::exit(1);                                                          \
    }                                                                        \
  } while (0)

using namespace itb;

static nn::TransformerConfig tiny_gpt() {
  auto c = nn::TransformerConfig::GPT2();
  c.block_size = 32, c.vocab_size = c.original_vocab_size = 128, c.n_layer = 2, c.n_head = c.n_kv_head = 4, c.n_embd = 32;
  return c;
}
static nn::TransformerConfig tiny_llama() {
  auto c = nn::TransformerConfig::LLaMA3();
  c.block_size = 32, c.vocab_size = c.original_vocab_size = 128, c.n_layer = 2, c.n_head = 4, c.n_kv_head = 2, c.n_embd = 32;
  c.multiple_of = 16;
  return c;
}

int main(int argc, char** argv) {
  const std::string tmp = argc > 1 ? argv[1] : "/tmp";
  torch::manual_seed(0);

  // layers: shapes, names, parameter counts
  nn::Linear lin(16, 8);
  EXPECT(lin.weight.sizes() == torch::IntArrayRef({8, 16}) && lin.bias.sizes() == torch::IntArrayRef({8}));
  EXPECT(lin.Parameters().size() == 2 && lin.StateDict().count("weight") && lin.StateDict().count("bias"));
  EXPECT(lin.weight.abs().max().item<float>() <= 0.25f + 1e-6f);               // Kaiming-uniform bound 1/sqrt(16)
  EXPECT(nn::MLP(tiny_gpt()).Parameters().size() == 4 && nn::MLP(tiny_llama()).Parameters().size() == 3);
  EXPECT(nn::CausalSelfAttention(tiny_gpt()).Parameters().size() == 4);
  EXPECT(nn::CausalSelfAttention(tiny_llama()).Parameters().size() == 2);
  EXPECT(tiny_llama().ffn_hidden() == (static_cast<int64_t>(std::llround((2 * 128 / 3) * 1.5)) + 15) / 16 * 16);
  auto freqs = ops::precompute_freqs_cis(64, 128);
  EXPECT(freqs.sizes() == torch::IntArrayRef({128, 32, 2}));

  // model: shapes, tying, state-dict names, no duplicate parameters
  auto gpt = std::make_shared<nn::TransformerModel>(tiny_gpt());
  auto idx = torch::randint(0, 128, {2, 8}, torch::kInt64);
  EXPECT(gpt->forward(idx).sizes() == torch::IntArrayRef({2, 8, 128}));
  auto sd = gpt->StateDict();
  for (const char* k : {"transformer.wte.weight", "transformer.wpe.weight", "transformer.h.0.ln_1.weight",
                        "transformer.h.0.attn.c_attn.weight", "transformer.h.1.mlp.c_proj.bias", "transformer.ln_f.bias",
                        "lm_head.weight"})
    EXPECT(sd.count(k) == 1);
  EXPECT(sd["transformer.wte.weight"].data_ptr() == sd["lm_head.weight"].data_ptr());
  EXPECT(gpt->Parameters().size() == 2 + 2 * 12 + 2 && sd.size() >= gpt->Parameters().size());
  auto llama = std::make_shared<nn::TransformerModel>(tiny_llama());
  EXPECT(llama->Parameters().size() == 1 + 2 * 7 + 1 + 1);
  EXPECT(llama->forward(idx).sizes() == torch::IntArrayRef({2, 8, 128}));

  // every parameter receives a gradient
  ops::cross_entropy(gpt->forward(idx), torch::randint(0, 128, {2, 8}, torch::kInt64)).backward();
  for (auto& p : gpt->Parameters()) EXPECT(p.grad().defined());

  // hooks and handles
  int pre = 0, post = 0;
  auto h1 = lin.RegisterForwardPreHook([&](Module*, const TensorList&) { ++pre; });
  auto h2 = lin.RegisterForwardPostHook([&](Module*, const TensorList&, const TensorList&) { ++post; });
  lin(torch::randn({3, 16}));
  h1->Remove();
  lin(torch::randn({3, 16}));
  EXPECT(pre == 1 && post == 2);
  int bwd = 0;
  auto h3 = lin.RegisterBackwardPostHook([&](Module*, size_t i, const Tensor& g) {
    if (i == 0 && g.sizes() == torch::IntArrayRef({3, 8})) ++bwd;
  });
  lin(torch::randn({3, 16})).sum().backward();
  h3->Remove();
  lin(torch::randn({3, 16})).sum().backward();
  EXPECT(bwd == 1);

  // strict loading; extra keys ignored; dtype conversion keeps tensor identity
  auto other = std::make_shared<nn::TransformerModel>(tiny_gpt());
  auto sd2 = other->StateDict();
  sd2["transformer.h.0.attn.bias"] = torch::zeros({1});                          // a buffer only the reference writes
  gpt->LoadStateDict(sd2);
  EXPECT(torch::equal(gpt->lm_head()->weight, other->lm_head()->weight));
  sd2.erase("transformer.ln_f.bias");
  bool threw = false;
  try {
    gpt->LoadStateDict(sd2);
  } catch (const c10::Error&) {
    threw = true;
  }
  EXPECT(threw);
  Tensor w = lin.weight;
  lin.To(torch::kBFloat16);
  EXPECT(w.scalar_type() == torch::kBFloat16 && lin.weight.scalar_type() == torch::kBFloat16);

  // optimizers: Adam's step counter advances without gradients; state-dict round trip; SGD has no state
  nn::Linear a(4, 4), b(4, 4);
  optim::Adam oa(a.Parameters(), 1e-2), ob(b.Parameters(), 1e-2);
  for (int i = 0; i < 3; ++i) {
    oa.ZeroGrad();
    a(torch::ones({2, 4})).sum().backward();
    oa.Step();
  }
  oa.ZeroGrad();
  oa.Step();
  EXPECT(oa.StateDict().at("adam.t").item<int64_t>() == 4);
  io::SaveStateDict(tmp + "/adam.ckpt", oa.StateDict());
  ob.LoadStateDict(io::LoadStateDict(tmp + "/adam.ckpt"));
  EXPECT(ob.t() == 4 && torch::allclose(ob.StateDict().at("adam.m.0"), oa.StateDict().at("adam.m.0")));
  EXPECT(optim::SGD(a.Parameters(), 0.1).StateDict().empty());

  // Adam against the closed form of its first step: p -= lr * g / (|g| + eps)
  nn::Linear c(3, 1, false);
  Tensor before = c.weight.detach().clone();
  optim::Adam oc(c.Parameters(), 0.1);
  c(torch::ones({1, 3})).sum().backward();
  oc.Step();
  EXPECT(torch::allclose(c.weight.detach(), before - 0.1, 1e-5, 1e-6));

  // checkpoint files: model + trainer state
  io::TrainerState st;
  st.global_step = 7, st.consumed_batches = 14, st.last_lr = 1e-4, st.n_layer = 2, st.n_embd = 32;
  std::string dir = io::SaveCheckpoint(tmp, st, *gpt, {});
  auto st2 = io::LoadTrainerState(dir + "/trainer_state.json");
  EXPECT(st2.global_step == 7 && st2.consumed_batches == 14 && st2.n_layer == 2 && st2.n_embd == 32);
  auto loaded = io::LoadStateDict(dir + "/model.ckpt");
  EXPECT(loaded.size() == gpt->StateDict().size() && torch::equal(loaded.at("lm_head.weight"), gpt->lm_head()->weight));

  // bf16 autocast emulation changes Linear only
  {
    nn::Linear l(8, 8);
    Tensor x = torch::randn({4, 8});
    Tensor full = l(x);
    AutocastGuard guard(torch::kBFloat16);
    Tensor low = l(x);
    EXPECT(!torch::equal(full, low) && torch::allclose(full, low, 5e-2, 5e-2));
  }
  // LoRA: target matching, shapes, frozen base, merge == unmerged forward, merge-and-unload
  {
    namespace lora = nn::lora;
    lora::LoRAConfig lc;
    lc.rank = 4, lc.alpha = 8.0;
    EXPECT(lc.Scaling() == 2.0);
    lc.target_modules = lora::ParseLoRATargetModules(" c_attn , attn.c_proj ,, ");
    EXPECT(lc.target_modules == (std::set<std::string>{"c_attn", "attn.c_proj"}));
    EXPECT(lc.ShouldApplyLoRA("transformer.h.0.attn.c_proj") && !lc.ShouldApplyLoRA("transformer.h.0.mlp.c_proj"));
    EXPECT(lc.ShouldApplyLoRA("c_attn") && !lc.ShouldApplyLoRA("xc_attn"));
    std::shared_ptr<Module> m = std::make_shared<nn::TransformerModel>(tiny_gpt());
    int64_t total_before = lora::CountTotalParameters(m);
    lora::GetLoRAModel(m, lc);
    auto mods = lora::LoRAModules(m);
    EXPECT(mods.size() == 4);                                                       // c_attn and attn.c_proj of 2 layers
    EXPECT(mods[0]->lora_A.size(0) == 4 && mods[0]->lora_A.size(1) == 32 && mods[0]->lora_B.size(1) == 4);
    EXPECT(!mods[0]->weight.requires_grad() && mods[0]->lora_A.requires_grad());
    EXPECT(lora::CountTrainableParameters(m) == lora::CountTotalParameters(m) - total_before);
    EXPECT(m->StateDict().count("transformer.h.0.attn.c_attn.lora_A") == 1);
    {
      torch::NoGradGuard g;
      for (auto& p : lora::GetLoRAParameters(m)) p.normal_(0, 0.3);
    }
    auto tm = std::static_pointer_cast<nn::TransformerModel>(m);
    Tensor before = tm->forward(idx).detach();
    lora::MergeLoRAWeights(m);
    EXPECT(mods[0]->IsMerged() && !mods[0]->lora_A.requires_grad());
    EXPECT(torch::allclose(tm->forward(idx).detach(), before, 1e-4, 1e-4));
    lora::UnmergeLoRAWeights(m);
    EXPECT(!mods[0]->IsMerged() && mods[0]->lora_A.requires_grad());
    EXPECT(torch::allclose(tm->forward(idx).detach(), before, 1e-4, 1e-4));
    lora::SaveLoRAWeights(m, tmp + "/adapter.bin");
    std::shared_ptr<Module> m2 = std::make_shared<nn::TransformerModel>(tiny_gpt());
    m2->LoadStateDict([&] {
      auto sd0 = m->StateDict();
      for (auto it = sd0.begin(); it != sd0.end();) it = it->first.find("lora_") != std::string::npos ? sd0.erase(it) : std::next(it);
      return sd0;
    }());
    lora::GetLoRAModel(m2, lc);
    lora::LoadLoRAWeights(m2, tmp + "/adapter.bin");
    EXPECT(torch::allclose(std::static_pointer_cast<nn::TransformerModel>(m2)->forward(idx).detach(), before, 1e-5, 1e-5));
    lora::MergeAndUnload(m);
    EXPECT(lora::LoRAModules(m).empty() && lora::LoRAStateDict(m).empty());
    EXPECT(lora::CountTrainableParameters(m) == total_before);
    EXPECT(torch::allclose(tm->forward(idx).detach(), before, 1e-4, 1e-4));
  }
  std::printf("ok %d\n", g_checks);
  return 0;
}
