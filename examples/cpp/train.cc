// GPT-2 / LLaMA-3 training loop on the C++ frontend, with the flag names and the per-step log line of
// the reference's example/gpt2/main.cc and example/llama3/main.cc: one process per device, data
// parallel over the ranks that infini_run / torchrun start (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT).
//
//   itb_train --family gpt2 --llmc_filepath model.bin --input_bin tokens.bin --batch_size 4
//             --sequence_length 64 --total_batch_size 256 --num_iteration 10 --learning_rate 1e-4
//             --device cpu|cuda --dtype float32|bfloat16 --optimizer sgd|adam|adamw
//             [--lora_rank 8 --lora_alpha 16 --lora_target_modules c_attn,c_proj --lora_load_path F --lora_save_path F]
//             [--save DIR --save_interval N] [--load DIR/checkpoint_step_000004]
#include <chrono>
#include <cstdio>
#include <iostream>
#include <map>
#include <string>

#include "itb/itb.h"

namespace {

struct Flags {
  std::map<std::string, std::string> kv;
  std::string get(const std::string& k, const std::string& d) const {
    auto it = kv.find(k);
    return it == kv.end() ? d : it->second;
  }
  int64_t geti(const std::string& k, int64_t d) const { return kv.count(k) ? std::stoll(kv.at(k)) : d; }
  double getd(const std::string& k, double d) const { return kv.count(k) ? std::stod(kv.at(k)) : d; }
  bool getb(const std::string& k, bool d) const {
    if (!kv.count(k)) return d;
    const std::string& v = kv.at(k);
    return v.empty() || v == "1" || v == "true";
  }
};
// --name value, --name=value, --flag
Flags parse(int argc, char** argv) {
  Flags f;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    TORCH_CHECK(a.rfind("--", 0) == 0, "unexpected argument ", a);
    a = a.substr(2);
    auto eq = a.find('=');
    if (eq != std::string::npos) {
      f.kv[a.substr(0, eq)] = a.substr(eq + 1);
    } else if (i + 1 < argc && std::string(argv[i + 1]).rfind("--", 0) != 0) {
      f.kv[a] = argv[++i];
    } else {
      f.kv[a] = "";
    }
  }
  return f;
}

itb::nn::TransformerConfig from_scratch_config(const std::string& family, const std::string& model) {
  using itb::nn::TransformerConfig;
  if (family == "gpt2") {
    auto c = TransformerConfig::GPT2();
    const std::map<std::string, std::array<int64_t, 3>> sizes = {
        {"d12", {12, 12, 768}}, {"d24", {24, 16, 1024}}, {"d36", {36, 20, 1280}}, {"d48", {48, 25, 1600}},
        {"gpt2", {12, 12, 768}}, {"gpt2-medium", {24, 16, 1024}}, {"gpt2-large", {36, 20, 1280}}, {"gpt2-xl", {48, 25, 1600}}};
    auto it = sizes.find(model);
    TORCH_CHECK(it != sizes.end(), "unknown GPT-2 model ", model);
    c.n_layer = it->second[0], c.n_head = c.n_kv_head = it->second[1], c.n_embd = it->second[2];
    return c;
  }
  auto c = TransformerConfig::LLaMA3();
  if (model == "llama3-8b") {
    c.n_layer = 32, c.n_embd = 4096, c.ffn_dim_multiplier = 1.3, c.multiple_of = 1024;
  } else if (model == "llama3-3b") {
    c.n_layer = 28, c.n_embd = 3072, c.n_head = 24, c.ffn_dim_multiplier = 1.0;
  }
  return c;
}

}  // namespace

int main(int argc, char** argv) {
  Flags fl = parse(argc, argv);
  const std::string family = fl.get("family", "gpt2");
  const int64_t B = fl.geti("batch_size", 4), T = fl.geti("sequence_length", 64);
  const int64_t total = fl.geti("total_batch_size", 256), iters = fl.geti("num_iteration", 10);
  const double lr = fl.getd("learning_rate", family == "gpt2" ? 1e-4 : 1e-5);
  const std::string opt_name = fl.get("optimizer", family == "gpt2" ? "sgd" : "adam");
  const bool bf16 = fl.get("dtype", "float32") == "bfloat16";
  const int64_t world_env = itb::dist::Env::FromEnvironment().world;
  TORCH_CHECK(total % (B * T * world_env) == 0, "total_batch_size must be a multiple of batch_size * sequence_length * ranks");
  const int64_t grad_accum = total / (B * T * world_env);
  const itb::dist::Env env = itb::dist::Env::FromEnvironment();    // one process per device (infini_run / torchrun)
  torch::Device device = fl.get("device", "cpu") == "cuda" ? torch::Device(torch::kCUDA, env.local_rank) : torch::Device(torch::kCPU);
  const int64_t dp = env.world;
  itb::nn::ManualSeed(static_cast<uint32_t>(fl.geti("seed", 42)));

  std::shared_ptr<itb::nn::TransformerModel> model;
  if (!fl.get("llmc_filepath", "").empty()) {
    model = family == "gpt2" ? itb::io::LoadGPT2FromLLMC(fl.get("llmc_filepath", ""))
                             : itb::io::LoadLLaMA3FromLLMC(fl.get("llmc_filepath", ""));
  } else {
    auto cfg = from_scratch_config(family, fl.get("model", family == "gpt2" ? "d12" : "llama3-1b"));
    if (fl.kv.count("n_layer")) cfg.n_layer = fl.geti("n_layer", cfg.n_layer);
    model = std::make_shared<itb::nn::TransformerModel>(cfg);
  }
  model->To(device);
  const auto& cfg = model->config;
  std::fprintf(stderr, "[I] model: %lld layers, %lld wide, %lld/%lld heads, vocab %lld; %zu parameter tensors\n",
               (long long)cfg.n_layer, (long long)cfg.n_embd, (long long)cfg.n_head, (long long)cfg.n_kv_head,
               (long long)cfg.vocab_size, model->Parameters().size());

  auto loss_module = std::make_shared<itb::nn::CrossEntropyLoss>();
  if (!fl.get("precision_check", "").empty()) {   // "level=1,format=simple,path=DIR,save_tensors=true"
    itb::utils::PrecisionChecker::Instance().Init(fl.get("precision_check", ""), env.rank);
    itb::utils::PrecisionChecker::Instance().Attach(model);
    itb::utils::PrecisionChecker::Instance().Attach(loss_module);
  }
  const int64_t lora_rank = fl.geti("lora_rank", 0);
  if (lora_rank > 0) {
    namespace lora = itb::nn::lora;
    lora::LoRAConfig lc;
    lc.rank = lora_rank, lc.alpha = fl.getd("lora_alpha", 16.0);
    lc.target_modules = lora::ParseLoRATargetModules(fl.get("lora_target_modules", "c_attn,c_proj"));
    lora::GetLoRAModel(model, lc);
    model->To(device);
    if (!fl.get("lora_load_path", "").empty()) lora::LoadLoRAWeights(model, fl.get("lora_load_path", ""));
    std::fprintf(stderr, "[I] %s\n", lora::PrintLoRASummary(model).c_str());
  }
  std::shared_ptr<itb::dist::Comm> comm;
  std::unique_ptr<itb::dist::DistributedDataParallel> ddp;
  if (dp > 1) {
    comm = itb::dist::MakeComm(env, device);
    ddp = std::make_unique<itb::dist::DistributedDataParallel>(model, comm);   // parameters become rank 0's
  }
  itb::TensorList trainable = itb::nn::lora::TrainableParameters(model);

  std::unique_ptr<itb::optim::Optimizer> optimizer;
  if (opt_name == "sgd") optimizer = std::make_unique<itb::optim::SGD>(trainable, lr);
  else optimizer = std::make_unique<itb::optim::Adam>(trainable, lr, 0.9, 0.999, 1e-8,
                                                      opt_name == "adamw" ? fl.getd("weight_decay", 0.1) : 0.0);

  itb::io::TokenLoader loader(fl.get("input_bin", ""), B, T, env.rank, dp);
  int64_t start_step = 0, consumed = 0;
  if (!fl.get("load", "").empty()) {
    const std::string dir = fl.get("load", "");
    auto st = itb::io::LoadTrainerState(dir + "/trainer_state.json");
    TORCH_CHECK(st.n_layer == cfg.n_layer && st.n_embd == cfg.n_embd, "checkpoint and model shapes differ");
    model->LoadStateDict(itb::io::LoadStateDict(dir + "/model.ckpt"));
    if (std::filesystem::exists(dir + "/optimizer.ckpt")) optimizer->LoadStateDict(itb::io::LoadStateDict(dir + "/optimizer.ckpt"));
    start_step = st.global_step;
    itb::Tensor x, y;
    for (int64_t i = 0; i < st.consumed_batches; ++i) loader.next(&x, &y);
    consumed = st.consumed_batches;
  }
  const int64_t save_interval = fl.geti("save_interval", 0);
  std::unique_ptr<itb::data::Tokenizer> tokenizer;
  if (!fl.get("tokenizer_bin", "").empty()) tokenizer = std::make_unique<itb::data::Tokenizer>(fl.get("tokenizer_bin", ""));
  const int64_t freq_generate = fl.geti("freq_generate_txt", 10), text_length = fl.geti("text_length", 64);

  for (int64_t step = start_step; step < iters; ++step) {
    auto t0 = std::chrono::steady_clock::now();
    itb::utils::PrecisionChecker::Instance().ResetCounters();
    optimizer->ZeroGrad();
    double lossf = 0.0;
    for (int64_t micro = 0; micro < grad_accum; ++micro) {
      itb::Tensor x, y;
      loader.next(&x, &y);
      ++consumed;
      x = x.to(device), y = y.to(device);
      itb::Tensor loss;
      {
        itb::AutocastGuard autocast(bf16 ? torch::kBFloat16 : torch::kFloat32);
        itb::Tensor logits = (*model)(itb::TensorList{x})[0];   // through the call operator: hooks see the model's output
        loss = (*loss_module)(itb::TensorList{logits, y})[0] / static_cast<double>(grad_accum);
      }
      lossf += loss.item<float>();
      loss.backward();
    }
    if (ddp) {
      ddp->SyncGradients();
      itb::Tensor l = torch::full({1}, lossf, torch::dtype(torch::kFloat32).device(device));
      comm->AllReduceSum(l);
      lossf = l.item<float>() / static_cast<double>(dp);
    }
    optimizer->Step();
    double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (env.rank == dp - 1)   // the last rank logs, as in the reference
      std::fprintf(stderr, "[E] step %4lld/%lld | train loss %.6f | lr %.2e | (%.2f ms | %.0f tok/s | peak used: %5.0f MB | "
                           "peak reserved: %5.0f MB, DP=%lld, TP=1, SP=1, PP=1)\n",
                   (long long)(step + 1), (long long)iters, lossf, lr, ms, total / (ms / 1e3), 0.0, 0.0, (long long)dp);
    if (tokenizer && freq_generate > 0 && (step + 1) % freq_generate == 0 && env.rank == 0) {
      std::vector<int64_t> ids;
      std::string text = tokenizer->GenerateText([&](const itb::Tensor& ids_in) { return model->forward(ids_in); }, B, T,
                                                 text_length, device, &ids);
      std::printf("%s\n[generated ids]", text.c_str());
      for (int64_t id : ids) std::printf(" %lld", (long long)id);
      std::printf("\n");
    }
    if (save_interval > 0 && (step + 1) % save_interval == 0 && !fl.get("save", "").empty() && env.rank == 0) {
      itb::io::TrainerState st;
      st.global_step = step + 1, st.consumed_batches = consumed, st.last_lr = lr;
      st.n_layer = cfg.n_layer, st.n_head = cfg.n_head, st.n_kv_head = cfg.n_kv_head, st.n_embd = cfg.n_embd;
      st.vocab_size = cfg.vocab_size, st.ddp_size = dp;
      itb::io::SaveCheckpoint(fl.get("save", ""), st, *model, optimizer->StateDict());
    }
  }
  if (comm) comm->Barrier();
  if (lora_rank > 0 && !fl.get("lora_save_path", "").empty() && env.rank == 0) itb::nn::lora::SaveLoRAWeights(model, fl.get("lora_save_path", ""));
  return 0;
}
