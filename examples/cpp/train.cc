// GPT-2 / LLaMA-3 training loop on the C++ frontend, with the flag names and the per-step log line of
// the reference's example/gpt2/main.cc and example/llama3/main.cc: one process per device, started by
// infini_run / torchrun (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT).
//
//   itb_train --family gpt2 --llmc_filepath model.bin --input_bin tokens.bin --batch_size 4
//             --sequence_length 64 --total_batch_size 256 --num_iteration 10 --learning_rate 1e-4
//             --device cpu|cuda --dtype float32|bfloat16 --optimizer sgd|adam|adamw
//             (without --llmc_filepath: a from-scratch --model d12|...|llama3-1b|llama3-8b, optionally reshaped by
//              --n_layer --n_embd --n_head --n_kv_head --vocab_size; without --input_bin: synthetic token ids)
//             [--lora_rank 8 --lora_alpha 16 --lora_target_modules c_attn,c_proj --lora_load_path F --lora_save_path F]
//             [--save DIR --save_interval N --save_optimizer_state --max_checkpoint_keep K] [--load DIR/checkpoint_step_000004]
//             [--elastic_resume]   --load a checkpoint written by another number of data-parallel ranks (ZeRO state is re-cut)
//             [--tensor_parallel N --sequence_parallel --pipeline_parallel N --virtual_pipeline_parallel N
//              --pipeline_schedule 1f1b|gpipe --zero_stage 0|1|2 --no_overlap_grad_reduce]
//             [--overfit_single_batch] [--input_val_bin F --val_loss_every N --val_max_batches M] [--sample_every N]
//             [--heartbeat_timeout S]   step heartbeats through the job's store and a watchdog thread: when a peer is
//                           silent for S seconds, or asks for an abort, the process groups are aborted and the rank
//                           ends with exit code 75 instead of waiting inside a collective (0 = off, the default;
//                           S must exceed the longest healthy step, checkpoint writes included);
//                           ITB_FAULT="<rank>:<step>:raise|exit|stall|mute[:arg]" injects a host-side fault
//             [--profile]   per-op / per-collective records, written as <family>.report.rank<r>,
//                           <family>.records.log.rank<r> and <family>.trace.rank<r>.json (Chrome trace) into
//                           the working directory
// The ranks are laid out TP fastest, then DP, then PP; data parallelism takes what is left of the
// world size.  CPU ranks talk through the job's TCP store, GPU ranks through NCCL.
#include <chrono>
#include <cstdio>
#include <iostream>
#include <map>
#include <random>
#include <string>
#include <unistd.h>
#include <thread>

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
  namespace par = itb::parallel;
  Flags fl = parse(argc, argv);
  const std::string family = fl.get("family", "gpt2");
  const int64_t B = fl.geti("batch_size", 4), T = fl.geti("sequence_length", 64);
  const int64_t total = fl.geti("total_batch_size", 256), iters = fl.geti("num_iteration", 10);
  const double lr = fl.getd("learning_rate", family == "gpt2" ? 1e-4 : 1e-5);
  const std::string opt_name = fl.get("optimizer", family == "gpt2" ? "sgd" : "adam");
  const bool bf16 = fl.get("dtype", "float32") == "bfloat16";
  const int zero_stage = static_cast<int>(fl.geti("zero_stage", 0));

  // ---- topology: one process per device; TP fastest, then DP, then PP
  par::GlobalEnv& env = par::env();
  env.InitAllEnv(static_cast<int>(fl.geti("tensor_parallel", 1)), fl.getb("sequence_parallel", false),
                 static_cast<int>(fl.geti("pipeline_parallel", 1)), static_cast<int>(fl.geti("virtual_pipeline_parallel", 1)));
  const int64_t dp = env.dp(), tp = env.tp(), pp = env.pp();
  TORCH_CHECK(total % (B * T * dp) == 0, "total_batch_size must be a multiple of batch_size * sequence_length * data-parallel ranks");
  const int64_t grad_accum = total / (B * T * dp);
  TORCH_CHECK(!env.sequence_parallel || T % tp == 0, "sequence_length must be divisible by the tensor-parallel size");
  torch::Device device = fl.get("device", "cpu") == "cuda" ? torch::Device(torch::kCUDA, env.local_rank) : torch::Device(torch::kCPU);
  if (env.world > 1) {
    par::ProcessGroupFactory::Instance().Init(device);
    if (env.rank == 0) std::fprintf(stderr, "%s", env.ProcessGroupOverview().c_str());
  }
  auto dp_group = par::dp_group();
  auto pp_group = par::pp_group();
  itb::nn::ManualSeed(static_cast<uint32_t>(fl.geti("seed", 42)));

  std::shared_ptr<itb::nn::TransformerModel> model;
  if (!fl.get("llmc_filepath", "").empty()) {
    model = family == "gpt2" ? itb::io::LoadGPT2FromLLMC(fl.get("llmc_filepath", ""))
                             : itb::io::LoadLLaMA3FromLLMC(fl.get("llmc_filepath", ""));
  } else {
    auto cfg = from_scratch_config(family, fl.get("model", family == "gpt2" ? "d12" : "llama3-1b"));
    // a from-scratch model of another shape (smoke runs, the configuration matrix)
    if (fl.kv.count("n_layer")) cfg.n_layer = fl.geti("n_layer", cfg.n_layer);
    if (fl.kv.count("n_embd")) cfg.n_embd = fl.geti("n_embd", cfg.n_embd);
    if (fl.kv.count("n_head")) cfg.n_head = cfg.n_kv_head = fl.geti("n_head", cfg.n_head);
    if (fl.kv.count("n_kv_head")) cfg.n_kv_head = fl.geti("n_kv_head", cfg.n_kv_head);
    if (fl.kv.count("vocab_size")) cfg.vocab_size = cfg.original_vocab_size = fl.geti("vocab_size", cfg.vocab_size);
    TORCH_CHECK(cfg.n_embd % cfg.n_head == 0 && cfg.n_head % cfg.n_kv_head == 0, "n_embd / n_head / n_kv_head do not divide");
    model = std::make_shared<itb::nn::TransformerModel>(cfg);
  }
  model->To(device);
  const auto& cfg = model->config;
  std::fprintf(stderr, "[I] rank %d: model: %lld layers (%zu here), %lld wide, %lld/%lld heads, vocab %lld; %zu parameter tensors\n", env.rank,
               (long long)cfg.n_layer, model->h->size(), (long long)cfg.n_embd, (long long)cfg.n_head, (long long)cfg.n_kv_head,
               (long long)cfg.vocab_size, model->Parameters().size());

  std::shared_ptr<itb::Module> loss_module;
  if (tp > 1) loss_module = std::make_shared<par::VocabParallelCrossEntropyLoss>(cfg.original_vocab_size);
  else loss_module = std::make_shared<itb::nn::CrossEntropyLoss>();
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
    // the adapters' draws must not depend on the layout: every adapter draws from a generator of its own, keyed by
    // its module's path in the whole model
    lc.seed = (static_cast<uint32_t>(fl.geti("seed", 42)) ^ 0x4C6F5241u) | 1u;
    lora::GetLoRAModel(model, lc);
    model->To(device);
    // one adapter file for the whole model: every rank keeps its own rows / columns / layers of it
    if (!fl.get("lora_load_path", "").empty()) lora::LoadFullLoRAWeights(model, fl.get("lora_load_path", ""));
    std::fprintf(stderr, "[I] %s\n", lora::PrintLoRASummary(model).c_str());
  }
  // ---- data parallelism: the wrapper broadcasts rank 0's parameters and reduces gradients during backward
  std::shared_ptr<par::DistributedDataParallel> ddp;
  if (dp > 1) {
    par::DistributedDataParallelConfig dc;
    dc.zero_stage = zero_stage;
    dc.overlap_grad_reduce = !fl.getb("no_overlap_grad_reduce", false);
    ddp = std::make_shared<par::DistributedDataParallel>(model, dp_group, dc);
  }
  itb::TensorList trainable = itb::nn::lora::TrainableParameters(model);

  auto make_base = [&](itb::TensorList params) -> std::unique_ptr<itb::optim::Optimizer> {
    if (opt_name == "sgd") return std::make_unique<itb::optim::SGD>(std::move(params), lr);
    return std::make_unique<itb::optim::Adam>(std::move(params), lr, 0.9, 0.999, 1e-8, opt_name == "adamw" ? fl.getd("weight_decay", 0.1) : 0.0);
  };
  std::unique_ptr<itb::optim::Optimizer> optimizer;
  if (ddp && zero_stage >= 1) optimizer = std::make_unique<par::DistributedOptimizer>(make_base, std::vector<par::DistributedDataParallel*>{ddp.get()});
  else optimizer = make_base(trainable);

  // ---- pipeline
  std::unique_ptr<par::PipelineParallel> pipeline;
  if (pp > 1) {
    par::PipelineConfig pc;
    pc.num_stages = static_cast<int>(pp), pc.stage = env.pp_rank, pc.vpp = env.vpp;
    pc.num_micro_batches = static_cast<int>(grad_accum);
    pc.schedule = fl.get("pipeline_schedule", "1f1b");
    pc.boundary_shape = {B, T / env.sp(), cfg.n_embd};
    pc.boundary_dtype = (bf16 && device.is_cuda()) ? torch::kBFloat16 : torch::kFloat32;
    pc.device = device;
    pipeline = std::make_unique<par::PipelineParallel>(
        pc, [&](int64_t ci, const itb::Tensor& in) {
          itb::AutocastGuard autocast(bf16 ? torch::kBFloat16 : torch::kFloat32);
          return model->forward_chunk(ci, in, T);
        }, pp_group);
    if (env.rank == 0) std::fprintf(stderr, "[I] pipeline schedule (%s)\n%s", pc.schedule.c_str(), pipeline->ScheduleTable().c_str());
  }

  // without --input_bin: uniform random ids from a fixed seed in a token file of this rank's own, removed at the end
  std::string data_path = fl.get("input_bin", ""), synthetic_path;
  if (data_path.empty()) {
    synthetic_path = data_path = "/tmp/itb_synth_" + family + "_" + std::to_string(::getpid()) + "_" + std::to_string(env.rank) + ".bin";
    std::mt19937 gen(1234);
    std::uniform_int_distribution<int64_t> draw(0, cfg.original_vocab_size - 1);
    std::vector<int64_t> ids(static_cast<size_t>(std::max<int64_t>(B * T * (grad_accum * dp * (iters + 2) + 4), 4 * T)));
    for (auto& id : ids) id = draw(gen);
    itb::io::WriteTokenFile(data_path, ids, family != "gpt2");
  }
  itb::io::TokenLoader loader(data_path, B, T, env.dp_rank, dp);
  int64_t start_step = 0, consumed = 0;
  const bool model_parallel = tp * pp > 1;
  // which ranks hold state nobody else has: every model-parallel slice, and under ZeRO every shard of the optimizer state
  const bool own_state = model_parallel || (dp > 1 && zero_stage >= 1);
  // A job that its launcher started again after a failure (ITB_RESTART_COUNT > 0, infini_run --max_restarts) goes on
  // from the newest checkpoint under --save that every rank finds complete, unless --load says otherwise.
  std::string load_dir = fl.get("load", "");
  const int restart_count = par::GlobalEnv::EnvInt("ITB_RESTART_COUNT", nullptr, 0);
  if (load_dir.empty() && restart_count > 0 && !fl.get("save", "").empty()) {
    // every rank looks at the directory it would read: its own when it saves, else that of data-parallel rank 0
    const bool saves_own = own_state && (env.dp_rank == 0 || zero_stage >= 1);
    const int probe = !own_state ? -1 : (saves_own ? env.rank : env.layout.RankOf(env.tp_rank, 0, env.pp_rank));
    int64_t step = itb::io::NewestCompleteCheckpointStep(fl.get("save", ""), probe);
    if (auto world_group = par::ProcessGroupFactory::Instance().GetDefaultProcessGroup()) {
      itb::Tensor s = torch::full({1}, static_cast<double>(step), torch::dtype(torch::kFloat64).device(device));
      world_group->AllReduce(s, par::ReduceOp::kMin);
      step = static_cast<int64_t>(s.item<double>());
    }
    if (step > 0) load_dir = itb::io::CheckpointDirOfStep(fl.get("save", ""), step);
    if (env.rank == 0)
      std::fprintf(stderr, "[I] restart %d: %s\n", restart_count,
                   step > 0 ? ("resuming from " + load_dir).c_str() : "no complete checkpoint yet, starting over");
  }
  if (!load_dir.empty()) {
    const std::string root = load_dir;
    // Which directory this rank reads.  A one-rank or pure data-parallel job without ZeRO wrote into the step
    // directory itself.  Otherwise the files are under rank_%06d of the rank that held this rank's (tensor,
    // pipeline) coordinates in the job that saved: its own data-parallel rank when every data-parallel rank saved
    // (ZeRO: optimizer shards) and the data-parallel size is unchanged, else data-parallel rank 0 (weights are the
    // same on every data-parallel rank).  --elastic_resume: another data-parallel size (same tensor / pipeline
    // layout); the slices of a ZeRO optimizer state are put together from the old ranks' files and cut again.
    const bool elastic = fl.getb("elastic_resume", false);
    const bool in_rank_dirs = !std::filesystem::exists(root + "/trainer_state.json");
    auto st = itb::io::LoadTrainerState(in_rank_dirs ? root + "/" + itb::io::RankDirName(0) + "/trainer_state.json" : root + "/trainer_state.json");
    TORCH_CHECK(st.n_layer == cfg.n_layer && st.n_embd == cfg.n_embd, "checkpoint and model shapes differ");
    const bool resized = st.ddp_size != dp;
    TORCH_CHECK(st.tp_size == tp && st.pp_size == pp && st.sp_size == env.sp() && (!resized || !own_state || elastic),
                "the checkpoint was written under another parallel layout (DP=", st.ddp_size, " TP=", st.tp_size, " SP=", st.sp_size,
                " PP=", st.pp_size, "); --elastic_resume accepts another data-parallel size");
    auto old_rank_dir = [&](int64_t old_dp, int64_t d) {   // the rank that held (tp_rank, d, pp_rank) in the job that saved
      return root + "/" + itb::io::RankDirName(static_cast<int>(env.tp_rank + tp * (d + old_dp * env.pp_rank)));
    };
    std::string dir = root;
    if (in_rank_dirs) {
      dir = old_rank_dir(st.ddp_size, !resized && env.dp_rank < st.ddp_size ? env.dp_rank : 0);
      if (!std::filesystem::exists(dir + "/model.ckpt")) dir = old_rank_dir(st.ddp_size, 0);   // only data-parallel rank 0 saved
      st = itb::io::LoadTrainerState(dir + "/trainer_state.json");
    }
    model->LoadStateDict(itb::io::LoadStateDict(dir + "/model.ckpt"));
    if (std::filesystem::exists(dir + "/optimizer.ckpt")) {
      if (resized && ddp && zero_stage >= 1) {
        std::vector<std::map<std::string, itb::Tensor>> old_states;
        for (int64_t d = 0; d < st.ddp_size; ++d) old_states.push_back(itb::io::LoadStateDict(old_rank_dir(st.ddp_size, d) + "/optimizer.ckpt"));
        std::vector<int64_t> numels;
        for (const auto& p : ddp->buffer()->params()) numels.push_back(p.numel());
        optimizer->LoadStateDict(par::ReshardZeroState(old_states, {numels}, static_cast<int>(dp), env.dp_rank));
        if (env.rank == 0)
          std::fprintf(stderr, "[I] elastic resume: ZeRO optimizer state of %lld data-parallel ranks re-cut for %lld\n",
                       (long long)st.ddp_size, (long long)dp);
      } else {
        optimizer->LoadStateDict(itb::io::LoadStateDict(dir + "/optimizer.ckpt"));
      }
    }
    start_step = st.global_step;
    // a rank consumes 1/dp of the batches: keep the position in the token stream
    const int64_t to_skip = resized ? st.consumed_batches * st.ddp_size / dp : st.consumed_batches;
    itb::Tensor x, y;
    for (int64_t i = 0; i < to_skip; ++i) loader.next(&x, &y);
    consumed = to_skip;
  }
  const int64_t save_interval = fl.geti("save_interval", 0);
  std::unique_ptr<itb::data::Tokenizer> tokenizer;
  if (!fl.get("tokenizer_bin", "").empty()) tokenizer = std::make_unique<itb::data::Tokenizer>(fl.get("tokenizer_bin", ""));
  const int64_t freq_generate = fl.geti("freq_generate_txt", 10), text_length = fl.geti("text_length", 64);
  // --sample_every N: the llm.c name for the same sampling period (a placeholder in the reference's loop)
  const int64_t sample_every = fl.geti("sample_every", 0);
  // --overfit_single_batch: every micro-batch of every step is the first batch of the file
  const bool overfit = fl.getb("overfit_single_batch", false);
  itb::Tensor first_x, first_y;
  auto next_batch = [&](itb::Tensor* x, itb::Tensor* y) {
    if (overfit && first_x.defined()) {
      *x = first_x, *y = first_y;
      return;
    }
    loader.next(x, y);
    ++consumed;
    if (overfit) first_x = x->clone(), first_y = y->clone(), *x = first_x, *y = first_y;
  };
  // --input_val_bin F --val_loss_every N: every N steps and after the last one, the mean loss over the first
  // --val_max_batches batches of this rank's share of F, averaged over the data-parallel group (a
  // placeholder in the reference's loop, example/gpt2/main.cc:401-404); not under pipeline parallelism
  const int64_t val_every = fl.geti("val_loss_every", 0), val_max_batches = fl.geti("val_max_batches", 20);
  std::unique_ptr<itb::data::DistributedDataLoader> val_loader;
  if (!fl.get("input_val_bin", "").empty() && val_every > 0 && pp == 1)
    val_loader = std::make_unique<itb::data::DistributedDataLoader>(
        std::make_shared<itb::data::TinyShakespeareDataset>(fl.get("input_val_bin", ""), T), B, env.dp_rank, dp);
  auto loss_of = [&](const itb::Tensor& logits, const itb::Tensor& y) {
    itb::AutocastGuard autocast(bf16 ? torch::kBFloat16 : torch::kFloat32);
    return (*loss_module)(itb::TensorList{logits, y})[0];
  };

  const bool profile = fl.getb("profile", false);
  if (profile) itb::utils::Profiler::Instance().Enable(env.rank);
  // failure detection: heartbeats and a watchdog over the job's store; faults are injected between steps
  const double heartbeat_timeout = fl.getd("heartbeat_timeout", 0.0);
  std::unique_ptr<itb::utils::Heartbeat> heartbeat;
  if (heartbeat_timeout > 0 && env.world > 1) {
    auto& factory = par::ProcessGroupFactory::Instance();
    factory.SetAbortable(true);
    heartbeat = std::make_unique<itb::utils::Heartbeat>(factory.store(), env.rank, env.world, heartbeat_timeout,
                                                        std::min(0.5, heartbeat_timeout / 4), [&factory] { return factory.AllGroups(); });
    heartbeat->Start();
  }
  itb::utils::FaultInjector injector(env.rank, nullptr, heartbeat.get(), device.is_cuda());
  auto rank_failed = [&](const std::string& why) {
    std::fprintf(stderr, "[E] rank %d stops: %s\n", env.rank, why.c_str());
    std::fflush(stderr);
    std::_Exit(75);   // EX_TEMPFAIL, as the Python trainer; peers are gone: no ordered shutdown, no collective in a destructor
  };
  for (int64_t step = start_step; step < iters; ++step) {
    injector.MaybeFire(step + 1);
    if (heartbeat) {
      try {
        heartbeat->Step(step + 1);
        heartbeat->WaitPeers(step + 1);   // every peer is alive and here before this step's first collective
      } catch (const itb::utils::RankFailure& e) {
        rank_failed(e.what());
      }
    }
    try {
    auto t0 = std::chrono::steady_clock::now();
    if (profile) itb::utils::Profiler::Instance().SetTag("Step_" + std::to_string(step + 1));
    itb::utils::PrecisionChecker::Instance().ResetCounters();
    optimizer->ZeroGrad();
    if (ddp) ddp->ZeroGrad();
    double lossf = 0.0;
    if (pipeline) {
      std::vector<itb::Tensor> xs, ys;
      for (int64_t micro = 0; micro < grad_accum; ++micro) {
        itb::Tensor x, y;
        next_batch(&x, &y);
        // the loader's tensors alias a ring slot that the next calls reuse: the schedule needs its own copies
        xs.push_back(device.is_cpu() ? x.clone() : x.to(device)), ys.push_back(device.is_cpu() ? y.clone() : y.to(device));
      }
      lossf = pipeline->StepMicroBatches(xs, ys, loss_of, [&](int64_t, bool last) {
        if (ddp) ddp->set_sync(last);
      });
    } else {
      for (int64_t micro = 0; micro < grad_accum; ++micro) {
        itb::Tensor x, y;
        next_batch(&x, &y);
        x = x.to(device), y = y.to(device);
        if (ddp) ddp->set_sync(micro == grad_accum - 1);   // earlier micro-batches only accumulate
        itb::Tensor loss;
        {
          itb::AutocastGuard autocast(bf16 ? torch::kBFloat16 : torch::kFloat32);
          // through the call operator: hooks see the model's output
          itb::Tensor logits = ddp ? (*ddp)(itb::TensorList{x})[0] : (*model)(itb::TensorList{x})[0];
          loss = loss_of(logits, y) / static_cast<double>(grad_accum);
        }
        lossf += loss.item<float>();
        loss.backward();
      }
    }
    if (ddp) ddp->FinishGradSync();
    // under sequence parallelism the parameters that every tensor-parallel rank holds whole saw a
    // slice of the sequence each: their gradients are partial sums
    if (env.sequence_parallel) par::AllReduceSequenceParallelGrads(model->SequenceParallelReplicated());
    // replicated adapter factors next to a split one hold this rank's part of their gradient
    if (lora_rank > 0 && tp > 1) par::AllReduceSequenceParallelGrads(itb::nn::lora::PartialGradParameters(model), /*always=*/true);
    optimizer->Step();
    if (dp_group) {
      itb::Tensor l = torch::full({1}, lossf, torch::dtype(torch::kFloat32).device(device));
      dp_group->AllReduce(l, par::ReduceOp::kAvg);
      lossf = l.item<float>();
    }
    double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    // high-water marks of the tensors' memory pool since the previous step (0 on the CPU, which has no pool)
    auto [peak_used_mb, peak_reserved_mb] = itb::core::Runtime::For(device).GetMemPoolPeakMB(device);
    itb::core::Runtime::For(device).ResetMemPoolHighWatermarks(device);
    if (env.rank == env.world - 1)   // the last rank logs, as in the reference (it holds the last pipeline stage)
      std::fprintf(stderr, "[E] step %4lld/%lld | train loss %.6f | lr %.2e | (%.2f ms | %.0f tok/s | peak used: %5.0f MB | "
                           "peak reserved: %5.0f MB, DP=%lld, TP=%lld, SP=%d, PP=%lld)\n",
                   (long long)(step + 1), (long long)iters, lossf, lr, ms, total / (ms / 1e3), static_cast<double>(peak_used_mb), static_cast<double>(peak_reserved_mb), (long long)dp, (long long)tp,
                   env.sp(), (long long)pp);
    if (val_loader && ((step + 1) % val_every == 0 || step + 1 == iters)) {
      torch::NoGradGuard no_grad;
      double sum = 0.0;
      int64_t n = 0;
      for (auto it = val_loader->begin(); it != val_loader->end() && n < val_max_batches; ++it, ++n) {
        auto [vx, vy] = *it;
        itb::AutocastGuard autocast(bf16 ? torch::kBFloat16 : torch::kFloat32);
        sum += loss_of(model->forward(vx.to(device)), vy.to(device)).item<float>();
      }
      itb::Tensor v = torch::tensor({sum, static_cast<double>(n)}, torch::dtype(torch::kFloat32).device(device));
      if (dp_group) dp_group->AllReduce(v, par::ReduceOp::kSum);
      v = v.cpu();
      if (env.rank == env.world - 1 && v[1].item<float>() > 0)
        std::fprintf(stderr, "[E] step %4lld/%lld | val loss %.6f (%lld batches)\n", (long long)(step + 1), (long long)iters,
                     v[0].item<float>() / v[1].item<float>(), (long long)n);
    }
    const bool sample_now = (freq_generate > 0 && (step + 1) % freq_generate == 0) ||
                            (sample_every > 0 && ((step + 1) % sample_every == 0 || step + 1 == iters));
    if (tokenizer && sample_now && env.rank == 0 && !model_parallel) {
      std::vector<int64_t> ids;
      std::string text = tokenizer->GenerateText([&](const itb::Tensor& ids_in) { return model->forward(ids_in); }, B, T,
                                                 text_length, device, &ids);
      std::printf("%s\n[generated ids]", text.c_str());
      for (int64_t id : ids) std::printf(" %lld", (long long)id);
      std::printf("\n");
    }
    // a rank saves what only it holds: its model-parallel slice, its shard of a ZeRO optimizer state
    const bool saver = own_state ? (env.dp_rank == 0 || zero_stage >= 1) : env.rank == 0;
    if (save_interval > 0 && (step + 1) % save_interval == 0 && !fl.get("save", "").empty()) {
      if (saver) {
        itb::io::TrainerState st;
        st.global_step = step + 1, st.consumed_batches = consumed, st.last_lr = lr;
        st.n_layer = cfg.n_layer, st.n_head = cfg.n_head, st.n_kv_head = cfg.n_kv_head, st.n_embd = cfg.n_embd;
        st.vocab_size = cfg.vocab_size, st.ddp_size = dp, st.tp_size = tp, st.sp_size = env.sp(), st.pp_size = pp;
        const bool with_optimizer = fl.getb("save_optimizer_state", true);
        itb::io::SaveCheckpoint(fl.get("save", ""), st, *model,
                                with_optimizer ? optimizer->StateDict() : std::map<std::string, itb::Tensor>{}, own_state ? env.rank : -1);
      }
      // every rank's part of this step is on disk before the oldest step directory goes
      if (auto world = par::ProcessGroupFactory::Instance().GetDefaultProcessGroup()) world->Barrier();
      if (env.rank == 0) itb::io::PruneCheckpoints(fl.get("save", ""), fl.geti("max_checkpoint_keep", 0));
    }
    } catch (const c10::Error& e) {
      // a collective that the watchdog aborted comes back as an error: report the failure it saw
      // (an error of the store itself can arrive before the watchdog's next look: give it two polls)
      for (int i = 0; heartbeat && !heartbeat->failure() && i < 100; ++i)
        std::this_thread::sleep_for(std::chrono::duration<double>(std::min(0.5, heartbeat_timeout / 4) / 50));
      if (heartbeat && heartbeat->failure()) rank_failed(heartbeat->failure()->str());
      throw;
    }
  }
  if (heartbeat) heartbeat->Stop();
  if (profile) {
    auto& prof = itb::utils::Profiler::Instance();
    prof.Disable();
    prof.Report(family + ".report.rank" + std::to_string(env.rank));
    prof.PrintRecords(family + ".records.log.rank" + std::to_string(env.rank));
    prof.ExportChromeTrace(family + ".trace.rank" + std::to_string(env.rank) + ".json");
  }
  if (auto world = par::ProcessGroupFactory::Instance().GetDefaultProcessGroup()) world->Barrier();
  // the adapters of a model-parallel run are gathered into ONE ordinary adapter file (a collective over every
  // tensor-parallel and pipeline group), loadable on any layout
  if (lora_rank > 0 && !fl.get("lora_save_path", "").empty()) itb::nn::lora::SaveFullLoRAWeights(model, fl.get("lora_save_path", ""));
  ddp.reset();
  if (!synthetic_path.empty()) std::remove(synthetic_path.c_str());
  par::ProcessGroupFactory::Instance().Shutdown();
  return 0;
}
