// File IO of the C++ frontend: llm.c weight files (reference: example/gpt2/checkpoint_loader.cc,
// example/llama3/checkpoint_loader.cc), llm.c token files behind a prefetching loader
// (example/common/tiny_shakespeare_dataset.cc, src/dataloader.cc), checkpoints
// (src/checkpoint/checkpoint.cc).
#pragma once
#include <dirent.h>
#include <ftw.h>
#include <sys/stat.h>

#include <algorithm>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <regex>
#include <sstream>

#include "../../runtime/state_dict_io.h"
#include "../../runtime/token_io.h"
#include "transformer.h"

namespace itb {
namespace io {

// ------------------------------------------------------------------ llm.c weight files
inline Tensor read_f32(std::ifstream& f, std::vector<int64_t> shape) {
  Tensor t = torch::empty(shape, torch::kFloat32);
  f.read(static_cast<char*>(t.data_ptr()), static_cast<std::streamsize>(t.numel() * 4));
  TORCH_CHECK(f.good(), "llm.c weight file is truncated");
  return t;
}
inline void assign(std::map<std::string, Tensor>& sd, const std::string& key, const Tensor& value) {
  auto it = sd.find(key);
  TORCH_CHECK(it != sd.end(), "model has no parameter '", key, "'");
  TORCH_CHECK(it->second.sizes() == value.sizes(), "shape mismatch for '", key, "'");
  torch::NoGradGuard g;
  it->second.copy_(value);
}

// How one tensor of a weight file maps onto this rank's slice of a tensor- / pipeline-parallel model
// (reference: the loaders of example/gpt2/net.cc:263-520 and example/llama3/net.cc:236-530 read every
// tensor and keep the rows or columns of their rank).
enum class Shard { kReplicated, kRows, kCols, kQKVRows };
class ShardedAssigner {
 public:
  ShardedAssigner(std::ifstream& f, nn::TransformerModel& model) : f_(f), model_(model), sd_(model.StateDict()) {}
  // Reads the next tensor of the file (full shape `shape`) into parameter `name`, given in the
  // single-process naming with GLOBAL layer numbers; skips it when this rank does not hold it.
  void next(const std::string& name, const std::vector<int64_t>& shape, Shard how, int64_t keep_rows = -1) {
    const std::string local = LocalName(name);
    int64_t numel = 1;
    for (int64_t d : shape) numel *= d;
    if (local.empty() || sd_.find(local) == sd_.end()) {
      f_.seekg(static_cast<std::streamoff>(numel * 4), std::ios::cur);
      TORCH_CHECK(f_.good(), "llm.c weight file is truncated");
      return;
    }
    Tensor t = read_f32(f_, shape);
    if (keep_rows >= 0) t = t.slice(0, 0, keep_rows);
    assign(sd_, local, Slice(t, how));
  }
  // The same tensor into a second parameter (an untied copy of a tied weight).
  void also(const std::string& name, const std::string& from) {
    const std::string dst = LocalName(name), src = LocalName(from);
    if (dst.empty() || src.empty() || sd_.find(dst) == sd_.end() || sd_.find(src) == sd_.end()) return;
    if (sd_.at(dst).data_ptr() != sd_.at(src).data_ptr()) assign(sd_, dst, sd_.at(src));
  }

 private:
  std::string LocalName(const std::string& name) const {
    static const std::string kLayer = "transformer.h.";
    if (name.rfind(kLayer, 0) != 0) return name;
    const size_t dot = name.find('.', kLayer.size());
    const int64_t local = model_.local_layer(std::stoll(name.substr(kLayer.size(), dot - kLayer.size())));
    return local < 0 ? std::string() : kLayer + std::to_string(local) + name.substr(dot);
  }
  Tensor Slice(const Tensor& t, Shard how) const {
    const auto& pe = parallel::env();
    const int64_t tp = pe.tp(), r = pe.tp_rank;
    if (tp == 1 || how == Shard::kReplicated) return t;
    if (how == Shard::kRows) return t.chunk(tp, 0)[r];
    if (how == Shard::kCols) return t.chunk(tp, 1)[r];
    // fused QKV: the file stacks [q | k | v]; a rank holds [q_r | k_r | v_r]
    const auto& c = model_.config;
    const int64_t q = c.n_head * c.head_dim(), kv = c.n_kv_head * c.head_dim();
    return torch::cat({t.slice(0, 0, q).chunk(tp, 0)[r], t.slice(0, q, q + kv).chunk(tp, 0)[r], t.slice(0, q + kv, q + 2 * kv).chunk(tp, 0)[r]}, 0);
  }
  std::ifstream& f_;
  nn::TransformerModel& model_;
  std::map<std::string, Tensor> sd_;
};

// GPT-2: 256 int32 header {magic 20240326, version 3 (fp32), block_size, vocab, layers, heads, width,
// padded vocab}, then the tensors kind by kind, each kind stacked over the layers.  Under tensor
// parallelism the vocabulary keeps the file's padding so that it divides among the ranks.
inline std::shared_ptr<nn::TransformerModel> LoadGPT2FromLLMC(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  TORCH_CHECK(f.is_open(), "File not found: ", path);
  int32_t h[256];
  f.read(reinterpret_cast<char*>(h), sizeof(h));
  TORCH_CHECK(f.good() && h[0] == 20240326, "not an llm.c GPT-2 weight file: ", path);
  TORCH_CHECK(h[1] == 3, "only fp32 llm.c GPT-2 files (version 3) are supported");
  auto cfg = nn::TransformerConfig::GPT2();
  const int64_t Vp = h[7];
  cfg.block_size = h[2], cfg.original_vocab_size = h[3];
  cfg.vocab_size = parallel::env().tp() > 1 ? Vp : h[3];
  cfg.n_layer = h[4], cfg.n_head = cfg.n_kv_head = h[5], cfg.n_embd = h[6];
  const int64_t L = cfg.n_layer, C = cfg.n_embd, F = cfg.ffn_hidden();
  auto model = std::make_shared<nn::TransformerModel>(cfg);
  ShardedAssigner put(f, *model);
  if (model->stage.is_last_stage) {   // one tensor in the file: the projection, and (tied or copied) the lookup table
    put.next("lm_head.weight", {Vp, C}, Shard::kRows, cfg.vocab_size);
    put.also("transformer.wte.weight", "lm_head.weight");
  } else {
    put.next("transformer.wte.weight", {Vp, C}, Shard::kRows, cfg.vocab_size);
  }
  put.next("transformer.wpe.weight", {cfg.block_size, C}, Shard::kReplicated);
  const std::vector<std::tuple<std::string, std::vector<int64_t>, Shard>> kinds = {
      {"ln_1.weight", {C}, Shard::kReplicated},          {"ln_1.bias", {C}, Shard::kReplicated},
      {"attn.c_attn.weight", {3 * C, C}, Shard::kQKVRows}, {"attn.c_attn.bias", {3 * C}, Shard::kQKVRows},
      {"attn.c_proj.weight", {C, C}, Shard::kCols},      {"attn.c_proj.bias", {C}, Shard::kReplicated},
      {"ln_2.weight", {C}, Shard::kReplicated},          {"ln_2.bias", {C}, Shard::kReplicated},
      {"mlp.c_fc.weight", {F, C}, Shard::kRows},         {"mlp.c_fc.bias", {F}, Shard::kRows},
      {"mlp.c_proj.weight", {C, F}, Shard::kCols},       {"mlp.c_proj.bias", {C}, Shard::kReplicated}};
  for (const auto& [kind, shape, how] : kinds)
    for (int64_t i = 0; i < L; ++i) put.next("transformer.h." + std::to_string(i) + "." + kind, shape, how);
  put.next("transformer.ln_f.weight", {C}, Shard::kReplicated);
  put.next("transformer.ln_f.bias", {C}, Shard::kReplicated);
  return model;
}

// LLaMA-3: 1024-byte header {magic 20240803, version 3, block_size, vocab, layers, heads, kv heads, width,
// ffn_dim_multiplier, multiple_of, norm_eps, rope_theta, use_scaled_rope, max_gen_batch, versions}.
inline std::shared_ptr<nn::TransformerModel> LoadLLaMA3FromLLMC(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  TORCH_CHECK(f.is_open(), "File not found: ", path);
  char raw[1024];
  f.read(raw, sizeof(raw));
  int32_t h[16];
  std::memcpy(h, raw, sizeof(h));
  TORCH_CHECK(f.good() && h[0] == 20240803, "not an llm.c LLaMA-3 weight file: ", path);
  TORCH_CHECK(h[1] == 3, "only fp32 llm.c LLaMA-3 files (version 3) are supported");
  float fl[4];
  std::memcpy(fl, raw + 32, 4);
  std::memcpy(fl + 1, raw + 40, 8);
  auto cfg = nn::TransformerConfig::LLaMA3();
  cfg.block_size = h[2], cfg.vocab_size = cfg.original_vocab_size = h[3];
  cfg.n_layer = h[4], cfg.n_head = h[5], cfg.n_kv_head = h[6], cfg.n_embd = h[7];
  cfg.ffn_dim_multiplier = static_cast<double>(fl[0]);
  cfg.multiple_of = h[9];
  cfg.norm_eps = fl[1], cfg.rope_theta = fl[2];
  cfg.use_scaled_rope = h[12] != 0, cfg.max_gen_batch_size = h[13];
  const int64_t L = cfg.n_layer, C = cfg.n_embd, V = cfg.vocab_size, F = cfg.ffn_hidden();
  const int64_t Q = (cfg.n_head + 2 * cfg.n_kv_head) * cfg.head_dim();
  auto model = std::make_shared<nn::TransformerModel>(cfg);
  ShardedAssigner put(f, *model);
  put.next("transformer.wte.weight", {V, C}, Shard::kRows);
  const std::vector<std::tuple<std::string, std::vector<int64_t>, Shard>> kinds = {
      {"ln_1.weight", {C}, Shard::kReplicated},    {"attn.c_attn.weight", {Q, C}, Shard::kQKVRows},
      {"attn.c_proj.weight", {C, C}, Shard::kCols}, {"ln_2.weight", {C}, Shard::kReplicated},
      {"mlp.c_fc.weight", {F, C}, Shard::kRows},   {"mlp.c_fc2.weight", {F, C}, Shard::kRows},
      {"mlp.c_proj.weight", {C, F}, Shard::kCols}};
  for (const auto& [kind, shape, how] : kinds)
    for (int64_t i = 0; i < L; ++i) put.next("transformer.h." + std::to_string(i) + "." + kind, shape, how);
  put.next("transformer.ln_f.weight", {C}, Shard::kReplicated);
  put.next("lm_head.weight", {V, C}, Shard::kRows);
  return model;
}

// ------------------------------------------------------------------ token files
// Sequential batches (x, y = x shifted by one token) of an llm.c token file; this data-parallel rank
// reads batches rank, rank + world, ...  A background thread keeps `depth` batches assembled ahead.
// Writes an llm.c token file: a 1024-byte header (magic, version, token count as int32), then the ids as
// uint16 (GPT-2: magic 20240520, version 1) or uint32 (LLaMA-3: magic 20240801, version 7)
// (reference: example/common/tiny_shakespeare_dataset.cc:27-100 reads exactly this).
inline void WriteTokenFile(const std::string& path, const std::vector<int64_t>& tokens, bool llama3 = false) {
  std::ofstream f(path, std::ios::binary);
  TORCH_CHECK(f.is_open(), "cannot write ", path);
  int32_t header[256] = {llama3 ? 20240801 : 20240520, llama3 ? 7 : 1, static_cast<int32_t>(tokens.size())};
  f.write(reinterpret_cast<const char*>(header), sizeof(header));
  for (int64_t t : tokens) {
    if (llama3) {
      const uint32_t v = static_cast<uint32_t>(t);
      f.write(reinterpret_cast<const char*>(&v), 4);
    } else {
      TORCH_CHECK(t >= 0 && t < 65536, "token ", t, " does not fit the 16-bit ids of a GPT-2 token file");
      const uint16_t v = static_cast<uint16_t>(t);
      f.write(reinterpret_cast<const char*>(&v), 2);
    }
  }
}

class TokenLoader {
 public:
  TokenLoader(const std::string& path, int64_t batch_size, int64_t sequence_length, int64_t ddp_rank = 0,
              int64_t ddp_world = 1, int64_t depth = 4)
      : file_(std::make_shared<TokenFile>(path)), B_(batch_size), T_(sequence_length) {
    for (int64_t i = 0; i < depth; ++i) {
      xs_.push_back(torch::empty({B_, T_}, torch::kInt64));
      ys_.push_back(torch::empty({B_, T_}, torch::kInt64));
    }
    std::vector<int64_t*> xp, yp;
    for (auto& t : xs_) xp.push_back(t.data_ptr<int64_t>());
    for (auto& t : ys_) yp.push_back(t.data_ptr<int64_t>());
    ring_ = std::make_unique<BatchRing>(file_, B_, T_, ddp_rank, ddp_world, xp, yp);
  }
  int64_t num_batches() const { return ring_->num_batches(); }
  // The next batch; after the last batch of the file the loader starts over.  The returned tensors
  // alias a ring slot that stays valid until two further calls.
  void next(Tensor* x, Tensor* y) {
    int64_t slot = ring_->next_slot();
    *x = xs_[slot];
    *y = ys_[slot];
  }

 private:
  std::shared_ptr<TokenFile> file_;
  int64_t B_, T_;
  std::vector<Tensor> xs_, ys_;
  std::unique_ptr<BatchRing> ring_;
};

// ------------------------------------------------------------------ checkpoints
struct TrainerState {
  int64_t global_step = 0, consumed_batches = 0;
  double last_lr = 0.0;
  int64_t n_layer = 0, n_head = 0, n_kv_head = 0, n_embd = 0, vocab_size = 0;
  int64_t ddp_size = 1, tp_size = 1, sp_size = 1, pp_size = 1;
};
inline void SaveStateDict(const std::string& path, const std::map<std::string, Tensor>& sd) {
  std::vector<std::string> names;
  std::vector<Tensor> tensors;
  for (const auto& [k, v] : sd) {
    names.push_back(k);
    tensors.push_back(v);
  }
  save_state_dict(path, names, tensors);
}
inline std::map<std::string, Tensor> LoadStateDict(const std::string& path) {
  std::map<std::string, Tensor> out;
  for (auto& [k, v] : load_state_dict(path)) out[k] = v;
  return out;
}
// Written last of a checkpoint's files and through a temporary file + rename: a trainer_state.json that exists is
// whole, and marks its directory as a complete checkpoint of its rank.
inline void SaveTrainerState(const std::string& path, const TrainerState& s) {
  const std::string tmp = path + ".tmp";
  {
    std::ofstream f(tmp);
    TORCH_CHECK(f.is_open(), "cannot write ", tmp);
    f << "{\n  \"n_layer\": " << s.n_layer << ",\n  \"n_head\": " << s.n_head << ",\n  \"n_kv_head\": " << s.n_kv_head
      << ",\n  \"n_embd\": " << s.n_embd << ",\n  \"vocab_size\": " << s.vocab_size << ",\n  \"global_step\": " << s.global_step
      << ",\n  \"consumed_batches\": " << s.consumed_batches << ",\n  \"last_lr\": " << s.last_lr << ",\n  \"ddp_size\": "
      << s.ddp_size << ",\n  \"tp_size\": " << s.tp_size << ",\n  \"sp_size\": " << s.sp_size << ",\n  \"pp_size\": " << s.pp_size
      << "\n}\n";
    f.flush();
    TORCH_CHECK(f.good(), "cannot write ", tmp);
  }
  TORCH_CHECK(std::rename(tmp.c_str(), path.c_str()) == 0, "cannot move ", tmp, " to ", path);
}
// Tolerant field scan (the reference's writer leaves out a comma after vocab_size).
inline TrainerState LoadTrainerState(const std::string& path) {
  std::ifstream f(path);
  TORCH_CHECK(f.is_open(), "Failed to open ", path);
  std::stringstream ss;
  ss << f.rdbuf();
  const std::string text = ss.str();
  auto num = [&](const char* key, double dflt) {
    std::smatch m;
    std::regex re(std::string("\"") + key + "\"\\s*:\\s*(-?[0-9.eE+-]+)");
    return std::regex_search(text, m, re) ? std::stod(m[1].str()) : dflt;
  };
  TrainerState s;
  s.global_step = static_cast<int64_t>(num("global_step", 0)), s.consumed_batches = static_cast<int64_t>(num("consumed_batches", 0));
  s.last_lr = num("last_lr", 0);
  s.n_layer = static_cast<int64_t>(num("n_layer", 0)), s.n_head = static_cast<int64_t>(num("n_head", 0));
  s.n_kv_head = static_cast<int64_t>(num("n_kv_head", 0)), s.n_embd = static_cast<int64_t>(num("n_embd", 0));
  s.vocab_size = static_cast<int64_t>(num("vocab_size", 0));
  s.ddp_size = static_cast<int64_t>(num("ddp_size", 1)), s.tp_size = static_cast<int64_t>(num("tp_size", 1));
  s.sp_size = static_cast<int64_t>(num("sp_size", 1)), s.pp_size = static_cast<int64_t>(num("pp_size", 1));
  return s;
}
// <root>/checkpoint_step_%06d/{model.ckpt, optimizer.ckpt, trainer_state.json}; a rank of a parallel job
// (global_rank >= 0) writes its slice under .../rank_%06d/ of the step directory, as the reference does
// (src/checkpoint/checkpoint_manager.cc:33-39).
inline std::string RankDirName(int global_rank) {
  char name[32];
  std::snprintf(name, sizeof(name), "rank_%06d", global_rank);
  return name;
}
inline std::string SaveCheckpoint(const std::string& root, const TrainerState& state, const Module& model,
                                  const std::map<std::string, Tensor>& optimizer_state, int global_rank = -1) {
  char name[64];
  std::snprintf(name, sizeof(name), "checkpoint_step_%06lld", static_cast<long long>(state.global_step));
  auto dir = std::filesystem::path(root) / name;
  if (global_rank >= 0) dir /= RankDirName(global_rank);
  std::filesystem::create_directories(dir);
  SaveStateDict((dir / "model.ckpt").string(), model.StateDict());
  if (!optimizer_state.empty()) SaveStateDict((dir / "optimizer.ckpt").string(), optimizer_state);
  SaveTrainerState((dir / "trainer_state.json").string(), state);
  return dir.string();
}

// <root>/checkpoint_step_* directories by step, oldest first.
inline std::vector<std::pair<int64_t, std::string>> ListCheckpoints(const std::string& root) {
  std::vector<std::pair<int64_t, std::string>> out;
  DIR* d = ::opendir(root.c_str());
  if (!d) return out;
  while (dirent* e = ::readdir(d)) {
    const std::string name = e->d_name, prefix = "checkpoint_step_";
    if (name.rfind(prefix, 0) != 0 || name.find_first_not_of("0123456789", prefix.size()) != std::string::npos) continue;
    struct stat st;
    if (::stat((root + "/" + name).c_str(), &st) == 0 && S_ISDIR(st.st_mode))
      out.emplace_back(std::stoll(name.substr(prefix.size())), root + "/" + name);
  }
  ::closedir(d);
  std::sort(out.begin(), out.end());
  return out;
}
// The newest step under <root> whose checkpoint is complete for this rank -- its trainer_state.json, the file a
// rank writes last, is there and parses (global_rank >= 0: under rank_%06d/, else in the step directory) -- or 0.
// Ranks of one job agree on a step by taking the minimum of what each of them finds.
inline int64_t NewestCompleteCheckpointStep(const std::string& root, int global_rank = -1) {
  auto all = ListCheckpoints(root);
  for (auto it = all.rbegin(); it != all.rend(); ++it) {
    const std::string dir = global_rank >= 0 ? it->second + "/" + RankDirName(global_rank) : it->second;
    try {
      if (LoadTrainerState(dir + "/trainer_state.json").global_step == it->first) return it->first;
    } catch (const std::exception&) {
    }
  }
  return 0;
}
inline std::string CheckpointDirOfStep(const std::string& root, int64_t step) {
  char name[64];
  std::snprintf(name, sizeof(name), "checkpoint_step_%06lld", static_cast<long long>(step));
  return root + "/" + name;
}

// Keeps the `keep` newest <root>/checkpoint_step_* directories (zero-padded names sort by step) and removes
// the rest (reference: src/checkpoint/checkpoint_manager.cc:103-118).  Returns how many were removed.
// Directory listing and recursive removal go through POSIX calls: std::filesystem's iterators are not
// ABI-stable across the libstdc++ the binary was compiled against and the one libtorch loads.
inline int PruneCheckpoints(const std::string& root, int64_t keep) {
  if (keep <= 0) return 0;
  auto all = ListCheckpoints(root);   // numbered step directories only, oldest first
  int removed = 0;
  while (static_cast<int64_t>(all.size()) > keep) {
    ::nftw(all.front().second.c_str(), [](const char* path, const struct stat*, int, struct FTW*) { return ::remove(path); }, 16,
           FTW_DEPTH | FTW_PHYS);
    all.erase(all.begin());
    ++removed;
  }
  return removed;
}

}  // namespace io
}  // namespace itb
