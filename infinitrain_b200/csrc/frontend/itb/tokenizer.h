// llm.c tokenizer files and the sampling loop of the reference's examples
// (example/common/tokenizer.cc:39-146).  File: 1024-byte header {uint32 magic 20240328 (GPT-2) or
// 20240801 (LLaMA-3), uint32 version 1|2, uint32 vocab_size, [uint32 eot when version 2]}, then
// vocab_size entries {uint8 length, bytes}.  Sampling: xorshift* generator seeded with 1337,
// multinomial draw from the softmax of position t - 1, prompt "The meaning of life is".
#pragma once
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "module.h"

namespace itb {
namespace data {

inline uint32_t RandomU32(uint64_t& state) {
  state ^= state >> 12;
  state ^= state << 25;
  state ^= state >> 27;
  return static_cast<uint32_t>((state * 0x2545F4914F6CDD1Dull) >> 32);
}
inline float RandomF32(uint64_t& state) { return (RandomU32(state) >> 8) / 16777216.0f; }
// Index of the first cumulative probability above `coin` (the last index when rounding leaves none).
inline int64_t SampleMult(const float* probabilities, int64_t n, float coin) {
  float cdf = 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    cdf += probabilities[i];
    if (coin < cdf) return i;
  }
  return n - 1;
}

class Tokenizer {
 public:
  static constexpr uint32_t kGpt2Magic = 20240328, kLlama3Magic = 20240801;
  explicit Tokenizer(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    TORCH_CHECK(f.is_open(), "Failed to open tokenizer file: ", path);
    char header[1024];
    f.read(header, sizeof(header));
    uint32_t h[4];
    std::memcpy(h, header, sizeof(h));
    magic_ = h[0];
    TORCH_CHECK(magic_ == kGpt2Magic || magic_ == kLlama3Magic, "Unsupported tokenizer magic: ", magic_);
    if (h[1] == 1) eot_ = magic_ == kGpt2Magic ? 50256 : 128001;
    else if (h[1] == 2) eot_ = h[3];
    else TORCH_CHECK(false, "Unsupported tokenizer version: ", h[1]);
    table_.resize(h[2]);
    for (auto& tok : table_) {
      uint8_t len = 0;
      f.read(reinterpret_cast<char*>(&len), 1);
      tok.resize(len);
      f.read(tok.data(), len);
    }
    TORCH_CHECK(f.good(), "tokenizer file is truncated: ", path);
  }
  std::string Decode(int64_t token) const {
    return token >= 0 && token < static_cast<int64_t>(table_.size()) ? table_[token] : "[INVALID_TOKEN]";
  }
  int64_t GetEndOfText() const { return eot_; }
  int64_t vocab_size() const { return static_cast<int64_t>(table_.size()); }
  std::vector<int64_t> Prompt() const {
    return magic_ == kGpt2Magic ? std::vector<int64_t>{464, 3616, 286, 1204, 318} : std::vector<int64_t>{791, 7438, 315, 2324, 374};
  }

  // Re-runs the whole [batch, sequence] window for every new token and samples position t - 1 of row
  // 0; `forward` maps token ids [B, T] to logits [B, T, V].  Returns the text; `tokens` gets the ids.
  template <class Forward>
  std::string GenerateText(Forward&& forward, int64_t batch_size, int64_t sequence_length, int64_t text_length,
                           torch::Device device, std::vector<int64_t>* tokens = nullptr) const {
    torch::NoGradGuard no_grad;
    Tensor x = torch::full({batch_size, sequence_length}, eot_, torch::kInt64);
    auto prompt = Prompt();
    int64_t* xb = x.data_ptr<int64_t>();
    for (size_t i = 0; i < prompt.size(); ++i) xb[i] = prompt[i];
    uint64_t rng = 1337;
    std::string text = "The meaning of life is";
    for (int64_t t = static_cast<int64_t>(prompt.size()); t < text_length; ++t) {
      Tensor logits = forward(x.to(device));
      Tensor probs = torch::softmax(logits[0][t - 1].to(torch::kFloat32), -1).to(torch::kCPU).contiguous();
      int64_t next = SampleMult(probs.data_ptr<float>(), probs.numel(), RandomF32(rng));
      xb[t] = next;
      if (tokens) tokens->push_back(next);
      text += Decode(next);
    }
    return text;
  }

 private:
  uint32_t magic_ = 0;
  int64_t eot_ = 0;
  std::vector<std::string> table_;
};

}  // namespace data
}  // namespace itb
