// llm.c token files and the prefetching batch ring, free of any framework dependency so that they
// can be built and exercised on their own (unit tests under ThreadSanitizer / AddressSanitizer).
//
// File: 1024-byte header (int32 magic 20240520 -> uint16 tokens, 20240801 -> uint32 tokens; int32
// version; int32 num_tokens), then the tokens.  Sample i is x = tok[i*T, i*T+T), y = x shifted by 1
// (reference: example/common/tiny_shakespeare_dataset.cc:27-118).
#pragma once
#include <fcntl.h>
#include <stdint.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <condition_variable>
#include <cstring>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace itb {

class TokenFile {
 public:
  explicit TokenFile(const std::string& path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("cannot open token file: " + path);
    struct stat st;
    if (fstat(fd_, &st) != 0) fail("fstat failed: " + path);
    size_ = static_cast<size_t>(st.st_size);
    if (size_ < 1024) fail("token file too small: " + path);
    void* m = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (m == MAP_FAILED) fail("mmap failed: " + path);
    base_ = static_cast<const uint8_t*>(m);
    int32_t h[3];
    std::memcpy(h, base_, sizeof(h));
    magic_ = h[0];
    version_ = h[1];
    num_tokens_ = h[2];
    if (magic_ == 20240520) bytes_per_token_ = 2;
    else if (magic_ == 20240801) bytes_per_token_ = 4;
    else fail("unknown token file magic " + std::to_string(magic_));
    if (num_tokens_ < 0 || 1024 + static_cast<size_t>(num_tokens_) * bytes_per_token_ > size_)
      fail("token file truncated: " + path);
  }
  TokenFile(const TokenFile&) = delete;
  TokenFile& operator=(const TokenFile&) = delete;
  ~TokenFile() { release(); }
  int64_t num_tokens() const { return num_tokens_; }
  int64_t magic() const { return magic_; }
  int64_t version() const { return version_; }
  inline int64_t token(int64_t i) const {
    const uint8_t* p = base_ + 1024 + i * bytes_per_token_;
    if (bytes_per_token_ == 2) {
      uint16_t v;
      std::memcpy(&v, p, 2);
      return v;
    }
    uint32_t v;
    std::memcpy(&v, p, 4);
    return v;
  }
  // x[b, t] = tok[(first + b) * T + t], y shifted by one token.
  void fill(int64_t first_sample, int64_t B, int64_t T, int64_t* x, int64_t* y) const {
    for (int64_t b = 0; b < B; ++b) {
      const int64_t s = (first_sample + b) * T;
      for (int64_t t = 0; t < T; ++t) {
        x[b * T + t] = token(s + t);
        y[b * T + t] = token(s + t + 1);
      }
    }
  }

 private:
  void release() {
    if (base_) munmap(const_cast<uint8_t*>(base_), size_);
    if (fd_ >= 0) ::close(fd_);
    base_ = nullptr;
    fd_ = -1;
  }
  [[noreturn]] void fail(const std::string& what) {
    release();
    throw std::runtime_error(what);
  }
  int fd_ = -1;
  size_t size_ = 0;
  const uint8_t* base_ = nullptr;
  int32_t magic_ = 0, version_ = 0, num_tokens_ = 0;
  int bytes_per_token_ = 2;
};

// Assembles batches on a background thread into a ring of caller-owned buffers (x and y of B*T
// int64 each per slot); `next_slot()` hands out the oldest ready slot, which stays untouched until two
// further calls.  Batch k covers samples [(start_batch + k * stride) * B, ... + B), wrapping around:
// rank r of dp ranks uses start_batch = r, stride = dp.
class BatchRing {
 public:
  BatchRing(std::shared_ptr<TokenFile> file, int64_t B, int64_t T, int64_t start_batch, int64_t stride,
            std::vector<int64_t*> xs, std::vector<int64_t*> ys)
      : file_(std::move(file)), B_(B), T_(T), start_(start_batch), stride_(stride),
        depth_(static_cast<int64_t>(xs.size())), xs_(std::move(xs)), ys_(std::move(ys)) {
    if (!(B > 0 && T > 0 && stride > 0 && depth_ >= 3 && ys_.size() == xs_.size()))
      throw std::runtime_error("TokenBatcher: bad arguments (depth >= 3)");
    num_samples_ = file_->num_tokens() / T - 1;   // the last sample needs one token of look-ahead
    if (num_samples_ < B) throw std::runtime_error("token file holds fewer samples than one batch");
    num_batches_ = num_samples_ / B;
    worker_ = std::thread([this] { this->run(); });
  }
  BatchRing(const BatchRing&) = delete;
  BatchRing& operator=(const BatchRing&) = delete;
  ~BatchRing() {
    {
      std::lock_guard<std::mutex> g(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    if (worker_.joinable()) worker_.join();
  }
  int64_t num_batches() const { return num_batches_; }
  int64_t next_slot() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [this] { return produced_ > consumed_ || stop_; });
    const int64_t slot = consumed_ % depth_;
    ++consumed_;
    lk.unlock();
    cv_.notify_all();
    return slot;
  }

 private:
  void run() {
    int64_t k = 0, produced = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> lk(mu_);
        // the two slots handed out last may still be read by the consumer: never refill them
        cv_.wait(lk, [this] { return stop_ || produced_ - consumed_ < depth_ - 2; });
        if (stop_) return;
      }
      const int64_t batch = (start_ + k * stride_) % num_batches_;
      const int64_t slot = produced % depth_;
      file_->fill(batch * B_, B_, T_, xs_[slot], ys_[slot]);
      ++k;
      ++produced;
      {
        std::lock_guard<std::mutex> g(mu_);
        produced_ = produced;
      }
      cv_.notify_all();
    }
  }
  std::shared_ptr<TokenFile> file_;
  int64_t B_, T_, start_, stride_, depth_;
  std::vector<int64_t*> xs_, ys_;
  int64_t num_samples_ = 0, num_batches_ = 0;
  std::thread worker_;
  std::mutex mu_;
  std::condition_variable cv_;
  int64_t produced_ = 0, consumed_ = 0;
  bool stop_ = false;
};

}  // namespace itb
