// Datasets and loaders of the C++ frontend in the reference's shape: an indexable Dataset of
// (input, target) samples, a DataLoader that stacks `batch_size` consecutive samples, and a
// DistributedDataLoader whose rank r reads batches r, r + W, r + 2 W, ...; no shuffling.
//
// Reference: infini_train/include/dataset.h:11-17, include/dataloader.h:11-58, src/dataloader.cc:17-102
// (iterators compared by batch index, samples stacked on the training thread),
// example/common/tiny_shakespeare_dataset.cc:27-118 (llm.c token file: sample i is tokens
// [i T, (i + 1) T) with the target shifted by one token inside the flat stream).
// TokenLoader (io.h) is the prefetching equivalent the trainer uses: same batches, assembled by a
// background thread; these classes are for programs written against the reference's iteration
// protocol and for datasets that are not token files.
#pragma once
#include <cstdint>
#include <fstream>
#include <memory>
#include <string>
#include <utility>

#include "../../runtime/token_io.h"
#include "module.h"

namespace itb {
namespace data {

class Dataset {
 public:
  virtual ~Dataset() = default;
  virtual std::pair<Tensor, Tensor> operator[](size_t idx) const = 0;
  virtual size_t Size() const = 0;
};

// Samples of `sequence_length` tokens out of an llm.c token file (uint16 GPT-2 ids or uint32 LLaMA-3 ids).
class TinyShakespeareDataset : public Dataset {
 public:
  TinyShakespeareDataset(const std::string& path, int64_t sequence_length)
      : file_(std::make_shared<TokenFile>(path)), T_(sequence_length) {
    TORCH_CHECK(T_ > 0, "sequence_length must be positive");
    // every sample needs one token past its end for the shifted target
    n_ = file_->num_tokens() > 0 ? static_cast<size_t>((file_->num_tokens() - 1) / T_) : 0;
  }
  std::pair<Tensor, Tensor> operator[](size_t idx) const override {
    TORCH_CHECK(idx < n_, "sample ", idx, " of ", n_);
    Tensor x = torch::empty({T_}, torch::kInt64), y = torch::empty({T_}, torch::kInt64);
    int64_t *xp = x.data_ptr<int64_t>(), *yp = y.data_ptr<int64_t>();
    const int64_t base = static_cast<int64_t>(idx) * T_;
    for (int64_t t = 0; t < T_; ++t) {
      xp[t] = file_->token(base + t);
      yp[t] = file_->token(base + t + 1);
    }
    return {x, y};
  }
  size_t Size() const override { return n_; }
  int64_t sequence_length() const { return T_; }

 private:
  std::shared_ptr<TokenFile> file_;
  int64_t T_;
  size_t n_;
};

// Any pair of tensors whose first dimension indexes the samples.
class TensorDataset : public Dataset {
 public:
  TensorDataset(Tensor inputs, Tensor targets) : x_(std::move(inputs)), y_(std::move(targets)) {
    TORCH_CHECK(x_.size(0) == y_.size(0), "inputs and targets differ in their number of samples");
  }
  std::pair<Tensor, Tensor> operator[](size_t idx) const override { return {x_[static_cast<int64_t>(idx)], y_[static_cast<int64_t>(idx)]}; }
  size_t Size() const override { return static_cast<size_t>(x_.size(0)); }

 private:
  Tensor x_, y_;
};

// An IDX file of unsigned bytes (the MNIST distribution format): big-endian magic 0x0000 08 <ndim>, then one
// big-endian uint32 per dimension, then the bytes (reference: example/mnist/dataset.cc:45-80).
inline Tensor ReadIdxFile(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  TORCH_CHECK(f.good(), "cannot open IDX file ", path);
  unsigned char head[4];
  f.read(reinterpret_cast<char*>(head), 4);
  TORCH_CHECK(f.gcount() == 4 && head[0] == 0 && head[1] == 0, "not an IDX file: ", path);
  TORCH_CHECK(head[2] == 0x08, "IDX file ", path, " does not hold unsigned bytes (type code ", int(head[2]), ")");
  const int ndim = head[3];
  TORCH_CHECK(ndim >= 1 && ndim <= 8, "IDX file ", path, " has ", ndim, " dimensions");
  std::vector<int64_t> dims;
  int64_t count = 1;
  for (int i = 0; i < ndim; ++i) {
    unsigned char b[4];
    f.read(reinterpret_cast<char*>(b), 4);
    TORCH_CHECK(f.gcount() == 4, "IDX file ", path, " ends inside its header");
    dims.push_back((int64_t(b[0]) << 24) | (int64_t(b[1]) << 16) | (int64_t(b[2]) << 8) | int64_t(b[3]));
    count *= dims.back();
  }
  Tensor out = torch::empty(dims, torch::kUInt8);
  f.read(reinterpret_cast<char*>(out.data_ptr<uint8_t>()), count);
  TORCH_CHECK(f.gcount() == count, "IDX file ", path, " holds ", f.gcount(), " of the ", count, " bytes its header announces");
  return out;
}

// MNIST out of `<dir>/{train,t10k}-images-idx3-ubyte` and `-labels-idx1-ubyte`: sample i is the image as
// fp32 [28, 28] scaled to [0, 1] and its label as one uint8 (reference: example/mnist/dataset.cc:82-125).
class MNISTDataset : public Dataset {
 public:
  MNISTDataset(const std::string& dir, bool train) {
    const std::string prefix = dir + "/" + (train ? "train" : "t10k");
    Tensor images = ReadIdxFile(prefix + "-images-idx3-ubyte");
    labels_ = ReadIdxFile(prefix + "-labels-idx1-ubyte");
    TORCH_CHECK(images.dim() == 3 && labels_.dim() == 1 && images.size(0) == labels_.size(0),
                "MNIST files under ", dir, " disagree: images ", images.sizes(), ", labels ", labels_.sizes());
    images_ = images.to(torch::kFloat32) / 255.0f;
  }
  std::pair<Tensor, Tensor> operator[](size_t idx) const override {
    TORCH_CHECK(idx < Size(), "sample ", idx, " of ", Size());
    return {images_[static_cast<int64_t>(idx)], labels_[static_cast<int64_t>(idx)]};
  }
  size_t Size() const override { return static_cast<size_t>(labels_.size(0)); }

 private:
  Tensor images_, labels_;
};

class DataLoaderIterator {
 public:
  DataLoaderIterator(const Dataset* dataset, size_t batch_size, size_t batch_idx, size_t max_batch_idx, size_t stride = 1)
      : dataset_(dataset), batch_size_(batch_size), batch_idx_(batch_idx), max_batch_idx_(max_batch_idx), stride_(stride) {
    if (batch_idx_ > max_batch_idx_) batch_idx_ = max_batch_idx_;
  }
  // [batch, ...] inputs and targets of batch `BatchIndex()`
  std::pair<Tensor, Tensor> operator*() const {
    TORCH_CHECK(batch_idx_ < max_batch_idx_, "dereferenced the end of a DataLoader");
    std::vector<Tensor> xs, ys;
    for (size_t i = 0; i < batch_size_; ++i) {
      auto s = (*dataset_)[batch_idx_ * batch_size_ + i];
      xs.push_back(s.first);
      ys.push_back(s.second);
    }
    return {torch::stack(xs), torch::stack(ys)};
  }
  DataLoaderIterator& operator++() {
    batch_idx_ = batch_idx_ + stride_ < max_batch_idx_ ? batch_idx_ + stride_ : max_batch_idx_;
    return *this;
  }
  DataLoaderIterator operator++(int) {
    DataLoaderIterator old = *this;
    ++*this;
    return old;
  }
  friend bool operator<(const DataLoaderIterator& a, const DataLoaderIterator& b) { return a.batch_idx_ < b.batch_idx_; }
  friend bool operator!=(const DataLoaderIterator& a, const DataLoaderIterator& b) { return a.batch_idx_ != b.batch_idx_; }
  friend bool operator==(const DataLoaderIterator& a, const DataLoaderIterator& b) { return a.batch_idx_ == b.batch_idx_; }
  size_t BatchIndex() const { return batch_idx_; }

 private:
  const Dataset* dataset_;   // not owned
  size_t batch_size_, batch_idx_, max_batch_idx_, stride_;
};

// Full batches only: a ragged last batch is dropped (the reference yields it and is undefined past it).
class DataLoader {
 public:
  DataLoader(std::shared_ptr<Dataset> dataset, size_t batch_size) : dataset_(std::move(dataset)), batch_size_(batch_size) {
    TORCH_CHECK(batch_size_ > 0, "batch_size must be positive");
    max_batch_idx_ = dataset_->Size() / batch_size_;
  }
  virtual ~DataLoader() = default;
  virtual DataLoaderIterator begin() const { return DataLoaderIterator(dataset_.get(), batch_size_, 0, max_batch_idx_); }
  virtual DataLoaderIterator end() const { return DataLoaderIterator(dataset_.get(), batch_size_, max_batch_idx_, max_batch_idx_); }
  size_t num_batches() const { return max_batch_idx_; }

 protected:
  std::shared_ptr<Dataset> dataset_;
  size_t batch_size_, max_batch_idx_ = 0;
};

class DistributedDataLoader : public DataLoader {
 public:
  DistributedDataLoader(std::shared_ptr<Dataset> dataset, size_t batch_size, size_t ddp_rank, size_t ddp_world_size)
      : DataLoader(std::move(dataset), batch_size), ddp_rank_(ddp_rank), ddp_world_size_(ddp_world_size) {
    TORCH_CHECK(ddp_world_size_ > 0 && ddp_rank_ < ddp_world_size_, "bad data-parallel coordinates");
  }
  DataLoaderIterator begin() const override {
    return DataLoaderIterator(dataset_.get(), batch_size_, ddp_rank_, max_batch_idx_, ddp_world_size_);
  }
  DataLoaderIterator end() const override {
    return DataLoaderIterator(dataset_.get(), batch_size_, max_batch_idx_, max_batch_idx_, ddp_world_size_);
  }

 private:
  size_t ddp_rank_, ddp_world_size_;
};

}  // namespace data
}  // namespace itb
