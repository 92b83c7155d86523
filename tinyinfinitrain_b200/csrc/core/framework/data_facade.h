// Dataset / DataLoader / TinyShakespeareDataset / Tokenizer with the reference's C++ signatures
// (infini_train/include/dataset.h:10-16, dataloader.h:11-42, example/common/tiny_shakespeare_dataset.h,
// example/common/tokenizer.h), as thin adapters over the data core (core/data.h), which works on at::Tensor.
//
// Differences from the reference, on purpose: tokens are widened to int64 once at load (the reference's
// operator[] returns views shifted by sizeof(int64_t) into a pre-widened buffer: tiny_shakespeare_dataset.cc:74-82);
// the loader takes an optional (rank, world) pair so data-parallel ranks read disjoint batches; batches can be
// assembled in pinned memory.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "core/data.h"
#include "core/framework/nn.h"
#include "core/framework/tensor.h"

namespace infini_train {

using TensorPair = std::pair<std::shared_ptr<Tensor>, std::shared_ptr<Tensor>>;

class Dataset {
 public:
  virtual ~Dataset() = default;
  virtual TensorPair operator[](size_t idx) const = 0;
  virtual size_t Size() const = 0;
};

class DataLoaderIterator {
 public:
  DataLoaderIterator(const Dataset& dataset, size_t batch_size, size_t batch_idx, size_t max_batch_idx, size_t rank,
                     size_t world);
  // Two [batch, ...] CPU tensors stacked from `batch_size` consecutive samples (the last batch may be short).
  TensorPair operator*() const;
  DataLoaderIterator& operator++();      // saturates at the end, as in the reference
  DataLoaderIterator operator++(int);
  friend bool operator<(const DataLoaderIterator& a, const DataLoaderIterator& b) { return a.batch_idx_ < b.batch_idx_; }
  friend bool operator!=(const DataLoaderIterator& a, const DataLoaderIterator& b) { return a.batch_idx_ != b.batch_idx_; }
  friend bool operator==(const DataLoaderIterator& a, const DataLoaderIterator& b) { return a.batch_idx_ == b.batch_idx_; }

 private:
  const Dataset* dataset_ = nullptr;  // not owned
  size_t batch_size_ = 0, batch_idx_ = 0, max_batch_idx_ = 0, rank_ = 0, world_ = 1;
};

class DataLoader {
 public:
  DataLoader(const std::shared_ptr<Dataset>& dataset, size_t batch_size, size_t rank = 0, size_t world = 1);
  DataLoaderIterator begin() const;
  DataLoaderIterator end() const;
  size_t NumBatches() const { return max_batch_idx_; }

 private:
  std::shared_ptr<Dataset> dataset_;
  size_t batch_size_ = 0, max_batch_idx_ = 0, rank_ = 0, world_ = 1;
};

class Tokenizer {
 public:
  enum class Version : uint32_t { kV1 = 1, kV2 = 2 };
  explicit Tokenizer(const std::string& filepath) : impl_(filepath) {}
  std::string Decode(uint32_t token_id) const { return impl_.Decode(token_id); }
  uint32_t GetEndToken() const { return impl_.GetEndToken(); }
  // Fills a [batch, seq] window with the end token, writes the prompt "The meaning of life is" into row 0 and samples
  // `text_length` - prompt tokens one at a time with llm.c's generator (state 1337), re-running the whole window per
  // token like the reference (tokenizer.cc:91-116).  Prints the text to stdout and returns it.
  std::string GenerateText(nn::Module& model, uint32_t batch_size, uint32_t sequence_length, uint32_t text_length,
                           Device device) const;

 private:
  titb::data::Tokenizer impl_;
};

}  // namespace infini_train

// The reference declares this class in the global namespace (example/common/tiny_shakespeare_dataset.h).
class TinyShakespeareDataset : public infini_train::Dataset {
 public:
  using TinyShakespeareType = titb::data::TinyShakespeareDataset::TinyShakespeareType;
  TinyShakespeareDataset(const std::string& filepath, size_t sequence_length) : impl_(filepath, sequence_length) {}
  infini_train::TensorPair operator[](size_t idx) const override;
  size_t Size() const override { return impl_.Size(); }
  TinyShakespeareType type() const { return impl_.type(); }

 private:
  titb::data::TinyShakespeareDataset impl_;
};
