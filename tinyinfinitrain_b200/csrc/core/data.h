// Datasets, the batching data loader and the llm.c tokenizer.
//
// Reference: infini_train/include/dataset.h:10-16, dataloader.h:11-42 (sequential, no
// shuffle, memcpy-stacks samples into [batch, seq] CPU tensors), example/common/
// tiny_shakespeare_dataset.{h,cc} (llm.c token .bin, tokens widened to int64 so that the
// embedding kernel can index with them) and example/common/tokenizer.{h,cc}.
// Additions: batches are assembled straight into pinned host memory so the training loop
// can issue an asynchronous H2D copy; a data-parallel rank sees every world-th batch; a
// synthetic uniform-token dataset (std::mt19937 + std::uniform_int_distribution) stands in
// where no corpus is on disk.
#pragma once
#include <ATen/ATen.h>

#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace titb {
namespace data {

class Dataset {
 public:
  virtual ~Dataset() = default;
  // (x, y): two int64 tensors of length seq_len; y is x shifted by one token.
  virtual std::pair<at::Tensor, at::Tensor> Get(size_t idx) const = 0;
  virtual size_t Size() const = 0;
  virtual int64_t SequenceLength() const = 0;
  virtual const int64_t* Tokens() const = 0;  // contiguous token stream backing the samples
};

class TinyShakespeareDataset : public Dataset {
 public:
  enum class TinyShakespeareType : int { kUINT16, kUINT32, kINVALID };
  TinyShakespeareDataset(const std::string& filepath, size_t sequence_length);
  std::pair<at::Tensor, at::Tensor> Get(size_t idx) const override;
  size_t Size() const override { return num_samples_; }
  int64_t SequenceLength() const override { return static_cast<int64_t>(sequence_length_); }
  const int64_t* Tokens() const override { return tokens_.data_ptr<int64_t>(); }
  TinyShakespeareType type() const { return type_; }
  int64_t NumTokens() const { return tokens_.numel(); }

 private:
  TinyShakespeareType type_ = TinyShakespeareType::kINVALID;
  at::Tensor tokens_;  // int64 [num_tokens]
  size_t sequence_length_ = 0;
  size_t num_samples_ = 0;
};

class SyntheticDataset : public Dataset {
 public:
  // num_samples * seq_len + 1 token ids drawn uniformly from [0, vocab_size) with mt19937(seed).
  SyntheticDataset(uint32_t seed, int64_t vocab_size, size_t sequence_length, size_t num_samples);
  std::pair<at::Tensor, at::Tensor> Get(size_t idx) const override;
  size_t Size() const override { return num_samples_; }
  int64_t SequenceLength() const override { return static_cast<int64_t>(sequence_length_); }
  const int64_t* Tokens() const override { return tokens_.data_ptr<int64_t>(); }

 private:
  at::Tensor tokens_;
  size_t sequence_length_ = 0;
  size_t num_samples_ = 0;
};

class DataLoader {
 public:
  // Rank `rank` of `world` takes batches rank, rank + world, ...  (world = 1: every batch).
  // drop_last: only full batches are served and every rank gets the same number of them (floor(full / world)),
  // which is what a job with static shapes or collectives per batch needs.
  DataLoader(std::shared_ptr<Dataset> dataset, size_t batch_size, bool pin_memory = false, size_t rank = 0,
             size_t world = 1, bool drop_last = false);
  size_t NumBatches() const { return num_batches_; }
  // Batch `i` of this rank as two [batch, seq] int64 tensors (the last batch may be short).
  std::pair<at::Tensor, at::Tensor> Batch(size_t i) const;

 private:
  std::shared_ptr<Dataset> dataset_;
  size_t batch_size_, rank_, world_, num_batches_;
  bool pin_;
};

class Tokenizer {
 public:
  enum class Version : uint32_t { kV1 = 1, kV2 = 2 };
  explicit Tokenizer(const std::string& filepath);
  std::string Decode(uint32_t token_id) const;
  uint32_t GetEndToken() const { return eot_token_; }
  uint32_t VocabSize() const { return vocab_size_; }
  uint32_t Magic() const { return magic_number_; }
  std::vector<uint32_t> Prompt() const;  // "The meaning of life is" for the file's model family

 private:
  uint32_t magic_number_ = 0, vocab_size_ = 0, eot_token_ = 0;
  std::vector<std::string> token_table_;
};

// llm.c's sampling helpers (xorshift* generator, multinomial draw from a probability row).
uint32_t RandomU32(uint64_t* state);
float RandomF32(uint64_t* state);
int SampleMult(const float* probabilities, int n, float coin);
void WriteTokenizer(const std::string& path, const std::vector<std::string>& table, uint32_t magic, uint32_t eot);

}  // namespace data
}  // namespace titb
