#include "core/data.h"

#include <c10/util/Exception.h>

#include <cstdio>
#include <cstring>
#include <random>

#include "core/llmc_io.h"
#include "core/rng.h"

namespace titb {
namespace data {

namespace {
std::pair<at::Tensor, at::Tensor> sample_views(const at::Tensor& tokens, size_t idx, size_t T) {
  const int64_t off = static_cast<int64_t>(idx * T);
  return {tokens.narrow(0, off, T), tokens.narrow(0, off + 1, T)};
}
}  // namespace

TinyShakespeareDataset::TinyShakespeareDataset(const std::string& filepath, size_t sequence_length)
    : sequence_length_(sequence_length) {
  TORCH_CHECK(sequence_length > 0, "sequence_length must be positive");
  int32_t magic = 0;
  tokens_ = llmc::read_tokens(filepath, &magic);
  type_ = magic == llmc::kDataMagicU16 ? TinyShakespeareType::kUINT16 : TinyShakespeareType::kUINT32;
  const int64_t n = tokens_.numel();
  num_samples_ = n > 1 ? static_cast<size_t>((n - 1) / static_cast<int64_t>(sequence_length)) : 0;
}

std::pair<at::Tensor, at::Tensor> TinyShakespeareDataset::Get(size_t idx) const {
  TORCH_CHECK(idx < num_samples_, "sample index ", idx, " out of range (", num_samples_, ")");
  return sample_views(tokens_, idx, sequence_length_);
}

SyntheticDataset::SyntheticDataset(uint32_t seed, int64_t vocab_size, size_t sequence_length, size_t num_samples)
    : sequence_length_(sequence_length), num_samples_(num_samples) {
  tokens_ = at::empty({static_cast<int64_t>(num_samples * sequence_length + 1)}, at::kLong);
  rng::fill_randint(tokens_.data_ptr<int64_t>(), tokens_.numel(), 0, vocab_size, seed);
}

std::pair<at::Tensor, at::Tensor> SyntheticDataset::Get(size_t idx) const {
  TORCH_CHECK(idx < num_samples_, "sample index ", idx, " out of range (", num_samples_, ")");
  return sample_views(tokens_, idx, sequence_length_);
}

DataLoader::DataLoader(std::shared_ptr<Dataset> dataset, size_t batch_size, bool pin_memory, size_t rank, size_t world,
                       bool drop_last)
    : dataset_(std::move(dataset)), batch_size_(batch_size), rank_(rank), world_(world), pin_(pin_memory) {
  TORCH_CHECK(batch_size_ > 0 && world_ > 0 && rank_ < world_, "bad DataLoader arguments");
  if (drop_last) {
    num_batches_ = (dataset_->Size() / batch_size_) / world_;
  } else {
    const size_t total = (dataset_->Size() + batch_size_ - 1) / batch_size_;
    num_batches_ = total > rank_ ? (total - rank_ + world_ - 1) / world_ : 0;
  }
}

std::pair<at::Tensor, at::Tensor> DataLoader::Batch(size_t i) const {
  TORCH_CHECK(i < num_batches_, "batch index ", i, " out of range (", num_batches_, ")");
  const size_t global = rank_ + i * world_;
  const size_t first = global * batch_size_;
  const size_t n = std::min(batch_size_, dataset_->Size() - first);
  const int64_t T = dataset_->SequenceLength();
  auto opts = at::TensorOptions().dtype(at::kLong).pinned_memory(pin_);
  at::Tensor x = at::empty({static_cast<int64_t>(n), T}, opts), y = at::empty({static_cast<int64_t>(n), T}, opts);
  const int64_t* tok = dataset_->Tokens();
  for (size_t s = 0; s < n; ++s) {  // samples are contiguous windows of the token stream
    const int64_t off = static_cast<int64_t>((first + s)) * T;
    std::memcpy(x.data_ptr<int64_t>() + s * T, tok + off, sizeof(int64_t) * T);
    std::memcpy(y.data_ptr<int64_t>() + s * T, tok + off + 1, sizeof(int64_t) * T);
  }
  return {x, y};
}

// --------------------------------------------------------------------------- tokenizer
namespace {
constexpr uint32_t kTokMagicGpt2 = 20240328, kTokMagicLlama3 = 20240801;
}

Tokenizer::Tokenizer(const std::string& filepath) {
  FILE* f = std::fopen(filepath.c_str(), "rb");
  TORCH_CHECK(f != nullptr, "File not found: ", filepath);
  uint32_t h[256];
  const bool ok = std::fread(h, sizeof(uint32_t), 256, f) == 256;
  if (!ok) std::fclose(f);
  TORCH_CHECK(ok, "tokenizer file too short");
  magic_number_ = h[0];
  const uint32_t version = h[1];
  vocab_size_ = h[2];
  if (magic_number_ == kTokMagicGpt2) eot_token_ = 50256;
  else if (magic_number_ == kTokMagicLlama3) eot_token_ = 128001;
  else { std::fclose(f); TORCH_CHECK(false, "unknown tokenizer magic ", magic_number_); }
  if (version == static_cast<uint32_t>(Version::kV2)) eot_token_ = h[3];
  token_table_.resize(vocab_size_);
  for (uint32_t i = 0; i < vocab_size_; ++i) {
    unsigned char len = 0;
    if (std::fread(&len, 1, 1, f) != 1) break;
    std::string s(len, '\0');
    if (len && std::fread(s.data(), 1, len, f) != len) break;
    token_table_[i] = std::move(s);
  }
  std::fclose(f);
}

std::string Tokenizer::Decode(uint32_t token_id) const {
  return token_id < token_table_.size() ? token_table_[token_id] : std::string();
}

std::vector<uint32_t> Tokenizer::Prompt() const {
  if (magic_number_ == kTokMagicLlama3) return {791, 7438, 315, 2324, 374};
  return {464, 3616, 286, 1204, 318};
}

uint32_t RandomU32(uint64_t* state) {
  uint64_t s = *state;
  s ^= s >> 12;
  s ^= s << 25;
  s ^= s >> 27;
  *state = s;
  return static_cast<uint32_t>((s * 0x2545F4914F6CDD1Dull) >> 32);
}
float RandomF32(uint64_t* state) { return (RandomU32(state) >> 8) / 16777216.0f; }

int SampleMult(const float* probabilities, int n, float coin) {
  float cdf = 0.f;
  for (int i = 0; i < n; ++i) {
    cdf += probabilities[i];
    if (coin < cdf) return i;
  }
  return n - 1;  // rounding
}

void WriteTokenizer(const std::string& path, const std::vector<std::string>& table, uint32_t magic, uint32_t eot) {
  FILE* f = std::fopen(path.c_str(), "wb");
  TORCH_CHECK(f != nullptr, "cannot write ", path);
  uint32_t h[256];
  std::memset(h, 0, sizeof(h));
  h[0] = magic; h[1] = 2; h[2] = static_cast<uint32_t>(table.size()); h[3] = eot;
  std::fwrite(h, sizeof(uint32_t), 256, f);
  for (const auto& s : table) {
    const unsigned char len = static_cast<unsigned char>(std::min<size_t>(s.size(), 255));
    std::fwrite(&len, 1, 1, f);
    std::fwrite(s.data(), 1, len, f);
  }
  std::fclose(f);
}

}  // namespace data
}  // namespace titb
