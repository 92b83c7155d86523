#include "core/framework/data_facade.h"

#include <algorithm>
#include <iostream>

namespace infini_train {

DataLoaderIterator::DataLoaderIterator(const Dataset& dataset, size_t batch_size, size_t batch_idx, size_t max_batch_idx,
                                       size_t rank, size_t world)
    : dataset_(&dataset), batch_size_(batch_size), batch_idx_(batch_idx), max_batch_idx_(max_batch_idx), rank_(rank),
      world_(world) {}

TensorPair DataLoaderIterator::operator*() const {
  TORCH_CHECK(batch_idx_ < max_batch_idx_, "DataLoaderIterator dereferenced at the end");
  const size_t global = rank_ + batch_idx_ * world_;          // this rank's batch_idx-th batch
  const size_t first = global * batch_size_;
  const size_t n = std::min(batch_size_, dataset_->Size() - first);
  std::vector<at::Tensor> xs, ys;
  xs.reserve(n);
  ys.reserve(n);
  for (size_t i = 0; i < n; ++i) {
    auto [x, y] = (*dataset_)[first + i];
    xs.push_back(x->data());
    ys.push_back(y->data());
  }
  return {std::make_shared<Tensor>(at::stack(xs, 0)), std::make_shared<Tensor>(at::stack(ys, 0))};
}

DataLoaderIterator& DataLoaderIterator::operator++() {
  batch_idx_ = std::min(batch_idx_ + 1, max_batch_idx_);
  return *this;
}
DataLoaderIterator DataLoaderIterator::operator++(int) {
  DataLoaderIterator tmp = *this;
  ++(*this);
  return tmp;
}

DataLoader::DataLoader(const std::shared_ptr<Dataset>& dataset, size_t batch_size, size_t rank, size_t world)
    : dataset_(dataset), batch_size_(batch_size), rank_(rank), world_(world) {
  TORCH_CHECK(dataset && batch_size > 0 && world > 0 && rank < world, "DataLoader: bad arguments");
  const size_t total = (dataset->Size() + batch_size - 1) / batch_size;
  max_batch_idx_ = total > rank ? (total - rank + world - 1) / world : 0;
}
DataLoaderIterator DataLoader::begin() const { return {*dataset_, batch_size_, 0, max_batch_idx_, rank_, world_}; }
DataLoaderIterator DataLoader::end() const { return {*dataset_, batch_size_, max_batch_idx_, max_batch_idx_, rank_, world_}; }

std::string Tokenizer::GenerateText(nn::Module& model, uint32_t batch_size, uint32_t sequence_length, uint32_t text_length,
                                    Device device) const {
  const int64_t eot = GetEndToken();
  at::Tensor window = at::full({static_cast<int64_t>(batch_size), static_cast<int64_t>(sequence_length)}, eot, at::kLong);
  const std::vector<uint32_t> prompt = impl_.Prompt();
  TORCH_CHECK(prompt.size() <= sequence_length, "sequence_length is shorter than the prompt");
  for (size_t i = 0; i < prompt.size(); ++i) window[0][static_cast<int64_t>(i)] = static_cast<int64_t>(prompt[i]);
  std::string text = "The meaning of life is";
  uint64_t state = 1337;
  const uint32_t limit = std::min(text_length, sequence_length);
  for (uint32_t t = static_cast<uint32_t>(prompt.size()); t < limit; ++t) {
    auto x = std::make_shared<Tensor>(Tensor(window.clone()).To(device));
    auto logits = model.Forward({x})[0];                      // [batch, seq, vocab]
    at::Tensor row = logits->data()[0][static_cast<int64_t>(t) - 1].to(at::kCPU, at::kFloat);
    at::Tensor probs = at::softmax(row, 0).contiguous();
    const float coin = titb::data::RandomF32(&state);
    const int tok = titb::data::SampleMult(probs.data_ptr<float>(), static_cast<int>(probs.numel()), coin);
    window[0][static_cast<int64_t>(t)] = static_cast<int64_t>(tok);
    text += Decode(static_cast<uint32_t>(tok));
  }
  std::cout << text << std::endl;
  return text;
}

}  // namespace infini_train

infini_train::TensorPair TinyShakespeareDataset::operator[](size_t idx) const {
  auto [x, y] = impl_.Get(idx);
  return {std::make_shared<infini_train::Tensor>(x), std::make_shared<infini_train::Tensor>(y)};
}
