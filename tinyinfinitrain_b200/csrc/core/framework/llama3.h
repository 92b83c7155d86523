// LLaMA-3 built from the C++ facade's modules: RMSNorm, rotary embedding (theta 500000, pairs (i, i + hd/2)),
// grouped-query causal attention, SwiGLU feed-forward, untied output head.  The reference ships no LLaMA model
// (only the dataset magic 20240801 and the tokenizer's end token 128001: example/common/tiny_shakespeare_dataset.cc:27-30,
// example/common/tokenizer.cc:14-25); module and parameter names follow the GPT-2 example so that StateDict keys
// line up with the Python model and with the llm.c-style checkpoint reader (core/llmc_io.h).
// Attention is composed from the facade's Functions (Slice / Rope / RepeatInterleave / Matmul / MaskedFill / Softmax);
// the production model with fused kernels is tinyinfinitrain_b200/models/llama3.py.
#pragma once
#include <memory>
#include <string>

#include "core/framework/nn.h"

namespace infini_train {

struct LLaMA3Config {
  int64_t block_size = 8192;
  int64_t vocab_size = 128256;
  int64_t n_layer = 16;
  int64_t n_head = 32;
  int64_t n_kv_head = 8;
  int64_t n_embd = 2048;
  int64_t ffn_dim = 8192;
  float norm_eps = 1e-5f;
  float rope_theta = 500000.f;
  int64_t head_dim() const { return n_embd / n_head; }
};

class LLaMA3Attention : public nn::Module {
 public:
  static constexpr char kCAttnLayerName[] = "c_attn";   // rows: q heads | k heads | v heads
  static constexpr char kCProjLayerName[] = "c_proj";
  explicit LLaMA3Attention(const LLaMA3Config& config);
  nn::TensorList Forward(const nn::TensorList& x) override;
  static constexpr char kMaskBufferName[] = "bias";  // buffer: 1 where attention is NOT allowed (min(block, 4096) square)
 private:
  LLaMA3Config config_;
};
class LLaMA3MLP : public nn::Module {
 public:
  static constexpr char kCFcLayerName[] = "c_fc";       // rows: gate | up
  static constexpr char kCProjLayerName[] = "c_proj";
  explicit LLaMA3MLP(const LLaMA3Config& config);
  nn::TensorList Forward(const nn::TensorList& x) override;
};
class LLaMA3Block : public nn::Module {
 public:
  explicit LLaMA3Block(const LLaMA3Config& config);
  nn::TensorList Forward(const nn::TensorList& x) override;
};
class LLaMA3 : public nn::Module {
 public:
  explicit LLaMA3(const LLaMA3Config& config);
  // {idx int64 [B, T]} -> {logits [B, T, vocab]}
  nn::TensorList Forward(const nn::TensorList& x) override;
  static std::unique_ptr<LLaMA3> FromLLMC(const std::string& filepath);
  const LLaMA3Config& config() const { return config_; }
 private:
  LLaMA3Config config_;
};

}  // namespace infini_train
