// GPT-2 built from the C++ facade's modules, op by op as in the reference
// (example/gpt2/net.h:13-78, net.cc:46-221): NewGELU out of elementwise ops, attention through
// Split / Transpose / Matmul / MaskedFill / Softmax.  It is the API-parity model and the C++
// oracle; the production model is the fused one in tinyinfinitrain_b200/models/gpt2.py.
// Differences from the reference: wte and lm_head are one tied tensor (listed once) and the
// lm_head has no bias.
#pragma once
#include <memory>
#include <string>

#include "core/framework/nn.h"

namespace infini_train {

struct GPT2Config {
  int64_t block_size = 1024;
  int64_t vocab_size = 50257;
  int64_t n_layer = 12;
  int64_t n_head = 12;
  int64_t n_embd = 768;
};

class NewGELU : public nn::Module {
 public:
  NewGELU() : Module("NewGELU") {}
  nn::TensorList Forward(const nn::TensorList& x) override;
};
class CausalSelfAttention : public nn::Module {
 public:
  static constexpr char kCAttnLayerName[] = "c_attn";
  static constexpr char kCProjLayerName[] = "c_proj";
  explicit CausalSelfAttention(const GPT2Config& config);
  nn::TensorList Forward(const nn::TensorList& x) override;
  static constexpr char kMaskBufferName[] = "bias";  // buffer: 1 where attention is NOT allowed, [block, block]
 private:
  GPT2Config config_;
};
class MLP : public nn::Module {
 public:
  static constexpr char kCFcLayerName[] = "c_fc";
  static constexpr char kGeluLayerName[] = "gelu";
  static constexpr char kCProjLayerName[] = "c_proj";
  explicit MLP(const GPT2Config& config);
  nn::TensorList Forward(const nn::TensorList& x) override;
};
class Block : public nn::Module {
 public:
  static constexpr char kLn1LayerName[] = "ln_1";
  static constexpr char kAttnLayerName[] = "attn";
  static constexpr char kLn2LayerName[] = "ln_2";
  static constexpr char kMlpLayerName[] = "mlp";
  explicit Block(const GPT2Config& config);
  nn::TensorList Forward(const nn::TensorList& x) override;
};
class GPT2 : public nn::Module {
 public:
  static constexpr char kTransformerLayerName[] = "transformer";
  static constexpr char kWTELayerName[] = "wte";
  static constexpr char kWPELayerName[] = "wpe";
  static constexpr char kHLayerName[] = "h";
  static constexpr char kLnFLayerName[] = "ln_f";
  static constexpr char kLMHeadLayerName[] = "lm_head";
  explicit GPT2(const GPT2Config& config);
  // {idx int64 [B, T]} -> {logits [B, T, vocab]}
  nn::TensorList Forward(const nn::TensorList& x) override;
  static std::unique_ptr<GPT2> FromLLMC(const std::string& filepath);
  static std::unique_ptr<GPT2> FromPretrained(const std::string& model_type);
  const GPT2Config& config() const { return config_; }
 private:
  GPT2Config config_;
};

}  // namespace infini_train
