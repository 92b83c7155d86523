#include "core/framework/llama3.h"

#include <c10/util/Exception.h>

#include <algorithm>
#include <cmath>
#include <limits>
#include <random>

#include "core/llmc_io.h"

namespace infini_train {

using TP = std::shared_ptr<Tensor>;
using nn::TensorList;

namespace {
std::shared_ptr<nn::Linear> linear_no_bias(int64_t in, int64_t out) { return std::make_shared<nn::Linear>(in, out, /*bias=*/false); }
}  // namespace

LLaMA3Attention::LLaMA3Attention(const LLaMA3Config& config) : Module("CausalSelfAttention"), config_(config) {
  TORCH_CHECK(config.n_embd % config.n_head == 0 && config.n_head % config.n_kv_head == 0, "bad head configuration");
  const int64_t hd = config.head_dim();
  AddModule(kCAttnLayerName, linear_no_bias(config.n_embd, (config.n_head + 2 * config.n_kv_head) * hd));
  AddModule(kCProjLayerName, linear_no_bias(config.n_embd, config.n_embd));
  const int64_t m = std::min<int64_t>(config.block_size, 4096);
  // a buffer, so that a To(device) issued on any ancestor moves it too
  buffers_[kMaskBufferName] = std::make_shared<Tensor>(at::triu(at::ones({m, m}, at::kFloat), 1));
}
TensorList LLaMA3Attention::Forward(const TensorList& in) {
  const TP& x = in[0];
  const int64_t B = x->Dims()[0], T = x->Dims()[1], C = x->Dims()[2];
  const int64_t Hq = config_.n_head, Hkv = config_.n_kv_head, hd = config_.head_dim(), group = Hq / Hkv;
  const TP& mask = buffers_.at(kMaskBufferName);
  TORCH_CHECK(T <= mask->Dims()[0], "sequence longer than the attention mask of this facade model");
  TP qkv = modules_[kCAttnLayerName]->Forward({x})[0];                                  // [B, T, (Hq + 2 Hkv) hd]
  auto part = [&](int64_t first_head, int64_t heads) {
    return qkv->Slice(2, first_head * hd, (first_head + heads) * hd)->View({B, T, heads, hd});
  };
  auto rope = [&](const TP& t) { return std::make_shared<autograd::Rope>(config_.rope_theta, 0)->Apply({t})[0]; };
  if (x->GetDevice().IsCUDA() && qkv->Dtype() == DataType::kBFLOAT16 && (hd == 64 || hd == 128)) {
    // bf16 on the GPU: one flash-attention kernel; grouped-query heads are mapped inside it, nothing is repeated
    TP y = std::make_shared<autograd::CausalAttention>()->Apply({rope(part(0, Hq)), rope(part(Hq, Hkv)), part(Hq + Hkv, Hkv)})[0];
    return modules_[kCProjLayerName]->Forward({y->View({B, T, C})});
  }
  TP q = rope(part(0, Hq))->Transpose(1, 2);                                              // [B, Hq, T, hd]
  TP k = rope(part(Hq, Hkv))->Transpose(1, 2);                                            // [B, Hkv, T, hd]
  TP v = part(Hq + Hkv, Hkv)->Transpose(1, 2);
  if (group > 1) {                                                                        // each kv head serves `group` query heads
    k = k->RepeatInterleave(group, 1);
    v = v->RepeatInterleave(group, 1);
  }
  TP att = q->Matmul(k->Transpose(-2, -1)) * (1.0f / std::sqrt(static_cast<float>(hd)));
  att = att->MaskedFill(mask->Slice({0, 0}, {T, T}, {1, 1}), -std::numeric_limits<float>::infinity());
  att = nn::function::Softmax(att, -1);
  TP y = att->Matmul(v)->Transpose(1, 2)->Contiguous()->View({B, T, C});
  return modules_[kCProjLayerName]->Forward({y});
}

LLaMA3MLP::LLaMA3MLP(const LLaMA3Config& config) : Module("MLP") {
  AddModule(kCFcLayerName, linear_no_bias(config.n_embd, 2 * config.ffn_dim));
  AddModule(kCProjLayerName, linear_no_bias(config.ffn_dim, config.n_embd));
}
TensorList LLaMA3MLP::Forward(const TensorList& in) {
  TP h = modules_[kCFcLayerName]->Forward(in)[0];
  h = std::make_shared<autograd::SwiGLU>()->Apply({h})[0];
  return modules_[kCProjLayerName]->Forward({h});
}

LLaMA3Block::LLaMA3Block(const LLaMA3Config& config) : Module("Block") {
  AddModule("ln_1", std::make_shared<nn::RMSNorm>(config.n_embd, config.norm_eps));
  AddModule("attn", std::make_shared<LLaMA3Attention>(config));
  AddModule("ln_2", std::make_shared<nn::RMSNorm>(config.n_embd, config.norm_eps));
  AddModule("mlp", std::make_shared<LLaMA3MLP>(config));
}
TensorList LLaMA3Block::Forward(const TensorList& in) {
  TP x = in[0];
  x = x + modules_["attn"]->Forward(modules_["ln_1"]->Forward({x}))[0];
  x = x + modules_["mlp"]->Forward(modules_["ln_2"]->Forward({x}))[0];
  return {x};
}

LLaMA3::LLaMA3(const LLaMA3Config& config) : Module("LLaMA3"), config_(config) {
  std::unordered_map<std::string, std::shared_ptr<nn::Module>> tr;
  tr["wte"] = std::make_shared<nn::Embedding>(config.vocab_size, config.n_embd);
  std::vector<std::shared_ptr<nn::Module>> blocks;
  for (int64_t i = 0; i < config.n_layer; ++i) blocks.push_back(std::make_shared<LLaMA3Block>(config));
  tr["h"] = std::make_shared<nn::Sequential>(std::move(blocks));
  tr["ln_f"] = std::make_shared<nn::RMSNorm>(config.n_embd, config.norm_eps);
  AddModule("transformer", std::make_shared<nn::ModuleDict>(std::move(tr)));
  AddModule("lm_head", linear_no_bias(config.n_embd, config.vocab_size));          // untied
  // N(0, 0.02); residual projections N(0, 0.02 / sqrt(2 L)); norms stay 1; each tensor from the head of the seed-42 stream
  const float resid_std = 0.02f / std::sqrt(2.0f * static_cast<float>(config.n_layer));
  for (auto& [name, p] : StateDict()) {
    if (name.find("ln_") != std::string::npos) continue;
    const bool resid = name.find("c_proj.weight") != std::string::npos;
    nn::init::Normal(p, 0.f, resid ? resid_std : 0.02f, std::mt19937(42));
  }
}

TensorList LLaMA3::Forward(const TensorList& in) {
  const TP& idx = in[0];
  TORCH_CHECK(idx->Dims()[1] <= config_.block_size, "Cannot forward sequence of length ", idx->Dims()[1], ", block size is only ",
              config_.block_size);
  nn::Module* tr = mutable_module("transformer");
  TP x = tr->mutable_module("wte")->Forward({idx})[0];
  x = tr->mutable_module("h")->Forward({x})[0];
  x = tr->mutable_module("ln_f")->Forward({x})[0];
  return mutable_module("lm_head")->Forward({x});
}

std::unique_ptr<LLaMA3> LLaMA3::FromLLMC(const std::string& filepath) {
  titb::llmc::Llama3Header h;
  auto sd = titb::llmc::read_llama3(filepath, &h);
  LLaMA3Config cfg;
  cfg.block_size = h.max_seq_len; cfg.vocab_size = h.vocab_size; cfg.n_layer = h.n_layer; cfg.n_head = h.n_head;
  cfg.n_kv_head = h.n_kv_head; cfg.n_embd = h.n_embd; cfg.ffn_dim = h.ffn_dim; cfg.norm_eps = h.norm_eps;
  cfg.rope_theta = h.rope_theta;
  auto model = std::make_unique<LLaMA3>(cfg);
  auto own = model->StateDict();
  for (auto& [name, t] : sd) {
    auto it = own.find(name);
    TORCH_CHECK(it != own.end(), "checkpoint tensor ", name, " has no counterpart in the model");
    TORCH_CHECK(it->second->data().sizes() == t.sizes(), "shape mismatch for ", name);
    it->second->data().copy_(t);
  }
  return model;
}

}  // namespace infini_train
