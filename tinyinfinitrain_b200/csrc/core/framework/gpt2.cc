#include "core/framework/gpt2.h"

#include <c10/util/Exception.h>

#include <cmath>
#include <limits>
#include <random>

#include "core/llmc_io.h"

namespace infini_train {

using TP = std::shared_ptr<Tensor>;
using nn::TensorList;

TensorList NewGELU::Forward(const TensorList& in) {
  const TP& x = in[0];
  // On the GPU the activation is one kernel; on the CPU it stays the reference's chain of element-wise
  // Functions so that CPU results match the reference operation for operation.
  if (x->GetDevice().IsCUDA()) return std::make_shared<autograd::Gelu>()->Apply({x});
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
  TP inner = (x + x->Pow(3.0f) * 0.044715f) * std::sqrt(2.0f / static_cast<float>(M_PI));
  return {(x * 0.5f) * (inner->Tanh() + 1.0f)};
}

CausalSelfAttention::CausalSelfAttention(const GPT2Config& config) : Module("CausalSelfAttention"), config_(config) {
  TORCH_CHECK(config.n_embd % config.n_head == 0, "n_embd must be divisible by n_head");
  AddModule(kCAttnLayerName, std::make_shared<nn::Linear>(config.n_embd, 3 * config.n_embd));
  AddModule(kCProjLayerName, std::make_shared<nn::Linear>(config.n_embd, config.n_embd));
  // registered as a buffer (the reference's "bias"), so that a To(device) issued on any ancestor moves it too
  buffers_[kMaskBufferName] = std::make_shared<Tensor>(at::triu(at::ones({config.block_size, config.block_size}, at::kFloat), 1));
}
TensorList CausalSelfAttention::Forward(const TensorList& in) {
  const TP& x = in[0];
  const int64_t B = x->Dims()[0], T = x->Dims()[1], C = x->Dims()[2];
  const int64_t H = config_.n_head, hd = C / H;
  auto qkv = modules_[kCAttnLayerName]->Forward({x})[0]->Split(static_cast<int>(C), 2);
  if (x->GetDevice().IsCUDA() && qkv[0]->Dtype() == DataType::kBFLOAT16 && (hd == 64 || hd == 128)) {
    // bf16 on the GPU: one flash-attention kernel instead of the Matmul / MaskedFill / Softmax / Matmul chain
    TP y = std::make_shared<autograd::CausalAttention>()->Apply(
        {qkv[0]->View({B, T, H, hd}), qkv[1]->View({B, T, H, hd}), qkv[2]->View({B, T, H, hd})})[0];
    return modules_[kCProjLayerName]->Forward({y->View({B, T, C})});
  }
  auto heads = [&](const TP& t) { return t->View({B, T, H, hd})->Transpose(1, 2); };  // [B, H, T, hd]
  TP q = heads(qkv[0]), k = heads(qkv[1]), v = heads(qkv[2]);
  TP att = q->Matmul(k->Transpose(-2, -1)) * (1.0f / std::sqrt(static_cast<float>(hd)));
  TP mask = buffers_.at(kMaskBufferName)->Slice({0, 0}, {T, T}, {1, 1});
  att = att->MaskedFill(mask, -std::numeric_limits<float>::infinity());
  att = nn::function::Softmax(att, -1);
  TP y = att->Matmul(v)->Transpose(1, 2)->Contiguous()->View({B, T, C});
  return modules_[kCProjLayerName]->Forward({y});
}

MLP::MLP(const GPT2Config& config) : Module("MLP") {
  AddModule(kCFcLayerName, std::make_shared<nn::Linear>(config.n_embd, 4 * config.n_embd));
  AddModule(kGeluLayerName, std::make_shared<NewGELU>());
  AddModule(kCProjLayerName, std::make_shared<nn::Linear>(4 * config.n_embd, config.n_embd));
}
TensorList MLP::Forward(const TensorList& in) {
  auto h = modules_[kCFcLayerName]->Forward(in);
  h = modules_[kGeluLayerName]->Forward(h);
  return modules_[kCProjLayerName]->Forward(h);
}

Block::Block(const GPT2Config& config) : Module("Block") {
  AddModule(kLn1LayerName, std::make_shared<nn::LayerNorm>(std::vector<int64_t>{config.n_embd}));
  AddModule(kAttnLayerName, std::make_shared<CausalSelfAttention>(config));
  AddModule(kLn2LayerName, std::make_shared<nn::LayerNorm>(std::vector<int64_t>{config.n_embd}));
  AddModule(kMlpLayerName, std::make_shared<MLP>(config));
}
TensorList Block::Forward(const TensorList& in) {
  TP x = in[0];
  x = x + modules_[kAttnLayerName]->Forward(modules_[kLn1LayerName]->Forward({x}))[0];
  x = x + modules_[kMlpLayerName]->Forward(modules_[kLn2LayerName]->Forward({x}))[0];
  return {x};
}

GPT2::GPT2(const GPT2Config& config) : Module("GPT2"), config_(config) {
  std::unordered_map<std::string, std::shared_ptr<nn::Module>> tr;
  tr[kWTELayerName] = std::make_shared<nn::Embedding>(config.vocab_size, config.n_embd);
  tr[kWPELayerName] = std::make_shared<nn::Embedding>(config.block_size, config.n_embd);
  std::vector<std::shared_ptr<nn::Module>> blocks;
  for (int64_t i = 0; i < config.n_layer; ++i) blocks.push_back(std::make_shared<Block>(config));
  tr[kHLayerName] = std::make_shared<nn::Sequential>(std::move(blocks));
  tr[kLnFLayerName] = std::make_shared<nn::LayerNorm>(std::vector<int64_t>{config.n_embd});
  AddModule(kTransformerLayerName, std::make_shared<nn::ModuleDict>(std::move(tr)));
  auto head = std::make_shared<nn::Linear>(config.n_embd, config.vocab_size, /*bias=*/false);
  // weight tying: lm_head.weight IS transformer.wte.weight
  *head->mutable_parameter(nn::Linear::kParamWeightName) =
      mutable_module(kTransformerLayerName)->mutable_module(kWTELayerName)->parameter(nn::Embedding::kParamWeightName);
  AddModule(kLMHeadLayerName, head);

  // N(0, 0.02), residual projections N(0, 0.02 / sqrt(2 L)); every tensor from the head of the
  // seed-42 stream (the reference copies its seeded generator per call, nn/init.h:12-13).
  const float resid_std = 0.02f / std::sqrt(2.0f * static_cast<float>(config.n_layer));
  for (auto& [name, p] : StateDict()) {
    const bool is_ln = name.find("ln_") != std::string::npos;
    const bool is_bias = name.size() >= 5 && name.compare(name.size() - 5, 5, ".bias") == 0;
    if (is_ln) continue;
    if (is_bias) { nn::init::Zeros(p); continue; }
    const bool resid = name.find("c_proj.weight") != std::string::npos;
    nn::init::Normal(p, 0.f, resid ? resid_std : 0.02f, std::mt19937(42));
  }
}

TensorList GPT2::Forward(const TensorList& in) {
  const TP& idx = in[0];
  const int64_t T = idx->Dims()[1];
  TORCH_CHECK(T <= config_.block_size, "Cannot forward sequence of length ", T, ", block size is only ", config_.block_size);
  nn::Module* tr = mutable_module(kTransformerLayerName);
  TP pos = nn::init::Arange(0, T, DataType::kINT64, idx->GetDevice());
  TP tok_emb = tr->mutable_module(kWTELayerName)->Forward({idx})[0];
  TP pos_emb = tr->mutable_module(kWPELayerName)->Forward({pos})[0];
  TP x = tok_emb + pos_emb;
  x = tr->mutable_module(kHLayerName)->Forward({x})[0];
  x = tr->mutable_module(kLnFLayerName)->Forward({x})[0];
  return mutable_module(kLMHeadLayerName)->Forward({x});
}

std::unique_ptr<GPT2> GPT2::FromLLMC(const std::string& filepath) {
  titb::llmc::Gpt2Header h;
  auto sd = titb::llmc::read_gpt2(filepath, &h, /*keep_padding=*/false);
  GPT2Config cfg;
  cfg.block_size = h.block_size; cfg.vocab_size = h.vocab_size; cfg.n_layer = h.n_layer; cfg.n_head = h.n_head;
  cfg.n_embd = h.n_embd;
  auto model = std::make_unique<GPT2>(cfg);
  auto own = model->StateDict();
  for (auto& [name, t] : sd) {
    auto it = own.find(name);
    TORCH_CHECK(it != own.end(), "checkpoint tensor ", name, " has no counterpart in the model");
    TORCH_CHECK(it->second->data().sizes() == t.sizes(), "shape mismatch for ", name);
    it->second->data().copy_(t);
  }
  return model;
}

std::unique_ptr<GPT2> GPT2::FromPretrained(const std::string&) {
  TORCH_CHECK(false, "FromPretrained needs network access; load an llm.c .bin file with FromLLMC");
}

}  // namespace infini_train
