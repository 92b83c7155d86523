#include "core/framework/nn.h"

#include <c10/util/Exception.h>

#include <cmath>
#include <unordered_set>

#include "core/framework/dispatcher.h"
#include "core/rng.h"

namespace infini_train::nn {

using TP = std::shared_ptr<Tensor>;

// ---------------------------------------------------------------------------------- Module
std::vector<TP> Module::Parameters() const {
  std::vector<TP> out;
  std::unordered_set<const Tensor*> seen;
  std::function<void(const Module*)> rec = [&](const Module* m) {
    for (const auto& name : m->order_) {
      const TP& p = m->parameters_.at(name);
      if (p && seen.insert(p.get()).second) out.push_back(p);
    }
    for (const auto& name : m->module_order_) rec(m->modules_.at(name).get());
  };
  rec(this);
  return out;
}
TP* Module::mutable_parameter(const std::string& name) {
  TORCH_CHECK(parameters_.count(name), "no parameter named ", name);
  return &parameters_.at(name);
}
const TP& Module::parameter(const std::string& name) const {
  TORCH_CHECK(parameters_.count(name), "no parameter named ", name);
  return parameters_.at(name);
}
std::vector<Module*> Module::modules() {
  std::vector<Module*> out;
  for (const auto& name : module_order_) {
    Module* m = modules_.at(name).get();
    out.push_back(m);
    for (Module* c : m->modules()) out.push_back(c);
  }
  return out;
}
Module* Module::mutable_module(const std::string& name) {
  TORCH_CHECK(modules_.count(name), "no sub-module named ", name);
  return modules_.at(name).get();
}
const Module& Module::module(const std::string& name) const {
  TORCH_CHECK(modules_.count(name), "no sub-module named ", name);
  return *modules_.at(name);
}
std::unordered_map<std::string, TP> Module::StateDict() const {
  std::unordered_map<std::string, TP> out;
  for (const auto& [name, p] : parameters_) out.emplace(name, p);
  for (const auto& [mname, m] : modules_)
    for (const auto& [k, v] : m->StateDict()) out.emplace(mname + "." + k, v);
  return out;
}
std::unordered_map<std::string, TP> Module::Buffers() const {
  std::unordered_map<std::string, TP> out;
  for (const auto& [name, b] : buffers_) out.emplace(name, b);
  for (const auto& [mname, m] : modules_)
    for (const auto& [k, v] : m->Buffers()) out.emplace(mname + "." + k, v);
  return out;
}
TensorList Module::Forward(const TensorList&) { TORCH_CHECK(false, "Forward not implemented for ", type_); }
void Module::To(Device device) {
  if (device == device_) return;
  // move each distinct tensor once so that tied parameters stay tied
  std::unordered_map<const Tensor*, TP> moved;
  std::function<void(Module*)> rec = [&](Module* m) {
    for (auto& [name, p] : m->parameters_) {
      if (!p) continue;
      auto it = moved.find(p.get());
      if (it == moved.end()) {
        TP q = std::make_shared<Tensor>(p->To(device));
        it = moved.emplace(p.get(), q).first;
      }
      p = it->second;
    }
    for (auto& [name, b] : m->buffers_)
      if (b) b = std::make_shared<Tensor>(b->To(device));
    m->device_ = device;
    for (auto& [name, c] : m->modules_) rec(c.get());
  };
  rec(this);
}
void Module::To(DataType dtype) {
  std::unordered_map<const Tensor*, TP> cast;
  std::function<void(Module*)> rec = [&](Module* m) {
    for (auto& [name, p] : m->parameters_) {
      if (!p) continue;
      auto it = cast.find(p.get());
      if (it == cast.end()) {
        TP q = std::make_shared<Tensor>(p->To(dtype));
        if (p->requires_grad()) q->RequiresGrad();
        it = cast.emplace(p.get(), q).first;
      }
      p = it->second;
    }
    for (auto& [name, c] : m->modules_) rec(c.get());
  };
  rec(this);
}
void Module::Apply(const std::function<void(Module*)>& fn) {
  for (const auto& name : module_order_) modules_.at(name)->Apply(fn);
  fn(this);
}
void Module::AddModule(const std::string& name, std::shared_ptr<Module> m) {
  if (!modules_.count(name)) module_order_.push_back(name);
  modules_[name] = std::move(m);
}

Sequential::Sequential(std::vector<std::shared_ptr<Module>> layers) : Module("Sequential") {
  for (size_t i = 0; i < layers.size(); ++i) AddModule(std::to_string(i), std::move(layers[i]));
}
TensorList Sequential::Forward(const TensorList& input_tensors) {
  TensorList x = input_tensors;
  for (const auto& name : module_order_) x = modules_.at(name)->Forward(x);
  return x;
}
ModuleDict::ModuleDict(std::unordered_map<std::string, std::shared_ptr<Module>> modules) : Module("ModuleDict") {
  for (auto& [k, v] : modules) AddModule(k, std::move(v));
}
TensorList ModuleDict::Forward(const TensorList&) { TORCH_CHECK(false, "Not implemented: ModuleDict has no Forward"); }

// ---------------------------------------------------------------------------------- layers
Linear::Linear(int64_t in_features, int64_t out_features, bool bias, Device device)
    : Module("Linear"), in_features_(in_features), out_features_(out_features), bias_(bias) {
  device_ = device;
  AddParameter(kParamWeightName, std::make_shared<Tensor>(std::vector<int64_t>{out_features, in_features},
                                                          DataType::kFLOAT32, device)->RequiresGrad());
  if (bias) AddParameter(kParamBiasName, std::make_shared<Tensor>(std::vector<int64_t>{out_features}, DataType::kFLOAT32,
                                                                  device)->RequiresGrad());
  ResetParameters();
}
void Linear::ResetParameters() {
  init::KaimingUniform(parameters_[kParamWeightName], std::sqrt(5.0f));
  if (bias_) {
    const auto fan = init::CalculateFanInAndFanOut(parameters_[kParamWeightName]);
    const float bound = fan.first > 0 ? 1.0f / std::sqrt(static_cast<float>(fan.first)) : 0.f;
    init::Uniform(parameters_[kParamBiasName], -bound, bound);
  }
}
TensorList Linear::Forward(const TensorList& in) {
  TensorList args = {in[0], parameters_[kParamWeightName]};
  if (bias_) args.push_back(parameters_[kParamBiasName]);
  return std::make_shared<autograd::Linear>()->Apply(args);
}
Embedding::Embedding(int64_t num_embeddings, int64_t embedding_dim, Device device) : Module("Embedding") {
  device_ = device;
  AddParameter(kParamWeightName, std::make_shared<Tensor>(std::vector<int64_t>{num_embeddings, embedding_dim},
                                                          DataType::kFLOAT32, device)->RequiresGrad());
  init::Normal(parameters_[kParamWeightName]);
}
TensorList Embedding::Forward(const TensorList& in) {
  return std::make_shared<autograd::Embedding>()->Apply({in[0], parameters_[kParamWeightName]});
}
LayerNorm::LayerNorm(const std::vector<int64_t>& normalized_shape, float eps, Device device)
    : Module("LayerNorm"), eps_(eps) {
  device_ = device;
  AddParameter(kParamWeightName, std::make_shared<Tensor>(normalized_shape, DataType::kFLOAT32, device)->RequiresGrad());
  AddParameter(kParamBiasName, std::make_shared<Tensor>(normalized_shape, DataType::kFLOAT32, device)->RequiresGrad());
  init::Ones(parameters_[kParamWeightName]);
  init::Zeros(parameters_[kParamBiasName]);
}
TensorList LayerNorm::Forward(const TensorList& in) {
  return std::make_shared<autograd::LayerNorm>(eps_)->Apply({in[0], parameters_[kParamWeightName], parameters_[kParamBiasName]});
}
RMSNorm::RMSNorm(int64_t dim, float eps, Device device) : Module("RMSNorm"), eps_(eps) {
  device_ = device;
  AddParameter(kParamWeightName, std::make_shared<Tensor>(std::vector<int64_t>{dim}, DataType::kFLOAT32, device)->RequiresGrad());
  init::Ones(parameters_[kParamWeightName]);
}
TensorList RMSNorm::Forward(const TensorList& in) {
  return std::make_shared<autograd::RMSNorm>(eps_)->Apply({in[0], parameters_[kParamWeightName]});
}
TensorList CrossEntropyLoss::Forward(const TensorList& in) {
  return std::make_shared<autograd::CrossEntropy>()->Apply({in[0], in[1]});
}
TensorList Sigmoid::Forward(const TensorList& in) { return std::make_shared<autograd::Sigmoid>()->Apply({in[0]}); }

// ---------------------------------------------------------------------------------- nn::function
namespace function {
TP Tril(const TP& x, int64_t d) { return std::make_shared<autograd::Tril>(d)->Apply({x})[0]; }
TP Triu(const TP& x, int64_t d) { return std::make_shared<autograd::Triu>(d)->Apply({x})[0]; }
TP Ones(const std::vector<int64_t>& dims) { return std::make_shared<Tensor>(at::ones(dims, at::kFloat)); }
TP Reciprocal(const TP& x) { return x->Reciprocal(); }
TP Sin(const TP& x) { return x->Sin(); }
TP Cos(const TP& x) { return x->Cos(); }
TP Tanh(const TP& x) { return x->Tanh(); }
TP Pow(const TP& x, float e) { return x->Pow(e); }
TP Pow(float base, const TP& x) { return std::make_shared<autograd::Pow>(base, true)->Apply({x})[0]; }
TP Rsqrt(const TP& x) { return x->Rsqrt(); }
TP Mean(const TP& x, int64_t dim, bool keep) { return std::make_shared<autograd::Mean>(dim, keep)->Apply({x})[0]; }
TP Sum(const TP& x, int64_t dim, bool keep) { return std::make_shared<autograd::Sum>(dim, keep)->Apply({x})[0]; }
TP Max(const TP& x, int64_t dim, bool keep) { return std::make_shared<autograd::Max>(dim, keep)->Apply({x})[0]; }
TP Min(const TP& x, int64_t dim, bool keep) { return std::make_shared<autograd::Min>(dim, keep)->Apply({x})[0]; }
TP Sigmoid(const TP& x) { return std::make_shared<autograd::Sigmoid>()->Apply({x})[0]; }
TP Softmax(const TP& x, int64_t dim) { return std::make_shared<autograd::Softmax>(dim)->Apply({x})[0]; }
TP Slice(const TP& x, const std::vector<int64_t>& s, const std::vector<int64_t>& e, const std::vector<int64_t>& st) {
  return x->Slice(s, e, st);
}
TP Stack(const std::vector<TP>& xs, int64_t dim) { return std::make_shared<autograd::Stack>(dim)->Apply(xs)[0]; }
TP Cast(const TP& x, DataType dtype) { return std::make_shared<autograd::Cast>(dtype)->Apply({x})[0]; }
}  // namespace function

// ---------------------------------------------------------------------------------- nn::init
namespace init {
namespace {
// The generator arrives by value: a seeded call always starts from the head of that seed's stream.
template <class Dist>
TP fill_from(const TP& t, Dist dist, std::optional<std::mt19937> generator) {
  at::Tensor h = at::empty(t->Dims(), at::kFloat);
  float* p = h.data_ptr<float>();
  if (generator.has_value()) {
    for (int64_t i = 0; i < h.numel(); ++i) p[i] = dist(*generator);
  } else {
    auto& gen = titb::rng::global_generator();
    for (int64_t i = 0; i < h.numel(); ++i) p[i] = dist(gen);
  }
  t->data().copy_(h);
  return t;
}
float gain(NonLinearityType nl, float a) {
  switch (nl) {
    case NonLinearityType::kTanh: return 5.0f / 3.0f;
    case NonLinearityType::kReLU: return std::sqrt(2.0f);
    case NonLinearityType::kLeakyReLU: return std::sqrt(2.0f / (1.0f + a * a));
    default: return 1.0f;
  }
}
}  // namespace
TP Normal(const TP& t, float mean, float std, std::optional<std::mt19937> g) {
  return fill_from(t, std::normal_distribution<float>(mean, std), std::move(g));
}
TP Uniform(const TP& t, float a, float b, std::optional<std::mt19937> g) {
  return fill_from(t, std::uniform_real_distribution<float>(a, b), std::move(g));
}
std::pair<int64_t, int64_t> CalculateFanInAndFanOut(const TP& t) {
  const auto& d = t->Dims();
  TORCH_CHECK(d.size() >= 2, "Fan in and fan out can not be computed for tensor with fewer than 2 dimensions");
  int64_t rf = 1;
  for (size_t i = 2; i < d.size(); ++i) rf *= d[i];
  return {d[1] * rf, d[0] * rf};
}
TP KaimingUniform(const TP& t, float a, KaimingMode mode, NonLinearityType nl, std::optional<std::mt19937> g) {
  const auto fan = CalculateFanInAndFanOut(t);
  const float f = static_cast<float>(mode == KaimingMode::kFanIn ? fan.first : fan.second);
  const float bound = std::sqrt(3.0f) * gain(nl, a) / std::sqrt(f);
  return Uniform(t, -bound, bound, std::move(g));
}
TP Ones(const TP& t) { t->data().fill_(1); return t; }
TP Zeros(const TP& t) { t->data().zero_(); return t; }
TP Arange(int64_t start, int64_t end, DataType dtype, Device device) {
  return std::make_shared<Tensor>(at::arange(start, end, at::TensorOptions().dtype(ToTorch(dtype)).device(device.ToTorch())));
}
}  // namespace init

}  // namespace infini_train::nn

// ---------------------------------------------------------------------------------- optimizers
namespace infini_train {

Optimizer::Optimizer(const std::vector<std::shared_ptr<Tensor>>& params) {
  std::unordered_set<const Tensor*> seen;
  for (const auto& p : params)
    if (p && seen.insert(p.get()).second) params_.push_back(p);  // a tied tensor is stepped once
}
void Optimizer::ZeroGrad() {
  for (auto& p : params_) p->ZeroGrad();
}

namespace optimizers {
using TP = std::shared_ptr<Tensor>;
SGD::SGD(const std::vector<TP>& params, float learning_rate) : Optimizer(params), learning_rate_(learning_rate) {}
void SGD::Step() {
  for (auto& p : params_) {
    if (!p->grad()) continue;
    Dispatcher::Instance().GetKernel({p->GetDevice().Type(), "AccumulateGrad"})
        .Call<void, const TP&, float, const TP&>(p->grad(), -learning_rate_, p);
  }
}
Adam::Adam(const std::vector<TP>& params, float learning_rate, float beta1, float beta2, float eps, float weight_decay)
    : Optimizer(params), learning_rate_(learning_rate), beta1_(beta1), beta2_(beta2), eps_(eps), weight_decay_(weight_decay) {
  for (const auto& p : params_) {
    m_.push_back(std::make_shared<Tensor>(at::zeros_like(p->data(), at::kFloat)));
    v_.push_back(std::make_shared<Tensor>(at::zeros_like(p->data(), at::kFloat)));
  }
}
void Adam::Step() {
  ++t_;
  for (size_t i = 0; i < params_.size(); ++i) {
    auto& p = params_[i];
    if (!p->grad()) continue;
    if (weight_decay_ != 0.f) p->data().mul_(1.0 - static_cast<double>(learning_rate_) * weight_decay_);
    Dispatcher::Instance().GetKernel({p->GetDevice().Type(), "AdamAccumulateGrad"})
        .Call<void, const TP&, const TP&, const TP&, const TP&, float, float, float, float, int64_t>(
            p->grad(), p, m_[i], v_[i], learning_rate_, beta1_, beta2_, eps_, t_);
  }
}
}  // namespace optimizers

}  // namespace infini_train
