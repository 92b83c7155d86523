// nn layer API of the C++ facade: Module, containers, layers, nn::function, nn::init, optimizers.
//
// Reference: infini_train/include/nn/modules/*.h, nn/functional.h, nn/init.h, optimizer.h.
// Differences: Parameters() lists a tied tensor once and To(device) keeps ties (the reference
// duplicates, module.cc:12-19, and re-allocates per parameter, :58-71); Adam takes an optional
// decoupled weight decay.
#pragma once
#include <functional>
#include <memory>
#include <optional>
#include <random>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/framework/autograd.h"
#include "core/framework/tensor.h"

namespace infini_train::nn {

using TensorList = std::vector<std::shared_ptr<Tensor>>;

class Module : public std::enable_shared_from_this<Module> {
 public:
  static constexpr char kUndefinedType[] = "Undefined";
  explicit Module(std::string type = kUndefinedType) : type_(std::move(type)) {}
  virtual ~Module() = default;

  const std::string& type() const { return type_; }
  std::vector<std::shared_ptr<Tensor>> Parameters() const;
  bool has_parameter(const std::string& name) const { return parameters_.count(name) != 0; }
  std::shared_ptr<Tensor>* mutable_parameter(const std::string& name);
  const std::shared_ptr<Tensor>& parameter(const std::string& name) const;
  std::vector<Module*> modules();
  Module* mutable_module(const std::string& name);
  const Module& module(const std::string& name) const;
  std::unordered_map<std::string, std::shared_ptr<Tensor>> StateDict() const;
  // Non-parameter tensors (e.g. the attention mask "bias"), dotted names like StateDict(); To(Device) moves them too.
  std::unordered_map<std::string, std::shared_ptr<Tensor>> Buffers() const;
  virtual TensorList Forward(const TensorList& input_tensors);
  virtual void To(Device device);
  // Casts every parameter (ties kept) to `dtype`, e.g. kBFLOAT16 for tensor-core training on the GPU (not in the
  // reference, whose tensors are fp32 only).
  virtual void To(DataType dtype);
  void Apply(const std::function<void(Module*)>& fn);  // post-order

  void AddModule(const std::string& name, std::shared_ptr<Module> m);
  void AddParameter(const std::string& name, std::shared_ptr<Tensor> p) { parameters_[name] = std::move(p); order_.push_back(name); }

 protected:
  Device device_;
  std::string type_;
  std::unordered_map<std::string, std::shared_ptr<Module>> modules_;
  std::vector<std::string> module_order_;
  std::unordered_map<std::string, std::shared_ptr<Tensor>> parameters_;
  std::vector<std::string> order_;
  std::unordered_map<std::string, std::shared_ptr<Tensor>> buffers_;
};

class Sequential : public Module {
 public:
  explicit Sequential(std::vector<std::shared_ptr<Module>> layers);
  TensorList Forward(const TensorList& input_tensors) override;
};
class ModuleDict : public Module {
 public:
  explicit ModuleDict(std::unordered_map<std::string, std::shared_ptr<Module>> modules);
  TensorList Forward(const TensorList& input_tensors) override;
};

class Linear : public Module {
 public:
  static constexpr char kParamWeightName[] = "weight";
  static constexpr char kParamBiasName[] = "bias";
  Linear(int64_t in_features, int64_t out_features, bool bias = true, Device device = Device());
  TensorList Forward(const TensorList& input_tensors) override;
  void ResetParameters();
 private:
  int64_t in_features_, out_features_;
  bool bias_;
};
class Embedding : public Module {
 public:
  static constexpr char kParamWeightName[] = "weight";
  Embedding(int64_t num_embeddings, int64_t embedding_dim, Device device = Device());
  TensorList Forward(const TensorList& input_tensors) override;
};
class LayerNorm : public Module {
 public:
  static constexpr char kParamWeightName[] = "weight";
  static constexpr char kParamBiasName[] = "bias";
  explicit LayerNorm(const std::vector<int64_t>& normalized_shape, float eps = 1e-5f, Device device = Device());
  TensorList Forward(const TensorList& input_tensors) override;
 private:
  float eps_;
};
class RMSNorm : public Module {
 public:
  static constexpr char kParamWeightName[] = "weight";
  explicit RMSNorm(int64_t dim, float eps = 1e-5f, Device device = Device());
  TensorList Forward(const TensorList& input_tensors) override;
 private:
  float eps_;
};
class CrossEntropyLoss : public Module {
 public:
  CrossEntropyLoss() : Module("CrossEntropyLoss") {}
  TensorList Forward(const TensorList& input_tensors) override;
};
class Sigmoid : public Module {
 public:
  Sigmoid() : Module("Sigmoid") {}
  TensorList Forward(const TensorList& input_tensors) override;
};

namespace function {
std::shared_ptr<Tensor> Tril(const std::shared_ptr<Tensor>& x, int64_t diagonal = 0);
std::shared_ptr<Tensor> Triu(const std::shared_ptr<Tensor>& x, int64_t diagonal = 0);
std::shared_ptr<Tensor> Ones(const std::vector<int64_t>& dims);
std::shared_ptr<Tensor> Reciprocal(const std::shared_ptr<Tensor>& x);
std::shared_ptr<Tensor> Sin(const std::shared_ptr<Tensor>& x);
std::shared_ptr<Tensor> Cos(const std::shared_ptr<Tensor>& x);
std::shared_ptr<Tensor> Tanh(const std::shared_ptr<Tensor>& x);
std::shared_ptr<Tensor> Pow(const std::shared_ptr<Tensor>& x, float exponent);
std::shared_ptr<Tensor> Pow(float base, const std::shared_ptr<Tensor>& x);
std::shared_ptr<Tensor> Rsqrt(const std::shared_ptr<Tensor>& x);
std::shared_ptr<Tensor> Mean(const std::shared_ptr<Tensor>& x, int64_t dim, bool keep_dim = false);
std::shared_ptr<Tensor> Sum(const std::shared_ptr<Tensor>& x, int64_t dim, bool keep_dim = false);
std::shared_ptr<Tensor> Max(const std::shared_ptr<Tensor>& x, int64_t dim, bool keep_dim = false);
std::shared_ptr<Tensor> Min(const std::shared_ptr<Tensor>& x, int64_t dim, bool keep_dim = false);
std::shared_ptr<Tensor> Sigmoid(const std::shared_ptr<Tensor>& x);
std::shared_ptr<Tensor> Softmax(const std::shared_ptr<Tensor>& x, int64_t dim = -1);
std::shared_ptr<Tensor> Slice(const std::shared_ptr<Tensor>& x, const std::vector<int64_t>& starts,
                              const std::vector<int64_t>& ends, const std::vector<int64_t>& steps);
std::shared_ptr<Tensor> Stack(const std::vector<std::shared_ptr<Tensor>>& xs, int64_t dim = 0);
std::shared_ptr<Tensor> Cast(const std::shared_ptr<Tensor>& x, DataType dtype);
}  // namespace function

namespace init {
enum class KaimingMode { kFanIn, kFanOut };
enum class NonLinearityType { kLinear, kSigmoid, kTanh, kReLU, kLeakyReLU };
std::shared_ptr<Tensor> Normal(const std::shared_ptr<Tensor>& t, float mean = 0.f, float std = 1.f,
                               std::optional<std::mt19937> generator = std::nullopt);
std::shared_ptr<Tensor> Uniform(const std::shared_ptr<Tensor>& t, float a = 0.f, float b = 1.f,
                                std::optional<std::mt19937> generator = std::nullopt);
std::shared_ptr<Tensor> KaimingUniform(const std::shared_ptr<Tensor>& t, float a = 0.f, KaimingMode mode = KaimingMode::kFanIn,
                                       NonLinearityType nl = NonLinearityType::kLeakyReLU,
                                       std::optional<std::mt19937> generator = std::nullopt);
std::shared_ptr<Tensor> Ones(const std::shared_ptr<Tensor>& t);
std::shared_ptr<Tensor> Zeros(const std::shared_ptr<Tensor>& t);
std::shared_ptr<Tensor> Arange(int64_t start, int64_t end, DataType dtype, Device device = Device());
std::pair<int64_t, int64_t> CalculateFanInAndFanOut(const std::shared_ptr<Tensor>& t);
}  // namespace init

}  // namespace infini_train::nn

namespace infini_train {

class Optimizer {
 public:
  explicit Optimizer(const std::vector<std::shared_ptr<Tensor>>& params);
  virtual ~Optimizer() = default;
  void ZeroGrad();
  virtual void Step() = 0;
 protected:
  std::vector<std::shared_ptr<Tensor>> params_;
};

namespace optimizers {
class SGD : public Optimizer {
 public:
  SGD(const std::vector<std::shared_ptr<Tensor>>& params, float learning_rate);
  void Step() override;
 private:
  float learning_rate_;
};
class Adam : public Optimizer {
 public:
  Adam(const std::vector<std::shared_ptr<Tensor>>& params, float learning_rate = 1e-3f, float beta1 = 0.9f,
       float beta2 = 0.999f, float eps = 1e-8f, float weight_decay = 0.f);
  void Step() override;
 private:
  int64_t t_ = 0;
  float learning_rate_, beta1_, beta2_, eps_, weight_decay_;
  std::vector<std::shared_ptr<Tensor>> m_, v_;
};
}  // namespace optimizers

}  // namespace infini_train
