// Python bindings of the C++ framework facade (Tensor / autograd::Function / nn / optimizers / GPT-2),
// used by the tests that restate the reference's gtest cases and by users who script the C++ API.
#include <torch/extension.h>

#include <sstream>

#include "core/framework/autograd.h"
#include "core/framework/dispatcher.h"
#include "core/framework/gpt2.h"
#include "core/framework/llama3.h"
#include "core/framework/nn.h"
#include "core/framework/tensor.h"

namespace fw = infini_train;
using TP = std::shared_ptr<fw::Tensor>;

namespace {

fw::Device dev_of(const std::string& s) {
  if (s == "cpu") return fw::Device();
  if (s.rfind("cuda", 0) == 0) {
    int idx = 0;
    auto c = s.find(':');
    if (c != std::string::npos) idx = std::stoi(s.substr(c + 1));
    return fw::Device(fw::DeviceType::kCUDA, static_cast<int8_t>(idx));
  }
  TORCH_CHECK(false, "unknown device ", s);
}

std::shared_ptr<fw::autograd::Function> make_function(const std::string& name, const std::vector<double>& a) {
  using namespace fw::autograd;
  auto f = [&](size_t i, double d) { return i < a.size() ? a[i] : d; };
  if (name == "Neg") return std::make_shared<Neg>();
  if (name == "Reciprocal") return std::make_shared<Reciprocal>();
  if (name == "Sin") return std::make_shared<Sin>();
  if (name == "Cos") return std::make_shared<Cos>();
  if (name == "Tanh") return std::make_shared<Tanh>();
  if (name == "Rsqrt") return std::make_shared<Rsqrt>();
  if (name == "Sigmoid") return std::make_shared<Sigmoid>();
  if (name == "Gelu") return std::make_shared<Gelu>();
  if (name == "SwiGLU") return std::make_shared<SwiGLU>();
  if (name == "CausalAttention") return std::make_shared<CausalAttention>((float)f(0, 0.0));
  if (name == "Rope") return std::make_shared<Rope>((float)f(0, 500000.0), (int64_t)f(1, 0));
  if (name == "Pow") return std::make_shared<Pow>((float)f(0, 2), f(1, 0) != 0);
  if (name == "EqualsScalar") return std::make_shared<EqualsScalar>((float)f(0, 0));
  if (name == "AddScalar") return std::make_shared<AddScalar>((float)f(0, 0));
  if (name == "MulScalar") return std::make_shared<MulScalar>((float)f(0, 1));
  if (name == "Add") return std::make_shared<Add>();
  if (name == "Sub") return std::make_shared<Sub>();
  if (name == "Mul") return std::make_shared<Mul>();
  if (name == "Div") return std::make_shared<Div>();
  if (name == "Matmul") return std::make_shared<Matmul>();
  if (name == "Linear") return std::make_shared<Linear>();
  if (name == "Outer") return std::make_shared<Outer>();
  if (name == "LayerNorm") return std::make_shared<LayerNorm>((float)f(0, 1e-5));
  if (name == "RMSNorm") return std::make_shared<RMSNorm>((float)f(0, 1e-5));
  if (name == "Softmax") return std::make_shared<Softmax>((int64_t)f(0, -1));
  if (name == "CrossEntropy") return std::make_shared<CrossEntropy>();
  if (name == "Embedding") return std::make_shared<Embedding>();
  if (name == "Mean") return std::make_shared<Mean>((int64_t)f(0, 0), f(1, 0) != 0);
  if (name == "Sum") return std::make_shared<Sum>((int64_t)f(0, 0), f(1, 0) != 0);
  if (name == "Max") return std::make_shared<Max>((int64_t)f(0, 0), f(1, 0) != 0);
  if (name == "Min") return std::make_shared<Min>((int64_t)f(0, 0), f(1, 0) != 0);
  if (name == "Tril") return std::make_shared<Tril>((int64_t)f(0, 0));
  if (name == "Triu") return std::make_shared<Triu>((int64_t)f(0, 0));
  if (name == "Transpose") return std::make_shared<Transpose>((int64_t)f(0, 0), (int64_t)f(1, 1));
  if (name == "RepeatInterleave") return std::make_shared<RepeatInterleave>((int64_t)f(0, 1), (int64_t)f(1, 0));
  if (name == "Split") return std::make_shared<Split>((int64_t)f(0, 1), (int)f(1, 0));
  if (name == "Stack") return std::make_shared<Stack>((int64_t)f(0, 0));
  TORCH_CHECK(false, "unknown Function ", name);
}

// The reference's dispatcher tests (test/kernels/test_dispatcher.cc:17-56) restated.
void TestVoidKernel(int* counter) { ++*counter; }
int TestIntKernel(int a, int b) { return a + b; }
void register_selftest_kernels() {
  using fw::DeviceType;
  static bool registered = false;
  if (!registered) {
    REGISTER_KERNEL(DeviceType::kCPU, SelfTestVoid, &TestVoidKernel);   // block-scope registration
    REGISTER_KERNEL(DeviceType::kCUDA, SelfTestInt, &TestIntKernel);
    registered = true;
  }
}
py::dict dispatcher_selftest() {
  using fw::DeviceType;
  auto& d = fw::Dispatcher::Instance();
  register_selftest_kernels();
  py::dict r;
  int counter = 0;
  d.GetKernel({DeviceType::kCPU, "SelfTestVoid"}).Call<void, int*>(&counter);
  r["void_called"] = counter == 1;
  r["int_result"] = d.GetKernel({DeviceType::kCUDA, "SelfTestInt"}).Call<int, int, int>(2, 3);
  r["separate_device_keys"] = !d.HasKernel({DeviceType::kCUDA, "SelfTestVoid"});
  r["has_linear_cpu"] = d.HasKernel({DeviceType::kCPU, "LinearForward"});
  r["has_adam_cuda"] = d.HasKernel({DeviceType::kCUDA, "AdamAccumulateGrad"});
  return r;
}
// These two raise (the reference tests them with EXPECT_DEATH): duplicate registration, unknown kernel.
void dispatcher_register_duplicate() {
  register_selftest_kernels();
  fw::Dispatcher::Instance().Register({fw::DeviceType::kCPU, "SelfTestVoid"}, &TestVoidKernel);
}
void dispatcher_get_missing() { fw::Dispatcher::Instance().GetKernel({fw::DeviceType::kCPU, "NoSuchKernel"}); }

}  // namespace

void bind_framework(pybind11::module_& m) {
  py::class_<fw::Tensor, TP>(m, "FwTensor")
      .def(py::init([](const at::Tensor& t, bool requires_grad) {
             auto p = std::make_shared<fw::Tensor>(t.detach().clone());
             if (requires_grad) p->RequiresGrad();
             return p;
           }), py::arg("t"), py::arg("requires_grad") = false)
      .def_static("empty", [](const std::vector<int64_t>& dims, const std::string& device) {
        return std::make_shared<fw::Tensor>(dims, fw::DataType::kFLOAT32, dev_of(device));
      })
      .def("torch", [](const TP& t) { return t->data(); })
      .def("Dims", &fw::Tensor::Dims)
      .def("NumElements", &fw::Tensor::NumElements)
      .def("SizeInBytes", &fw::Tensor::SizeInBytes)
      .def("Dtype", [](const TP& t) { return std::string(fw::DataTypeName(t->Dtype())); })
      .def("GetDevice", [](const TP& t) { return t->GetDevice().ToString(); })
      .def("Fill", [](const TP& t, double v) { t->Fill<float>((float)v); })
      .def("To", [](const TP& t, const std::string& d) { return std::make_shared<fw::Tensor>(t->To(dev_of(d))); })
      .def("Cast", [](const TP& t, const std::string& dt) {
        return infini_train::nn::function::Cast(t, dt == "bfloat16" ? fw::DataType::kBFLOAT16 : fw::DataType::kFLOAT32);
      })
      .def("Add", py::overload_cast<const TP&>(&fw::Tensor::Add)).def("AddScalar", py::overload_cast<float>(&fw::Tensor::Add))
      .def("Sub", py::overload_cast<const TP&>(&fw::Tensor::Sub)).def("SubScalar", py::overload_cast<float>(&fw::Tensor::Sub))
      .def("Mul", py::overload_cast<const TP&>(&fw::Tensor::Mul)).def("MulScalar", py::overload_cast<float>(&fw::Tensor::Mul))
      .def("Div", py::overload_cast<const TP&>(&fw::Tensor::Div)).def("DivScalar", py::overload_cast<float>(&fw::Tensor::Div))
      .def("Neg", &fw::Tensor::Neg).def("Reciprocal", &fw::Tensor::Reciprocal).def("Sin", &fw::Tensor::Sin)
      .def("Cos", &fw::Tensor::Cos).def("Tanh", &fw::Tensor::Tanh).def("Pow", &fw::Tensor::Pow)
      .def("Rsqrt", &fw::Tensor::Rsqrt).def("Equals", &fw::Tensor::Equals)
      .def("Split", &fw::Tensor::Split, py::arg("split_size"), py::arg("dim") = 0)
      .def("Transpose", &fw::Tensor::Transpose)
      .def("Slice", py::overload_cast<const std::vector<int64_t>&, const std::vector<int64_t>&, const std::vector<int64_t>&>(&fw::Tensor::Slice))
      .def("RepeatInterleave", &fw::Tensor::RepeatInterleave)
      .def("View", &fw::Tensor::View).def("Contiguous", &fw::Tensor::Contiguous)
      .def("Flatten", &fw::Tensor::Flatten, py::arg("start") = 0, py::arg("end") = -1)
      .def("Squeeze", &fw::Tensor::Squeeze).def("Matmul", &fw::Tensor::Matmul).def("Outer", &fw::Tensor::Outer)
      .def("MaskedFill", &fw::Tensor::MaskedFill)
      .def("RequiresGrad", &fw::Tensor::RequiresGrad)
      .def("grad", &fw::Tensor::grad).def("requires_grad", &fw::Tensor::requires_grad)
      .def("is_leaf", &fw::Tensor::is_leaf).def("ZeroGrad", &fw::Tensor::ZeroGrad)
      .def("Backward", [](const TP& t, const TP& g) { t->Backward(g); }, py::arg("gradient") = nullptr)
      .def("SaveAsNpy", &fw::Tensor::SaveAsNpy)
      .def("__repr__", [](const TP& t) { std::ostringstream os; t->Print(os); return os.str(); });
  m.def("fw_set_print_options", &fw::SetPrintOptions, py::arg("precision") = -1, py::arg("threshold") = -1,
        py::arg("edge_items") = -1, py::arg("linewidth") = -1, py::arg("profile") = "", py::arg("sci_mode") = -1);

  py::class_<fw::autograd::Function, std::shared_ptr<fw::autograd::Function>>(m, "FwFunction")
      .def("Forward", &fw::autograd::Function::Forward)
      .def("SetupContext", &fw::autograd::Function::SetupContext)
      .def("Backward", &fw::autograd::Function::Backward)
      .def("Apply", &fw::autograd::Function::Apply);
  m.def("fw_function", &make_function, py::arg("name"), py::arg("args") = std::vector<double>{});
  m.def("fw_mask", [](const TP& x, const TP& mask, double v) {
    return std::make_shared<fw::autograd::Mask>(mask, (float)v)->Apply({x})[0];
  });
  m.def("fw_dispatcher_selftest", &dispatcher_selftest);
  m.def("fw_dispatcher_register_duplicate", &dispatcher_register_duplicate);
  m.def("fw_dispatcher_get_missing", &dispatcher_get_missing);

  namespace nn = fw::nn;
  py::class_<nn::Module, std::shared_ptr<nn::Module>>(m, "FwModule")
      .def("type", &nn::Module::type)
      .def("Parameters", &nn::Module::Parameters)
      .def("StateDict", &nn::Module::StateDict)
      .def("Buffers", &nn::Module::Buffers)
      .def("Forward", &nn::Module::Forward)
      .def("has_parameter", &nn::Module::has_parameter)
      .def("parameter", &nn::Module::parameter)
      .def("To", [](nn::Module& mod, const std::string& d) { mod.To(dev_of(d)); })
      .def("ToDtype", [](nn::Module& mod, const std::string& dt) {
        TORCH_CHECK(dt == "float32" || dt == "bfloat16", "ToDtype: float32 or bfloat16");
        mod.To(dt == "bfloat16" ? fw::DataType::kBFLOAT16 : fw::DataType::kFLOAT32);
      });
  py::class_<nn::Linear, nn::Module, std::shared_ptr<nn::Linear>>(m, "FwLinear")
      .def(py::init([](int64_t i, int64_t o, bool b) { return std::make_shared<nn::Linear>(i, o, b); }),
           py::arg("in_features"), py::arg("out_features"), py::arg("bias") = true);
  py::class_<nn::Embedding, nn::Module, std::shared_ptr<nn::Embedding>>(m, "FwEmbedding")
      .def(py::init([](int64_t n, int64_t d) { return std::make_shared<nn::Embedding>(n, d); }));
  py::class_<nn::LayerNorm, nn::Module, std::shared_ptr<nn::LayerNorm>>(m, "FwLayerNorm")
      .def(py::init([](int64_t d, double eps) { return std::make_shared<nn::LayerNorm>(std::vector<int64_t>{d}, (float)eps); }),
           py::arg("dim"), py::arg("eps") = 1e-5);
  py::class_<nn::RMSNorm, nn::Module, std::shared_ptr<nn::RMSNorm>>(m, "FwRMSNorm")
      .def(py::init([](int64_t d, double eps) { return std::make_shared<nn::RMSNorm>(d, (float)eps); }),
           py::arg("dim"), py::arg("eps") = 1e-5);
  py::class_<nn::CrossEntropyLoss, nn::Module, std::shared_ptr<nn::CrossEntropyLoss>>(m, "FwCrossEntropyLoss").def(py::init<>());
  py::class_<nn::Sigmoid, nn::Module, std::shared_ptr<nn::Sigmoid>>(m, "FwSigmoid").def(py::init<>());
  py::class_<nn::Sequential, nn::Module, std::shared_ptr<nn::Sequential>>(m, "FwSequential")
      .def(py::init<std::vector<std::shared_ptr<nn::Module>>>());
  py::class_<fw::GPT2, nn::Module, std::shared_ptr<fw::GPT2>>(m, "FwGPT2")
      .def(py::init([](int64_t block, int64_t vocab, int64_t L, int64_t H, int64_t C) {
        fw::GPT2Config c; c.block_size = block; c.vocab_size = vocab; c.n_layer = L; c.n_head = H; c.n_embd = C;
        return std::make_shared<fw::GPT2>(c);
      }))
      .def_static("FromLLMC", [](const std::string& p) { return std::shared_ptr<fw::GPT2>(fw::GPT2::FromLLMC(p)); });

  py::class_<fw::LLaMA3, nn::Module, std::shared_ptr<fw::LLaMA3>>(m, "FwLLaMA3")
      .def(py::init([](int64_t block, int64_t vocab, int64_t L, int64_t H, int64_t Hkv, int64_t C, int64_t F, double eps,
                       double theta) {
        fw::LLaMA3Config c;
        c.block_size = block; c.vocab_size = vocab; c.n_layer = L; c.n_head = H; c.n_kv_head = Hkv; c.n_embd = C;
        c.ffn_dim = F; c.norm_eps = (float)eps; c.rope_theta = (float)theta;
        return std::make_shared<fw::LLaMA3>(c);
      }), py::arg("block_size"), py::arg("vocab_size"), py::arg("n_layer"), py::arg("n_head"), py::arg("n_kv_head"),
           py::arg("n_embd"), py::arg("ffn_dim"), py::arg("norm_eps") = 1e-5, py::arg("rope_theta") = 500000.0)
      .def_static("FromLLMC", [](const std::string& p) { return std::shared_ptr<fw::LLaMA3>(fw::LLaMA3::FromLLMC(p)); });

  py::class_<fw::Optimizer, std::shared_ptr<fw::Optimizer>>(m, "FwOptimizer")
      .def("ZeroGrad", &fw::Optimizer::ZeroGrad).def("Step", &fw::Optimizer::Step);
  py::class_<fw::optimizers::SGD, fw::Optimizer, std::shared_ptr<fw::optimizers::SGD>>(m, "FwSGD")
      .def(py::init<const std::vector<TP>&, float>());
  py::class_<fw::optimizers::Adam, fw::Optimizer, std::shared_ptr<fw::optimizers::Adam>>(m, "FwAdam")
      .def(py::init<const std::vector<TP>&, float, float, float, float, float>(), py::arg("params"),
           py::arg("learning_rate") = 1e-3f, py::arg("beta1") = 0.9f, py::arg("beta2") = 0.999f, py::arg("eps") = 1e-8f,
           py::arg("weight_decay") = 0.f);
  m.def("fw_init_normal", [](const TP& t, double mean, double std, c10::optional<int64_t> seed) {
    return nn::init::Normal(t, (float)mean, (float)std, seed ? std::optional<std::mt19937>(std::mt19937((uint32_t)*seed)) : std::nullopt);
  }, py::arg("t"), py::arg("mean") = 0.0, py::arg("std") = 1.0, py::arg("seed") = py::none());
}
