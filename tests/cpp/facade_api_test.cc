// The reference's gtest cases, restated directly against the C++ API (no test framework dependency):
// test/autograd/test_elementwise.cc:11-59, test/kernels/test_matmul.cc:12-133, test/optimizer/test_adam.cc:11-60,
// test/tensor/test_tensor.cc:10-78, test/kernels/test_dispatcher.cc:17-56, plus the data layer and a short GPT-2
// training run.  Usage: facade_api_test [cpu|cuda] <scratch-dir>.  Exit code 0 = all checks passed.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include "core/framework/autograd.h"
#include "core/framework/data_facade.h"
#include "core/framework/dispatcher.h"
#include "core/framework/gpt2.h"
#include "core/framework/nn.h"
#include "core/framework/tensor.h"
#include "core/llmc_io.h"

using namespace infini_train;
using TP = std::shared_ptr<Tensor>;

static int g_failed = 0;
#define EXPECT(cond)                                                             \
  do {                                                                           \
    if (!(cond)) {                                                               \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);              \
      ++g_failed;                                                                \
    }                                                                            \
  } while (0)

static Device g_dev;

static TP T(std::vector<float> v, std::vector<int64_t> dims, bool requires_grad = false) {
  auto t = std::make_shared<Tensor>(dims, DataType::kFLOAT32, Device());
  std::memcpy(t->DataPtr(), v.data(), v.size() * sizeof(float));
  auto d = std::make_shared<Tensor>(t->To(g_dev));
  return requires_grad ? d->RequiresGrad() : d;
}
static std::vector<float> V(const TP& t) { return t->ToFloatVector(); }
static bool near(const std::vector<float>& a, const std::vector<float>& b, float tol) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (!(std::fabs(a[i] - b[i]) <= tol)) return false;
  return true;
}

static void TestNeg() {
  auto x = T({1.f, -2.f, 0.f}, {3});
  auto f = std::make_shared<autograd::Neg>();
  auto out = f->Forward({x});
  EXPECT(near(V(out[0]), {-1.f, 2.f, -0.f}, 0.f));
  f->SetupContext({x}, out);
  EXPECT(near(V(f->Backward({T({1.f, 1.f, 1.f}, {3})})[0]), {-1.f, -1.f, -1.f}, 0.f));
}

static void TestMatmul() {
  auto a = T({1, 2, 3, 4, 5, 6}, {2, 3});
  auto b = T({7, 8, 9, 10, 11, 12}, {3, 2});
  auto out = std::make_shared<autograd::Matmul>()->Forward({a, b})[0];
  EXPECT((out->Dims() == std::vector<int64_t>{2, 2}));
  EXPECT(near(V(out), {58, 64, 139, 154}, 0.f));
  std::vector<float> seq(12);
  for (int i = 0; i < 12; ++i) seq[i] = static_cast<float>(i + 1);
  auto o3 = std::make_shared<autograd::Matmul>()->Forward({T(seq, {2, 2, 3}), T(seq, {2, 3, 2})})[0];
  EXPECT(near(V(o3), {22, 28, 49, 64, 220, 244, 301, 334}, 0.f));
  auto f = std::make_shared<autograd::Matmul>();
  f->SetupContext({a, b}, {T({0, 0, 0, 0}, {2, 2})});
  auto g = f->Backward({T({0.1f, 0.2f, 0.3f, 0.4f}, {2, 2})});
  EXPECT(near(V(g[0]), {2.3f, 2.9f, 3.5f, 5.3f, 6.7f, 8.1f}, 1e-5f));
  EXPECT(near(V(g[1]), {1.3f, 1.8f, 1.7f, 2.4f, 2.1f, 3.0f}, 1e-5f));
}

static void TestAdam() {
  auto p = T({1.f, 2.f, 3.f}, {3}, true);
  const std::vector<float> grad = {0.1f, -0.2f, 0.3f};
  const float lr = 0.1f, b1 = 0.9f, b2 = 0.999f, eps = 1e-8f;
  optimizers::Adam opt({p}, lr, b1, b2, eps);
  std::vector<double> m(3, 0.0), v(3, 0.0), ref = {1.0, 2.0, 3.0};
  for (int t = 1; t <= 3; ++t) {
    p->grad()->data().copy_(T(grad, {3})->data());
    opt.Step();
    for (int i = 0; i < 3; ++i) {
      m[i] = b1 * m[i] + (1 - b1) * grad[i];
      v[i] = b2 * v[i] + (1 - b2) * grad[i] * grad[i];
      ref[i] -= lr * (m[i] / (1 - std::pow(b1, t))) / (std::sqrt(v[i] / (1 - std::pow(b2, t))) + eps);
    }
  }
  EXPECT(near(V(p), {static_cast<float>(ref[0]), static_cast<float>(ref[1]), static_cast<float>(ref[2])}, 1e-5f));
  EXPECT(V(p)[0] < 1.f && V(p)[1] > 2.f);
}

static void TestTensorAutograd() {
  auto x = T({2.f}, {1}, true);
  x->Pow(2)->Backward();
  EXPECT(near(V(x->grad()), {4.f}, 0.f));
  auto y = T({1.f, 1.f, 1.f}, {3}, true);
  auto y1 = y->Mul(2.f), y2 = y->Pow(3);
  y1->Backward(T({1, 1, 1}, {3}));
  y2->Backward(T({2, 2, 2}, {3}));
  EXPECT(near(V(y->grad()), {8.f, 8.f, 8.f}, 0.f));
  std::vector<float> seq(12);
  for (int i = 0; i < 12; ++i) seq[i] = static_cast<float>(i + 1);
  auto flat = T(seq, {3, 4})->Flatten(0, 1);
  EXPECT((flat->Dims() == std::vector<int64_t>{12}) && near(V(flat), seq, 0.f));
  EXPECT((T(std::vector<float>(24, 0.f), {2, 3, 4})->Flatten(1, -1)->Dims() == std::vector<int64_t>{2, 12}));
  auto tr = T(seq, {4, 3})->Transpose(0, 1)->Flatten(0, -1);
  EXPECT(tr->NumElements() == 12 && near(V(tr), {1, 4, 7, 10, 2, 5, 8, 11, 3, 6, 9, 12}, 0.f));
  // operators with a scalar on either side
  auto z = 2.f * T({1.f, 2.f}, {2}) + 1.f;
  EXPECT(near(V(z), {3.f, 5.f}, 0.f));
  EXPECT(near(V(1.f / T({2.f, 4.f}, {2})), {0.5f, 0.25f}, 0.f));
}

// Tensor::Uniform(from, to, generator) and the static Tensor::SetPrintOptions of the reference's tensor.h:124,151.
static void TestUniformAndPrintOptions() {
  auto a = std::make_shared<Tensor>(std::vector<int64_t>{4, 5}, DataType::kFLOAT32, g_dev);
  auto b = std::make_shared<Tensor>(std::vector<int64_t>{4, 5}, DataType::kFLOAT32, g_dev);
  std::mt19937 gen(7);
  auto ra = a->Uniform(-2.f, 3.f, gen);
  b->Uniform(-2.f, 3.f, gen);                     // the generator is copied: same seed, same values
  EXPECT(ra.get() == a.get());
  const auto va = V(a), vb = V(b);
  EXPECT(near(va, vb, 0.f));
  bool in_range = true, varied = false;
  for (float x : va) {
    in_range = in_range && x >= -2.f && x < 3.f;
    varied = varied || x != va[0];
  }
  EXPECT(in_range && varied);
  std::mt19937 expect(7);
  std::uniform_real_distribution<float> dist(-2.f, 3.f);
  EXPECT(std::fabs(va[0] - dist(expect)) == 0.f);  // libstdc++ stream, element order = memory order
  Tensor::SetPrintOptions(2, std::nullopt, std::nullopt, 120);
  EXPECT(PrintOptions::Get().precision == 2 && PrintOptions::Get().linewidth == 120);
  Tensor::SetPrintOptions(std::nullopt, std::nullopt, std::nullopt, std::nullopt, std::string("default"));
  EXPECT(PrintOptions::Get().precision == 4 && PrintOptions::Get().linewidth == 80);
}

static void CounterKernel(int* c) { ++*c; }
static int AddKernel(int a, int b) { return a + b; }
static void TestDispatcher() {
  REGISTER_KERNEL(DeviceType::kCPU, ApiTestVoid, &CounterKernel);      // block scope, as the reference's test does
  REGISTER_KERNEL(DeviceType::kCUDA, ApiTestInt, &AddKernel);
  auto& d = Dispatcher::Instance();
  int c = 0;
  d.GetKernel({DeviceType::kCPU, "ApiTestVoid"}).Call<void, int*>(&c);
  EXPECT(c == 1);
  EXPECT((d.GetKernel({DeviceType::kCUDA, "ApiTestInt"}).Call<int, int, int>(2, 3) == 5));
  EXPECT(!d.HasKernel({DeviceType::kCUDA, "ApiTestVoid"}));
  bool dup = false, missing = false;
  try { d.Register({DeviceType::kCPU, "ApiTestVoid"}, &CounterKernel); } catch (const std::runtime_error& e) {
    dup = std::string(e.what()).find("Kernel already registered") != std::string::npos;
  }
  try { d.GetKernel({DeviceType::kCPU, "NoSuchKernel"}); } catch (const std::runtime_error& e) {
    missing = std::string(e.what()).find("Kernel not found") != std::string::npos;
  }
  EXPECT(dup && missing);
  EXPECT(d.HasKernel({DeviceType::kCPU, "LinearForward"}) && d.HasKernel({DeviceType::kCUDA, "AdamAccumulateGrad"}));
}

static void TestDataAndTraining(const std::string& dir) {
  // 4 * 33 + 1 tokens below a 97-word vocabulary -> 8 windows of 16 tokens (+ the shifted target)
  at::Tensor toks = at::arange(0, 8 * 16 + 1, at::kLong).remainder(97);
  const std::string tok_path = dir + "/tokens.bin";
  titb::llmc::write_tokens(tok_path, toks, titb::llmc::kDataMagicU16);
  auto ds = std::make_shared<TinyShakespeareDataset>(tok_path, 16);
  EXPECT(ds->Size() == 8);
  auto [x0, y0] = (*ds)[1];
  EXPECT(x0->Dims() == std::vector<int64_t>{16} && x0->Dtype() == DataType::kINT64);
  EXPECT(x0->data()[0].item<int64_t>() == 16 && y0->data()[0].item<int64_t>() == 17);
  DataLoader loader(ds, 3);
  size_t batches = 0, rows = 0;
  for (auto it = loader.begin(); it != loader.end(); ++it) {
    auto [x, y] = *it;
    rows += static_cast<size_t>(x->Dims()[0]);
    EXPECT(x->Dims()[1] == 16 && y->Dims() == x->Dims());
    ++batches;
  }
  EXPECT(batches == 3 && rows == 8);
  auto end = loader.end();
  ++end;                                          // saturates
  EXPECT(end == loader.end());
  DataLoader r1(ds, 3, /*rank=*/1, /*world=*/2);
  EXPECT(r1.NumBatches() == 1);

  std::vector<std::string> table;
  for (int i = 0; i < 50300; ++i) table.push_back("<" + std::to_string(i) + ">");
  const std::string tk_path = dir + "/tokenizer.bin";
  titb::data::WriteTokenizer(tk_path, table, 20240328, 50256);
  Tokenizer tokenizer(tk_path);
  EXPECT(tokenizer.GetEndToken() == 50256 && tokenizer.Decode(7) == "<7>");

  GPT2Config cfg;
  cfg.block_size = 16; cfg.vocab_size = 97; cfg.n_layer = 2; cfg.n_head = 2; cfg.n_embd = 32;
  GPT2 model(cfg);
  model.To(g_dev);
  EXPECT(model.StateDict().count("transformer.h.1.attn.c_attn.weight") == 1);
  EXPECT(model.StateDict().at("lm_head.weight") == model.StateDict().at("transformer.wte.weight"));   // tied: one tensor
  optimizers::SGD opt(model.Parameters(), 0.05f);
  nn::CrossEntropyLoss loss_fn;
  std::vector<float> losses;
  for (int step = 0; step < 4; ++step) {
    auto it = loader.begin();                     // the reference restarts its loader every step
    opt.ZeroGrad();
    auto [x, y] = *it;
    auto xd = std::make_shared<Tensor>(x->To(g_dev)), yd = std::make_shared<Tensor>(y->To(g_dev));
    auto logits = model.Forward({xd})[0];
    EXPECT((logits->Dims() == std::vector<int64_t>{3, 16, 97}));
    auto loss = loss_fn.Forward({logits, yd})[0];
    losses.push_back(loss->ToFloatVector()[0]);
    loss->Backward();
    opt.Step();
  }
  EXPECT(std::fabs(losses[0] - std::log(97.f)) < 0.3f && losses[3] < losses[0]);
}

int main(int argc, char** argv) {
  const std::string dev = argc > 1 ? argv[1] : "cpu";
  const std::string dir = argc > 2 ? argv[2] : "/tmp";
  g_dev = dev == "cuda" ? Device(DeviceType::kCUDA, 0) : Device();
  // optional third argument: run one case group only (the reference has one test program per group)
  const std::string only = argc > 3 ? argv[3] : "";
  auto want = [&](const char* name) { return only.empty() || only == name; };
  try {
    if (want("elementwise")) TestNeg();
    if (want("matmul")) TestMatmul();
    if (want("adam")) TestAdam();
    if (want("autograd")) TestTensorAutograd();
    if (want("dispatcher")) TestDispatcher();
    if (want("tensor")) TestUniformAndPrintOptions();
    if (want("gpt2")) TestDataAndTraining(dir);
  } catch (const std::exception& e) {
    std::printf("EXCEPTION: %s\n", e.what());
    return 2;
  }
  std::printf(g_failed ? "%d check(s) failed\n" : "all checks passed\n", g_failed);
  return g_failed ? 1 : 0;
}
