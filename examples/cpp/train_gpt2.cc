// GPT-2 training through the C++ API, following the reference's fixture (test/example/test_gpt2.cc:104-227): load an
// llm.c checkpoint (or start from the seeded random initialisation), read a TinyShakespeare token file, accumulate
// gradients over total_batch_size / (batch_size * sequence_length) micro-steps, take SGD steps, and optionally compare
// the last micro-step's logits with a reference blob and generate text.
//
//   train_gpt2 --input_bin tiny_shakespeare_train.bin [--llmc_filepath gpt2_124M.bin] [--tokenizer_bin gpt2_tokenizer.bin]
//              [--logits_reference gpt2_logits_reference.bin] [--device cuda|cpu] [--batch_size 2] [--sequence_length 64]
//              [--total_batch_size 256] [--num_iteration 10] [--learning_rate 1e-4] [--text_length 64]
//              [--freq_generate_txt 10] [--n_layer N --n_head N --n_embd N  (random-init model size)]
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "core/framework/data_facade.h"
#include "core/framework/gpt2.h"
#include "core/framework/nn.h"
#include "core/framework/tensor.h"

using namespace infini_train;

// Blob layout: uint64 ndims; int64 dims[ndims]; float data[].  100 evenly spaced elements, |diff| <= tolerance.
static bool ValidateLogits(const Tensor& logits, const std::string& path, float tolerance = 1e-3f) {
  std::ifstream in(path, std::ios::binary);
  if (!in) { std::printf("cannot open %s\n", path.c_str()); return false; }
  uint64_t nd = 0;
  in.read(reinterpret_cast<char*>(&nd), 8);
  std::vector<int64_t> dims(nd);
  in.read(reinterpret_cast<char*>(dims.data()), static_cast<std::streamsize>(8 * nd));
  if (dims != logits.Dims()) { std::printf("logits shape differs from the reference blob\n"); return false; }
  size_t n = 1;
  for (int64_t d : dims) n *= static_cast<size_t>(d);
  std::vector<float> ref(n);
  in.read(reinterpret_cast<char*>(ref.data()), static_cast<std::streamsize>(4 * n));
  const std::vector<float> cur = logits.ToFloatVector();
  float worst = 0.f;
  for (int i = 0; i < 100; ++i) {
    const size_t idx = static_cast<size_t>(i) * n / 100;
    worst = std::fmax(worst, std::fabs(ref[idx] - cur[idx]));
  }
  std::printf("logits check: worst sampled |diff| = %g (tolerance %g)\n", worst, tolerance);
  return worst <= tolerance;
}

int main(int argc, char** argv) {
  std::map<std::string, std::string> flag = {
      {"llmc_filepath", ""}, {"input_bin", ""}, {"tokenizer_bin", ""}, {"logits_reference", ""}, {"device", "cuda"},
      {"batch_size", "2"}, {"sequence_length", "64"}, {"total_batch_size", "256"}, {"num_iteration", "10"},
      {"learning_rate", "1e-4"}, {"text_length", "64"}, {"freq_generate_txt", "10"}, {"n_layer", "12"}, {"n_head", "12"},
      {"n_embd", "768"}};
  for (int i = 1; i + 1 < argc; i += 2) {
    std::string k = argv[i];
    if (k.rfind("--", 0) != 0 || !flag.count(k.substr(2))) { std::printf("unknown flag %s\n", argv[i]); return 2; }
    flag[k.substr(2)] = argv[i + 1];
  }
  if (flag["input_bin"].empty()) { std::printf("--input_bin is required\n"); return 2; }
  const Device device = flag["device"] == "cpu" ? Device() : Device(DeviceType::kCUDA, 0);
  const size_t B = std::stoul(flag["batch_size"]), T = std::stoul(flag["sequence_length"]);
  const int accum = std::max<int>(1, std::stoi(flag["total_batch_size"]) / static_cast<int>(B * T));
  const int iters = std::stoi(flag["num_iteration"]), gen_every = std::stoi(flag["freq_generate_txt"]);

  std::unique_ptr<GPT2> model;
  if (!flag["llmc_filepath"].empty()) {
    model = GPT2::FromLLMC(flag["llmc_filepath"]);
  } else {
    GPT2Config cfg;
    cfg.n_layer = std::stoi(flag["n_layer"]); cfg.n_head = std::stoi(flag["n_head"]); cfg.n_embd = std::stoi(flag["n_embd"]);
    model = std::make_unique<GPT2>(cfg);
  }
  model->To(device);
  DataLoader loader(std::make_shared<TinyShakespeareDataset>(flag["input_bin"], T), B);
  optimizers::SGD optimizer(model->Parameters(), std::stof(flag["learning_rate"]));
  nn::CrossEntropyLoss loss_fn;
  std::unique_ptr<Tokenizer> tokenizer;
  if (!flag["tokenizer_bin"].empty()) tokenizer = std::make_unique<Tokenizer>(flag["tokenizer_bin"]);

  std::shared_ptr<Tensor> logits;
  for (int step = 0; step < iters + 1; ++step) {        // the reference runs num_iteration + 1 optimizer steps
    auto it = loader.begin();                           // ... and restarts the loader in each of them
    optimizer.ZeroGrad();
    float lossf = 0.f;
    for (int micro = 0; micro < accum; ++micro) {
      auto [x, y] = *it;
      ++it;
      auto xd = std::make_shared<Tensor>(x->To(device)), yd = std::make_shared<Tensor>(y->To(device));
      logits = model->Forward({xd})[0];
      auto loss = loss_fn.Forward({logits, yd})[0];
      lossf += loss->ToFloatVector()[0] / static_cast<float>(accum);
      loss->Backward();
    }
    optimizer.Step();
    std::printf("step %d/%d | loss %.6f\n", step + 1, iters + 1, lossf);
    if (tokenizer && gen_every > 0 && (step + 1) % gen_every == 0)
      tokenizer->GenerateText(*model, static_cast<uint32_t>(B), static_cast<uint32_t>(T),
                              static_cast<uint32_t>(std::stoul(flag["text_length"])), device);
  }
  if (!flag["logits_reference"].empty()) return ValidateLogits(*logits, flag["logits_reference"]) ? 0 : 1;
  return 0;
}
