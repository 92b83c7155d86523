#include "core/rng.h"

namespace titb {
namespace rng {

std::mt19937& global_generator() {
  static std::mt19937 gen{std::random_device{}()};
  return gen;
}
void seed_global(uint32_t seed) { global_generator().seed(seed); }

void fill_normal(float* out, int64_t n, float mean, float std, std::optional<uint32_t> seed) {
  std::normal_distribution<float> dist(mean, std);
  if (seed.has_value()) {
    std::mt19937 gen(*seed);
    for (int64_t i = 0; i < n; ++i) out[i] = dist(gen);
  } else {
    auto& gen = global_generator();
    for (int64_t i = 0; i < n; ++i) out[i] = dist(gen);
  }
}

void fill_uniform(float* out, int64_t n, float lo, float hi, std::optional<uint32_t> seed) {
  std::uniform_real_distribution<float> dist(lo, hi);
  if (seed.has_value()) {
    std::mt19937 gen(*seed);
    for (int64_t i = 0; i < n; ++i) out[i] = dist(gen);
  } else {
    auto& gen = global_generator();
    for (int64_t i = 0; i < n; ++i) out[i] = dist(gen);
  }
}

void fill_randint(int64_t* out, int64_t n, int64_t lo, int64_t hi, uint32_t seed) {
  std::mt19937 gen(seed);
  std::uniform_int_distribution<int64_t> dist(lo, hi - 1);
  for (int64_t i = 0; i < n; ++i) out[i] = dist(gen);
}

}  // namespace rng
}  // namespace titb
