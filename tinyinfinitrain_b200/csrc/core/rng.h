// Host random number generation with the reference's exact semantics.
//
// The reference initialises tensors on the host with std::mt19937 and libstdc++'s
// std::normal_distribution<float> / std::uniform_real_distribution<float>
// (infini_train/src/nn/init.cc:24-48, :50-70); "same seed => same weights" therefore
// depends on those library sequences, which is why this lives in C++ and not in
// torch.manual_seed.  A generator passed explicitly is used from a copy (the
// reference takes std::optional<std::mt19937> by value), the global one advances.
#pragma once
#include <cstdint>
#include <optional>
#include <random>

namespace titb {
namespace rng {

std::mt19937& global_generator();
void seed_global(uint32_t seed);

// Fills n floats from N(mean, std); `seed` engaged => a fresh mt19937(seed) is used.
void fill_normal(float* out, int64_t n, float mean, float std, std::optional<uint32_t> seed);
void fill_uniform(float* out, int64_t n, float lo, float hi, std::optional<uint32_t> seed);
// Uniform integers in [lo, hi) with std::uniform_int_distribution<int64_t>.
void fill_randint(int64_t* out, int64_t n, int64_t lo, int64_t hi, uint32_t seed);

}  // namespace rng
}  // namespace titb
