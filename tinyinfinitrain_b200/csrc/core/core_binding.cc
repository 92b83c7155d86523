// Python bindings of the C++ framework core.
#include <torch/extension.h>

#include "core/rng.h"

namespace {

std::optional<uint32_t> opt_seed(const c10::optional<int64_t>& s) {
  if (s.has_value()) return static_cast<uint32_t>(*s);
  return std::nullopt;
}

void rng_normal_(at::Tensor t, double mean, double std, c10::optional<int64_t> seed) {
  TORCH_CHECK(t.device().is_cpu() && t.scalar_type() == at::kFloat && t.is_contiguous(),
              "rng_normal_: contiguous CPU float tensor expected");
  titb::rng::fill_normal(t.data_ptr<float>(), t.numel(), (float)mean, (float)std, opt_seed(seed));
}
void rng_uniform_(at::Tensor t, double lo, double hi, c10::optional<int64_t> seed) {
  TORCH_CHECK(t.device().is_cpu() && t.scalar_type() == at::kFloat && t.is_contiguous(),
              "rng_uniform_: contiguous CPU float tensor expected");
  titb::rng::fill_uniform(t.data_ptr<float>(), t.numel(), (float)lo, (float)hi, opt_seed(seed));
}
void rng_randint_(at::Tensor t, int64_t lo, int64_t hi, int64_t seed) {
  TORCH_CHECK(t.device().is_cpu() && t.scalar_type() == at::kLong && t.is_contiguous(),
              "rng_randint_: contiguous CPU int64 tensor expected");
  titb::rng::fill_randint(t.data_ptr<int64_t>(), t.numel(), lo, hi, (uint32_t)seed);
}

}  // namespace

void bind_core(pybind11::module_& m) {
  m.def("rng_seed", [](int64_t s) { titb::rng::seed_global((uint32_t)s); });
  m.def("rng_normal_", &rng_normal_, py::arg("t"), py::arg("mean"), py::arg("std"), py::arg("seed") = py::none());
  m.def("rng_uniform_", &rng_uniform_, py::arg("t"), py::arg("lo"), py::arg("hi"), py::arg("seed") = py::none());
  m.def("rng_randint_", &rng_randint_);
}
