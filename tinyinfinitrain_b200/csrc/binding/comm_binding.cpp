// Python bindings of the NVLink communication kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kernels/api.h"

namespace {
using at::Tensor;

void check(int rc, const char* what) {
  TORCH_CHECK(rc < 20000, "titb200: ", what, ": unsupported arguments (world > 16, bad channel or shard size)");
  TORCH_CHECK(rc == 0, "titb200: ", what, " failed: ", cudaGetErrorString(static_cast<cudaError_t>(rc)));
}
std::vector<unsigned long long> to_u64(const std::vector<int64_t>& v) {
  std::vector<unsigned long long> r(v.size());
  for (size_t i = 0; i < v.size(); ++i) r[i] = static_cast<unsigned long long>(v[i]);
  return r;
}

void comm_barrier(const std::vector<int64_t>& pad_ptrs, int64_t rank, int64_t channel, const Tensor& epoch,
                  double timeout_s) {
  TORCH_CHECK(epoch.is_cuda() && epoch.scalar_type() == at::kInt && epoch.numel() >= 1);
  c10::cuda::CUDAGuard guard(epoch.device());
  auto p = to_u64(pad_ptrs);
  check(titb_comm_barrier(p.data(), (int)rank, (int)p.size(), (int)channel,
                          reinterpret_cast<unsigned int*>(epoch.data_ptr<int>()), timeout_s,
                          at::cuda::getCurrentCUDAStream().stream()), "comm_barrier");
}

void rs_adam_ag(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& param_ptrs, int64_t grad_mc,
                int64_t param_mc, const Tensor& master, const Tensor& m, const Tensor& v, int64_t shard_off,
                int64_t rank, double lr, double b1, double b2, double eps, double wd, int64_t step, double grad_scale,
                const c10::optional<Tensor>& dev_state, int64_t max_blocks) {
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous());
  c10::cuda::CUDAGuard guard(master.device());
  auto g = to_u64(grad_ptrs), p = to_u64(param_ptrs);
  TORCH_CHECK(g.size() == p.size());
  TitbRsAdamDesc d{};
  d.grad_ptrs = g.data(); d.param_ptrs = p.data();
  d.grad_mc = reinterpret_cast<const void*>(grad_mc); d.param_mc = reinterpret_cast<void*>(param_mc);
  d.master = master.data_ptr<float>(); d.m = m.data_ptr<float>(); d.v = v.data_ptr<float>();
  d.shard_off = shard_off; d.shard_n = master.numel();
  d.world = (int)g.size(); d.rank = (int)rank;
  d.lr = (float)lr; d.beta1 = (float)b1; d.beta2 = (float)b2; d.eps = (float)eps; d.weight_decay = (float)wd;
  d.bc1 = (float)(1.0 - std::pow(b1, (double)step)); d.bc2 = (float)(1.0 - std::pow(b2, (double)step));
  d.grad_scale = (float)grad_scale;
  d.dev_state = dev_state.has_value() && dev_state->defined() ? dev_state->data_ptr<float>() : nullptr;
  d.max_blocks = (int)max_blocks;
  check(titb_rs_adam_ag(&d, at::cuda::getCurrentCUDAStream().stream()), "rs_adam_ag");
}

void allreduce_small(const std::vector<int64_t>& buf_ptrs, const Tensor& out, int64_t op) {
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous());
  c10::cuda::CUDAGuard guard(out.device());
  auto b = to_u64(buf_ptrs);
  check(titb_allreduce_small(b.data(), out.data_ptr<float>(), (int)out.numel(), (int)b.size(), (int)op,
                             at::cuda::getCurrentCUDAStream().stream()), "allreduce_small");
}
}  // namespace

void bind_comm(pybind11::module_& m) {
  m.def("comm_barrier", &comm_barrier);
  m.def("rs_adam_ag", &rs_adam_ag, py::arg("grad_ptrs"), py::arg("param_ptrs"), py::arg("grad_mc"),
        py::arg("param_mc"), py::arg("master"), py::arg("m"), py::arg("v"), py::arg("shard_off"), py::arg("rank"),
        py::arg("lr"), py::arg("b1"), py::arg("b2"), py::arg("eps"), py::arg("wd"), py::arg("step"),
        py::arg("grad_scale"), py::arg("dev_state") = py::none(), py::arg("max_blocks") = 0);
  m.def("allreduce_small", &allreduce_small);
}
