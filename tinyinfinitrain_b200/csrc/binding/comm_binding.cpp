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

// In-place sum (times scale) / gather over the ranks of a byte range of a symmetric buffer; the caller brackets the
// call with the device barrier.
void symm_allreduce(const std::vector<int64_t>& buf_ptrs, int64_t mc_ptr, int64_t byte_off, int64_t nbytes, int64_t dtype,
                    int64_t rank, double scale, int64_t max_blocks) {
  auto b = to_u64(buf_ptrs);
  check(titb_symm_allreduce(b.data(), (unsigned long long)mc_ptr, byte_off, nbytes, (int)dtype, (int)b.size(), (int)rank,
                            (float)scale, (int)max_blocks, at::cuda::getCurrentCUDAStream().stream()), "symm_allreduce");
}
void symm_allgather(const std::vector<int64_t>& buf_ptrs, int64_t mc_ptr, int64_t byte_off, int64_t nbytes, int64_t rank,
                    int64_t max_blocks) {
  auto b = to_u64(buf_ptrs);
  check(titb_symm_allgather(b.data(), (unsigned long long)mc_ptr, byte_off, nbytes, (int)b.size(), (int)rank,
                            (int)max_blocks, at::cuda::getCurrentCUDAStream().stream()), "symm_allgather");
}

void symm_signal(int64_t remote_word, int64_t value) {
  check(titb_symm_signal((unsigned long long)remote_word, (unsigned int)value, at::cuda::getCurrentCUDAStream().stream()),
        "symm_signal");
}
void symm_wait(int64_t local_word, int64_t value, double timeout_s) {
  check(titb_symm_wait((unsigned long long)local_word, (unsigned int)value, timeout_s,
                       at::cuda::getCurrentCUDAStream().stream()), "symm_wait");
}

// ---- gradient-norm clipping ---------------------------------------------------------------------------------------
// Clips a flat fp32 gradient buffer in place to `max_norm` (norm taken of pre_scale * grad); `out` is a device
// tensor of two floats that receives {norm, coefficient}.  Everything stays on the device.
void clip_grad_norm_(const Tensor& grad, double max_norm, double pre_scale, const Tensor& out) {
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == at::kFloat && grad.is_contiguous());
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.numel() >= 2 && max_norm > 0);
  c10::cuda::CUDAGuard guard(grad.device());
  auto st = at::cuda::getCurrentCUDAStream().stream();
  Tensor partials = at::empty({titb_clip_max_partials()}, grad.options());
  int np = 0;
  check(titb_sumsq_partials(grad.data_ptr<float>(), grad.numel(), partials.data_ptr<float>(), &np, st), "sumsq");
  check(titb_clip_coef(partials.data_ptr<float>(), np, (float)pre_scale, (float)max_norm, out.data_ptr<float>(), st), "clip_coef");
  check(titb_scale_by_dev(grad.data_ptr<float>(), grad.numel(), out.data_ptr<float>() + 1, st), "scale_by_dev");
}
// out[0] = squared norm of this rank's shard of the cross-rank gradient sum (no scaling applied).
void rs_grad_sumsq(const std::vector<int64_t>& grad_ptrs, int64_t grad_mc, int64_t shard_off, int64_t shard_n, int64_t rank,
                   const Tensor& out) {
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.numel() >= 1);
  c10::cuda::CUDAGuard guard(out.device());
  auto st = at::cuda::getCurrentCUDAStream().stream();
  auto g = to_u64(grad_ptrs);
  Tensor partials = at::empty({titb_clip_max_partials()}, out.options());
  int np = 0;
  check(titb_rs_sumsq_partials(g.data(), reinterpret_cast<const void*>(grad_mc), shard_off, shard_n, (int)g.size(), (int)rank,
                               partials.data_ptr<float>(), &np, st), "rs_sumsq");
  check(titb_clip_coef(partials.data_ptr<float>(), np, 1.f, 0.f, out.data_ptr<float>(), st), "sum_partials");
}
// total: device tensor whose first n values are summed (e.g. the ranks' squared norms); out = {norm, coefficient}.
void clip_coef_from_totals(const Tensor& totals, int64_t n, double pre_scale, double max_norm, const Tensor& out) {
  TORCH_CHECK(totals.is_cuda() && totals.scalar_type() == at::kFloat && totals.numel() >= n && out.numel() >= 2 && max_norm > 0);
  c10::cuda::CUDAGuard guard(out.device());
  check(titb_clip_coef(totals.data_ptr<float>(), (int)n, (float)pre_scale, (float)max_norm, out.data_ptr<float>(),
                       at::cuda::getCurrentCUDAStream().stream()), "clip_coef");
}
// out[0] = sum of squares of a flat fp32 tensor (fixed summation order).
void sumsq_(const Tensor& x, const Tensor& out) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous() && out.is_cuda() &&
              out.scalar_type() == at::kFloat && out.numel() >= 1);
  c10::cuda::CUDAGuard guard(x.device());
  auto st = at::cuda::getCurrentCUDAStream().stream();
  if (x.numel() == 0) { out.narrow(0, 0, 1).zero_(); return; }
  Tensor partials = at::empty({titb_clip_max_partials()}, x.options());
  int np = 0;
  check(titb_sumsq_partials(x.data_ptr<float>(), x.numel(), partials.data_ptr<float>(), &np, st), "sumsq");
  check(titb_clip_coef(partials.data_ptr<float>(), np, 1.f, 0.f, out.data_ptr<float>(), st), "sum_partials");
}
void scale_by_dev_(const Tensor& x, const Tensor& coef) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous() && coef.is_cuda() &&
              coef.scalar_type() == at::kFloat && coef.numel() >= 1);
  c10::cuda::CUDAGuard guard(x.device());
  check(titb_scale_by_dev(x.data_ptr<float>(), x.numel(), coef.data_ptr<float>(), at::cuda::getCurrentCUDAStream().stream()),
        "scale_by_dev");
}
}  // namespace

void bind_comm(pybind11::module_& m) {
  m.def("comm_barrier", &comm_barrier);
  m.def("rs_adam_ag", &rs_adam_ag, py::arg("grad_ptrs"), py::arg("param_ptrs"), py::arg("grad_mc"),
        py::arg("param_mc"), py::arg("master"), py::arg("m"), py::arg("v"), py::arg("shard_off"), py::arg("rank"),
        py::arg("lr"), py::arg("b1"), py::arg("b2"), py::arg("eps"), py::arg("wd"), py::arg("step"),
        py::arg("grad_scale"), py::arg("dev_state") = py::none(), py::arg("max_blocks") = 0);
  m.def("allreduce_small", &allreduce_small);
  m.def("symm_allreduce", &symm_allreduce, py::arg("buf_ptrs"), py::arg("mc_ptr"), py::arg("byte_off"), py::arg("nbytes"),
        py::arg("dtype"), py::arg("rank"), py::arg("scale") = 1.0, py::arg("max_blocks") = 0);
  m.def("symm_signal", &symm_signal);
  m.def("symm_wait", &symm_wait, py::arg("local_word"), py::arg("value"), py::arg("timeout_s") = 2.0);
  m.def("symm_allgather", &symm_allgather, py::arg("buf_ptrs"), py::arg("mc_ptr"), py::arg("byte_off"), py::arg("nbytes"),
        py::arg("rank"), py::arg("max_blocks") = 0);
  m.def("clip_grad_norm_", &clip_grad_norm_);
  m.def("rs_grad_sumsq", &rs_grad_sumsq);
  m.def("clip_coef_from_totals", &clip_coef_from_totals);
  m.def("scale_by_dev_", &scale_by_dev_);
  m.def("sumsq_", &sumsq_);
}
