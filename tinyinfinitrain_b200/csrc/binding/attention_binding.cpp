// Python bindings of the fused causal attention kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "kernels/api.h"

namespace {
using at::Tensor;

// [B, T, H, hd] view whose head dim is dense and whose batch stride is T * token stride,
// i.e. a column slice of a [B*T, W] row-major buffer.
bool is_token_major(const Tensor& t) {
  return t.dim() == 4 && t.stride(3) == 1 && t.stride(2) == t.size(3) && t.stride(0) == t.size(1) * t.stride(1) &&
         (t.stride(1) % 8) == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16) == 0;
}
Tensor token_major(const Tensor& t) { return is_token_major(t) ? t : t.contiguous(); }

void check(int rc, const char* what) {
  TORCH_CHECK(rc != TITB_ERR_SHAPE, "titb200: ", what, ": head_dim must be 64 or 128 and Hq % Hkv == 0");
  TORCH_CHECK(rc != TITB_ERR_ALIGNMENT, "titb200: ", what, ": operands must be 16-byte aligned");
  TORCH_CHECK(rc != TITB_ERR_TENSOR_MAP, "titb200: ", what, ": TMA tensor map could not be encoded");
  TORCH_CHECK(rc == 0, "titb200: ", what, " failed: ", cudaGetErrorString(static_cast<cudaError_t>(rc)));
}

std::vector<Tensor> attn_fwd(const Tensor& q_, const Tensor& k_, const Tensor& v_, double scale) {
  TORCH_CHECK(q_.is_cuda() && q_.scalar_type() == at::kBFloat16, "titb200 attention: bf16 CUDA tensors");
  c10::cuda::CUDAGuard guard(q_.device());
  Tensor q = token_major(q_), k = token_major(k_), v = token_major(v_);
  const int64_t B = q.size(0), T = q.size(1), Hq = q.size(2), hd = q.size(3), Hkv = k.size(2);
  Tensor o = at::empty({B, T, Hq, hd}, q.options());
  Tensor lse = at::empty({B, Hq, T}, q.options().dtype(at::kFloat));
  TitbAttnDesc d{};
  d.q = q.data_ptr(); d.k = k.data_ptr(); d.v = v.data_ptr(); d.o = o.data_ptr(); d.lse = lse.data_ptr<float>();
  d.B = (int)B; d.T = (int)T; d.Hq = (int)Hq; d.Hkv = (int)Hkv; d.hd = (int)hd;
  d.q_stride_t = q.stride(1); d.k_stride_t = k.stride(1); d.v_stride_t = v.stride(1); d.o_stride_t = Hq * hd;
  d.scale = (float)scale;
  check(titb_attn_fwd(&d, at::cuda::getCurrentCUDAStream().stream()), "attn_fwd");
  return {o, lse};
}

// Gradients are written into dq/dk/dv when given (token-major views, e.g. slices of one fused
// dQKV buffer); otherwise fresh contiguous tensors are returned.
std::vector<Tensor> attn_bwd(const Tensor& d_o_, const Tensor& q_, const Tensor& k_, const Tensor& v_, const Tensor& o,
                             const Tensor& lse, double scale, const c10::optional<Tensor>& dq_,
                             const c10::optional<Tensor>& dk_, const c10::optional<Tensor>& dv_) {
  c10::cuda::CUDAGuard guard(q_.device());
  Tensor q = token_major(q_), k = token_major(k_), v = token_major(v_), d_o = token_major(d_o_);
  const int64_t B = q.size(0), T = q.size(1), Hq = q.size(2), hd = q.size(3), Hkv = k.size(2);
  Tensor dq = dq_.has_value() && dq_->defined() ? *dq_ : at::empty({B, T, Hq, hd}, q.options());
  Tensor dk = dk_.has_value() && dk_->defined() ? *dk_ : at::empty({B, T, Hkv, hd}, q.options());
  Tensor dv = dv_.has_value() && dv_->defined() ? *dv_ : at::empty({B, T, Hkv, hd}, q.options());
  TORCH_CHECK(is_token_major(dq) && is_token_major(dk) && is_token_major(dv), "titb200 attention: bad gradient views");
  Tensor delta = at::empty({B, Hq, T}, q.options().dtype(at::kFloat));
  Tensor acc = at::empty({B, T, Hq, hd}, q.options().dtype(at::kFloat));
  TitbAttnDesc d{};
  d.q = q.data_ptr(); d.k = k.data_ptr(); d.v = v.data_ptr(); d.o = o.data_ptr(); d.lse = lse.data_ptr<float>();
  d.d_o = d_o.data_ptr(); d.dq = dq.data_ptr(); d.dk = dk.data_ptr(); d.dv = dv.data_ptr();
  d.delta = delta.data_ptr<float>(); d.dq_accum = acc.data_ptr<float>();
  d.B = (int)B; d.T = (int)T; d.Hq = (int)Hq; d.Hkv = (int)Hkv; d.hd = (int)hd;
  d.q_stride_t = q.stride(1); d.k_stride_t = k.stride(1); d.v_stride_t = v.stride(1); d.o_stride_t = o.stride(1);
  d.do_stride_t = d_o.stride(1); d.dq_stride_t = dq.stride(1); d.dk_stride_t = dk.stride(1); d.dv_stride_t = dv.stride(1);
  d.scale = (float)scale;
  check(titb_attn_bwd(&d, at::cuda::getCurrentCUDAStream().stream()), "attn_bwd");
  return {dq, dk, dv};
}
}  // namespace

void bind_attention(pybind11::module_& m) {
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd, py::arg("d_o"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("lse"),
        py::arg("scale"), py::arg("dq") = py::none(), py::arg("dk") = py::none(), py::arg("dv") = py::none());
}
