#include "core/framework/autograd.h"

#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <tuple>

#include "core/framework/dispatcher.h"

namespace infini_train::autograd {

namespace {
using TP = std::shared_ptr<Tensor>;
using Dims = std::vector<int64_t>;
using TPPair = std::pair<TP, TP>;
using TPTriple = std::tuple<TP, TP, TP>;

// TITB200_NVTX=1: every kernel dispatch drops an NVTX marker with the kernel's registered name ("LinearForward",
// "LayerNormBackward", ...), so an Nsight timeline of a C++ program shows the op sequence (the reference has no tracing).
const bool kNvtxMarkers = [] { const char* e = std::getenv("TITB200_NVTX"); return e != nullptr && e[0] == '1'; }();

const KernelFunction& K(const TP& t, const char* name) {
  if (kNvtxMarkers) nvtxMarkA(name);
  return Dispatcher::Instance().GetKernel({t->GetDevice().Type(), name});
}
}  // namespace

// ---------------------------------------------------------------------------------- engine
TensorList Function::Apply(const TensorList& input_tensors) {
  TensorList outputs = Forward(input_tensors);
  SetupContext(input_tensors, outputs);
  bool any_requires_grad = false;
  for (const auto& in : input_tensors) {
    if (!in) { next_functions_.emplace_back(nullptr, -1); continue; }
    if (in->requires_grad() && in->is_leaf()) {
      next_functions_.emplace_back(std::make_shared<AccumulateGrad>(in->grad()), 0);
    } else {
      next_functions_.emplace_back(in->grad_fn(), in->output_idx());
      if (in->grad_fn()) in->grad_fn()->IncreaseDependenciesNumber();
    }
    any_requires_grad = any_requires_grad || in->requires_grad();
  }
  grad_outputs_.assign(outputs.size(), nullptr);
  for (size_t i = 0; i < outputs.size(); ++i) {
    auto& out = outputs[i];
    if (!out) continue;
    out->set_requires_grad(any_requires_grad);
    out->set_is_leaf(!any_requires_grad);
    if (any_requires_grad) {
      out->set_grad_fn(shared_from_this());
      out->set_output_idx(static_cast<int>(i));
    }
  }
  return outputs;
}

void Function::BackwardPartial(const TP& grad_output, int idx) {
  TORCH_CHECK(idx >= 0 && idx < static_cast<int>(grad_outputs_.size()), "bad output index in backward");
  if (!grad_outputs_[idx]) {
    grad_outputs_[idx] = grad_output;
    ++grad_outputs_reached_;
  } else {
    // a second consumer of the same output: sum the gradients
    TP acc = std::make_shared<Tensor>(grad_outputs_[idx]->data().clone());
    K(acc, "AccumulateGrad").Call<void, const TP&, float, const TP&>(grad_output, 1.0f, acc);
    grad_outputs_[idx] = acc;
  }
  ++dependencies_reached_;
  const bool all_slots = grad_outputs_reached_ == static_cast<int>(grad_outputs_.size());
  const bool all_consumers = dependencies_reached_ >= dependencies_number_ || dependencies_number_ == 0;
  if (!(all_slots && all_consumers)) return;
  TensorList grads = Backward(grad_outputs_);
  saved_tensors_.clear();
  grad_outputs_.assign(grad_outputs_.size(), nullptr);
  grad_outputs_reached_ = 0;
  dependencies_reached_ = 0;
  TORCH_CHECK(grads.size() == next_functions_.size(), "Backward returned ", grads.size(), " gradients for ",
              next_functions_.size(), " inputs");
  for (size_t i = 0; i < grads.size(); ++i) {
    auto& [fn, out_idx] = next_functions_[i];
    if (fn && grads[i]) fn->BackwardPartial(grads[i], out_idx);
  }
}

TensorList AccumulateGrad::Forward(const TensorList&) { TORCH_CHECK(false, "AccumulateGrad has no Forward"); }
TensorList AccumulateGrad::Backward(const TensorList&) { TORCH_CHECK(false, "AccumulateGrad has no Backward"); }
void AccumulateGrad::BackwardPartial(const TP& grad_output, int) {
  if (!grad_) return;
  K(grad_, "AccumulateGrad").Call<void, const TP&, float, const TP&>(grad_output, learning_rate_, grad_);
}

// ---------------------------------------------------------------------------------- unary
#define UNARY_IMPL(Name, SAVE_OUTPUT)                                                                   \
  TensorList Name::Forward(const TensorList& in) {                                                      \
    return {K(in[0], #Name "Forward").Call<TP, const TP&>(in[0])};                                      \
  }                                                                                                     \
  void Name::SetupContext(const TensorList& in, const TensorList& out) {                                \
    saved_tensors_ = {SAVE_OUTPUT ? out[0] : in[0]};                                                    \
  }                                                                                                     \
  TensorList Name::Backward(const TensorList& g) {                                                      \
    return {K(g[0], #Name "Backward").Call<TP, const TP&, const TP&>(g[0], saved_tensors_[0])};         \
  }
UNARY_IMPL(Neg, false)
UNARY_IMPL(Reciprocal, false)
UNARY_IMPL(Sin, false)
UNARY_IMPL(Cos, false)
UNARY_IMPL(Tanh, true)
UNARY_IMPL(Rsqrt, false)
UNARY_IMPL(Sigmoid, true)
UNARY_IMPL(Gelu, false)

TensorList Pow::Forward(const TensorList& in) {
  return {K(in[0], "PowForward").Call<TP, const TP&, float, bool>(in[0], exponent_, scalar_is_base_)};
}
void Pow::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0]}; }
TensorList Pow::Backward(const TensorList& g) {
  return {K(g[0], "PowBackward").Call<TP, const TP&, const TP&, float, bool>(g[0], saved_tensors_[0], exponent_, scalar_is_base_)};
}
TensorList EqualsScalar::Forward(const TensorList& in) {
  return {K(in[0], "EqualsScalarForward").Call<TP, const TP&, float>(in[0], scalar_)};
}
void EqualsScalar::SetupContext(const TensorList&, const TensorList&) {}
TensorList EqualsScalar::Backward(const TensorList&) { TORCH_CHECK(false, "EqualsScalar::Backward shall not be called"); }
TensorList AddScalar::Forward(const TensorList& in) {
  return {K(in[0], "AddScalarForward").Call<TP, const TP&, float>(in[0], scalar_)};
}
void AddScalar::SetupContext(const TensorList&, const TensorList&) {}
TensorList AddScalar::Backward(const TensorList& g) { return {K(g[0], "AddScalarBackward").Call<TP, const TP&>(g[0])}; }
TensorList MulScalar::Forward(const TensorList& in) {
  return {K(in[0], "MulScalarForward").Call<TP, const TP&, float>(in[0], scalar_)};
}
void MulScalar::SetupContext(const TensorList&, const TensorList&) {}
TensorList MulScalar::Backward(const TensorList& g) {
  return {K(g[0], "MulScalarBackward").Call<TP, const TP&, float>(g[0], scalar_)};
}

// ---------------------------------------------------------------------------------- binary
#define BINARY_DIMS_IMPL(Name)                                                                              \
  TensorList Name::Forward(const TensorList& in) {                                                          \
    return {K(in[0], #Name "Forward").Call<TP, const TP&, const TP&>(in[0], in[1])};                        \
  }                                                                                                         \
  void Name::SetupContext(const TensorList& in, const TensorList&) {                                        \
    a_dims_ = in[0]->Dims();                                                                                \
    b_dims_ = in[1]->Dims();                                                                                \
  }                                                                                                         \
  TensorList Name::Backward(const TensorList& g) {                                                          \
    auto [da, db] = K(g[0], #Name "Backward").Call<TPPair, const TP&, const Dims&, const Dims&>(g[0], a_dims_, b_dims_); \
    return {da, db};                                                                                        \
  }
BINARY_DIMS_IMPL(Add)
BINARY_DIMS_IMPL(Sub)
#define BINARY_SAVED_IMPL(Name)                                                                             \
  TensorList Name::Forward(const TensorList& in) {                                                          \
    return {K(in[0], #Name "Forward").Call<TP, const TP&, const TP&>(in[0], in[1])};                        \
  }                                                                                                         \
  void Name::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0], in[1]}; }     \
  TensorList Name::Backward(const TensorList& g) {                                                          \
    auto [da, db] = K(g[0], #Name "Backward").Call<TPPair, const TP&, const TP&, const TP&>(g[0], saved_tensors_[0], saved_tensors_[1]); \
    return {da, db};                                                                                        \
  }
BINARY_SAVED_IMPL(Mul)
BINARY_SAVED_IMPL(Div)

// ---------------------------------------------------------------------------------- GEMM family
TensorList Matmul::Forward(const TensorList& in) {
  return {K(in[0], "MatmulForward").Call<TP, const TP&, const TP&>(in[0], in[1])};
}
void Matmul::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0], in[1]}; }
TensorList Matmul::Backward(const TensorList& g) {
  auto [da, db] = K(g[0], "MatmulBackward").Call<TPPair, const TP&, const TP&, const TP&>(saved_tensors_[0], saved_tensors_[1], g[0]);
  return {da, db};
}
TensorList Linear::Forward(const TensorList& in) {
  TP bias = in.size() > 2 ? in[2] : nullptr;
  return {K(in[0], "LinearForward").Call<TP, const TP&, const TP&, bool, const TP&>(in[0], in[1], true, bias)};
}
void Linear::SetupContext(const TensorList& in, const TensorList&) {
  saved_tensors_ = {in[0], in[1]};
  bias_ = in.size() > 2 && in[2] != nullptr;
  out_features_ = in[1]->Dims()[0];
}
TensorList Linear::Backward(const TensorList& g) {
  auto [dx, dw, db] = K(g[0], "LinearBackward").Call<TPTriple, const TP&, const TP&, bool, int64_t, const TP&, bool>(
      saved_tensors_[0], saved_tensors_[1], true, out_features_, g[0], bias_);
  if (bias_) return {dx, dw, db};
  return {dx, dw};
}
TensorList Outer::Forward(const TensorList& in) {
  return {K(in[0], "OuterForward").Call<TP, const TP&, const TP&>(in[0], in[1])};
}
void Outer::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0], in[1]}; }
TensorList Outer::Backward(const TensorList& g) {
  auto [da, db] = K(g[0], "OuterBackward").Call<TPPair, const TP&, const TP&, const TP&>(saved_tensors_[0], saved_tensors_[1], g[0]);
  return {da, db};
}

// ---------------------------------------------------------------------------------- norm / softmax / loss / embedding
TensorList LayerNorm::Forward(const TensorList& in) {
  auto [y, mean, rstd] = K(in[0], "LayerNormForward").Call<TPTriple, const TP&, const TP&, const TP&, float>(in[0], in[1], in[2], eps_);
  mean_ = mean;
  rstd_ = rstd;
  return {y};
}
void LayerNorm::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0], in[1], in[2], mean_, rstd_}; }
TensorList LayerNorm::Backward(const TensorList& g) {
  auto [dx, dw, db] = K(g[0], "LayerNormBackward").Call<TPTriple, const TP&, const TP&, const TP&, const TP&, const TP&, const TP&>(
      saved_tensors_[0], saved_tensors_[1], saved_tensors_[2], saved_tensors_[3], saved_tensors_[4], g[0]);
  return {dx, dw, db};
}
TensorList RMSNorm::Forward(const TensorList& in) {
  auto [y, rstd] = K(in[0], "RMSNormForward").Call<std::pair<TP, TP>, const TP&, const TP&, float>(in[0], in[1], eps_);
  rstd_ = rstd;
  return {y};
}
void RMSNorm::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0], in[1], rstd_}; }
TensorList RMSNorm::Backward(const TensorList& g) {
  auto [dx, dw] = K(g[0], "RMSNormBackward").Call<std::pair<TP, TP>, const TP&, const TP&, const TP&, const TP&>(
      saved_tensors_[0], saved_tensors_[1], saved_tensors_[2], g[0]);
  return {dx, dw};
}
TensorList Rope::Forward(const TensorList& in) {
  return {K(in[0], "RopeForward").Call<TP, const TP&, float, int64_t, bool>(in[0], theta_, pos_offset_, false)};
}
void Rope::SetupContext(const TensorList&, const TensorList&) {}
TensorList Rope::Backward(const TensorList& g) {
  // the rotation is orthogonal: its transpose is the rotation by the negative angle
  return {K(g[0], "RopeForward").Call<TP, const TP&, float, int64_t, bool>(g[0], theta_, pos_offset_, true)};
}
TensorList CausalAttention::Forward(const TensorList& in) {
  auto [o, lse] = K(in[0], "CausalAttentionForward").Call<std::pair<TP, TP>, const TP&, const TP&, const TP&, float>(
      in[0], in[1], in[2], scale_);
  out_ = o;
  lse_ = lse;
  return {o};
}
void CausalAttention::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0], in[1], in[2], out_, lse_}; }
TensorList CausalAttention::Backward(const TensorList& g) {
  auto [dq, dk, dv] = K(g[0], "CausalAttentionBackward")
                          .Call<TPTriple, const TP&, const TP&, const TP&, const TP&, const TP&, const TP&, float>(
                              g[0], saved_tensors_[0], saved_tensors_[1], saved_tensors_[2], saved_tensors_[3],
                              saved_tensors_[4], scale_);
  return {dq, dk, dv};
}
TensorList SwiGLU::Forward(const TensorList& in) { return {K(in[0], "SwiGLUForward").Call<TP, const TP&>(in[0])}; }
void SwiGLU::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0]}; }
TensorList SwiGLU::Backward(const TensorList& g) {
  return {K(g[0], "SwiGLUBackward").Call<TP, const TP&, const TP&>(g[0], saved_tensors_[0])};
}
TensorList Softmax::Forward(const TensorList& in) {
  return {K(in[0], "SoftmaxForward").Call<TP, const TP&, int64_t>(in[0], dim_)};
}
void Softmax::SetupContext(const TensorList&, const TensorList& out) { saved_tensors_ = {out[0]}; }
TensorList Softmax::Backward(const TensorList& g) {
  return {K(g[0], "SoftmaxBackward").Call<TP, const TP&, const TP&, int64_t>(g[0], saved_tensors_[0], dim_)};
}
TensorList CrossEntropy::Forward(const TensorList& in) {
  return {K(in[0], "CrossEntropyForward").Call<TP, const TP&, const TP&>(in[0], in[1])};
}
void CrossEntropy::SetupContext(const TensorList& in, const TensorList&) { saved_tensors_ = {in[0], in[1]}; }
TensorList CrossEntropy::Backward(const TensorList& g) {
  return {K(g[0], "CrossEntropyBackward").Call<TP, const TP&, const TP&, const TP&>(saved_tensors_[0], saved_tensors_[1], g[0]), nullptr};
}
TensorList Embedding::Forward(const TensorList& in) {
  return {K(in[1], "EmbeddingForward").Call<TP, const TP&, const TP&>(in[0], in[1])};
}
void Embedding::SetupContext(const TensorList& in, const TensorList&) {
  saved_tensors_ = {in[0]};
  weight_dims_ = in[1]->Dims();
}
TensorList Embedding::Backward(const TensorList& g) {
  return {nullptr, K(g[0], "EmbeddingBackward").Call<TP, const TP&, const Dims&, const TP&>(saved_tensors_[0], weight_dims_, g[0])};
}

// ---------------------------------------------------------------------------------- reductions
#define REDUCE_DIMS_IMPL(Name)                                                                                   \
  TensorList Name::Forward(const TensorList& in) {                                                               \
    return {K(in[0], #Name "Forward").Call<TP, const TP&, int64_t, bool>(in[0], dim_, keep_dim_)};               \
  }                                                                                                              \
  void Name::SetupContext(const TensorList& in, const TensorList&) { input_dims_ = in[0]->Dims(); }              \
  TensorList Name::Backward(const TensorList& g) {                                                               \
    return {K(g[0], #Name "Backward").Call<TP, const TP&, const Dims&, int64_t, bool>(g[0], input_dims_, dim_, keep_dim_)}; \
  }
REDUCE_DIMS_IMPL(Mean)
REDUCE_DIMS_IMPL(Sum)
#define REDUCE_SAVED_IMPL(Name)                                                                                  \
  TensorList Name::Forward(const TensorList& in) {                                                               \
    return {K(in[0], #Name "Forward").Call<TP, const TP&, int64_t, bool>(in[0], dim_, keep_dim_)};               \
  }                                                                                                              \
  void Name::SetupContext(const TensorList& in, const TensorList& out) { saved_tensors_ = {in[0], out[0]}; }     \
  TensorList Name::Backward(const TensorList& g) {                                                               \
    return {K(g[0], #Name "Backward").Call<TP, const TP&, const TP&, const TP&, int64_t, bool>(g[0], saved_tensors_[0], saved_tensors_[1], dim_, keep_dim_)}; \
  }
REDUCE_SAVED_IMPL(Max)
REDUCE_SAVED_IMPL(Min)

// ---------------------------------------------------------------------------------- transforms
TensorList Tril::Forward(const TensorList& in) { return {K(in[0], "TrilForward").Call<TP, const TP&, int64_t>(in[0], diagonal_)}; }
void Tril::SetupContext(const TensorList&, const TensorList&) {}
TensorList Tril::Backward(const TensorList& g) { return {K(g[0], "TrilBackward").Call<TP, const TP&, int64_t>(g[0], diagonal_)}; }
TensorList Triu::Forward(const TensorList& in) { return {K(in[0], "TriuForward").Call<TP, const TP&, int64_t>(in[0], diagonal_)}; }
void Triu::SetupContext(const TensorList&, const TensorList&) {}
TensorList Triu::Backward(const TensorList& g) { return {K(g[0], "TriuBackward").Call<TP, const TP&, int64_t>(g[0], diagonal_)}; }
TensorList Transpose::Forward(const TensorList& in) {
  return {K(in[0], "TransposeForward").Call<TP, const TP&, int64_t, int64_t>(in[0], dim0_, dim1_)};
}
void Transpose::SetupContext(const TensorList&, const TensorList&) {}
TensorList Transpose::Backward(const TensorList& g) {
  return {K(g[0], "TransposeBackward").Call<TP, const TP&, int64_t, int64_t>(g[0], dim0_, dim1_)};
}
TensorList Mask::Forward(const TensorList& in) {
  return {K(in[0], "MaskForward").Call<TP, const TP&, const TP&, float>(in[0], mask_, value_)};
}
void Mask::SetupContext(const TensorList&, const TensorList&) {}
TensorList Mask::Backward(const TensorList& g) { return {K(g[0], "MaskBackward").Call<TP, const TP&, const TP&>(g[0], mask_)}; }
TensorList RepeatInterleave::Forward(const TensorList& in) {
  return {K(in[0], "RepeatInterleaveForward").Call<TP, const TP&, int64_t, int64_t>(in[0], repeat_, dim_)};
}
void RepeatInterleave::SetupContext(const TensorList& in, const TensorList&) { input_dims_ = in[0]->Dims(); }
TensorList RepeatInterleave::Backward(const TensorList& g) {
  return {K(g[0], "RepeatInterleaveBackward").Call<TP, const TP&, const Dims&, int64_t>(g[0], input_dims_, dim_)};
}

// ---------------------------------------------------------------------------------- misc
TensorList Split::Forward(const TensorList& in) {
  return K(in[0], "SplitForward").Call<TensorList, const TP&, int64_t, int>(in[0], split_size_, dim_);
}
void Split::SetupContext(const TensorList& in, const TensorList&) { input_dims_ = in[0]->Dims(); }
TensorList Split::Backward(const TensorList& g) {
  return {K(g[0], "SplitBackward").Call<TP, const Dims&, int64_t, int, const TensorList&>(input_dims_, split_size_, dim_, g)};
}
TensorList NoOp::Forward(const TensorList& in) {
  return {K(in[0], "NoOpForward").Call<TP, const TP&, const Dims&>(in[0], output_dims_)};
}
void NoOp::SetupContext(const TensorList& in, const TensorList&) { input_dims_ = in[0]->Dims(); }
TensorList NoOp::Backward(const TensorList& g) {
  return {K(g[0], "NoOpBackward").Call<TP, const Dims&, const TP&>(input_dims_, g[0])};
}
TensorList Slice::Forward(const TensorList& in) {
  return {K(in[0], "SliceForward").Call<TP, const TP&, const Dims&, const Dims&, const Dims&>(in[0], starts_, ends_, steps_)};
}
void Slice::SetupContext(const TensorList& in, const TensorList&) { input_dims_ = in[0]->Dims(); }
TensorList Slice::Backward(const TensorList& g) {
  return {K(g[0], "SliceBackward").Call<TP, const TP&, const Dims&, const Dims&, const Dims&, const Dims&>(g[0], input_dims_, starts_, ends_, steps_)};
}
TensorList Stack::Forward(const TensorList& in) {
  return {K(in[0], "StackForward").Call<TP, const TensorList&, int64_t>(in, dim_)};
}
void Stack::SetupContext(const TensorList&, const TensorList&) {}
TensorList Stack::Backward(const TensorList& g) {
  return K(g[0], "StackBackward").Call<TensorList, const Dims&, int64_t, const TP&>(Dims{}, dim_, g[0]);
}
TensorList Cast::Forward(const TensorList& in) {
  src_dtype_ = in[0]->Dtype();
  return {MakeTensor(in[0]->data().to(ToTorch(dtype_)))};
}
void Cast::SetupContext(const TensorList&, const TensorList&) {}
TensorList Cast::Backward(const TensorList& g) { return {MakeTensor(g[0]->data().to(ToTorch(src_dtype_)))}; }

}  // namespace infini_train::autograd
