// Autograd engine and the op Functions of the C++ facade.
//
// Reference: infini_train/include/autograd/function.h:10-39, src/autograd/function.cc:24-91 and
// the 32 op classes under include/autograd/.  Same contract: Apply() runs Forward, then
// SetupContext, wires next_functions_ (a private AccumulateGrad node per leaf that requires
// grad), and BackwardPartial() fires Backward once every output slot has a gradient and every
// consumer has reported, frees the saved tensors and walks on depth first.
#pragma once
#include <memory>
#include <utility>
#include <vector>

#include "core/framework/tensor.h"

namespace infini_train::autograd {

using TensorList = std::vector<std::shared_ptr<Tensor>>;

class Function : public std::enable_shared_from_this<Function> {
 public:
  virtual ~Function() = default;
  virtual TensorList Forward(const TensorList& input_tensors) = 0;
  virtual void SetupContext(const TensorList& input_tensors, const TensorList& output_tensors) {}
  virtual TensorList Backward(const TensorList& grad_outputs) = 0;

  TensorList Apply(const TensorList& input_tensors);
  virtual void BackwardPartial(const std::shared_ptr<Tensor>& grad_output, int idx);
  void IncreaseDependenciesNumber() { ++dependencies_number_; }

 protected:
  TensorList saved_tensors_;

 private:
  std::vector<std::pair<std::shared_ptr<Function>, int>> next_functions_;
  int dependencies_number_ = 0;
  int dependencies_reached_ = 0;
  int grad_outputs_reached_ = 0;
  TensorList grad_outputs_;
};

class AccumulateGrad final : public Function {
 public:
  explicit AccumulateGrad(std::shared_ptr<Tensor> grad, float learning_rate = 1.0f)
      : grad_(std::move(grad)), learning_rate_(learning_rate) {}
  TensorList Forward(const TensorList&) override;
  TensorList Backward(const TensorList&) override;
  void BackwardPartial(const std::shared_ptr<Tensor>& grad_output, int idx) override;

 private:
  std::shared_ptr<Tensor> grad_;
  float learning_rate_;
};

#define TITB_DECLARE_FUNCTION_BODY                                                        \
  TensorList Forward(const TensorList& input_tensors) override;                           \
  void SetupContext(const TensorList& input_tensors, const TensorList& outputs) override; \
  TensorList Backward(const TensorList& grad_outputs) override;

// ---- unary elementwise ---------------------------------------------------------------------------
#define TITB_DECLARE_UNARY(Name) \
  class Name : public Function { \
   public:                       \
    TITB_DECLARE_FUNCTION_BODY   \
  };
TITB_DECLARE_UNARY(Neg)
TITB_DECLARE_UNARY(Reciprocal)
TITB_DECLARE_UNARY(Sin)
TITB_DECLARE_UNARY(Cos)
TITB_DECLARE_UNARY(Tanh)
TITB_DECLARE_UNARY(Rsqrt)
TITB_DECLARE_UNARY(Sigmoid)
// tanh-form GELU in one kernel (not in the reference, whose NewGELU module composes eight element-wise ops:
// example/gpt2/net.cc:46-51); saves the input
TITB_DECLARE_UNARY(Gelu)

class Pow : public Function {
 public:
  explicit Pow(float exponent, bool scalar_is_base = false) : exponent_(exponent), scalar_is_base_(scalar_is_base) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  float exponent_;
  bool scalar_is_base_;
};
class EqualsScalar : public Function {
 public:
  explicit EqualsScalar(float scalar) : scalar_(scalar) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  float scalar_;
};
class AddScalar : public Function {
 public:
  explicit AddScalar(float scalar) : scalar_(scalar) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  float scalar_;
};
class MulScalar : public Function {
 public:
  explicit MulScalar(float scalar) : scalar_(scalar) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  float scalar_;
};

// ---- binary elementwise (b is broadcast to a, right aligned) -----------------------------------------
#define TITB_DECLARE_BINARY(Name)  \
  class Name : public Function {   \
   public:                         \
    TITB_DECLARE_FUNCTION_BODY     \
   private:                        \
    std::vector<int64_t> a_dims_, b_dims_; \
  };
TITB_DECLARE_BINARY(Add)
TITB_DECLARE_BINARY(Sub)
TITB_DECLARE_BINARY(Mul)
TITB_DECLARE_BINARY(Div)

// ---- matmul / linear / outer ----------------------------------------------------------------------------
class Matmul : public Function {
 public:
  TITB_DECLARE_FUNCTION_BODY
};
class Linear : public Function {
 public:
  TITB_DECLARE_FUNCTION_BODY
 private:
  bool bias_ = true;
  int64_t out_features_ = 0;
};
class Outer : public Function {
 public:
  TITB_DECLARE_FUNCTION_BODY
};

// ---- normalisation, softmax, loss, embedding ---------------------------------------------------------------
class LayerNorm : public Function {
 public:
  explicit LayerNorm(float eps = 1e-5f) : eps_(eps) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  float eps_;
  std::shared_ptr<Tensor> mean_, rstd_;
};
class RMSNorm : public Function {  // not in the reference
 public:
  explicit RMSNorm(float eps = 1e-5f) : eps_(eps) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  float eps_;
  std::shared_ptr<Tensor> rstd_;
};
// Rotary position embedding on [B, T, H, hd]: element i is paired with i + hd/2, angle (t + pos_offset) * theta^(-2i/hd)
// (not in the reference)
class Rope : public Function {
 public:
  explicit Rope(float theta = 500000.f, int64_t pos_offset = 0) : theta_(theta), pos_offset_(pos_offset) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  float theta_;
  int64_t pos_offset_;
};
// silu(x[..., :F]) * x[..., F:] on a fused gate | up projection of width 2F (not in the reference); saves the input
class SwiGLU : public Function {
 public:
  TITB_DECLARE_FUNCTION_BODY
};
// Causal self-attention in one Function: inputs q [B, T, Hq, hd], k and v [B, T, Hkv, hd] (Hq % Hkv == 0), output
// [B, T, Hq, hd].  bf16 CUDA tensors with hd 64 or 128 run the tcgen05 flash-attention kernels (the score matrix is
// never materialised); everything else runs the same math through ATen.  The reference composes attention from
// Matmul / MaskedFill / Softmax (example/gpt2/net.cc:91-108), which the facade models still do for fp32.
class CausalAttention : public Function {
 public:
  explicit CausalAttention(float scale = 0.f) : scale_(scale) {}      // 0 = 1 / sqrt(hd)
  TITB_DECLARE_FUNCTION_BODY
 private:
  float scale_;
  std::shared_ptr<Tensor> out_, lse_;
};
class Softmax : public Function {
 public:
  explicit Softmax(int64_t dim = -1) : dim_(dim) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  int64_t dim_;
};
class CrossEntropy : public Function {
 public:
  TITB_DECLARE_FUNCTION_BODY
};
class Embedding : public Function {
 public:
  TITB_DECLARE_FUNCTION_BODY
 private:
  std::vector<int64_t> weight_dims_;
};

// ---- reductions ------------------------------------------------------------------------------------------------
#define TITB_DECLARE_REDUCTION(Name)                                                          \
  class Name : public Function {                                                              \
   public:                                                                                    \
    explicit Name(int64_t dim, bool keep_dim = false) : dim_(dim), keep_dim_(keep_dim) {}     \
    TITB_DECLARE_FUNCTION_BODY                                                                \
   private:                                                                                   \
    int64_t dim_;                                                                             \
    bool keep_dim_;                                                                           \
    std::vector<int64_t> input_dims_;                                                         \
  };
TITB_DECLARE_REDUCTION(Mean)
TITB_DECLARE_REDUCTION(Sum)
TITB_DECLARE_REDUCTION(Max)
TITB_DECLARE_REDUCTION(Min)

// ---- transforms ---------------------------------------------------------------------------------------------------
class Tril : public Function {
 public:
  explicit Tril(int64_t diagonal = 0) : diagonal_(diagonal) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  int64_t diagonal_;
};
class Triu : public Function {
 public:
  explicit Triu(int64_t diagonal = 0) : diagonal_(diagonal) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  int64_t diagonal_;
};
class Transpose : public Function {
 public:
  Transpose(int64_t dim0, int64_t dim1) : dim0_(dim0), dim1_(dim1) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  int64_t dim0_, dim1_;
};
class Mask : public Function {
 public:
  Mask(std::shared_ptr<Tensor> mask, float value) : mask_(std::move(mask)), value_(value) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  std::shared_ptr<Tensor> mask_;
  float value_;
};
class RepeatInterleave : public Function {
 public:
  RepeatInterleave(int64_t repeat, int64_t dim) : repeat_(repeat), dim_(dim) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  int64_t repeat_, dim_;
  std::vector<int64_t> input_dims_;
};

// ---- misc -------------------------------------------------------------------------------------------------------------
class Split : public Function {
 public:
  Split(int64_t split_size, int dim = 0) : split_size_(split_size), dim_(dim) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  int64_t split_size_;
  int dim_;
  std::vector<int64_t> input_dims_;
};
class NoOp : public Function {  // View / Contiguous / Flatten / Squeeze
 public:
  explicit NoOp(std::vector<int64_t> output_dims) : output_dims_(std::move(output_dims)) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  std::vector<int64_t> output_dims_, input_dims_;
};
class Slice : public Function {
 public:
  Slice(std::vector<int64_t> starts, std::vector<int64_t> ends, std::vector<int64_t> steps)
      : starts_(std::move(starts)), ends_(std::move(ends)), steps_(std::move(steps)) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  std::vector<int64_t> starts_, ends_, steps_, input_dims_;
};
class Stack : public Function {
 public:
  explicit Stack(int64_t dim) : dim_(dim) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  int64_t dim_;
};
class Cast : public Function {  // dtype conversion, not in the reference
 public:
  explicit Cast(DataType dtype) : dtype_(dtype) {}
  TITB_DECLARE_FUNCTION_BODY
 private:
  DataType dtype_, src_dtype_ = DataType::kFLOAT32;
};

}  // namespace infini_train::autograd
