// C++ framework facade: Device, DataType and Tensor with the reference's method names.
//
// Reference: infini_train/include/device.h:8-36, tensor.h:20-198, src/tensor.cc.  Storage and
// math are delegated to libtorch (at::Tensor); on CUDA the float32/bfloat16 ops go through the
// sm_100a kernel library.  The autograd engine is the framework's own (autograd/function.h),
// with the reference's dependency-counting semantics, so user-defined Function subclasses work
// the same way.  Deliberate differences from the reference:
//  * any CUDA device index 0..N-1 is valid (the reference aborts on index != 0, device.cc:11-17);
//  * views keep their byte offset (the reference's NoOp view rewinds to offset 0, no_op.cc:14);
//  * Fill writes the value in the tensor's own dtype (the reference reinterprets it as float).
#pragma once
#include <ATen/ATen.h>

#include <cstdint>
#include <iostream>
#include <memory>
#include <optional>
#include <random>
#include <string>
#include <vector>

namespace infini_train {

enum class DeviceType : int8_t { kCPU = 0, kCUDA = 1, kCount = 2 };

class Device {
 public:
  Device() : type_(DeviceType::kCPU), index_(0) {}
  Device(DeviceType type, int8_t index);
  DeviceType Type() const { return type_; }
  int8_t Index() const { return index_; }
  bool IsCPU() const { return type_ == DeviceType::kCPU; }
  bool IsCUDA() const { return type_ == DeviceType::kCUDA; }
  std::string ToString() const;
  at::Device ToTorch() const;
  bool operator==(const Device& o) const { return type_ == o.type_ && index_ == o.index_; }
  friend std::ostream& operator<<(std::ostream& os, const Device& d) { return os << d.ToString(); }

 private:
  DeviceType type_;
  int8_t index_;
};

enum class DataType : int8_t {
  kUINT8, kINT8, kUINT16, kINT16, kUINT32, kINT32, kUINT64, kINT64, kBFLOAT16, kFLOAT16, kFLOAT32, kFLOAT64,
};
size_t DataTypeSize(DataType t);
const char* DataTypeName(DataType t);
at::ScalarType ToTorch(DataType t);
DataType FromTorch(at::ScalarType t);

struct PrintOptions {
  int precision = 4;
  int threshold = 1000;
  int edge_items = 3;
  int linewidth = 80;
  bool sci_mode = false;
  static PrintOptions& Get();
};
void SetPrintOptions(int precision = -1, int threshold = -1, int edge_items = -1, int linewidth = -1,
                     const std::string& profile = "", int sci_mode = -1);

namespace autograd { class Function; }

class Tensor : public std::enable_shared_from_this<Tensor> {
 public:
  Tensor() = default;
  Tensor(const std::vector<int64_t>& dims, DataType dtype, Device device = Device());
  // View of `tensor` starting `offset` bytes into its buffer.
  Tensor(const Tensor& tensor, size_t offset, const std::vector<int64_t>& dims);
  explicit Tensor(at::Tensor t);

  // ---- data -----------------------------------------------------------------------------------
  const std::vector<int64_t>& Dims() const { return dims_; }
  size_t NumElements() const { return static_cast<size_t>(data_.numel()); }
  DataType Dtype() const { return FromTorch(data_.scalar_type()); }
  Device GetDevice() const;
  void* DataPtr() { return data_.data_ptr(); }
  const void* DataPtr() const { return data_.data_ptr(); }
  size_t SizeInBytes() const { return NumElements() * DataTypeSize(Dtype()); }
  at::Tensor& data() { return data_; }
  const at::Tensor& data() const { return data_; }
  template <typename T> void Fill(T value) { data_.fill_(value); }
  Tensor To(Device device) const;      // same device: aliasing view (reference tensor.cc:177-183)
  Tensor To(DataType dtype) const;     // dtype cast (not in the reference)
  std::vector<float> ToFloatVector() const;

  // ---- operator sugar (each call records an autograd::Function) ------------------------------------
  std::shared_ptr<Tensor> Equals(float scalar);
  std::shared_ptr<Tensor> Add(const std::shared_ptr<Tensor>& other);
  std::shared_ptr<Tensor> Add(float scalar);
  std::shared_ptr<Tensor> Sub(const std::shared_ptr<Tensor>& other);
  std::shared_ptr<Tensor> Sub(float scalar);
  std::shared_ptr<Tensor> Mul(const std::shared_ptr<Tensor>& other);
  std::shared_ptr<Tensor> Mul(float scalar);
  std::shared_ptr<Tensor> Div(const std::shared_ptr<Tensor>& other);
  std::shared_ptr<Tensor> Div(float scalar);
  std::shared_ptr<Tensor> Neg();
  std::shared_ptr<Tensor> Reciprocal();
  std::shared_ptr<Tensor> Sin();
  std::shared_ptr<Tensor> Cos();
  std::shared_ptr<Tensor> Tanh();
  std::shared_ptr<Tensor> Pow(float exponent);
  std::shared_ptr<Tensor> Rsqrt();
  std::vector<std::shared_ptr<Tensor>> Split(int split_size, int dim = 0);
  std::shared_ptr<Tensor> Transpose(int dim0, int dim1);
  std::shared_ptr<Tensor> Slice(const std::vector<int64_t>& starts, const std::vector<int64_t>& ends,
                                const std::vector<int64_t>& steps);
  std::shared_ptr<Tensor> Slice(int dim, int64_t start, int64_t end, int64_t step = 1);
  std::shared_ptr<Tensor> RepeatInterleave(int64_t repeat, int64_t dim);
  std::shared_ptr<Tensor> View(const std::vector<int64_t>& dims);
  std::shared_ptr<Tensor> Contiguous();
  std::shared_ptr<Tensor> Flatten(int64_t start = 0, int64_t end = -1);
  std::shared_ptr<Tensor> Squeeze(int64_t dim);
  std::shared_ptr<Tensor> Matmul(const std::shared_ptr<Tensor>& other);
  std::shared_ptr<Tensor> Outer(const std::shared_ptr<Tensor>& other);
  std::shared_ptr<Tensor> MaskedFill(const std::shared_ptr<Tensor>& mask, float value);
  // Fills the tensor with U[from, to) drawn on the host (libstdc++ uniform_real_distribution over std::mt19937) and
  // returns it; `generator` is copied, as in the reference (infini_train/include/tensor.h:124), so the same seeded
  // generator gives the same values on every call.  Without one a process-wide generator advances.
  std::shared_ptr<Tensor> Uniform(float from = 0.f, float to = 1.f, std::optional<std::mt19937> generator = std::nullopt);
  // Same options as torch.set_printoptions; unset arguments keep their value (reference tensor.h:151-153).
  static void SetPrintOptions(std::optional<int64_t> precision = std::nullopt, std::optional<int64_t> threshold = std::nullopt,
                              std::optional<int64_t> edge_items = std::nullopt, std::optional<int64_t> linewidth = std::nullopt,
                              std::optional<std::string> profile = std::nullopt, std::optional<bool> sci_mode = std::nullopt);

  // ---- autograd ---------------------------------------------------------------------------------
  std::shared_ptr<Tensor> RequiresGrad();
  std::shared_ptr<Tensor> grad() const { return grad_; }
  bool requires_grad() const { return requires_grad_; }
  void set_requires_grad(bool v) { requires_grad_ = v; }
  bool is_leaf() const { return is_leaf_; }
  void set_is_leaf(bool v) { is_leaf_ = v; }
  std::shared_ptr<autograd::Function> grad_fn() const { return grad_fn_; }
  void set_grad_fn(std::shared_ptr<autograd::Function> f) { grad_fn_ = std::move(f); }
  int output_idx() const { return output_idx_; }
  void set_output_idx(int i) { output_idx_ = i; }
  void ZeroGrad();
  void Backward(std::shared_ptr<Tensor> gradient = nullptr, bool retain_graph = false, bool create_graph = false);

  // ---- debugging -----------------------------------------------------------------------------------
  void SaveAsNpy(const std::string& path) const;
  void Print(std::ostream& os = std::cout) const;
  friend std::ostream& operator<<(std::ostream& os, const Tensor& t) { t.Print(os); return os; }

 private:
  at::Tensor data_;
  std::vector<int64_t> dims_;
  bool requires_grad_ = false;
  bool is_leaf_ = true;
  std::shared_ptr<Tensor> grad_;
  std::shared_ptr<autograd::Function> grad_fn_;
  int output_idx_ = -1;
};

using TensorPtr = std::shared_ptr<Tensor>;
inline TensorPtr MakeTensor(at::Tensor t) { return std::make_shared<Tensor>(std::move(t)); }

TensorPtr operator==(const TensorPtr& t, float s);
TensorPtr operator+(const TensorPtr& a, const TensorPtr& b);
TensorPtr operator+(const TensorPtr& a, float s);
TensorPtr operator+(float s, const TensorPtr& a);
TensorPtr operator-(const TensorPtr& a, const TensorPtr& b);
TensorPtr operator-(const TensorPtr& a, float s);
TensorPtr operator-(float s, const TensorPtr& a);
TensorPtr operator-(const TensorPtr& a);
TensorPtr operator*(const TensorPtr& a, const TensorPtr& b);
TensorPtr operator*(const TensorPtr& a, float s);
TensorPtr operator*(float s, const TensorPtr& a);
TensorPtr operator/(const TensorPtr& a, const TensorPtr& b);
TensorPtr operator/(const TensorPtr& a, float s);
TensorPtr operator/(float s, const TensorPtr& a);

}  // namespace infini_train
