#include "core/framework/tensor.h"

#include <c10/util/Exception.h>

#include <cstring>
#include <fstream>
#include <functional>
#include <sstream>

#include "core/framework/autograd.h"
#include "core/rng.h"

namespace infini_train {

// ---------------------------------------------------------------------------------- Device / DataType
Device::Device(DeviceType type, int8_t index) : type_(type), index_(index) {
  TORCH_CHECK(index >= 0, "device index must be non-negative");
  if (type == DeviceType::kCPU) TORCH_CHECK(index == 0, "CPU device index must be 0");
}
std::string Device::ToString() const {
  std::ostringstream os;
  os << "Device(" << (IsCPU() ? "CPU" : "CUDA") << ", " << static_cast<int>(index_) << ")";
  return os.str();
}
at::Device Device::ToTorch() const {
  return IsCPU() ? at::Device(at::kCPU) : at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(index_));
}

size_t DataTypeSize(DataType t) {
  static const size_t sizes[] = {1, 1, 2, 2, 4, 4, 8, 8, 2, 2, 4, 8};
  return sizes[static_cast<int>(t)];
}
const char* DataTypeName(DataType t) {
  static const char* names[] = {"uint8", "int8", "uint16", "int16", "uint32", "int32", "uint64", "int64",
                                "bfloat16", "float16", "float32", "float64"};
  return names[static_cast<int>(t)];
}
at::ScalarType ToTorch(DataType t) {
  switch (t) {
    case DataType::kUINT8: return at::kByte;
    case DataType::kINT8: return at::kChar;
    case DataType::kUINT16: return at::kUInt16;
    case DataType::kINT16: return at::kShort;
    case DataType::kUINT32: return at::kUInt32;
    case DataType::kINT32: return at::kInt;
    case DataType::kUINT64: return at::kUInt64;
    case DataType::kINT64: return at::kLong;
    case DataType::kBFLOAT16: return at::kBFloat16;
    case DataType::kFLOAT16: return at::kHalf;
    case DataType::kFLOAT32: return at::kFloat;
    case DataType::kFLOAT64: return at::kDouble;
  }
  return at::kFloat;
}
DataType FromTorch(at::ScalarType t) {
  switch (t) {
    case at::kByte: return DataType::kUINT8;
    case at::kChar: return DataType::kINT8;
    case at::kUInt16: return DataType::kUINT16;
    case at::kShort: return DataType::kINT16;
    case at::kUInt32: return DataType::kUINT32;
    case at::kInt: return DataType::kINT32;
    case at::kUInt64: return DataType::kUINT64;
    case at::kLong: return DataType::kINT64;
    case at::kBFloat16: return DataType::kBFLOAT16;
    case at::kHalf: return DataType::kFLOAT16;
    case at::kDouble: return DataType::kFLOAT64;
    default: return DataType::kFLOAT32;
  }
}

PrintOptions& PrintOptions::Get() {
  static PrintOptions opts;
  return opts;
}
void SetPrintOptions(int precision, int threshold, int edge_items, int linewidth, const std::string& profile,
                     int sci_mode) {
  PrintOptions& o = PrintOptions::Get();
  if (profile == "default") o = PrintOptions();
  else if (profile == "short") { o.precision = 2; o.edge_items = 2; o.linewidth = 80; }
  else if (profile == "full") { o.threshold = 1 << 30; }
  if (precision >= 0) o.precision = precision;
  if (threshold >= 0) o.threshold = threshold;
  if (edge_items >= 0) o.edge_items = edge_items;
  if (linewidth >= 0) o.linewidth = linewidth;
  if (sci_mode >= 0) o.sci_mode = sci_mode != 0;
}

// ---------------------------------------------------------------------------------- Tensor basics
Tensor::Tensor(const std::vector<int64_t>& dims, DataType dtype, Device device)
    : data_(at::empty(dims, at::TensorOptions().dtype(ToTorch(dtype)).device(device.ToTorch()))), dims_(dims) {}

Tensor::Tensor(const Tensor& tensor, size_t offset, const std::vector<int64_t>& dims) : dims_(dims) {
  const size_t esz = DataTypeSize(tensor.Dtype());
  TORCH_CHECK(offset % esz == 0, "view offset must be a multiple of the element size");
  int64_t n = 1;
  for (auto d : dims) n *= d;
  at::Tensor flat = tensor.data_.reshape({-1});
  data_ = flat.narrow(0, static_cast<int64_t>(offset / esz), n).view(dims);
}

Tensor::Tensor(at::Tensor t) : data_(t.contiguous()) { dims_ = data_.sizes().vec(); }

Device Tensor::GetDevice() const {
  if (data_.is_cuda()) return Device(DeviceType::kCUDA, static_cast<int8_t>(data_.device().index()));
  return Device();
}

Tensor Tensor::To(Device device) const {
  Tensor out(data_.to(device.ToTorch()));
  out.requires_grad_ = requires_grad_;
  if (requires_grad_) {
    out.grad_ = std::make_shared<Tensor>(at::zeros_like(out.data_));
  }
  return out;
}
Tensor Tensor::To(DataType dtype) const { return Tensor(data_.to(ToTorch(dtype))); }

std::vector<float> Tensor::ToFloatVector() const {
  at::Tensor c = data_.to(at::kCPU, at::kFloat).contiguous();
  return std::vector<float>(c.data_ptr<float>(), c.data_ptr<float>() + c.numel());
}

std::shared_ptr<Tensor> Tensor::Uniform(float from, float to, std::optional<std::mt19937> generator) {
  at::Tensor h = at::empty(dims_, at::kFloat);
  float* p = h.data_ptr<float>();
  const int64_t n = h.numel();
  if (generator.has_value()) {
    std::mt19937 g = *generator;                       // a copy: the caller's generator does not advance
    std::uniform_real_distribution<float> dist(from, to);
    for (int64_t i = 0; i < n; ++i) p[i] = dist(g);
  } else {
    titb::rng::fill_uniform(p, n, from, to, std::nullopt);
  }
  data_.copy_(h);
  return shared_from_this();
}
void Tensor::SetPrintOptions(std::optional<int64_t> precision, std::optional<int64_t> threshold, std::optional<int64_t> edge_items,
                             std::optional<int64_t> linewidth, std::optional<std::string> profile, std::optional<bool> sci_mode) {
  infini_train::SetPrintOptions(precision ? static_cast<int>(*precision) : -1, threshold ? static_cast<int>(*threshold) : -1,
                                edge_items ? static_cast<int>(*edge_items) : -1, linewidth ? static_cast<int>(*linewidth) : -1,
                                profile ? *profile : std::string(), sci_mode ? (*sci_mode ? 1 : 0) : -1);
}

// ---------------------------------------------------------------------------------- autograd fields
std::shared_ptr<Tensor> Tensor::RequiresGrad() {
  requires_grad_ = true;
  if (!grad_) grad_ = std::make_shared<Tensor>(at::zeros_like(data_));
  return shared_from_this();
}
void Tensor::ZeroGrad() {
  if (grad_) grad_->data().zero_();
}
void Tensor::Backward(std::shared_ptr<Tensor> gradient, bool, bool) {
  TORCH_CHECK(requires_grad_, "Backward() on a tensor that does not require grad");
  if (!gradient) gradient = std::make_shared<Tensor>(at::ones_like(data_));
  TORCH_CHECK(gradient->Dims() == dims_, "gradient shape does not match the tensor");
  if (grad_fn_) grad_fn_->BackwardPartial(gradient, output_idx_);
  else if (grad_) grad_->data().add_(gradient->data());
}

// ---------------------------------------------------------------------------------- operator sugar
namespace {
template <class F, class... A>
std::shared_ptr<Tensor> apply1(const autograd::TensorList& in, A&&... a) {
  return std::make_shared<F>(std::forward<A>(a)...)->Apply(in)[0];
}
std::shared_ptr<Tensor> scalar_like(const Tensor& t, float s) {
  return std::make_shared<Tensor>(at::full({1}, s, t.data().options()));
}
}  // namespace

std::shared_ptr<Tensor> Tensor::Equals(float s) { return apply1<autograd::EqualsScalar>({shared_from_this()}, s); }
std::shared_ptr<Tensor> Tensor::Add(const std::shared_ptr<Tensor>& o) { return apply1<autograd::Add>({shared_from_this(), o}); }
std::shared_ptr<Tensor> Tensor::Add(float s) { return apply1<autograd::AddScalar>({shared_from_this()}, s); }
std::shared_ptr<Tensor> Tensor::Sub(const std::shared_ptr<Tensor>& o) { return apply1<autograd::Sub>({shared_from_this(), o}); }
std::shared_ptr<Tensor> Tensor::Sub(float s) { return apply1<autograd::AddScalar>({shared_from_this()}, -s); }
std::shared_ptr<Tensor> Tensor::Mul(const std::shared_ptr<Tensor>& o) { return apply1<autograd::Mul>({shared_from_this(), o}); }
std::shared_ptr<Tensor> Tensor::Mul(float s) { return apply1<autograd::MulScalar>({shared_from_this()}, s); }
std::shared_ptr<Tensor> Tensor::Div(const std::shared_ptr<Tensor>& o) { return apply1<autograd::Div>({shared_from_this(), o}); }
std::shared_ptr<Tensor> Tensor::Div(float s) { return apply1<autograd::MulScalar>({shared_from_this()}, 1.0f / s); }
std::shared_ptr<Tensor> Tensor::Neg() { return apply1<autograd::Neg>({shared_from_this()}); }
std::shared_ptr<Tensor> Tensor::Reciprocal() { return apply1<autograd::Reciprocal>({shared_from_this()}); }
std::shared_ptr<Tensor> Tensor::Sin() { return apply1<autograd::Sin>({shared_from_this()}); }
std::shared_ptr<Tensor> Tensor::Cos() { return apply1<autograd::Cos>({shared_from_this()}); }
std::shared_ptr<Tensor> Tensor::Tanh() { return apply1<autograd::Tanh>({shared_from_this()}); }
std::shared_ptr<Tensor> Tensor::Pow(float e) { return apply1<autograd::Pow>({shared_from_this()}, e); }
std::shared_ptr<Tensor> Tensor::Rsqrt() { return apply1<autograd::Rsqrt>({shared_from_this()}); }
std::vector<std::shared_ptr<Tensor>> Tensor::Split(int split_size, int dim) {
  return std::make_shared<autograd::Split>(split_size, dim)->Apply({shared_from_this()});
}
std::shared_ptr<Tensor> Tensor::Transpose(int d0, int d1) {
  const int nd = static_cast<int>(dims_.size());
  return apply1<autograd::Transpose>({shared_from_this()}, (d0 + nd) % nd, (d1 + nd) % nd);
}
std::shared_ptr<Tensor> Tensor::Slice(const std::vector<int64_t>& s, const std::vector<int64_t>& e,
                                      const std::vector<int64_t>& st) {
  return apply1<autograd::Slice>({shared_from_this()}, s, e, st);
}
std::shared_ptr<Tensor> Tensor::Slice(int dim, int64_t start, int64_t end, int64_t step) {
  std::vector<int64_t> s(dims_.size(), 0), e = dims_, st(dims_.size(), 1);
  s[dim] = start; e[dim] = end; st[dim] = step;
  return Slice(s, e, st);
}
std::shared_ptr<Tensor> Tensor::RepeatInterleave(int64_t repeat, int64_t dim) {
  return apply1<autograd::RepeatInterleave>({shared_from_this()}, repeat, dim);
}
std::shared_ptr<Tensor> Tensor::View(const std::vector<int64_t>& dims) {
  std::vector<int64_t> out = dims;
  int64_t known = 1, infer = -1;
  for (size_t i = 0; i < out.size(); ++i) {
    if (out[i] == -1) infer = static_cast<int64_t>(i);
    else known *= out[i];
  }
  if (infer >= 0) out[infer] = static_cast<int64_t>(NumElements()) / known;
  return apply1<autograd::NoOp>({shared_from_this()}, out);
}
std::shared_ptr<Tensor> Tensor::Contiguous() { return apply1<autograd::NoOp>({shared_from_this()}, dims_); }
std::shared_ptr<Tensor> Tensor::Flatten(int64_t start, int64_t end) {
  const int64_t nd = static_cast<int64_t>(dims_.size());
  if (start < 0) start += nd;
  if (end < 0) end += nd;
  TORCH_CHECK(0 <= start && start <= end && end < nd, "Flatten: bad dims");
  std::vector<int64_t> out(dims_.begin(), dims_.begin() + start);
  int64_t merged = 1;
  for (int64_t i = start; i <= end; ++i) merged *= dims_[i];
  out.push_back(merged);
  out.insert(out.end(), dims_.begin() + end + 1, dims_.end());
  return Contiguous()->View(out);
}
std::shared_ptr<Tensor> Tensor::Squeeze(int64_t dim) {
  if (dim < 0) dim += static_cast<int64_t>(dims_.size());
  std::vector<int64_t> out = dims_;
  if (out[dim] == 1) out.erase(out.begin() + dim);
  return View(out);
}
std::shared_ptr<Tensor> Tensor::Matmul(const std::shared_ptr<Tensor>& o) { return apply1<autograd::Matmul>({shared_from_this(), o}); }
std::shared_ptr<Tensor> Tensor::Outer(const std::shared_ptr<Tensor>& o) { return apply1<autograd::Outer>({shared_from_this(), o}); }
std::shared_ptr<Tensor> Tensor::MaskedFill(const std::shared_ptr<Tensor>& mask, float value) {
  return apply1<autograd::Mask>({shared_from_this()}, mask, value);
}

TensorPtr operator==(const TensorPtr& t, float s) { return t->Equals(s); }
TensorPtr operator+(const TensorPtr& a, const TensorPtr& b) { return a->Add(b); }
TensorPtr operator+(const TensorPtr& a, float s) { return a->Add(s); }
TensorPtr operator+(float s, const TensorPtr& a) { return a->Add(s); }
TensorPtr operator-(const TensorPtr& a, const TensorPtr& b) { return a->Sub(b); }
TensorPtr operator-(const TensorPtr& a, float s) { return a->Sub(s); }
TensorPtr operator-(float s, const TensorPtr& a) { return a->Neg()->Add(s); }
TensorPtr operator-(const TensorPtr& a) { return a->Neg(); }
TensorPtr operator*(const TensorPtr& a, const TensorPtr& b) { return a->Mul(b); }
TensorPtr operator*(const TensorPtr& a, float s) { return a->Mul(s); }
TensorPtr operator*(float s, const TensorPtr& a) { return a->Mul(s); }
TensorPtr operator/(const TensorPtr& a, const TensorPtr& b) { return a->Div(b); }
TensorPtr operator/(const TensorPtr& a, float s) { return a->Div(s); }
TensorPtr operator/(float s, const TensorPtr& a) { return a->Reciprocal()->Mul(s); }

// ---------------------------------------------------------------------------------- debugging
void Tensor::SaveAsNpy(const std::string& path) const {
  // NumPy .npy version 1.0, little-endian float32, C order; header padded so data starts at a multiple of 16.
  at::Tensor c = data_.to(at::kCPU, at::kFloat).contiguous();
  std::ostringstream shape;
  shape << "(";
  for (size_t i = 0; i < dims_.size(); ++i) shape << dims_[i] << (dims_.size() == 1 || i + 1 < dims_.size() ? "," : "");
  shape << ")";
  std::string dict = "{'descr': '<f4', 'fortran_order': False, 'shape': " + shape.str() + ", }";
  const size_t preamble = 10;
  size_t total = preamble + dict.size() + 1;
  const size_t pad = (16 - total % 16) % 16;
  dict.append(pad, ' ');
  dict.push_back('\n');
  std::ofstream out(path, std::ios::binary);
  TORCH_CHECK(out.good(), "cannot write ", path);
  const char magic[] = {'\x93', 'N', 'U', 'M', 'P', 'Y', 1, 0};
  out.write(magic, 8);
  const uint16_t hlen = static_cast<uint16_t>(dict.size());
  out.write(reinterpret_cast<const char*>(&hlen), 2);
  out.write(dict.data(), dict.size());
  out.write(reinterpret_cast<const char*>(c.data_ptr<float>()), sizeof(float) * c.numel());
}

void Tensor::Print(std::ostream& os) const {
  const PrintOptions& o = PrintOptions::Get();
  at::Tensor c = data_.to(at::kCPU, at::kDouble).contiguous();
  const double* p = c.data_ptr<double>();
  const bool summarize = static_cast<int64_t>(c.numel()) > o.threshold;
  std::ostringstream fmt;
  fmt.precision(o.precision);
  fmt << (o.sci_mode ? std::scientific : std::fixed);
  std::function<void(size_t, int64_t, int)> rec = [&](size_t dim, int64_t off, int indent) {
    if (dim == dims_.size()) { fmt << p[off]; return; }
    int64_t stride = 1;
    for (size_t d = dim + 1; d < dims_.size(); ++d) stride *= dims_[d];
    fmt << "[";
    const int64_t n = dims_[dim];
    for (int64_t i = 0; i < n; ++i) {
      if (summarize && n > 2 * o.edge_items && i == o.edge_items) {
        fmt << "..., ";
        if (dim + 1 < dims_.size()) fmt << "\n" << std::string(indent + 1, ' ');
        i = n - o.edge_items - 1;
        continue;
      }
      rec(dim + 1, off + i * stride, indent + 1);
      if (i + 1 < n) {
        fmt << ",";
        if (dim + 1 < dims_.size()) fmt << "\n" << std::string(indent + 1, ' ');
        else fmt << " ";
      }
    }
    fmt << "]";
  };
  fmt << "tensor(";
  rec(0, 0, 7);
  fmt << ", dtype=" << DataTypeName(Dtype());
  if (data_.is_cuda()) fmt << ", device='cuda:" << static_cast<int>(data_.device().index()) << "'";
  if (requires_grad_) fmt << ", requires_grad=True";
  fmt << ")";
  os << fmt.str() << std::endl;
}

}  // namespace infini_train
