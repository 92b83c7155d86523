// Kernel functions behind the facade's Dispatcher, registered under the reference's names
// ("LinearForward", "AdamAccumulateGrad", ...) for both device types.
//
// CPU tensors: ATen fp32 math restating infini_train/src/kernels/cpu/*.cc (the numerical oracle).
// CUDA float32/bfloat16 tensors: the sm_100a kernel library (tcgen05 GEMM for bf16 Linear/Matmul,
// the SIMT SGEMM for fp32, fused LayerNorm / softmax / cross-entropy / embedding / Adam kernels);
// reductions, outer product, mask, tril/triu and every materialised view (transpose, slice, split, stack,
// repeat-interleave) go through the library's reduce / gather / scatter kernels as well.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cmath>
#include <tuple>

#include "core/framework/dispatcher.h"
#include "kernels/api.h"

namespace infini_train::kernels {

using TP = std::shared_ptr<Tensor>;
static bool native(const at::Tensor& t) {
  return t.is_cuda() && (t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16);
}
static int dt(const at::Tensor& t) { return t.scalar_type() == at::kBFloat16 ? 1 : 0; }
static cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static void ok(int rc, const char* what) { TORCH_CHECK(rc == 0, "kernel ", what, " failed with code ", rc); }

// Contiguous copy of a (possibly strided, possibly stride-0 expanded) view.  CUDA views of up to six dimensions
// are materialised by the library's gather kernel; everything else by ATen.
static at::Tensor materialize(const at::Tensor& t) {
  if (t.is_contiguous()) return t;
  const int64_t es = t.element_size();
  if (!t.is_cuda() || t.dim() > 6 || !(es == 2 || es == 4 || es == 8) || t.numel() == 0) return t.contiguous();
  c10::cuda::CUDAGuard guard(t.device());
  at::Tensor out = at::empty(t.sizes(), t.options());
  std::vector<long long> sz(t.sizes().begin(), t.sizes().end()), st(t.strides().begin(), t.strides().end());
  ok(titb_gather_nd(t.storage().data(), out.data_ptr(), (int)sz.size(), sz.data(), st.data(), t.storage_offset(), (int)es,
                    stream()), "gather_nd");
  return out;
}
// Writes the contiguous `src` into `view`, a view of the contiguous tensor `dst` (same dtype, <= 6 dimensions).
static void scatter_into(at::Tensor& dst, const at::Tensor& view, const at::Tensor& src_) {
  if (!native(dst) || view.dim() > 6 || src_.scalar_type() != dst.scalar_type()) {
    const_cast<at::Tensor&>(view).copy_(src_);
    return;
  }
  c10::cuda::CUDAGuard guard(dst.device());
  at::Tensor src = materialize(src_);
  std::vector<long long> sz(view.sizes().begin(), view.sizes().end()), st(view.strides().begin(), view.strides().end());
  ok(titb_scatter_nd(src.data_ptr(), dst.data_ptr(), (int)sz.size(), sz.data(), st.data(),
                     view.storage_offset() - dst.storage_offset(), dt(dst), 0, stream()), "scatter_nd");
}
static TP W(at::Tensor t) { return std::make_shared<Tensor>(materialize(t)); }
// [outer, n, inner] factorisation of a reduction over `dim`.
struct Axis3 { int64_t outer = 1, n = 1, inner = 1; };
static Axis3 axis3(c10::IntArrayRef dims, int64_t dim) {
  Axis3 a;
  for (int64_t d = 0; d < dim; ++d) a.outer *= dims[d];
  a.n = dims[dim];
  for (int64_t d = dim + 1; d < (int64_t)dims.size(); ++d) a.inner *= dims[d];
  return a;
}

// ---- accumulate / optimizers ------------------------------------------------------------------------
void AccumulateGrad(const TP& gradient, float rate, const TP& tensor) {
  at::Tensor& t = tensor->data();
  const at::Tensor& g = gradient->data();
  if (t.is_cuda() && t.scalar_type() == at::kFloat && native(g) && t.is_contiguous() && g.is_contiguous()) {
    c10::cuda::CUDAGuard guard(t.device());
    ok(titb_axpy(t.data_ptr<float>(), g.data_ptr(), rate, t.numel(), dt(g), stream()), "AccumulateGrad");
    return;
  }
  t.add_(g.to(t.scalar_type()), rate);
}

void AdamAccumulateGrad(const TP& grad, const TP& param, const TP& m, const TP& v, float learning_rate, float beta1,
                        float beta2, float eps, int64_t t) {
  at::Tensor& p = param->data();
  const at::Tensor& g = grad->data();
  const double bc1 = 1.0 - std::pow(beta1, static_cast<double>(t)), bc2 = 1.0 - std::pow(beta2, static_cast<double>(t));
  if (p.is_cuda() && p.scalar_type() == at::kFloat && g.scalar_type() == at::kFloat && p.is_contiguous()) {
    c10::cuda::CUDAGuard guard(p.device());
    ok(titb_adam_flat(p.data_ptr<float>(), nullptr, g.data_ptr<float>(), m->data().data_ptr<float>(),
                      v->data().data_ptr<float>(), p.numel(), learning_rate, beta1, beta2, eps, 0.f, (float)bc1,
                      (float)bc2, 1.f, 0, nullptr, stream()), "AdamAccumulateGrad");
    return;
  }
  at::Tensor gf = g.to(at::kFloat);
  m->data().mul_(beta1).add_(gf, 1.0 - beta1);
  v->data().mul_(beta2).addcmul_(gf, gf, 1.0 - beta2);
  at::Tensor mh = m->data() / bc1, vh = v->data() / bc2;
  p.sub_((mh / (vh.sqrt() + eps)).mul_(learning_rate).to(p.scalar_type()));
}

void Fill(const TP& tensor, void* value_ptr) {
  at::Tensor& t = tensor->data();
  const float v = *static_cast<float*>(value_ptr);
  if (native(t) && t.is_contiguous()) {
    c10::cuda::CUDAGuard guard(t.device());
    ok(titb_fill(t.data_ptr(), t.numel(), v, dt(t), stream()), "Fill");
    return;
  }
  t.fill_(v);
}

// ---- unary elementwise ------------------------------------------------------------------------------------
static TP unary(int op, const TP& x, float s, at::Tensor (*ref)(const at::Tensor&, float)) {
  const at::Tensor& a = x->data();
  if (native(a) && a.is_contiguous()) {
    c10::cuda::CUDAGuard guard(a.device());
    at::Tensor y = at::empty_like(a);
    ok(titb_unary_fwd(op, a.data_ptr(), y.data_ptr(), a.numel(), s, dt(a), stream()), "unary");
    return W(y);
  }
  return W(ref(a, s));
}
static TP unary_bwd(int op, const TP& dy, const TP& saved, float s, at::Tensor (*ref)(const at::Tensor&, const at::Tensor&, float)) {
  const at::Tensor& g = dy->data();
  const at::Tensor& sv = saved ? saved->data() : g;
  if (native(g) && g.is_contiguous() && sv.is_contiguous() && sv.scalar_type() == g.scalar_type()) {
    c10::cuda::CUDAGuard guard(g.device());
    at::Tensor dx = at::empty_like(g);
    ok(titb_unary_bwd(op, g.data_ptr(), sv.data_ptr(), dx.data_ptr(), g.numel(), s, dt(g), stream()), "unary_bwd");
    return W(dx);
  }
  return W(ref(g, sv, s));
}
#define UNARY_KERNEL(Name, OP, FWD, BWD)                                                                          \
  TP Name##Forward(const TP& x) { return unary(OP, x, 0.f, [](const at::Tensor& a, float) -> at::Tensor { return FWD; }); } \
  TP Name##Backward(const TP& dy, const TP& saved) {                                                              \
    return unary_bwd(OP, dy, saved, 0.f, [](const at::Tensor& g, const at::Tensor& a, float) -> at::Tensor { return BWD; }); \
  }
UNARY_KERNEL(Neg, TITB_NEG, -a, -g + 0 * a)
UNARY_KERNEL(Reciprocal, TITB_RECIPROCAL, a.reciprocal(), -g / (a * a))
UNARY_KERNEL(Sin, TITB_SIN, a.sin(), g * a.cos())
UNARY_KERNEL(Cos, TITB_COS, a.cos(), -g * a.sin())
UNARY_KERNEL(Tanh, TITB_TANH, a.tanh(), g * (1 - a * a))          // saved = output
UNARY_KERNEL(Rsqrt, TITB_RSQRT, a.rsqrt(), g * (-0.5 / (a * a.sqrt())))
UNARY_KERNEL(Sigmoid, TITB_SIGMOID, a.sigmoid(), g * a * (1 - a))  // saved = output

// GELU, tanh form: 0.5 x (1 + tanh(k (x + 0.044715 x^3))), k = sqrt(2 / pi); saved = input
static at::Tensor gelu_inner(const at::Tensor& x) { return (x + x.pow(3) * 0.044715) * 0.7978845608028654; }
TP GeluForward(const TP& x) {
  const at::Tensor& a = x->data();
  if (native(a) && a.is_contiguous()) {
    c10::cuda::CUDAGuard guard(a.device());
    at::Tensor y = at::empty_like(a);
    ok(titb_gelu_fwd(a.data_ptr(), y.data_ptr(), a.numel(), dt(a), stream()), "Gelu");
    return W(y);
  }
  return W(a * 0.5 * (gelu_inner(a).tanh() + 1));
}
TP GeluBackward(const TP& dy, const TP& saved) {
  const at::Tensor &g = dy->data(), &a = saved->data();
  if (native(g) && g.is_contiguous() && a.is_contiguous() && a.scalar_type() == g.scalar_type()) {
    c10::cuda::CUDAGuard guard(g.device());
    at::Tensor dx = at::empty_like(g);
    ok(titb_gelu_bwd(g.data_ptr(), a.data_ptr(), dx.data_ptr(), g.numel(), dt(g), stream()), "GeluBackward");
    return W(dx);
  }
  at::Tensor t = gelu_inner(a).tanh();
  at::Tensor dinner = (a.pow(2) * (3 * 0.044715) + 1) * 0.7978845608028654;
  return W(g * (0.5 * (t + 1) + 0.5 * a * (1 - t * t) * dinner));
}

TP PowForward(const TP& x, float e, bool scalar_is_base) {
  return unary(scalar_is_base ? TITB_POW_SCALAR_BASE : TITB_POW_SCALAR_EXP, x, e,
               scalar_is_base ? +[](const at::Tensor& a, float s) -> at::Tensor { return at::pow(s, a); }
                              : +[](const at::Tensor& a, float s) -> at::Tensor { return a.pow(s); });
}
TP PowBackward(const TP& dy, const TP& x, float e, bool scalar_is_base) {
  return unary_bwd(scalar_is_base ? TITB_POW_SCALAR_BASE : TITB_POW_SCALAR_EXP, dy, x, e,
                   scalar_is_base
                       ? +[](const at::Tensor& g, const at::Tensor& a, float s) -> at::Tensor { return g * std::log(s) * at::pow(s, a); }
                       : +[](const at::Tensor& g, const at::Tensor& a, float s) -> at::Tensor { return g * s * a.pow(s - 1); });
}
TP EqualsScalarForward(const TP& x, float s) {
  return unary(TITB_EQUALS_SCALAR, x, s, [](const at::Tensor& a, float v) -> at::Tensor { return (a == v).to(a.scalar_type()); });
}
TP AddScalarForward(const TP& x, float s) {
  return unary(TITB_ADD_SCALAR, x, s, [](const at::Tensor& a, float v) -> at::Tensor { return a + v; });
}
TP AddScalarBackward(const TP& dy) { return W(dy->data().clone()); }
TP MulScalarForward(const TP& x, float s) {
  return unary(TITB_MUL_SCALAR, x, s, [](const at::Tensor& a, float v) -> at::Tensor { return a * v; });
}
TP MulScalarBackward(const TP& dy, float s) {
  return unary(TITB_MUL_SCALAR, dy, s, [](const at::Tensor& a, float v) -> at::Tensor { return a * v; });
}

// ---- binary elementwise: result has a's shape, b broadcast right-aligned --------------------------------------------
static at::Tensor reduce_to(at::Tensor g, const std::vector<int64_t>& dims) {
  while (g.dim() > static_cast<int64_t>(dims.size())) g = g.sum(0);
  for (size_t d = 0; d < dims.size(); ++d)
    if (dims[d] == 1 && g.size(d) != 1) g = g.sum(static_cast<int64_t>(d), true);
  return g.contiguous();
}
// b right-aligned against a and broadcast one way (b -> a), as in the reference's elementwise.cu:23-48
static bool broadcast_desc(const at::Tensor& a, const at::Tensor& b, TitbBroadcast* bc) {
  if (a.dim() > 8 || b.dim() > a.dim()) return false;
  bc->ndim = (int)a.dim();
  const int64_t off = a.dim() - b.dim();
  int64_t bstride = 1;
  for (int64_t d = a.dim() - 1; d >= 0; --d) {
    bc->a_dims[d] = a.size(d);
    bc->b_strides[d] = 0;
    if (d >= off) {
      const int64_t bd = b.size(d - off);
      if (bd != a.size(d) && bd != 1) return false;
      bc->b_strides[d] = (bd == 1) ? 0 : bstride;
      bstride *= bd;
    }
  }
  return true;
}
static TP binary(int op, const TP& a, const TP& b) {
  const at::Tensor &x = a->data(), &y = b->data();
  TORCH_CHECK(x.numel() % std::max<int64_t>(1, y.numel()) == 0, "binary op: b does not broadcast to a");
  TitbBroadcast bc{};
  if (native(x) && native(y) && x.scalar_type() == y.scalar_type() && x.numel() > 0 && broadcast_desc(x, y, &bc)) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = materialize(x), yc = materialize(y), out = at::empty_like(xc);
    ok(titb_binary_fwd(op, xc.data_ptr(), yc.data_ptr(), out.data_ptr(), xc.numel(), bc, dt(xc), stream()), "binary");
    return W(out);
  }
  switch (op) {
    case 0: return W(x + y);
    case 1: return W(x - y);
    case 2: return W(x * y);
    default: return W(x / y);
  }
}
TP AddForward(const TP& a, const TP& b) { return binary(0, a, b); }
TP SubForward(const TP& a, const TP& b) { return binary(1, a, b); }
TP MulForward(const TP& a, const TP& b) { return binary(2, a, b); }
TP DivForward(const TP& a, const TP& b) { return binary(3, a, b); }
std::pair<TP, TP> AddBackward(const TP& dy, const std::vector<int64_t>& a_dims, const std::vector<int64_t>& b_dims) {
  return {W(dy->data().clone()), W(reduce_to(dy->data(), b_dims))};
}
std::pair<TP, TP> SubBackward(const TP& dy, const std::vector<int64_t>& a_dims, const std::vector<int64_t>& b_dims) {
  return {W(dy->data().clone()), W(reduce_to(-dy->data(), b_dims))};
}
std::pair<TP, TP> MulBackward(const TP& dy, const TP& a, const TP& b) {
  return {W(dy->data() * b->data()), W(reduce_to(dy->data() * a->data(), b->Dims()))};
}
std::pair<TP, TP> DivBackward(const TP& dy, const TP& a, const TP& b) {
  const at::Tensor &g = dy->data(), &x = a->data(), &y = b->data();
  return {W(g / y), W(reduce_to(-g * x / (y * y), b->Dims()))};
}

// ---- GEMM family ------------------------------------------------------------------------------------------------
// D[M,N] = A op B for 2-D row-major operands; ta/tb select the transposed reading of the stored matrix.
static at::Tensor gemm2d(const at::Tensor& a_, const at::Tensor& b_, bool ta, bool tb) {
  at::Tensor a = a_.contiguous(), b = b_.contiguous();
  const int64_t M = ta ? a.size(1) : a.size(0), K = ta ? a.size(0) : a.size(1), N = tb ? b.size(0) : b.size(1);
  if (a.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && (K % 8 == 0) &&
      ((ta ? M : K) % 8 == 0) && ((tb ? K : N) % 8 == 0)) {
    c10::cuda::CUDAGuard guard(a.device());
    at::Tensor out = at::empty({M, N}, a.options());
    TitbGemmDesc d{};
    d.a = a.data_ptr(); d.b = b.data_ptr(); d.out = out.data_ptr();
    d.M = (int)M; d.N = (int)N; d.K = (int)K;
    d.a_mn_major = ta;         // stored [K, M]
    d.b_mn_major = !tb;        // stored [K, N]
    d.lda = a.stride(0); d.ldb = b.stride(0); d.ldo = N; d.splits = 1;
    ok(titb_gemm_bf16(&d, stream()), "gemm_bf16");
    return out;
  }
  if (a.is_cuda() && a.scalar_type() == at::kFloat && b.scalar_type() == at::kFloat) {
    c10::cuda::CUDAGuard guard(a.device());
    at::Tensor out = at::empty({M, N}, a.options());
    ok(titb_sgemm(a.data_ptr<float>(), b.data_ptr<float>(), out.data_ptr<float>(), (int)M, (int)N, (int)K, ta, tb, 0,
                  stream()), "sgemm");
    return out;
  }
  return at::matmul(ta ? a.t() : a, tb ? b.t() : b);
}

TP MatmulForward(const TP& a, const TP& b) {
  const at::Tensor &x = a->data(), &y = b->data();
  if (x.dim() == 2 && y.dim() == 2) return W(gemm2d(x, y, false, false));
  const int64_t M = x.size(-2), K = x.size(-1), N = y.size(-1);
  at::Tensor x3 = x.reshape({-1, M, K}), y3 = y.reshape({-1, K, N});
  TORCH_CHECK(x3.size(0) == y3.size(0), "Matmul: both operands must carry the same batch dims");
  std::vector<at::Tensor> outs;
  for (int64_t i = 0; i < x3.size(0); ++i) outs.push_back(gemm2d(x3[i], y3[i], false, false));
  auto shape = x.sizes().vec();
  shape.back() = N;
  return W(at::stack(outs).reshape(shape));
}
std::pair<TP, TP> MatmulBackward(const TP& a, const TP& b, const TP& dc) {
  const at::Tensor &x = a->data(), &y = b->data(), &g = dc->data();
  const int64_t M = x.size(-2), K = x.size(-1), N = y.size(-1);
  at::Tensor x3 = x.reshape({-1, M, K}), y3 = y.reshape({-1, K, N}), g3 = g.reshape({-1, M, N});
  std::vector<at::Tensor> da, db;
  for (int64_t i = 0; i < x3.size(0); ++i) {
    da.push_back(gemm2d(g3[i], y3[i], false, true));   // dA = dC B^T
    db.push_back(gemm2d(x3[i], g3[i], true, false));   // dB = A^T dC
  }
  return {W(at::stack(da).reshape(x.sizes())), W(at::stack(db).reshape(y.sizes()))};
}

// y = x W^T + b when transpose (weight [out, in]) else x W + b (weight [in, out]).
TP LinearForward(const TP& input, const TP& weight, bool transpose, const TP& bias) {
  const at::Tensor& x = input->data();
  at::Tensor x2 = x.reshape({-1, x.size(-1)});
  at::Tensor y = gemm2d(x2, weight->data(), false, transpose);
  if (bias) y = y + bias->data();
  auto shape = x.sizes().vec();
  shape.back() = y.size(1);
  return W(y.reshape(shape));
}
std::tuple<TP, TP, TP> LinearBackward(const TP& input, const TP& weight, bool transpose, int64_t out_features,
                                      const TP& grad_output, bool has_bias) {
  const at::Tensor &x = input->data(), &w = weight->data(), &g = grad_output->data();
  at::Tensor x2 = x.reshape({-1, x.size(-1)}), g2 = g.reshape({-1, out_features});
  at::Tensor dx = gemm2d(g2, w, false, !transpose).reshape(x.sizes());  // dY W  (or dY W^T)
  at::Tensor dw = transpose ? gemm2d(g2, x2, true, false) : gemm2d(x2, g2, true, false);
  TP db = nullptr;  // column sums (the reference's CUDA path sums the wrong axis)
  if (has_bias && native(g2)) {
    c10::cuda::CUDAGuard guard(g2.device());
    at::Tensor gc = materialize(g2);
    auto fopt = gc.options().dtype(at::kFloat);
    at::Tensor sum = at::empty({out_features}, fopt), scratch = at::empty({titb_colsum_blocks(gc.size(0)), out_features}, fopt);
    ok(titb_colsum(gc.data_ptr(), sum.data_ptr<float>(), gc.size(0), (int)out_features, dt(gc), 0, scratch.data_ptr<float>(),
                   stream()), "bias gradient");
    db = W(sum.to(gc.scalar_type()));
  } else if (has_bias) {
    db = W(g2.sum(0));
  }
  return {W(dx), W(dw), db};
}

TP OuterForward(const TP& a, const TP& b) {
  const at::Tensor &x = a->data(), &y = b->data();
  if (native(x) && native(y) && x.scalar_type() == y.scalar_type() && x.dim() == 1 && y.dim() == 1) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = materialize(x), yc = materialize(y), out = at::empty({x.numel(), y.numel()}, x.options());
    ok(titb_outer(xc.data_ptr(), yc.data_ptr(), out.data_ptr(), x.numel(), y.numel(), dt(x), stream()), "Outer");
    return W(out);
  }
  return W(at::outer(x, y));
}
std::pair<TP, TP> OuterBackward(const TP& a, const TP& b, const TP& g) {
  const at::Tensor &x = a->data(), &y = b->data(), &go = g->data();
  if (native(x) && native(y) && native(go) && x.scalar_type() == y.scalar_type() && go.scalar_type() == x.scalar_type()) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = materialize(x), yc = materialize(y), gc = materialize(go);
    at::Tensor da = at::empty_like(xc), db = at::empty_like(yc);
    ok(titb_outer_bwd(gc.data_ptr(), xc.data_ptr(), yc.data_ptr(), da.data_ptr(), db.data_ptr(), xc.numel(), yc.numel(),
                      dt(x), stream()), "OuterBackward");
    return {W(da), W(db)};
  }
  return {W(at::mv(go, y)), W(at::mv(go.t(), x))};
}

// ---- normalisation ------------------------------------------------------------------------------------------------------
std::tuple<TP, TP, TP> LayerNormForward(const TP& input, const TP& weight, const TP& bias, float eps) {
  const at::Tensor& x = input->data();
  const int64_t C = x.size(-1), rows = x.numel() / C;
  if (native(x) && x.is_contiguous() && weight->data().scalar_type() == x.scalar_type()) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor y = at::empty_like(x), mean = at::empty({rows}, x.options().dtype(at::kFloat)), rstd = at::empty_like(mean);
    ok(titb_layernorm_fwd(x.data_ptr(), weight->data().data_ptr(), bias->data().data_ptr(), y.data_ptr(),
                          mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, (int)C, eps, dt(x), stream()), "LayerNormForward");
    return {W(y), W(mean), W(rstd)};
  }
  at::Tensor xf = x.to(at::kFloat).reshape({rows, C});
  at::Tensor mean = xf.mean(1), var = xf.var(1, false);
  at::Tensor rstd = (var + eps).rsqrt();
  at::Tensor y = (xf - mean.unsqueeze(1)) * rstd.unsqueeze(1) * weight->data().to(at::kFloat) + bias->data().to(at::kFloat);
  return {W(y.reshape(x.sizes()).to(x.scalar_type())), W(mean), W(rstd)};
}
std::tuple<TP, TP, TP> LayerNormBackward(const TP& input, const TP& weight, const TP& bias, const TP& mean, const TP& rstd,
                                         const TP& grad_output) {
  const at::Tensor& x = input->data();
  const int64_t C = x.size(-1), rows = x.numel() / C;
  const at::Tensor& go = grad_output->data();
  if (native(x) && x.is_contiguous() && go.is_contiguous() && go.scalar_type() == x.scalar_type() &&
      weight->data().scalar_type() == x.scalar_type()) {
    c10::cuda::CUDAGuard guard(x.device());
    auto fopt = x.options().dtype(at::kFloat);
    at::Tensor dx = at::empty_like(x), dw = at::empty({C}, fopt), db = at::empty({C}, fopt);
    at::Tensor scratch = at::empty({2, titb_layernorm_bwd_blocks(rows), C}, fopt);
    ok(titb_layernorm_bwd(go.data_ptr(), x.data_ptr(), weight->data().data_ptr(), mean->data().data_ptr<float>(),
                          rstd->data().data_ptr<float>(), dx.data_ptr(), dw.data_ptr<float>(), db.data_ptr<float>(),
                          scratch.data_ptr<float>(), rows, (int)C, dt(x), 0, nullptr, stream()), "LayerNormBackward");
    return {W(dx), W(dw.to(weight->data().scalar_type())), W(db.to(weight->data().scalar_type()))};
  }
  at::Tensor xf = x.to(at::kFloat).reshape({rows, C}), g = go.to(at::kFloat).reshape({rows, C});
  at::Tensor w = weight->data().to(at::kFloat);
  at::Tensor norm = (xf - mean->data().unsqueeze(1)) * rstd->data().unsqueeze(1);
  at::Tensor dnorm = g * w;
  at::Tensor dx = (dnorm - dnorm.mean(1, true) - norm * (dnorm * norm).mean(1, true)) * rstd->data().unsqueeze(1);
  return {W(dx.reshape(x.sizes()).to(x.scalar_type())), W((g * norm).sum(0).to(weight->data().scalar_type())),
          W(g.sum(0).to(weight->data().scalar_type()))};
}

// ---- RMSNorm / RoPE / SwiGLU (LLaMA-3 building blocks; not in the reference) ---------------------------------------------
std::pair<TP, TP> RMSNormForward(const TP& input, const TP& weight, float eps) {
  const at::Tensor& x = input->data();
  const int64_t C = x.size(-1), rows = x.numel() / C;
  if (native(x) && x.is_contiguous() && weight->data().scalar_type() == x.scalar_type()) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor y = at::empty_like(x), rstd = at::empty({rows}, x.options().dtype(at::kFloat));
    ok(titb_rmsnorm_fwd(x.data_ptr(), weight->data().data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, (int)C, eps,
                        dt(x), stream()), "RMSNormForward");
    return {W(y), W(rstd)};
  }
  at::Tensor xf = x.to(at::kFloat).reshape({rows, C});
  at::Tensor rstd = (xf.pow(2).mean(1) + eps).rsqrt();
  at::Tensor y = xf * rstd.unsqueeze(1) * weight->data().to(at::kFloat);
  return {W(y.reshape(x.sizes()).to(x.scalar_type())), W(rstd)};
}
std::pair<TP, TP> RMSNormBackward(const TP& input, const TP& weight, const TP& rstd, const TP& grad_output) {
  const at::Tensor& x = input->data();
  const at::Tensor& g = grad_output->data();
  const int64_t C = x.size(-1), rows = x.numel() / C;
  if (native(x) && x.is_contiguous() && g.is_contiguous() && g.scalar_type() == x.scalar_type() &&
      weight->data().scalar_type() == x.scalar_type()) {
    c10::cuda::CUDAGuard guard(x.device());
    auto fopt = x.options().dtype(at::kFloat);
    at::Tensor dx = at::empty_like(x), dw = at::empty({C}, fopt);
    at::Tensor scratch = at::empty({2, titb_layernorm_bwd_blocks(rows), C}, fopt);
    ok(titb_rmsnorm_bwd(g.data_ptr(), x.data_ptr(), weight->data().data_ptr(), rstd->data().data_ptr<float>(), dx.data_ptr(),
                        dw.data_ptr<float>(), scratch.data_ptr<float>(), rows, (int)C, dt(x), 0, nullptr, stream()), "RMSNormBackward");
    return {W(dx), W(dw.to(weight->data().scalar_type()))};
  }
  at::Tensor xf = x.to(at::kFloat).reshape({rows, C}), gf = g.to(at::kFloat).reshape({rows, C});
  at::Tensor w = weight->data().to(at::kFloat), r = rstd->data().to(at::kFloat).unsqueeze(1);
  at::Tensor n = xf * r, dn = gf * w;
  at::Tensor dx = (dn - n * (dn * n).mean(1, true)) * r;
  return {W(dx.reshape(x.sizes()).to(x.scalar_type())), W((gf * n).sum(0).to(weight->data().scalar_type()))};
}
TP RopeForward(const TP& input, float theta, int64_t pos_offset, bool inverse) {
  const at::Tensor& x = input->data();
  TORCH_CHECK(x.dim() == 4 && x.size(3) % 2 == 0, "Rope expects [B, T, H, hd] with an even head size");
  const int64_t B = x.size(0), T = x.size(1), H = x.size(2), hd = x.size(3), half = hd / 2;
  if (native(x)) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = materialize(x), y = at::empty_like(xc);
    ok(titb_rope(xc.data_ptr(), y.data_ptr(), (int)B, (int)T, (int)H, (int)hd, (int)pos_offset, theta, inverse, dt(xc),
                 stream()), "Rope");
    return W(y);
  }
  at::Tensor inv = at::pow(theta, -at::arange(0, half, at::kFloat) * 2.0 / static_cast<double>(hd));
  at::Tensor ang = (at::arange(T, at::kFloat) + static_cast<double>(pos_offset)).unsqueeze(1) * inv.unsqueeze(0);   // [T, half]
  at::Tensor cos = ang.cos().reshape({1, T, 1, half}), sin = ang.sin().reshape({1, T, 1, half});
  if (inverse) sin = -sin;
  at::Tensor a = x.narrow(3, 0, half).to(at::kFloat), b = x.narrow(3, half, half).to(at::kFloat);
  return W(at::cat({a * cos - b * sin, b * cos + a * sin}, 3).to(x.scalar_type()));
}
TP SwiGLUForward(const TP& input) {
  const at::Tensor& x = input->data();
  const int64_t F = x.size(-1) / 2, rows = x.numel() / (2 * F);
  auto sizes = x.sizes().vec();
  sizes.back() = F;
  if (native(x) && x.is_contiguous()) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor y = at::empty(sizes, x.options());
    ok(titb_swiglu_fwd(x.data_ptr(), y.data_ptr(), rows, (int)F, dt(x), stream()), "SwiGLU");
    return W(y);
  }
  at::Tensor gate = x.narrow(-1, 0, F).to(at::kFloat), up = x.narrow(-1, F, F).to(at::kFloat);
  return W((at::silu(gate) * up).to(x.scalar_type()));
}
TP SwiGLUBackward(const TP& grad_output, const TP& input) {
  const at::Tensor &g = grad_output->data(), &x = input->data();
  const int64_t F = x.size(-1) / 2, rows = x.numel() / (2 * F);
  if (native(x) && x.is_contiguous() && g.is_contiguous() && g.scalar_type() == x.scalar_type()) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor dx = at::empty_like(x);
    ok(titb_swiglu_bwd(g.data_ptr(), x.data_ptr(), dx.data_ptr(), rows, (int)F, dt(x), stream()), "SwiGLUBackward");
    return W(dx);
  }
  at::Tensor gate = x.narrow(-1, 0, F).to(at::kFloat), up = x.narrow(-1, F, F).to(at::kFloat), gf = g.to(at::kFloat);
  at::Tensor sg = gate.sigmoid();
  at::Tensor dgate = gf * up * (sg * (1 + gate * (1 - sg)));        // d silu(z) / dz = s (1 + z (1 - s))
  at::Tensor dup = gf * gate * sg;
  return W(at::cat({dgate, dup}, -1).to(x.scalar_type()));
}

// ---- fused causal attention -------------------------------------------------------------------------------------------------
static bool attn_kernel_ok(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
  const int64_t hd = q.size(3);
  return q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
         v.scalar_type() == at::kBFloat16 && (hd == 64 || hd == 128) && q.size(2) % k.size(2) == 0;
}
// softmax(mask(q k^T scale)) per head as [B, Hq, T, T] fp32, plus the head-major fp32 operands
static at::Tensor attn_probs(const at::Tensor& q, const at::Tensor& k, float scale, at::Tensor* qh, at::Tensor* kh) {
  const int64_t T = q.size(1), group = q.size(2) / k.size(2);
  *qh = q.to(at::kFloat).transpose(1, 2);                                            // [B, Hq, T, hd]
  *kh = k.to(at::kFloat).transpose(1, 2).repeat_interleave(group, 1);
  at::Tensor s = at::matmul(*qh, kh->transpose(-2, -1)) * scale;
  at::Tensor mask = at::triu(at::ones({T, T}, s.options().dtype(at::kBool)), 1);
  return at::softmax(s.masked_fill(mask, -INFINITY), -1);
}
std::pair<TP, TP> CausalAttentionForward(const TP& q_, const TP& k_, const TP& v_, float scale) {
  const at::Tensor &q = q_->data(), &k = k_->data(), &v = v_->data();
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.sizes() == k.sizes() && q.size(3) == k.size(3), "CausalAttention: bad shapes");
  const int64_t B = q.size(0), T = q.size(1), Hq = q.size(2), hd = q.size(3), Hkv = k.size(2);
  if (scale == 0.f) scale = 1.f / std::sqrt(static_cast<float>(hd));
  if (attn_kernel_ok(q, k, v)) {
    c10::cuda::CUDAGuard guard(q.device());
    at::Tensor qc = materialize(q), kc = materialize(k), vc = materialize(v);
    at::Tensor o = at::empty({B, T, Hq, hd}, q.options()), lse = at::empty({B, Hq, T}, q.options().dtype(at::kFloat));
    TitbAttnDesc d{};
    d.q = qc.data_ptr(); d.k = kc.data_ptr(); d.v = vc.data_ptr(); d.o = o.data_ptr(); d.lse = lse.data_ptr<float>();
    d.B = (int)B; d.T = (int)T; d.Hq = (int)Hq; d.Hkv = (int)Hkv; d.hd = (int)hd;
    d.q_stride_t = Hq * hd; d.k_stride_t = Hkv * hd; d.v_stride_t = Hkv * hd; d.o_stride_t = Hq * hd;
    d.scale = scale;
    ok(titb_attn_fwd(&d, stream()), "CausalAttentionForward");
    return {W(o), W(lse)};
  }
  at::Tensor qh, kh;
  at::Tensor p = attn_probs(q, k, scale, &qh, &kh);
  at::Tensor vh = v.to(at::kFloat).transpose(1, 2).repeat_interleave(Hq / Hkv, 1);
  at::Tensor o = at::matmul(p, vh).transpose(1, 2).contiguous().to(q.scalar_type());
  return {W(o), W(at::zeros({1}, o.options().dtype(at::kFloat)))};                   // no saved statistics on this path
}
std::tuple<TP, TP, TP> CausalAttentionBackward(const TP& go_, const TP& q_, const TP& k_, const TP& v_, const TP& o_,
                                               const TP& lse_, float scale) {
  const at::Tensor &go = go_->data(), &q = q_->data(), &k = k_->data(), &v = v_->data();
  const int64_t B = q.size(0), T = q.size(1), Hq = q.size(2), hd = q.size(3), Hkv = k.size(2), group = Hq / Hkv;
  if (scale == 0.f) scale = 1.f / std::sqrt(static_cast<float>(hd));
  if (attn_kernel_ok(q, k, v) && go.scalar_type() == at::kBFloat16) {
    c10::cuda::CUDAGuard guard(q.device());
    at::Tensor qc = materialize(q), kc = materialize(k), vc = materialize(v), gc = materialize(go), oc = materialize(o_->data());
    at::Tensor dq = at::empty_like(qc), dk = at::empty_like(kc), dv = at::empty_like(vc);
    auto fopt = q.options().dtype(at::kFloat);
    at::Tensor delta = at::empty({B, Hq, T}, fopt), acc = at::empty({B, T, Hq, hd}, fopt);
    TitbAttnDesc d{};
    d.q = qc.data_ptr(); d.k = kc.data_ptr(); d.v = vc.data_ptr(); d.o = oc.data_ptr(); d.lse = lse_->data().data_ptr<float>();
    d.d_o = gc.data_ptr(); d.dq = dq.data_ptr(); d.dk = dk.data_ptr(); d.dv = dv.data_ptr();
    d.delta = delta.data_ptr<float>(); d.dq_accum = acc.data_ptr<float>();
    d.B = (int)B; d.T = (int)T; d.Hq = (int)Hq; d.Hkv = (int)Hkv; d.hd = (int)hd;
    d.q_stride_t = d.o_stride_t = d.do_stride_t = d.dq_stride_t = Hq * hd;
    d.k_stride_t = d.v_stride_t = d.dk_stride_t = d.dv_stride_t = Hkv * hd;
    d.scale = scale;
    ok(titb_attn_bwd(&d, stream()), "CausalAttentionBackward");
    return {W(dq), W(dk), W(dv)};
  }
  // dV = P^T dO; dP = dO V^T; dS = P (dP - rowsum(dP P)); dQ = dS K scale; dK = dS^T Q scale; kv heads sum their group
  at::Tensor qh, kh;
  at::Tensor p = attn_probs(q, k, scale, &qh, &kh);
  at::Tensor vh = v.to(at::kFloat).transpose(1, 2).repeat_interleave(group, 1);
  at::Tensor gh = go.to(at::kFloat).transpose(1, 2);                                 // [B, Hq, T, hd]
  at::Tensor dvh = at::matmul(p.transpose(-2, -1), gh);
  at::Tensor dp = at::matmul(gh, vh.transpose(-2, -1));
  at::Tensor ds = p * (dp - (dp * p).sum(-1, true));
  at::Tensor dqh = at::matmul(ds, kh) * scale, dkh = at::matmul(ds.transpose(-2, -1), qh) * scale;
  auto fold = [&](const at::Tensor& t) {                                             // [B, Hq, T, hd] -> [B, T, Hkv, hd]
    return t.reshape({B, Hkv, group, T, hd}).sum(2).transpose(1, 2).contiguous();
  };
  return {W(dqh.transpose(1, 2).contiguous().to(q.scalar_type())), W(fold(dkh).to(k.scalar_type())),
          W(fold(dvh).to(v.scalar_type()))};
}

// ---- softmax / cross entropy / embedding -------------------------------------------------------------------------------
TP SoftmaxForward(const TP& input, int64_t dim) {
  const at::Tensor& x = input->data();
  if (native(x) && x.dim() >= 1) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = materialize(x), y = at::empty_like(xc);
    const Axis3 a = axis3(xc.sizes(), dim < 0 ? dim + xc.dim() : dim);
    ok(titb_softmax_fwd(xc.data_ptr(), y.data_ptr(), a.outer, (int)a.n, a.inner, dt(xc), stream()), "Softmax");
    return W(y);
  }
  return W(at::softmax(x, dim));
}
TP SoftmaxBackward(const TP& grad_output, const TP& output, int64_t dim) {
  const at::Tensor &g = grad_output->data(), &y = output->data();
  if (native(g) && native(y) && g.scalar_type() == y.scalar_type() && y.dim() >= 1) {
    c10::cuda::CUDAGuard guard(y.device());
    at::Tensor gc = materialize(g), yc = materialize(y), dx = at::empty_like(yc);
    const Axis3 a = axis3(yc.sizes(), dim < 0 ? dim + yc.dim() : dim);
    ok(titb_softmax_bwd(gc.data_ptr(), yc.data_ptr(), dx.data_ptr(), a.outer, (int)a.n, a.inner, dt(yc), stream()),
       "SoftmaxBackward");
    return W(dx);
  }
  return W(y * (g - (g * y).sum(dim, true)));
}
TP CrossEntropyForward(const TP& input, const TP& target) {
  const at::Tensor& x = input->data();
  const int64_t V = x.size(-1), rows = x.numel() / V;
  at::Tensor tgt = target->data().reshape({rows}).to(at::kLong);
  if (native(x) && x.is_contiguous()) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor losses = at::empty({rows}, x.options().dtype(at::kFloat)), loss = at::empty({}, losses.options());
    ok(titb_xent_fwd_bwd(x.data_ptr(), (const long long*)tgt.data_ptr<int64_t>(), losses.data_ptr<float>(), nullptr, rows,
                         (int)V, V, 0.f, dt(x), stream()), "CrossEntropyForward");
    ok(titb_mean(losses.data_ptr<float>(), loss.data_ptr<float>(), rows, 1.f / rows, stream()), "mean");
    return W(loss);
  }
  at::Tensor lsm = at::log_softmax(x.to(at::kFloat).reshape({rows, V}), 1);
  return W(-lsm.gather(1, tgt.unsqueeze(1)).mean());
}
TP CrossEntropyBackward(const TP& input, const TP& target, const TP& grad_output) {
  const at::Tensor& x = input->data();
  const int64_t V = x.size(-1), rows = x.numel() / V;
  at::Tensor tgt = target->data().reshape({rows}).to(at::kLong);
  if (native(x) && x.is_contiguous() && tgt.is_cuda()) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor d = at::empty_like(x), up = grad_output->data().to(at::kFloat).reshape({-1}).contiguous(), tc = tgt.contiguous();
    ok(titb_xent_bwd(x.data_ptr(), reinterpret_cast<const long long*>(tc.data_ptr<int64_t>()), d.data_ptr(), up.data_ptr<float>(),
                     rows, (int)V, V, 1.f / static_cast<float>(rows), dt(x), stream()), "CrossEntropyBackward");
    return W(d);
  }
  at::Tensor p = at::softmax(x.to(at::kFloat).reshape({rows, V}), 1);
  p.scatter_add_(1, tgt.unsqueeze(1), at::full({rows, 1}, -1.0, p.options()));
  at::Tensor d = p * (grad_output->data().to(at::kFloat) / static_cast<double>(rows));  // honours the upstream gradient
  return W(d.reshape(x.sizes()).to(x.scalar_type()));
}
TP EmbeddingForward(const TP& input, const TP& weight) {
  TORCH_CHECK(input->data().scalar_type() == at::kLong, "Embedding indices must be INT64");
  const at::Tensor &idx = input->data(), &w = weight->data();
  const int64_t C = w.size(-1);
  if (native(w) && idx.is_cuda() && w.is_contiguous() && C % (w.scalar_type() == at::kBFloat16 ? 8 : 4) == 0 && idx.dim() >= 1) {
    c10::cuda::CUDAGuard guard(w.device());
    at::Tensor ic = materialize(idx);
    auto sizes = ic.sizes().vec();
    sizes.push_back(C);
    at::Tensor out = at::empty(sizes, w.options());
    ok(titb_embedding_fwd(reinterpret_cast<const long long*>(ic.data_ptr<int64_t>()), w.data_ptr(), nullptr, out.data_ptr(),
                          ic.numel(), (int)ic.size(-1), (int)C, 0, dt(w), stream()), "EmbeddingForward");
    return W(out);
  }
  return W(at::embedding(w, idx));
}
TP EmbeddingBackward(const TP& input, const std::vector<int64_t>& weight_dims, const TP& grad_output) {
  const at::Tensor& g = grad_output->data();
  const at::Tensor& idx = input->data();
  at::Tensor dw = at::zeros(weight_dims, g.options().dtype(at::kFloat));
  const int64_t C = g.size(-1);
  if (native(g) && idx.is_cuda() && C % (g.scalar_type() == at::kBFloat16 ? 8 : 4) == 0 && idx.dim() >= 1) {
    c10::cuda::CUDAGuard guard(g.device());
    at::Tensor ic = materialize(idx), gc = materialize(g);
    ok(titb_embedding_bwd(reinterpret_cast<const long long*>(ic.data_ptr<int64_t>()), gc.data_ptr(), dw.data_ptr<float>(), nullptr,
                          ic.numel(), (int)ic.size(-1), (int)C, 0, (int)weight_dims[0], dt(gc), stream()), "EmbeddingBackward");
    return W(dw.to(g.scalar_type()));
  }
  dw.index_add_(0, idx.reshape({-1}), g.reshape({-1, C}).to(at::kFloat));
  return W(dw.to(g.scalar_type()));
}

// ---- reductions -----------------------------------------------------------------------------------------------------------
static at::Tensor expand_back(const at::Tensor& g, const std::vector<int64_t>& in_dims, int64_t dim, bool keep_dim) {
  at::Tensor gg = keep_dim ? g : g.unsqueeze(dim);
  return gg.expand(in_dims).contiguous();
}
// op: 0 sum, 1 mean, 2 max, 3 min
static TP reduce_forward(const TP& x, int64_t dim, bool keep, int op) {
  const at::Tensor& t = x->data();
  const int64_t d = dim < 0 ? dim + t.dim() : dim;
  if (native(t) && t.dim() >= 1 && t.numel() > 0) {
    c10::cuda::CUDAGuard guard(t.device());
    at::Tensor tc = materialize(t);
    auto sizes = tc.sizes().vec();
    if (keep) sizes[d] = 1; else sizes.erase(sizes.begin() + d);
    at::Tensor y = at::empty(sizes, tc.options());
    const Axis3 a = axis3(tc.sizes(), d);
    ok(titb_reduce(tc.data_ptr(), y.data_ptr(), nullptr, a.outer, a.n, a.inner, op, dt(tc), stream()), "reduce");
    return W(y);
  }
  switch (op) {
    case 0: return W(t.sum(d, keep));
    case 1: return W(t.mean(d, keep));
    case 2: return W(t.amax(d, keep));
    default: return W(t.amin(d, keep));
  }
}
static TP reduce_broadcast_backward(const TP& g, const std::vector<int64_t>& in_dims, int64_t dim, bool keep, float scale) {
  const at::Tensor& go = g->data();
  const int64_t d = dim < 0 ? dim + (int64_t)in_dims.size() : dim;
  if (native(go)) {
    c10::cuda::CUDAGuard guard(go.device());
    at::Tensor gc = materialize(go), dx = at::empty(in_dims, go.options());
    const Axis3 a = axis3(in_dims, d);
    ok(titb_reduce_bwd(gc.data_ptr(), nullptr, dx.data_ptr(), a.outer, a.n, a.inner, scale, dt(gc), stream()), "reduce_bwd");
    return W(dx);
  }
  at::Tensor e = expand_back(go, in_dims, d, keep);
  return W(scale == 1.f ? e : e * static_cast<double>(scale));
}
TP MeanForward(const TP& x, int64_t dim, bool keep) { return reduce_forward(x, dim, keep, 1); }
TP SumForward(const TP& x, int64_t dim, bool keep) { return reduce_forward(x, dim, keep, 0); }
TP MaxForward(const TP& x, int64_t dim, bool keep) { return reduce_forward(x, dim, keep, 2); }
TP MinForward(const TP& x, int64_t dim, bool keep) { return reduce_forward(x, dim, keep, 3); }
TP MeanBackward(const TP& g, const std::vector<int64_t>& in_dims, int64_t dim, bool keep) {
  const int64_t d = dim < 0 ? dim + (int64_t)in_dims.size() : dim;
  return reduce_broadcast_backward(g, in_dims, dim, keep, 1.f / static_cast<float>(in_dims[d]));
}
TP SumBackward(const TP& g, const std::vector<int64_t>& in_dims, int64_t dim, bool keep) {
  return reduce_broadcast_backward(g, in_dims, dim, keep, 1.f);
}
// Max/Min route the gradient to every element equal to the extremum (reference reduction.cc:13-167).
TP MaxBackward(const TP& g, const TP& input, const TP& output, int64_t dim, bool keep) {
  const at::Tensor& x = input->data();
  const int64_t d = dim < 0 ? dim + x.dim() : dim;
  at::Tensor o = keep ? output->data() : output->data().unsqueeze(d);
  return W(expand_back(g->data(), x.sizes().vec(), d, keep) * (x == o).to(x.scalar_type()));
}
TP MinBackward(const TP& g, const TP& input, const TP& output, int64_t dim, bool keep) {
  return MaxBackward(g, input, output, dim, keep);
}

// ---- transforms -------------------------------------------------------------------------------------------------------------
static TP tri(const TP& x, int64_t diag, bool upper) {
  const at::Tensor& t = x->data();
  if (native(t) && t.dim() == 2) {
    c10::cuda::CUDAGuard guard(t.device());
    at::Tensor tc = materialize(t), y = at::empty_like(tc);
    ok(titb_tri(tc.data_ptr(), y.data_ptr(), (int)tc.size(0), (int)tc.size(1), (int)diag, upper, dt(tc), stream()), "tri");
    return W(y);
  }
  return W(upper ? at::triu(t, diag) : at::tril(t, diag));
}
TP TrilForward(const TP& x, int64_t diag) { return tri(x, diag, false); }
TP TrilBackward(const TP& g, int64_t diag) { return tri(g, diag, false); }
TP TriuForward(const TP& x, int64_t diag) { return tri(x, diag, true); }
TP TriuBackward(const TP& g, int64_t diag) { return tri(g, diag, true); }
TP TransposeForward(const TP& x, int64_t d0, int64_t d1) { return W(x->data().transpose(d0, d1)); }
TP TransposeBackward(const TP& g, int64_t d0, int64_t d1) { return W(g->data().transpose(d0, d1)); }
// mask is broadcast by modulo over the flattened input (reference transform.cc:121-152).
static at::Tensor mask_like(const at::Tensor& x, const at::Tensor& mask) {
  const int64_t n = x.numel(), m = mask.numel();
  at::Tensor flat = mask.reshape({-1});
  if (m != n) flat = flat.repeat({(n + m - 1) / m}).narrow(0, 0, n);
  return (flat == 1).reshape(x.sizes());
}
// flags: bit 0 = backward (masked positions become 0), bit 1 = an element is masked when its entry equals 1
static TP mask_apply(const at::Tensor& x, const at::Tensor& mask, float value, int backward) {
  int mdt = -1;
  if (mask.scalar_type() == at::kFloat) mdt = 0;
  else if (mask.scalar_type() == at::kBFloat16) mdt = 1;
  else if (mask.scalar_type() == at::kBool || mask.scalar_type() == at::kByte) mdt = 2;
  if (native(x) && mask.is_cuda() && mdt >= 0 && mask.numel() > 0) {
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = materialize(x), mc = materialize(mask), y = at::empty_like(xc);
    ok(titb_mask_fill(xc.data_ptr(), mc.data_ptr(), y.data_ptr(), xc.numel(), mc.numel(), value, backward | 2, dt(xc), mdt,
                      stream()), "Mask");
    return W(y);
  }
  return W(x.masked_fill(mask_like(x, mask), backward ? 0.0 : static_cast<double>(value)));
}
TP MaskForward(const TP& x, const TP& mask, float value) { return mask_apply(x->data(), mask->data(), value, 0); }
TP MaskBackward(const TP& g, const TP& mask) { return mask_apply(g->data(), mask->data(), 0.f, 1); }
TP RepeatInterleaveForward(const TP& x, int64_t repeat, int64_t dim) {
  const at::Tensor& t = x->data();
  const int64_t d = dim < 0 ? dim + t.dim() : dim;
  if (native(t) && t.dim() <= 5) {
    // [.., n, ..] -> stride-0 view [.., n, repeat, ..] materialised by the gather kernel -> [.., n * repeat, ..]
    std::vector<int64_t> ex = t.sizes().vec(), out = t.sizes().vec();
    ex.insert(ex.begin() + d + 1, repeat);
    out[d] *= repeat;
    return W(materialize(materialize(t).unsqueeze(d + 1).expand(ex)).reshape(out));
  }
  return W(t.repeat_interleave(repeat, d));
}
TP RepeatInterleaveBackward(const TP& g, const std::vector<int64_t>& in_dims, int64_t dim) {
  std::vector<int64_t> shape = in_dims;
  const int64_t d = dim < 0 ? dim + (int64_t)in_dims.size() : dim;
  const int64_t repeat = g->data().size(d) / in_dims[d];
  shape.insert(shape.begin() + d + 1, repeat);
  return reduce_forward(std::make_shared<Tensor>(materialize(g->data()).reshape(shape)), d + 1, false, 0);
}

// ---- misc ---------------------------------------------------------------------------------------------------------------------
std::vector<TP> SplitForward(const TP& x, int64_t split_size, int dim) {
  std::vector<TP> out;
  for (auto& t : x->data().split(split_size, dim)) out.push_back(W(t));
  return out;
}
TP SplitBackward(const std::vector<int64_t>& in_dims, int64_t split_size, int dim, const std::vector<TP>& grads) {
  TORCH_CHECK(!grads.empty(), "SplitBackward: no gradients");
  at::Tensor dx = at::empty(in_dims, grads[0]->data().options());
  int64_t pos = 0;
  for (auto& g : grads) {
    const int64_t len = g->data().size(dim);
    scatter_into(dx, dx.narrow(dim, pos, len), g->data());
    pos += len;
  }
  TORCH_CHECK(pos == in_dims[dim], "SplitBackward: gradients do not cover the split dimension");
  return W(dx);
}
TP NoOpForward(const TP& x, const std::vector<int64_t>& dims) { return std::make_shared<Tensor>(x->data().reshape(dims)); }
TP NoOpBackward(const std::vector<int64_t>& dims, const TP& g) { return std::make_shared<Tensor>(g->data().reshape(dims)); }
static at::Tensor slice_nd(at::Tensor t, const std::vector<int64_t>& s, const std::vector<int64_t>& e,
                           const std::vector<int64_t>& st) {
  for (size_t d = 0; d < s.size(); ++d) t = t.slice(static_cast<int64_t>(d), s[d], e[d], st[d]);
  return t;
}
TP SliceForward(const TP& x, const std::vector<int64_t>& s, const std::vector<int64_t>& e, const std::vector<int64_t>& st) {
  return W(slice_nd(x->data(), s, e, st));
}
TP SliceBackward(const TP& g, const std::vector<int64_t>& in_dims, const std::vector<int64_t>& s,
                 const std::vector<int64_t>& e, const std::vector<int64_t>& st) {
  at::Tensor dx = at::zeros(in_dims, g->data().options());
  scatter_into(dx, slice_nd(dx, s, e, st), g->data());
  return W(dx);
}
TP StackForward(const std::vector<TP>& xs, int64_t dim) {
  TORCH_CHECK(!xs.empty(), "StackForward: no inputs");
  std::vector<int64_t> shape = xs[0]->data().sizes().vec();
  const int64_t d = dim < 0 ? dim + (int64_t)shape.size() + 1 : dim;
  shape.insert(shape.begin() + d, (int64_t)xs.size());
  at::Tensor out = at::empty(shape, xs[0]->data().options());
  for (size_t i = 0; i < xs.size(); ++i) scatter_into(out, out.select(d, (int64_t)i), xs[i]->data());
  return W(out);
}
std::vector<TP> StackBackward(const std::vector<int64_t>&, int64_t dim, const TP& g) {
  std::vector<TP> out;
  for (auto& t : g->data().unbind(dim)) out.push_back(W(t));
  return out;
}

// ---- registration ----------------------------------------------------------------------------------------------------------------
#define REG_BOTH(Name)                                  \
  REGISTER_KERNEL(DeviceType::kCPU, Name, &Name);       \
  REGISTER_KERNEL(DeviceType::kCUDA, Name, &Name)

REG_BOTH(AccumulateGrad); REG_BOTH(AdamAccumulateGrad); REG_BOTH(Fill);
REG_BOTH(NegForward); REG_BOTH(NegBackward); REG_BOTH(ReciprocalForward); REG_BOTH(ReciprocalBackward);
REG_BOTH(SinForward); REG_BOTH(SinBackward); REG_BOTH(CosForward); REG_BOTH(CosBackward);
REG_BOTH(TanhForward); REG_BOTH(TanhBackward); REG_BOTH(RsqrtForward); REG_BOTH(RsqrtBackward);
REG_BOTH(SigmoidForward); REG_BOTH(SigmoidBackward); REG_BOTH(GeluForward); REG_BOTH(GeluBackward); REG_BOTH(PowForward); REG_BOTH(PowBackward);
REG_BOTH(EqualsScalarForward); REG_BOTH(AddScalarForward); REG_BOTH(AddScalarBackward);
REG_BOTH(MulScalarForward); REG_BOTH(MulScalarBackward);
REG_BOTH(AddForward); REG_BOTH(AddBackward); REG_BOTH(SubForward); REG_BOTH(SubBackward);
REG_BOTH(MulForward); REG_BOTH(MulBackward); REG_BOTH(DivForward); REG_BOTH(DivBackward);
REG_BOTH(MatmulForward); REG_BOTH(MatmulBackward); REG_BOTH(LinearForward); REG_BOTH(LinearBackward);
REG_BOTH(OuterForward); REG_BOTH(OuterBackward); REG_BOTH(LayerNormForward); REG_BOTH(LayerNormBackward);
REG_BOTH(CausalAttentionForward); REG_BOTH(CausalAttentionBackward);
REG_BOTH(RMSNormForward); REG_BOTH(RMSNormBackward); REG_BOTH(RopeForward); REG_BOTH(SwiGLUForward); REG_BOTH(SwiGLUBackward);
REG_BOTH(SoftmaxForward); REG_BOTH(SoftmaxBackward); REG_BOTH(CrossEntropyForward); REG_BOTH(CrossEntropyBackward);
REG_BOTH(EmbeddingForward); REG_BOTH(EmbeddingBackward);
REG_BOTH(MeanForward); REG_BOTH(MeanBackward); REG_BOTH(SumForward); REG_BOTH(SumBackward);
REG_BOTH(MaxForward); REG_BOTH(MaxBackward); REG_BOTH(MinForward); REG_BOTH(MinBackward);
REG_BOTH(TrilForward); REG_BOTH(TrilBackward); REG_BOTH(TriuForward); REG_BOTH(TriuBackward);
REG_BOTH(TransposeForward); REG_BOTH(TransposeBackward); REG_BOTH(MaskForward); REG_BOTH(MaskBackward);
REG_BOTH(RepeatInterleaveForward); REG_BOTH(RepeatInterleaveBackward);
REG_BOTH(SplitForward); REG_BOTH(SplitBackward); REG_BOTH(NoOpForward); REG_BOTH(NoOpBackward);
REG_BOTH(SliceForward); REG_BOTH(SliceBackward); REG_BOTH(StackForward); REG_BOTH(StackBackward);

}  // namespace infini_train::kernels
