// Python bindings of the sm_100a kernel library: at::Tensor in, at::Tensor out.
// Outputs are allocated with the torch caching allocator and every launch goes
// to the current CUDA stream, so the ops can be captured in CUDA graphs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGraphsC10Utils.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>

#include "kernels/api.h"

namespace {

using at::Tensor;
using c10::optional;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline int dt_code(const Tensor& t) {
  if (t.scalar_type() == at::kFloat) return 0;
  if (t.scalar_type() == at::kBFloat16) return 1;
  TORCH_CHECK(false, "titb200: only float32 and bfloat16 tensors are supported, got ", t.scalar_type());
}
inline void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), "titb200: ", name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), "titb200: ", name, " must be contiguous");
}
int64_t g_launches = 0;  // kernels launched through this module (host-side count)
inline void check_rc(int rc, const char* what, int nkernels = 1) {
  g_launches += nkernels;
  if (rc >= 20000) {
    const char* msg = rc == TITB_ERR_ALIGNMENT ? "operand base or row stride not 16-byte aligned"
                      : rc == TITB_ERR_TENSOR_MAP ? "TMA tensor map could not be encoded"
                                                  : "unsupported shape";
    TORCH_CHECK(false, "titb200: ", what, " failed: ", msg);
  }
  TORCH_CHECK(rc == 0, "titb200: ", what, " failed: ", cudaGetErrorString(static_cast<cudaError_t>(rc)));
}
// Clears any error left on this thread by an unrelated earlier CUDA call, then launches.
#define CHECK_RC(...)          \
  do {                         \
    (void)cudaGetLastError();  \
    check_rc(__VA_ARGS__);     \
  } while (0)
inline const void* opt_ptr(const optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// ----------------------------------------------------------------------- GEMM
// out[M,N] = A . B^T.  a: [M,K] (a_mn=0) or [K,M] (a_mn=1); b: [N,K] (b_mn=0) or [K,N] (b_mn=1).
// Row strides may exceed the logical width (2-D views with stride(1) == 1).
std::vector<Tensor> gemm(const Tensor& a, const Tensor& b, bool a_mn, bool b_mn, int64_t epilogue,
                         const optional<Tensor>& bias, const optional<Tensor>& aux_in, bool want_aux_out,
                         const optional<Tensor>& out_, bool accumulate, bool out_fp32, int64_t tile_n,
                         int64_t splits, const optional<Tensor>& alpha) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda(), "titb200 gemm: CUDA tensors required");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "titb200 gemm: bf16 operands");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "titb200 gemm: 2-D row-major");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "titb200 gemm: reduction sizes differ: ", K, " vs ", Kb);
  Tensor out;
  if (out_.has_value() && out_->defined()) {
    out = *out_;
    TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.stride(1) == 1, "titb200 gemm: bad out");
    out_fp32 = out.scalar_type() == at::kFloat;
    TORCH_CHECK(out_fp32 || out.scalar_type() == at::kBFloat16, "titb200 gemm: out must be fp32 or bf16");
  } else {
    out = at::empty({M, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
    accumulate = false;
  }
  Tensor aux_out;
  if (want_aux_out) aux_out = at::empty({M, N}, a.options());

  TitbGemmDesc d{};
  d.a = a.data_ptr(); d.b = b.data_ptr(); d.out = out.data_ptr();
  d.M = (int)M; d.N = (int)N; d.K = (int)K;
  d.a_mn_major = a_mn; d.b_mn_major = b_mn;
  d.lda = a.stride(0); d.ldb = b.stride(0); d.ldo = out.stride(0);
  d.out_fp32 = out_fp32; d.accumulate = accumulate; d.epilogue = (int)epilogue;
  d.bias = opt_ptr(bias);
  if (bias.has_value() && bias->defined())
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N, "titb200 gemm: bias must be bf16 [N]");
  if (aux_in.has_value() && aux_in->defined()) {
    TORCH_CHECK(aux_in->scalar_type() == at::kBFloat16 && aux_in->dim() == 2 && aux_in->size(0) == M &&
                    aux_in->size(1) == N && aux_in->stride(1) == 1, "titb200 gemm: aux_in must be bf16 [M,N]");
    d.aux_in = aux_in->data_ptr(); d.ld_aux_in = aux_in->stride(0);
  }
  if (want_aux_out) { d.aux_out = aux_out.data_ptr(); d.ld_aux_out = N; }
  d.tile_n = (int)tile_n;
  if (alpha.has_value() && alpha->defined()) {
    TORCH_CHECK(alpha->is_cuda() && alpha->scalar_type() == at::kFloat && alpha->numel() == 1, "titb200 gemm: alpha must be a CUDA fp32 scalar");
    d.alpha = alpha->data_ptr();
  }
  int s = splits > 0 ? (int)splits : titb_gemm_pick_splits((int)M, (int)N, (int)K);
  if (epilogue != TITB_EPI_NONE || (N & 3)) s = 1;
  // bf16 outputs go through an fp32 workspace and a reduction kernel: worth it only for very long reductions
  // (the vocabulary projection's input gradient, K = 50304)
  if (s > 1 && splits <= 0 && !out_fp32 && K < 16384) s = 1;
  Tensor ws;
  if (s > 1 && !titb_gemm_split_in_place(&d)) {
    ws = at::empty({s, M, N}, a.options().dtype(at::kFloat));
    d.workspace = ws.data_ptr();
  }
  d.splits = s;
  CHECK_RC(titb_gemm_bf16(&d, cur_stream()), "gemm_bf16", (s > 1 && ws.defined()) ? 2 : 1);
  if (want_aux_out) return {out, aux_out};
  return {out};
}

// all-gather -> GEMM.  `peer_ptrs`: every rank's [Ms, K] bf16 shard (symmetric memory, already
// separated from its writers by a cross-GPU barrier).  Returns {Y [M, N] (, pre-activation), X [M, K]}.
std::vector<Tensor> gemm_ag(const std::vector<int64_t>& peer_ptrs, int64_t rank, int64_t rows_per_rank, int64_t K,
                            const Tensor& b, bool b_mn, int64_t epilogue, const optional<Tensor>& bias,
                            bool want_aux_out, int64_t helper_ctas) {
  TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kBFloat16 && b.dim() == 2 && b.stride(1) == 1);
  c10::cuda::CUDAGuard guard(b.device());
  const int64_t world = (int64_t)peer_ptrs.size(), M = rows_per_rank * world;
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "titb200 gemm_ag: reduction sizes differ");
  Tensor X = at::empty({M, K}, b.options());
  Tensor flags = at::empty({M / 128 + 1}, b.options().dtype(at::kInt));
  Tensor out = at::empty({M, N}, b.options());
  Tensor aux_out;
  if (want_aux_out) aux_out = at::empty({M, N}, b.options());
  std::vector<unsigned long long> pp(peer_ptrs.begin(), peer_ptrs.end());
  TitbGemmColl c{};
  c.mode = 1; c.world = (int)world; c.rank = (int)rank; c.helper_ctas = (int)helper_ctas;
  c.rows_per_rank = (int)rows_per_rank; c.peer_ptrs = pp.data(); c.gathered = X.data_ptr(); c.flags = flags.data_ptr();
  TitbGemmDesc d{};
  d.a = X.data_ptr(); d.b = b.data_ptr(); d.out = out.data_ptr();
  d.M = (int)M; d.N = (int)N; d.K = (int)K; d.a_mn_major = 0; d.b_mn_major = b_mn;
  d.lda = K; d.ldb = b.stride(0); d.ldo = N; d.epilogue = (int)epilogue; d.bias = opt_ptr(bias);
  if (want_aux_out) { d.aux_out = aux_out.data_ptr(); d.ld_aux_out = N; }
  d.splits = 1; d.coll = &c;
  CHECK_RC(titb_gemm_bf16(&d, cur_stream()), "gemm_ag");
  if (want_aux_out) return {out, aux_out, X};
  return {out, X};
}

// Parameter all-gather -> GEMM.  `w`: this rank's full-size [N, K] copy of the weight (rows it does not own are
// overwritten by the kernel); `peer_ptrs[r]`: address of the first row rank r owns, in r's memory.  Returns
// {Y [M, N] (, pre-activation)}.
std::vector<Tensor> gemm_param_gather(const Tensor& x, const Tensor& w, const std::vector<int64_t>& peer_ptrs, int64_t rank,
                                      int64_t epilogue, const optional<Tensor>& bias, const optional<Tensor>& aux_in,
                                      bool want_aux_out, int64_t helper_ctas, int64_t tile_n) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1);
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t world = (int64_t)peer_ptrs.size(), M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "titb200 gemm_param_gather: reduction sizes differ");
  TORCH_CHECK(world >= 1 && N % (128 * world) == 0, "titb200 gemm_param_gather: weight rows must split into 128-row chunks per rank");
  Tensor flags = at::empty({N / 128 + 1}, x.options().dtype(at::kInt));
  Tensor out = at::empty({M, N}, x.options());
  Tensor aux_out;
  if (want_aux_out) aux_out = at::empty({M, N}, x.options());
  std::vector<unsigned long long> pp(peer_ptrs.begin(), peer_ptrs.end());
  TitbGemmColl c{};
  c.mode = 3; c.world = (int)world; c.rank = (int)rank; c.helper_ctas = (int)helper_ctas;
  c.rows_per_rank = (int)(N / world); c.peer_ptrs = pp.data(); c.gathered = w.data_ptr(); c.flags = flags.data_ptr();
  TitbGemmDesc d{};
  d.a = x.data_ptr(); d.b = w.data_ptr(); d.out = out.data_ptr();
  d.M = (int)M; d.N = (int)N; d.K = (int)K; d.a_mn_major = 0; d.b_mn_major = 0;
  d.lda = x.stride(0); d.ldb = K; d.ldo = N; d.epilogue = (int)epilogue; d.bias = opt_ptr(bias);
  if (aux_in.has_value() && aux_in->defined()) {
    TORCH_CHECK(aux_in->dim() == 2 && aux_in->size(0) == M && aux_in->size(1) == N && aux_in->stride(1) == 1);
    d.aux_in = aux_in->data_ptr(); d.ld_aux_in = aux_in->stride(0);
  }
  if (want_aux_out) { d.aux_out = aux_out.data_ptr(); d.ld_aux_out = N; }
  d.splits = 1; d.tile_n = (int)tile_n; d.coll = &c;
  if (d.tile_n == 0) d.tile_n = (N / world) % 256 == 0 ? 256 : 128;   // a B tile never straddles two owners
  CHECK_RC(titb_gemm_param_gather_bf16(&d, cur_stream()), "gemm_param_gather");
  if (want_aux_out) return {out, aux_out};
  return {out};
}

// GEMM -> reduce-scatter.  `recv_ptrs`: every rank's receive buffer bf16 [world][Ms][N]; `cnt_ptrs`:
// every rank's uint32 [Ms/128] counters.  Returns this rank's [Ms, N] rows of sum_r (a_r . b_r^T).
Tensor gemm_rs(const Tensor& a, const Tensor& b, bool b_mn, const std::vector<int64_t>& recv_ptrs,
               const std::vector<int64_t>& cnt_ptrs, int64_t rank, const optional<Tensor>& bias,
               const optional<Tensor>& residual, int64_t helper_ctas) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && a.dim() == 2 && a.stride(1) == 1);
  TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kBFloat16 && b.dim() == 2 && b.stride(1) == 1);
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t world = (int64_t)recv_ptrs.size(), M = a.size(0), K = a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "titb200 gemm_rs: reduction sizes differ");
  TORCH_CHECK(M % world == 0, "titb200 gemm_rs: rows not divisible by the group size");
  const int64_t Ms = M / world;
  Tensor out = at::empty({Ms, N}, a.options());
  std::vector<unsigned long long> rp(recv_ptrs.begin(), recv_ptrs.end()), cp(cnt_ptrs.begin(), cnt_ptrs.end());
  TitbGemmColl c{};
  c.mode = 2; c.world = (int)world; c.rank = (int)rank; c.helper_ctas = (int)helper_ctas; c.rows_per_rank = (int)Ms;
  c.peer_ptrs = rp.data(); c.cnt_ptrs = cp.data(); c.flags = reinterpret_cast<void*>(cp[rank]);
  c.rs_out = out.data_ptr(); c.rs_bias = opt_ptr(bias);
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->is_contiguous() && residual->numel() == Ms * N, "titb200 gemm_rs: residual must be [Ms, N]");
    c.rs_residual = residual->data_ptr();
  }
  TitbGemmDesc d{};
  d.a = a.data_ptr(); d.b = b.data_ptr(); d.out = out.data_ptr();
  d.M = (int)M; d.N = (int)N; d.K = (int)K; d.a_mn_major = 0; d.b_mn_major = b_mn;
  d.lda = a.stride(0); d.ldb = b.stride(0); d.ldo = N; d.splits = 1; d.coll = &c;
  CHECK_RC(titb_gemm_bf16(&d, cur_stream()), "gemm_rs");
  return out;
}

Tensor sgemm(const Tensor& a, const Tensor& b, bool ta, bool tb, const optional<Tensor>& out_, bool accumulate) {
  check_cuda(a, "a"); check_cuda(b, "b");
  TORCH_CHECK(a.scalar_type() == at::kFloat && b.scalar_type() == at::kFloat && a.dim() == 2 && b.dim() == 2);
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = ta ? a.size(1) : a.size(0), K = ta ? a.size(0) : a.size(1);
  const int64_t N = tb ? b.size(0) : b.size(1);
  TORCH_CHECK((tb ? b.size(1) : b.size(0)) == K, "titb200 sgemm: reduction sizes differ");
  Tensor out = (out_.has_value() && out_->defined()) ? *out_ : at::empty({M, N}, a.options());
  if (!(out_.has_value() && out_->defined())) accumulate = false;
  CHECK_RC(titb_sgemm(a.data_ptr<float>(), b.data_ptr<float>(), out.data_ptr<float>(), (int)M, (int)N, (int)K, ta, tb,
                      accumulate, cur_stream()), "sgemm");
  return out;
}

// ---------------------------------------------------------------------- norms
// `out`: where the normalised rows go (same shape and dtype as x, contiguous); a caller that feeds the result to a
// collective passes a view of its symmetric buffer here, which saves the staging copy.
static Tensor norm_out(const Tensor& x, const c10::optional<Tensor>& out) {
  if (!out.has_value()) return at::empty_like(x);
  TORCH_CHECK(out->is_cuda() && out->is_contiguous() && out->scalar_type() == x.scalar_type() &&
              out->numel() == x.numel(), "norm: out must be a contiguous CUDA tensor of x's size and dtype");
  return out->detach();   // a fresh handle on the same memory, so autograd metadata never lands on the caller's tensor
}
std::vector<Tensor> layernorm_fwd(const Tensor& x, const Tensor& w, const Tensor& b, double eps,
                                  const c10::optional<Tensor>& out) {
  check_cuda(x, "x"); check_cuda(w, "weight"); check_cuda(b, "bias");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t C = x.size(-1), rows = x.numel() / C;
  Tensor y = norm_out(x, out);
  Tensor mean = at::empty({rows}, x.options().dtype(at::kFloat)), rstd = at::empty_like(mean);
  CHECK_RC(titb_layernorm_fwd(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr<float>(),
                              rstd.data_ptr<float>(), rows, (int)C, (float)eps, dt_code(x), cur_stream()),
           "layernorm_fwd");
  return {y, mean, rstd};
}
// dw/db are written (or accumulated) into fp32 tensors supplied by the caller, or fresh ones.
// `dres`: gradient arriving through a residual connection around the norm, added to dx inside the kernel.
std::vector<Tensor> layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& mean,
                                  const Tensor& rstd, const optional<Tensor>& dw_, const optional<Tensor>& db_,
                                  bool accumulate, const optional<Tensor>& dres_) {
  check_cuda(dy, "dy"); check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t C = x.size(-1), rows = x.numel() / C;
  Tensor dx = at::empty_like(x);
  auto fopt = x.options().dtype(at::kFloat);
  const bool have = dw_.has_value() && dw_->defined();
  Tensor dw = have ? *dw_ : at::empty({C}, fopt);
  Tensor db = (db_.has_value() && db_->defined()) ? *db_ : at::empty({C}, fopt);
  TORCH_CHECK(dw.scalar_type() == at::kFloat && db.scalar_type() == at::kFloat, "titb200: fp32 weight grads");
  const bool have_res = dres_.has_value() && dres_->defined();
  Tensor dres;
  if (have_res) {
    dres = dres_->contiguous();
    TORCH_CHECK(dres.sizes() == x.sizes() && dres.scalar_type() == x.scalar_type(), "titb200: dres must match x");
  }
  Tensor scratch = at::empty({2, titb_layernorm_bwd_blocks(rows), C}, fopt);
  CHECK_RC(titb_layernorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr<float>(),
                              rstd.data_ptr<float>(), dx.data_ptr(), dw.data_ptr<float>(), db.data_ptr<float>(),
                              scratch.data_ptr<float>(), rows, (int)C, dt_code(x), have && accumulate,
                              have_res ? dres.data_ptr() : nullptr, cur_stream()),
           "layernorm_bwd", 2);
  return {dx, dw, db};
}
std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps, const c10::optional<Tensor>& out) {
  check_cuda(x, "x"); check_cuda(w, "weight");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t C = x.size(-1), rows = x.numel() / C;
  Tensor y = norm_out(x, out);
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  CHECK_RC(titb_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, (int)C,
                            (float)eps, dt_code(x), cur_stream()), "rmsnorm_fwd");
  return {y, rstd};
}
std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd,
                                const optional<Tensor>& dw_, bool accumulate, const optional<Tensor>& dres_) {
  check_cuda(dy, "dy"); check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t C = x.size(-1), rows = x.numel() / C;
  Tensor dx = at::empty_like(x);
  auto fopt = x.options().dtype(at::kFloat);
  const bool have = dw_.has_value() && dw_->defined();
  Tensor dw = have ? *dw_ : at::empty({C}, fopt);
  const bool have_res = dres_.has_value() && dres_->defined();
  Tensor dres;
  if (have_res) {
    dres = dres_->contiguous();
    TORCH_CHECK(dres.sizes() == x.sizes() && dres.scalar_type() == x.scalar_type(), "titb200: dres must match x");
  }
  Tensor scratch = at::empty({2, titb_layernorm_bwd_blocks(rows), C}, fopt);
  CHECK_RC(titb_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                            dw.data_ptr<float>(), scratch.data_ptr<float>(), rows, (int)C, dt_code(x),
                            have && accumulate, have_res ? dres.data_ptr() : nullptr, cur_stream()), "rmsnorm_bwd", 2);
  return {dx, dw};
}

// ---------------------------------------------------------------- activations
Tensor gelu_fwd(const Tensor& x) {
  check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  CHECK_RC(titb_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), dt_code(x), cur_stream()), "gelu_fwd");
  return y;
}
Tensor gelu_bwd(const Tensor& dy, const Tensor& x) {
  check_cuda(x, "x"); check_cuda(dy, "dy");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = at::empty_like(x);
  CHECK_RC(titb_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), dt_code(x), cur_stream()), "gelu_bwd");
  return dx;
}
Tensor swiglu_fwd(const Tensor& x) {
  check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t F = x.size(-1) / 2, rows = x.numel() / (2 * F);
  auto sizes = x.sizes().vec();
  sizes.back() = F;
  Tensor y = at::empty(sizes, x.options());
  CHECK_RC(titb_swiglu_fwd(x.data_ptr(), y.data_ptr(), rows, (int)F, dt_code(x), cur_stream()), "swiglu_fwd");
  return y;
}
Tensor swiglu_bwd(const Tensor& dy, const Tensor& x) {
  check_cuda(x, "x"); check_cuda(dy, "dy");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t F = x.size(-1) / 2, rows = x.numel() / (2 * F);
  Tensor dx = at::empty_like(x);
  CHECK_RC(titb_swiglu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), rows, (int)F, dt_code(x), cur_stream()),
           "swiglu_bwd");
  return dx;
}
// x: [B, T, H, hd] contiguous.
Tensor rope(const Tensor& x, int64_t pos_offset, double theta, bool inverse, bool inplace) {
  check_cuda(x, "x");
  TORCH_CHECK(x.dim() == 4, "titb200 rope: expects [B, T, H, hd]");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = inplace ? x : at::empty_like(x);
  CHECK_RC(titb_rope(x.data_ptr(), y.data_ptr(), (int)x.size(0), (int)x.size(1), (int)x.size(2), (int)x.size(3),
                     (int)pos_offset, (float)theta, inverse, dt_code(x), cur_stream()), "rope");
  return y;
}

// In-place rotary embedding on the first `n_heads` heads of a fused [B, T, W] projection buffer.
void rope_qkv_(const Tensor& qkv, int64_t n_heads, int64_t hd, int64_t pos_offset, double theta, bool inverse) {
  check_cuda(qkv, "qkv");
  TORCH_CHECK(qkv.dim() == 3 && n_heads * hd <= qkv.size(2), "titb200 rope_qkv_: expects [B, T, W] with W >= heads*hd");
  c10::cuda::CUDAGuard guard(qkv.device());
  CHECK_RC(titb_rope_strided(qkv.data_ptr(), qkv.data_ptr(), (int)qkv.size(0), (int)qkv.size(1), (int)n_heads, (int)hd,
                             qkv.size(2), (int)pos_offset, (float)theta, inverse, dt_code(qkv), cur_stream()),
           "rope_strided");
}

// ------------------------------------------------------------------ embedding
Tensor embedding_fwd(const Tensor& idx, const Tensor& wte, const optional<Tensor>& wpe, int64_t pos_offset) {
  check_cuda(idx, "idx"); check_cuda(wte, "wte");
  TORCH_CHECK(idx.scalar_type() == at::kLong, "titb200 embedding: indices must be int64");
  c10::cuda::CUDAGuard guard(wte.device());
  const int64_t C = wte.size(1), BT = idx.numel(), T = idx.dim() >= 1 ? idx.size(-1) : 1;
  auto sizes = idx.sizes().vec();
  sizes.push_back(C);
  Tensor out = at::empty(sizes, wte.options());
  CHECK_RC(titb_embedding_fwd(idx.data_ptr<int64_t>() ? (const long long*)idx.data_ptr<int64_t>() : nullptr,
                              wte.data_ptr(), opt_ptr(wpe), out.data_ptr(), BT, (int)T, (int)C, (int)pos_offset,
                              dt_code(wte), cur_stream()), "embedding_fwd");
  return out;
}
void embedding_bwd(const Tensor& idx, const Tensor& dout, const optional<Tensor>& dwte, const optional<Tensor>& dwpe,
                   int64_t vocab_lo, int64_t vocab_hi, bool deterministic) {
  check_cuda(idx, "idx"); check_cuda(dout, "dout");
  c10::cuda::CUDAGuard guard(dout.device());
  const int64_t C = dout.size(-1), BT = idx.numel(), T = idx.size(-1);
  float* pw = dwte.has_value() && dwte->defined() ? dwte->data_ptr<float>() : nullptr;
  float* pp = dwpe.has_value() && dwpe->defined() ? dwpe->data_ptr<float>() : nullptr;
  if (deterministic && pw != nullptr && BT <= titb_embedding_sorted_max_tokens()) {
    // sorted segment reduce for the token rows (no atomics); the position rows are a fixed-order sum already
    int64_t npad = 2;
    while (npad < BT) npad <<= 1;
    Tensor keys = at::empty({npad}, idx.options().dtype(at::kLong));
    CHECK_RC(titb_embedding_bwd_wte_sorted((const long long*)idx.data_ptr<int64_t>(), dout.data_ptr(), pw, BT, (int)C,
                                           (int)vocab_lo, (int)std::min<int64_t>(vocab_hi, INT32_MAX), dt_code(dout),
                                           reinterpret_cast<unsigned long long*>(keys.data_ptr<int64_t>()), cur_stream()),
             "embedding_bwd_wte_sorted", 2);
    pw = nullptr;
    if (pp == nullptr) return;
  }
  CHECK_RC(titb_embedding_bwd((const long long*)idx.data_ptr<int64_t>(), dout.data_ptr(), pw, pp, BT, (int)T, (int)C,
                              (int)vocab_lo, (int)std::min<int64_t>(vocab_hi, INT32_MAX), dt_code(dout), cur_stream()),
           "embedding_bwd");
}
// Vocabulary-parallel table, forward: rows of `w` (this rank's slice [vocab_lo, vocab_lo + w.size(0))) go to the
// [Ms, C] token-shard buffers behind dst_ptrs (one address per rank).  Barriers are the caller's.
void embedding_vp_push(const Tensor& idx, const Tensor& w, const std::vector<int64_t>& dst_ptrs, int64_t rows_per_rank,
                       int64_t vocab_lo, int64_t vocab_total, bool zero_strays) {
  check_cuda(idx, "idx"); check_cuda(w, "weight");
  TORCH_CHECK(idx.scalar_type() == at::kLong && idx.is_contiguous() && w.is_contiguous() && w.dim() == 2);
  c10::cuda::CUDAGuard guard(w.device());
  std::vector<unsigned long long> d(dst_ptrs.begin(), dst_ptrs.end());
  CHECK_RC(titb_embedding_vp_push((const long long*)idx.data_ptr<int64_t>(), w.data_ptr(), d.data(), (int)d.size(),
                                  idx.numel(), rows_per_rank, (int)w.size(1), vocab_lo, vocab_lo + w.size(0),
                                  vocab_total, zero_strays ? 1 : 0, dt_code(w), cur_stream()), "embedding_vp_push");
}
// Backward: gradient rows of the ids in this rank's slice, pulled from the token owners' [Ms, C] buffers (dtype of
// `like`) and added to dw (fp32 [rows of the slice, C]).
void embedding_vp_pull_bwd(const Tensor& idx, const std::vector<int64_t>& src_ptrs, const Tensor& dw,
                           int64_t rows_per_rank, int64_t vocab_lo, const Tensor& like) {
  check_cuda(idx, "idx"); check_cuda(dw, "dw");
  TORCH_CHECK(idx.scalar_type() == at::kLong && idx.is_contiguous() && dw.scalar_type() == at::kFloat &&
              dw.is_contiguous() && dw.dim() == 2);
  c10::cuda::CUDAGuard guard(dw.device());
  std::vector<unsigned long long> s(src_ptrs.begin(), src_ptrs.end());
  CHECK_RC(titb_embedding_vp_pull_bwd((const long long*)idx.data_ptr<int64_t>(), s.data(), (int)s.size(),
                                      dw.data_ptr<float>(), idx.numel(), rows_per_rank, (int)dw.size(1), vocab_lo,
                                      vocab_lo + dw.size(0), dt_code(like), cur_stream()), "embedding_vp_pull_bwd");
}

// ------------------------------------------------------- softmax / cross entropy
Tensor softmax_fwd(const Tensor& x, int64_t dim) {
  check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  dim = at::maybe_wrap_dim(dim, x.dim());
  int64_t outer = 1, inner = 1;
  for (int64_t i = 0; i < dim; ++i) outer *= x.size(i);
  for (int64_t i = dim + 1; i < x.dim(); ++i) inner *= x.size(i);
  Tensor y = at::empty_like(x);
  CHECK_RC(titb_softmax_fwd(x.data_ptr(), y.data_ptr(), outer, (int)x.size(dim), inner, dt_code(x), cur_stream()),
           "softmax_fwd");
  return y;
}
Tensor softmax_bwd(const Tensor& dy, const Tensor& y, int64_t dim) {
  check_cuda(dy, "dy"); check_cuda(y, "y");
  c10::cuda::CUDAGuard guard(y.device());
  dim = at::maybe_wrap_dim(dim, y.dim());
  int64_t outer = 1, inner = 1;
  for (int64_t i = 0; i < dim; ++i) outer *= y.size(i);
  for (int64_t i = dim + 1; i < y.dim(); ++i) inner *= y.size(i);
  Tensor dx = at::empty_like(y);
  CHECK_RC(titb_softmax_bwd(dy.data_ptr(), y.data_ptr(), dx.data_ptr(), outer, (int)y.size(dim), inner, dt_code(y),
                            cur_stream()), "softmax_bwd");
  return dx;
}
// logits: [rows, ld] (last dim may be padded beyond V).  Returns the mean loss (0-d fp32);
// when write_grad the gradient scaled by grad_scale overwrites `logits`.
Tensor xent_fused(const Tensor& logits, const Tensor& targets, int64_t V, double grad_scale, bool write_grad,
                  double mean_scale) {
  check_cuda(logits, "logits"); check_cuda(targets, "targets");
  TORCH_CHECK(targets.scalar_type() == at::kLong, "titb200 cross entropy: targets must be int64");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t ld = logits.size(-1), rows = logits.numel() / ld;
  TORCH_CHECK(targets.numel() == rows, "titb200 cross entropy: one target per row");
  Tensor losses = at::empty({rows}, logits.options().dtype(at::kFloat));
  CHECK_RC(titb_xent_fwd_bwd(logits.data_ptr(), (const long long*)targets.data_ptr<int64_t>(),
                             losses.data_ptr<float>(), write_grad ? logits.data_ptr() : nullptr, rows, (int)V, ld,
                             (float)grad_scale, dt_code(logits), cur_stream()), "xent_fwd_bwd");
  Tensor loss = at::empty({}, losses.options());
  CHECK_RC(titb_mean(losses.data_ptr<float>(), loss.data_ptr<float>(), rows, (float)mean_scale, cur_stream()), "mean");
  return loss;
}
Tensor xent_bwd(const Tensor& logits, const Tensor& targets, const Tensor& upstream, int64_t V, double grad_scale,
                bool inplace) {
  check_cuda(logits, "logits");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t ld = logits.size(-1), rows = logits.numel() / ld;
  Tensor up = upstream.to(at::kFloat).contiguous();
  Tensor d = inplace ? logits : at::empty_like(logits);
  CHECK_RC(titb_xent_bwd(logits.data_ptr(), (const long long*)targets.data_ptr<int64_t>(), d.data_ptr(),
                         up.data_ptr<float>(), rows, (int)V, ld, (float)grad_scale, dt_code(logits), cur_stream()),
           "xent_bwd");
  return d;
}

// Vocabulary-parallel cross entropy, pass 1: (max, sum-exp, target logit) of every row of this rank's logits slice,
// written to slot `rank` of the [world, rows, 3] fp32 table behind every address in dst_ptrs.
void xent_vp_stats(const Tensor& logits, const Tensor& targets, const std::vector<int64_t>& dst_ptrs, int64_t rank,
                   int64_t vocab_lo, int64_t vocab_size) {
  check_cuda(logits, "logits"); check_cuda(targets, "targets");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && logits.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t ld = logits.size(-1), rows = logits.numel() / ld;
  TORCH_CHECK(targets.numel() == rows, "titb200 cross entropy: one target per row");
  std::vector<unsigned long long> d(dst_ptrs.begin(), dst_ptrs.end());
  CHECK_RC(titb_xent_vp_stats(logits.data_ptr(), (const long long*)targets.data_ptr<int64_t>(), d.data(), (int)d.size(),
                              (int)rank, rows, ld, ld, vocab_lo, vocab_size, dt_code(logits), cur_stream()),
           "xent_vp_stats");
}
// Pass 2: per-row losses from the complete table; the slice is overwritten with grad_scale * (softmax - onehot).
Tensor xent_vp_grad(const Tensor& logits, const Tensor& targets, const Tensor& stats, int64_t vocab_lo,
                    int64_t vocab_size, double grad_scale) {
  check_cuda(logits, "logits"); check_cuda(stats, "stats");
  TORCH_CHECK(stats.scalar_type() == at::kFloat && stats.is_contiguous() && stats.dim() == 3 && stats.size(2) == 3);
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && logits.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t ld = logits.size(-1), rows = logits.numel() / ld;
  TORCH_CHECK(stats.size(1) == rows, "titb200 cross entropy: statistics table has the wrong number of rows");
  Tensor losses = at::empty({rows}, logits.options().dtype(at::kFloat));
  CHECK_RC(titb_xent_vp_grad(logits.data_ptr(), (const long long*)targets.data_ptr<int64_t>(), stats.data_ptr<float>(),
                             (int)stats.size(0), losses.data_ptr<float>(), rows, ld, ld, vocab_lo, vocab_size,
                             (float)grad_scale, dt_code(logits), cur_stream()), "xent_vp_grad");
  return losses;
}

// ------------------------------------------------------------------ optimizers
void adam_flat(const Tensor& master, const optional<Tensor>& lp, const Tensor& grad, const Tensor& m, const Tensor& v,
               double lr, double b1, double b2, double eps, double wd, int64_t step, double grad_scale,
               const optional<Tensor>& dev_state) {
  check_cuda(master, "master"); check_cuda(grad, "grad");
  TORCH_CHECK(master.scalar_type() == at::kFloat && grad.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat &&
              v.scalar_type() == at::kFloat, "titb200 adam: fp32 state");
  c10::cuda::CUDAGuard guard(master.device());
  const int64_t n = master.numel();
  TORCH_CHECK(grad.numel() == n && m.numel() == n && v.numel() == n, "titb200 adam: size mismatch");
  const double bc1 = 1.0 - std::pow(b1, (double)step), bc2 = 1.0 - std::pow(b2, (double)step);
  void* lpp = nullptr; int lpd = 0;
  if (lp.has_value() && lp->defined()) { TORCH_CHECK(lp->numel() == n); lpp = lp->data_ptr(); lpd = dt_code(*lp); }
  CHECK_RC(titb_adam_flat(master.data_ptr<float>(), lpp, grad.data_ptr<float>(), m.data_ptr<float>(),
                          v.data_ptr<float>(), n, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, (float)bc1,
                          (float)bc2, (float)grad_scale, lpd,
                          dev_state.has_value() && dev_state->defined() ? dev_state->data_ptr<float>() : nullptr,
                          cur_stream()), "adam_flat");
}
void adam_tick(const Tensor& state, double b1, double b2) {
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == at::kFloat && state.numel() >= 4);
  c10::cuda::CUDAGuard guard(state.device());
  CHECK_RC(titb_adam_tick(state.data_ptr<float>(), (float)b1, (float)b2, cur_stream()), "adam_tick");
}
void sgd_flat(const Tensor& master, const optional<Tensor>& lp, const Tensor& grad, double lr) {
  check_cuda(master, "master"); check_cuda(grad, "grad");
  c10::cuda::CUDAGuard guard(master.device());
  void* lpp = nullptr; int lpd = 0;
  if (lp.has_value() && lp->defined()) { lpp = lp->data_ptr(); lpd = dt_code(*lp); }
  CHECK_RC(titb_sgd_flat(master.data_ptr<float>(), lpp, grad.data_ptr<float>(), master.numel(), (float)lr, lpd,
                         cur_stream()), "sgd_flat");
}
void axpy(const Tensor& y, const Tensor& x, double a) {
  check_cuda(y, "y"); check_cuda(x, "x");
  TORCH_CHECK(y.scalar_type() == at::kFloat && y.numel() == x.numel());
  c10::cuda::CUDAGuard guard(y.device());
  CHECK_RC(titb_axpy(y.data_ptr<float>(), x.data_ptr(), (float)a, y.numel(), dt_code(x), cur_stream()), "axpy");
}

// ----------------------------------------------------------- elementwise family
Tensor unary_fwd(int64_t op, const Tensor& x, double s) {
  check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  CHECK_RC(titb_unary_fwd((int)op, x.data_ptr(), y.data_ptr(), x.numel(), (float)s, dt_code(x), cur_stream()), "unary");
  return y;
}
Tensor unary_bwd(int64_t op, const Tensor& dy, const Tensor& saved, double s) {
  check_cuda(dy, "dy"); check_cuda(saved, "saved");
  c10::cuda::CUDAGuard guard(dy.device());
  Tensor dx = at::empty_like(dy);
  CHECK_RC(titb_unary_bwd((int)op, dy.data_ptr(), saved.data_ptr(), dx.data_ptr(), dy.numel(), (float)s, dt_code(dy),
                          cur_stream()), "unary_bwd");
  return dx;
}
// y = a (op) b with b broadcast to a's shape (right-aligned, one-way).
Tensor binary_fwd(int64_t op, const Tensor& a, const Tensor& b) {
  check_cuda(a, "a"); check_cuda(b, "b");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "titb200 binary: dtype mismatch");
  TORCH_CHECK(a.dim() <= 8 && b.dim() <= a.dim(), "titb200 binary: b must broadcast to a (<= 8 dims)");
  c10::cuda::CUDAGuard guard(a.device());
  TitbBroadcast bc{};
  bc.ndim = (int)a.dim();
  const int64_t off = a.dim() - b.dim();
  int64_t bstride = 1;
  std::vector<int64_t> bs(a.dim(), 0);
  for (int64_t d = a.dim() - 1; d >= 0; --d) {
    bc.a_dims[d] = a.size(d);
    if (d >= off) {
      const int64_t bd = b.size(d - off);
      TORCH_CHECK(bd == a.size(d) || bd == 1, "titb200 binary: cannot broadcast dim ", d);
      bc.b_strides[d] = (bd == 1) ? 0 : bstride;
      bstride *= bd;
    } else {
      bc.b_strides[d] = 0;
    }
  }
  Tensor y = at::empty_like(a);
  CHECK_RC(titb_binary_fwd((int)op, a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), bc, dt_code(a), cur_stream()),
           "binary");
  return y;
}
Tensor cast(const Tensor& x, bool to_bf16) {
  check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty(x.sizes(), x.options().dtype(to_bf16 ? at::kBFloat16 : at::kFloat));
  CHECK_RC(titb_cast(x.data_ptr(), y.data_ptr(), x.numel(), dt_code(x), to_bf16 ? 1 : 0, cur_stream()), "cast");
  return y;
}
void fill_(const Tensor& y, double value) {
  check_cuda(y, "y");
  c10::cuda::CUDAGuard guard(y.device());
  CHECK_RC(titb_fill(y.data_ptr(), y.numel(), (float)value, dt_code(y), cur_stream()), "fill");
}
Tensor transpose_last2(const Tensor& x) {
  check_cuda(x, "x");
  TORCH_CHECK(x.dim() >= 2);
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t R = x.size(-2), C = x.size(-1), batch = x.numel() / (R * C);
  auto sizes = x.sizes().vec();
  std::swap(sizes[sizes.size() - 1], sizes[sizes.size() - 2]);
  Tensor y = at::empty(sizes, x.options());
  CHECK_RC(titb_transpose(x.data_ptr(), y.data_ptr(), batch, (int)R, (int)C, dt_code(x), cur_stream()), "transpose");
  return y;
}
Tensor tri(const Tensor& x, int64_t diagonal, bool upper) {
  check_cuda(x, "x");
  TORCH_CHECK(x.dim() == 2, "titb200 tril/triu: 2-D only");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  CHECK_RC(titb_tri(x.data_ptr(), y.data_ptr(), (int)x.size(0), (int)x.size(1), (int)diagonal, upper, dt_code(x),
                    cur_stream()), "tri");
  return y;
}
// ---------------------------------------------------------------------- reductions / view-like transforms
// x reduced along `dim` (op: 0 sum, 1 mean, 2 max, 3 min); returns {y, idx} (idx defined for max / min only).
std::vector<Tensor> reduce_dim(const Tensor& x_, int64_t op, int64_t dim, bool keepdim) {
  check_cuda(x_, "x");
  c10::cuda::CUDAGuard guard(x_.device());
  Tensor x = x_.contiguous();
  const int64_t nd = x.dim();
  TORCH_CHECK(nd >= 1, "titb200 reduce: needs at least one dimension");
  if (dim < 0) dim += nd;
  TORCH_CHECK(dim >= 0 && dim < nd, "titb200 reduce: dim out of range");
  int64_t outer = 1, inner = 1;
  for (int64_t d = 0; d < dim; ++d) outer *= x.size(d);
  for (int64_t d = dim + 1; d < nd; ++d) inner *= x.size(d);
  auto sizes = x.sizes().vec();
  if (keepdim) sizes[dim] = 1; else sizes.erase(sizes.begin() + dim);
  Tensor y = at::empty(sizes, x.options());
  Tensor idx;
  if (op >= 2) idx = at::empty(sizes, x.options().dtype(at::kLong));
  CHECK_RC(titb_reduce(x.data_ptr(), y.data_ptr(), idx.defined() ? reinterpret_cast<long long*>(idx.data_ptr<int64_t>()) : nullptr,
                       outer, x.size(dim), inner, (int)op, dt_code(x), cur_stream()), "reduce");
  return {y, idx};
}
Tensor reduce_dim_bwd(const Tensor& g_, const optional<Tensor>& idx_, std::vector<int64_t> in_sizes, int64_t dim, double scale) {
  check_cuda(g_, "grad");
  c10::cuda::CUDAGuard guard(g_.device());
  Tensor g = g_.contiguous();
  const int64_t nd = (int64_t)in_sizes.size();
  if (dim < 0) dim += nd;
  int64_t outer = 1, inner = 1;
  for (int64_t d = 0; d < dim; ++d) outer *= in_sizes[d];
  for (int64_t d = dim + 1; d < nd; ++d) inner *= in_sizes[d];
  Tensor dx = at::empty(in_sizes, g.options());
  const bool have = idx_.has_value() && idx_->defined();
  Tensor idx = have ? idx_->contiguous() : Tensor();
  CHECK_RC(titb_reduce_bwd(g.data_ptr(), have ? reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()) : nullptr,
                           dx.data_ptr(), outer, in_sizes[dim], inner, (float)scale, dt_code(g), cur_stream()), "reduce_bwd");
  return dx;
}
// Contiguous copy of the view (sizes, strides, offset -- in elements) of `base`'s storage.
Tensor gather_view(const Tensor& base, std::vector<int64_t> sizes, std::vector<int64_t> strides, int64_t offset) {
  check_cuda(base, "x");
  TORCH_CHECK(sizes.size() == strides.size() && sizes.size() <= 6, "titb200 gather_view: at most 6 dimensions");
  c10::cuda::CUDAGuard guard(base.device());
  Tensor out = at::empty(sizes, base.options());
  std::vector<long long> sz(sizes.begin(), sizes.end()), st(strides.begin(), strides.end());
  CHECK_RC(titb_gather_nd(base.data_ptr(), out.data_ptr(), (int)sz.size(), sz.data(), st.data(), offset,
                          (int)base.element_size(), cur_stream()), "gather_view");
  return out;
}
// Writes (or accumulates) the contiguous `src` into the view (sizes = src.sizes(), strides, offset) of `dst`.
void scatter_view_(const Tensor& dst, const Tensor& src_, std::vector<int64_t> strides, int64_t offset, bool accumulate) {
  check_cuda(dst, "dst"); check_cuda(src_, "src");
  TORCH_CHECK(dst.scalar_type() == src_.scalar_type() && dst.is_contiguous());
  c10::cuda::CUDAGuard guard(dst.device());
  Tensor src = src_.contiguous();
  TORCH_CHECK((size_t)src.dim() == strides.size() && src.dim() <= 6, "titb200 scatter_view: at most 6 dimensions");
  std::vector<long long> sz(src.sizes().begin(), src.sizes().end()), st(strides.begin(), strides.end());
  CHECK_RC(titb_scatter_nd(src.data_ptr(), dst.data_ptr(), (int)sz.size(), sz.data(), st.data(), offset, dt_code(dst),
                           accumulate, cur_stream()), "scatter_view");
}
Tensor mask_fill(const Tensor& x_, const Tensor& mask_, double value, bool backward) {
  check_cuda(x_, "x"); check_cuda(mask_, "mask");
  c10::cuda::CUDAGuard guard(x_.device());
  Tensor x = x_.contiguous(), mask = mask_.contiguous();
  int mdt;
  if (mask.scalar_type() == at::kFloat) mdt = 0;
  else if (mask.scalar_type() == at::kBFloat16) mdt = 1;
  else if (mask.scalar_type() == at::kBool || mask.scalar_type() == at::kByte) mdt = 2;
  else TORCH_CHECK(false, "titb200 mask_fill: mask must be float32, bfloat16, bool or uint8");
  TORCH_CHECK(mask.numel() > 0 && x.numel() % mask.numel() == 0, "titb200 mask_fill: mask must tile the trailing dims");
  Tensor y = at::empty_like(x);
  CHECK_RC(titb_mask_fill(x.data_ptr(), mask.data_ptr(), y.data_ptr(), x.numel(), mask.numel(), (float)value, backward,
                          dt_code(x), mdt, cur_stream()), "mask_fill");
  return y;
}
Tensor outer_fwd(const Tensor& a_, const Tensor& b_) {
  check_cuda(a_, "a"); check_cuda(b_, "b");
  TORCH_CHECK(a_.dim() == 1 && b_.dim() == 1 && a_.scalar_type() == b_.scalar_type());
  c10::cuda::CUDAGuard guard(a_.device());
  Tensor a = a_.contiguous(), b = b_.contiguous();
  Tensor y = at::empty({a.numel(), b.numel()}, a.options());
  CHECK_RC(titb_outer(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), b.numel(), dt_code(a), cur_stream()), "outer");
  return y;
}
std::vector<Tensor> outer_bwd(const Tensor& g_, const Tensor& a_, const Tensor& b_) {
  check_cuda(g_, "grad");
  c10::cuda::CUDAGuard guard(g_.device());
  Tensor g = g_.contiguous(), a = a_.contiguous(), b = b_.contiguous();
  Tensor da = at::empty_like(a), db = at::empty_like(b);
  CHECK_RC(titb_outer_bwd(g.data_ptr(), a.data_ptr(), b.data_ptr(), da.data_ptr(), db.data_ptr(), a.numel(), b.numel(),
                          dt_code(g), cur_stream()), "outer_bwd", 2);
  return {da, db};
}

// Column sums of a [rows, C] view into an fp32 [C] tensor (bias gradients).
Tensor colsum(const Tensor& x, const optional<Tensor>& out_, bool accumulate) {
  check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t C = x.size(-1), rows = x.numel() / C;
  auto fopt = x.options().dtype(at::kFloat);
  const bool have = out_.has_value() && out_->defined();
  Tensor out = have ? *out_ : at::empty({C}, fopt);
  Tensor scratch = at::empty({titb_colsum_blocks(rows), C}, fopt);
  CHECK_RC(titb_colsum(x.data_ptr(), out.data_ptr<float>(), rows, (int)C, dt_code(x), have && accumulate,
                       scratch.data_ptr<float>(), cur_stream()), "colsum", 2);
  return out;
}

int64_t status_read(bool clear) { return titb_status_read(clear, cur_stream()); }

}  // namespace

void bind_attention(pybind11::module_& m);
void bind_comm(pybind11::module_& m);
void bind_core(pybind11::module_& m);
void bind_symm(pybind11::module_& m);

PYBIND11_MODULE(_C, m) {
  m.doc() = "tinyinfinitrain_b200 native ops (sm_100a)";
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("a_mn") = false, py::arg("b_mn") = false,
        py::arg("epilogue") = 0, py::arg("bias") = py::none(), py::arg("aux_in") = py::none(),
        py::arg("want_aux_out") = false, py::arg("out") = py::none(), py::arg("accumulate") = false,
        py::arg("out_fp32") = false, py::arg("tile_n") = 0, py::arg("splits") = 0, py::arg("alpha") = py::none());
  m.def("gemm_ag", &gemm_ag, py::arg("peer_ptrs"), py::arg("rank"), py::arg("rows_per_rank"), py::arg("K"),
        py::arg("b"), py::arg("b_mn") = false, py::arg("epilogue") = 0, py::arg("bias") = py::none(),
        py::arg("want_aux_out") = false, py::arg("helper_ctas") = 16);
  m.def("gemm_param_gather", &gemm_param_gather, py::arg("x"), py::arg("w"), py::arg("peer_ptrs"), py::arg("rank"),
        py::arg("epilogue") = 0, py::arg("bias") = py::none(), py::arg("aux_in") = py::none(),
        py::arg("want_aux_out") = false, py::arg("helper_ctas") = 8, py::arg("tile_n") = 0);
  m.def("gemm_rs", &gemm_rs, py::arg("a"), py::arg("b"), py::arg("b_mn"), py::arg("recv_ptrs"), py::arg("cnt_ptrs"),
        py::arg("rank"), py::arg("bias") = py::none(), py::arg("residual") = py::none(), py::arg("helper_ctas") = 8);
  m.def("reduce_dim", &reduce_dim, py::arg("x"), py::arg("op"), py::arg("dim"), py::arg("keepdim") = false);
  m.def("reduce_dim_bwd", &reduce_dim_bwd, py::arg("g"), py::arg("idx"), py::arg("in_sizes"), py::arg("dim"),
        py::arg("scale") = 1.0);
  m.def("gather_view", &gather_view);
  m.def("scatter_view_", &scatter_view_, py::arg("dst"), py::arg("src"), py::arg("strides"), py::arg("offset"),
        py::arg("accumulate") = false);
  m.def("mask_fill", &mask_fill, py::arg("x"), py::arg("mask"), py::arg("value"), py::arg("backward") = false);
  m.def("outer_fwd", &outer_fwd);
  m.def("outer_bwd", &outer_bwd);
  m.def("sgemm", &sgemm, py::arg("a"), py::arg("b"), py::arg("ta") = false, py::arg("tb") = false,
        py::arg("out") = py::none(), py::arg("accumulate") = false);
  m.def("layernorm_fwd", &layernorm_fwd, py::arg("x"), py::arg("weight"), py::arg("bias"), py::arg("eps"),
        py::arg("out") = py::none());
  m.def("layernorm_bwd", &layernorm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("mean"), py::arg("rstd"),
        py::arg("dw") = py::none(), py::arg("db") = py::none(), py::arg("accumulate") = false,
        py::arg("dres") = py::none());
  m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("weight"), py::arg("eps"), py::arg("out") = py::none());
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("rstd"),
        py::arg("dw") = py::none(), py::arg("accumulate") = false,
        py::arg("dres") = py::none());
  m.def("gelu_fwd", &gelu_fwd);
  m.def("gelu_bwd", &gelu_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("rope", &rope, py::arg("x"), py::arg("pos_offset") = 0, py::arg("theta") = 10000.0, py::arg("inverse") = false,
        py::arg("inplace") = false);
  m.def("rope_qkv_", &rope_qkv_);
  m.def("embedding_fwd", &embedding_fwd, py::arg("idx"), py::arg("wte"), py::arg("wpe") = py::none(),
        py::arg("pos_offset") = 0);
  m.def("embedding_bwd", &embedding_bwd, py::arg("idx"), py::arg("dout"), py::arg("dwte") = py::none(),
        py::arg("dwpe") = py::none(), py::arg("vocab_lo") = 0, py::arg("vocab_hi") = (int64_t)1 << 40,
        py::arg("deterministic") = false);
  m.def("embedding_vp_push", &embedding_vp_push);
  m.def("embedding_vp_pull_bwd", &embedding_vp_pull_bwd);
  m.def("softmax_fwd", &softmax_fwd);
  m.def("softmax_bwd", &softmax_bwd);
  m.def("xent_fused", &xent_fused, py::arg("logits"), py::arg("targets"), py::arg("V"), py::arg("grad_scale"),
        py::arg("write_grad"), py::arg("mean_scale"));
  m.def("xent_bwd", &xent_bwd);
  m.def("xent_vp_stats", &xent_vp_stats);
  m.def("xent_vp_grad", &xent_vp_grad);
  m.def("adam_flat", &adam_flat, py::arg("master"), py::arg("lp"), py::arg("grad"), py::arg("m"), py::arg("v"),
        py::arg("lr"), py::arg("b1"), py::arg("b2"), py::arg("eps"), py::arg("wd"), py::arg("step"),
        py::arg("grad_scale"), py::arg("dev_state") = py::none());
  m.def("adam_tick", &adam_tick);
  m.def("launch_count", [] { return g_launches; });
  m.def("sgd_flat", &sgd_flat);
  m.def("axpy", &axpy);
  m.def("unary_fwd", &unary_fwd);
  m.def("unary_bwd", &unary_bwd);
  m.def("binary_fwd", &binary_fwd);
  m.def("cast", &cast);
  m.def("fill_", &fill_);
  m.def("transpose_last2", &transpose_last2);
  m.def("tri", &tri);
  m.def("colsum", &colsum, py::arg("x"), py::arg("out") = py::none(), py::arg("accumulate") = false);
  m.def("status_read", &status_read, py::arg("clear") = true);
  m.def("gemm_set_tma_store", [](bool on) { titb_gemm_set_tma_store(on ? 1 : 0); });
  bind_attention(m);
  bind_comm(m);
  bind_core(m);
  bind_symm(m);
}
