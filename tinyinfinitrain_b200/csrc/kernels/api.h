// C API of the sm_100a kernel library (libtitb200_kernels.so).
//
// Every function enqueues work on `stream` and returns a cudaError_t-compatible
// int (0 = success) from the launch; none of them synchronises.  Pointers are
// device pointers unless a comment says otherwise.  "bf16" buffers hold
// __nv_bfloat16, row-major, with the row stride given in elements.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TITB_API extern "C" __attribute__((visibility("default")))
#else
#define TITB_API extern "C"
#endif

// Error codes of this library (outside the cudaError_t range).
enum TitbError {
  TITB_ERR_ALIGNMENT = 20001,   // a base pointer or row stride is not 16-byte aligned
  TITB_ERR_TENSOR_MAP = 20002,  // cuTensorMapEncodeTiled rejected the operand description
  TITB_ERR_SHAPE = 20003,       // unsupported shape for this kernel
};

// ---- library status ---------------------------------------------------------
// One int per device, in device memory, written by kernels whose bounded waits
// ran out (see common.cuh StatusCode).  titb_status_ptr returns the device
// pointer (allocating it on first use); titb_status_read copies it to the host
// after synchronising `stream` and optionally clears it.
TITB_API int* titb_status_ptr(void);
TITB_API int titb_status_read(int clear, cudaStream_t stream);

// ---- tcgen05 GEMM -----------------------------------------------------------
// D[M,N] = A . B^T over a reduction of length K, bf16 inputs, fp32 accumulation in
// tensor memory.  Each operand is either K-major (stored [rows, K], ld >= K) or
// MN-major (stored [K, rows], ld >= rows): this covers forward (X W^T), dgrad
// (dY W) and wgrad (dY^T X) without a transpose pass.
enum TitbEpilogue {
  TITB_EPI_NONE = 0,
  TITB_EPI_BIAS = 1,           // out = acc + bias[col]
  TITB_EPI_BIAS_GELU = 2,      // aux_out = acc + bias ; out = gelu_tanh(aux_out)
  TITB_EPI_DGELU = 3,          // out = acc * gelu_tanh'(aux_in)
  TITB_EPI_BIAS_RESIDUAL = 4,  // out = acc + bias + aux_in   (bias may be null)
  TITB_EPI_SWIGLU = 5,         // reserved
};

// Optional collective fused into the GEMM (see gemm_tcgen05.cu, CollArgs).  All pointer tables are
// host arrays of `world` device addresses as mapped on the calling GPU (symmetric memory).
//  mode 1 (all-gather -> GEMM): A = all ranks' [rows_per_rank, K] shards; `peer_ptrs` are the shard
//    bases, `gathered` a local [M, K] buffer that receives the gathered rows (and must be passed as
//    TitbGemmDesc::a), `flags` a local uint32 [M / 128] array.
//  mode 2 (GEMM -> reduce-scatter): `peer_ptrs` are the receive buffers bf16 [world][rows_per_rank][N],
//    `cnt_ptrs` the per-rank counter arrays uint32 [rows_per_rank / 128] (zero before first use),
//    `flags` this rank's own counter array, `rs_out` the [rows_per_rank, N] result (+bias +residual).
//    TitbGemmDesc::out is unused.
// A cross-GPU barrier (titb_comm_barrier) must separate the writes of the peers' inputs from this call.
struct TitbGemmColl {
  int mode, world, rank, helper_ctas, rows_per_rank;
  const unsigned long long* peer_ptrs;
  const unsigned long long* cnt_ptrs;
  void* gathered;
  void* flags;
  void* rs_out;
  const void* rs_bias;
  const void* rs_residual;
};

struct TitbGemmDesc {
  const void* a;        // bf16
  const void* b;        // bf16
  void* out;            // bf16 or fp32, [M, ldo]
  int M, N, K;
  int a_mn_major, b_mn_major;
  long long lda, ldb, ldo;
  int out_fp32;         // 1: out is float
  int accumulate;       // 1: out += result (read-modify-write)
  int epilogue;         // TitbEpilogue
  const void* bias;     // bf16 [N] or null
  const void* aux_in;   // bf16 [M, ld_aux_in] or null
  long long ld_aux_in;
  void* aux_out;        // bf16 [M, ld_aux_out] or null
  long long ld_aux_out;
  int splits;           // split-K factor (>=1); >1 needs `workspace`
  void* workspace;      // fp32 [splits, M, N] scratch when splits > 1
  int tile_n;           // 0 = heuristic, else 128 or 256
  const void* alpha;    // optional device fp32 scalar: result = alpha * (A . B^T) before the epilogue
  const TitbGemmColl* coll;  // optional fused collective, or null
};
TITB_API int titb_gemm_bf16(const TitbGemmDesc* d, cudaStream_t stream);
// Same descriptor, collective mode 3 only (gemm_param_gather.cu): the B operand is a weight [N, K] (K-major,
// contiguous rows) whose rows are sharded over `world` ranks, rows_per_rank each (a multiple of 128).  `b` and
// `coll->gathered` are this rank's full-size copy, `coll->peer_ptrs[r]` the first row rank r owns, in r's memory
// as mapped on this GPU (for r == rank it may alias the local copy: then nothing is moved), `coll->flags` N / 128
// uint32 words of scratch.  The caller orders the launch after the owners' last writes (device barrier).
TITB_API int titb_gemm_param_gather_bf16(const TitbGemmDesc* d, cudaStream_t stream);
// Picks the split-K factor the heuristic would use (so callers can size the workspace).
TITB_API int titb_gemm_pick_splits(int M, int N, int K);
// Tile width (128, 192 or 256) the GEMM takes for this shape and split-K factor when the descriptor leaves tile_n 0.
TITB_API int titb_gemm_pick_tile(int M, int N, int K, int splits);
// 1 when a split-K call with this descriptor sums its partial tiles in the output itself (fp32 output, no fused
// epilogue, TMA reduce-add) and needs no workspace; 0 when it needs workspace [splits, M, N] fp32.
TITB_API int titb_gemm_split_in_place(const TitbGemmDesc* d);
// Switches the shared-memory-staged TMA store epilogue of bf16 outputs on (default) or off (A/B timing).
TITB_API void titb_gemm_set_tma_store(int enabled);
// fp32 SIMT GEMM for API parity with fp32 tensors: C[M,N] (+)= op(A) op(B), row-major.
TITB_API int titb_sgemm(const float* A, const float* B, float* C, int M, int N, int K, int trans_a, int trans_b,
                        int accumulate, cudaStream_t stream);

// ---- normalisation ------------------------------------------------------------
// dtype: 0 = fp32, 1 = bf16 for x/y/w/b; statistics are always fp32.
TITB_API int titb_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                long long rows, int C, float eps, int dtype, cudaStream_t stream);
// dw/db partial sums use `scratch` (fp32 [2, nblocks, C]); nblocks = titb_layernorm_bwd_blocks(rows).
// `dres` (optional, same shape and dtype as x): a gradient arriving through a residual connection around the norm;
// dx = norm backward + dres, added inside the kernel.
TITB_API int titb_layernorm_bwd_blocks(long long rows);
TITB_API int titb_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                void* dx, float* dw, float* db, float* scratch, long long rows, int C, int dtype,
                                int accumulate_wgrad, const void* dres, cudaStream_t stream);
TITB_API int titb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int C, float eps,
                              int dtype, cudaStream_t stream);
TITB_API int titb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                              float* scratch, long long rows, int C, int dtype, int accumulate_wgrad, const void* dres,
                              cudaStream_t stream);
// ---- activations ----------------------------------------------------------------
TITB_API int titb_gelu_fwd(const void* x, void* y, long long n, int dtype, cudaStream_t stream);
TITB_API int titb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, int dtype, cudaStream_t stream);
// SwiGLU on a fused [rows, 2*F] projection: y[r, f] = silu(x[r, f]) * x[r, F + f].
TITB_API int titb_swiglu_fwd(const void* x, void* y, long long rows, int F, int dtype, cudaStream_t stream);
TITB_API int titb_swiglu_bwd(const void* dy, const void* x, void* dx, long long rows, int F, int dtype,
                             cudaStream_t stream);

// ---- rotary embedding --------------------------------------------------------------
// x: [B, T, H, hd] (contiguous), rotates pairs (i, i + hd/2) with angle pos * theta^(-2i/hd).
// inverse = 1 applies the transpose rotation (the backward pass).  In place when y == x.
TITB_API int titb_rope(const void* x, void* y, int B, int T, int H, int hd, int pos_offset, float theta,
                       int inverse, int dtype, cudaStream_t stream);

// Same on the first H heads of rows that are stride_t elements apart (e.g. the q and k heads of a
// fused QKV buffer); x and y use the same stride.
TITB_API int titb_rope_strided(const void* x, void* y, int B, int T, int H, int hd, long long stride_t,
                               int pos_offset, float theta, int inverse, int dtype, cudaStream_t stream);

// ---- embedding ------------------------------------------------------------------------
// out[b,t,:] = wte[idx[b,t],:] (+ wpe[t + pos_offset,:] when wpe != null).
TITB_API int titb_embedding_fwd(const long long* idx, const void* wte, const void* wpe, void* out, long long BT,
                                int T, int C, int pos_offset, int dtype, cudaStream_t stream);
// dwte[idx[b,t],:] += dout[b,t,:] ; dwpe[t,:] += sum_b dout[b,t,:].  fp32 gradient buffers.
TITB_API int titb_embedding_bwd(const long long* idx, const void* dout, float* dwte, float* dwpe, long long BT,
                                int T, int C, int vocab_lo, int vocab_hi, int dtype, cudaStream_t stream);
// Vocabulary-parallel table: this rank holds rows [vocab_lo, vocab_hi) of the table; the M = world * Ms tokens are
// split by position, rank r owning tokens [r * Ms, (r + 1) * Ms).  `push` stores the rows this rank holds into the
// [Ms, C] buffer of each token's owner (dst_ptrs[r], 16-byte aligned, local or peer-mapped memory; world <= 16); with
// zero_strays != 0 it also writes zero rows for ids outside [0, vocab_total).  Across the ranks every destination row
// is written exactly once, so no reduction follows; the caller puts a cross-rank barrier before (destinations free)
// and after (all rows landed) the launch.  `pull_bwd` is the transpose: gradient rows of the ids this rank holds are
// read from the token owners' [Ms, C] buffers (src_ptrs) and added to dw [vocab_hi - vocab_lo, C] fp32 with atomics.
TITB_API int titb_embedding_vp_push(const long long* idx, const void* w, const unsigned long long* dst_ptrs, int world,
                                    long long M, long long Ms, int C, long long vocab_lo, long long vocab_hi,
                                    long long vocab_total, int zero_strays, int dtype, cudaStream_t stream);
TITB_API int titb_embedding_vp_pull_bwd(const long long* idx, const unsigned long long* src_ptrs, int world, float* dw,
                                        long long M, long long Ms, int C, long long vocab_lo, long long vocab_hi,
                                        int dtype, cudaStream_t stream);

// Deterministic variant of the token part (dwte only): the keys (row, position) of one step are sorted in the shared
// memory of one block and every run of equal rows is summed in position order, no atomics.  BT must not exceed
// titb_embedding_sorted_max_tokens(); scratch_keys: BT rounded up to a power of two, 64-bit words.
TITB_API int titb_embedding_sorted_max_tokens(void);
TITB_API int titb_embedding_bwd_wte_sorted(const long long* idx, const void* dout, float* dwte, long long BT, int C,
                                           int vocab_lo, int vocab_hi, int dtype, unsigned long long* scratch_keys,
                                           cudaStream_t stream);

// ---- softmax / cross entropy -------------------------------------------------------------
TITB_API int titb_softmax_fwd(const void* x, void* y, long long outer, int axis, long long inner, int dtype,
                              cudaStream_t stream);
TITB_API int titb_softmax_bwd(const void* dy, const void* y, void* dx, long long outer, int axis, long long inner,
                              int dtype, cudaStream_t stream);
// Fused loss + gradient.  logits: [rows, ld] with V valid columns (columns >= V are
// padding: ignored for the loss, gradient written as 0).  losses: fp32 [rows].  When
// dlogits != null it receives grad_scale * (softmax - onehot); it may alias logits.
TITB_API int titb_xent_fwd_bwd(const void* logits, const long long* targets, float* losses, void* dlogits,
                               long long rows, int V, long long ld, float grad_scale, int dtype,
                               cudaStream_t stream);
TITB_API int titb_xent_bwd(const void* logits, const long long* targets, void* dlogits, const float* upstream,
                           long long rows, int V, long long ld, float grad_scale, int dtype, cudaStream_t stream);
TITB_API int titb_mean(const float* x, float* out, long long n, float scale, cudaStream_t stream);
// Vocabulary-parallel cross entropy.  logits [rows, ld] is this rank's slice: column c is global column
// vocab_lo + c; columns >= V_local or with a global index >= vocab_size are padding.
// Pass 1 writes (row max, sum exp(x - max), target logit or 0) to slot `rank` of a [world, rows, 3] fp32 table at
// each of the n_dst (<= 16) destination addresses (the local table and/or peers' tables in peer-mapped memory).
TITB_API int titb_xent_vp_stats(const void* logits, const long long* targets, const unsigned long long* dst_ptrs,
                                int n_dst, int rank, long long rows, long long V_local, long long ld,
                                long long vocab_lo, long long vocab_size, int dtype, cudaStream_t stream);
// Pass 2 reads the complete table (all `world` slots), writes losses[row] = logsumexp - target logit (0 for rows
// whose target is outside [0, vocab_size)) and overwrites the slice with grad_scale * (softmax - onehot).
TITB_API int titb_xent_vp_grad(void* logits, const long long* targets, const float* stats, int world, float* losses,
                               long long rows, long long V_local, long long ld, long long vocab_lo,
                               long long vocab_size, float grad_scale, int dtype, cudaStream_t stream);

// ---- optimizers ----------------------------------------------------------------------------
// One launch over a flat range.  master/m/v fp32; grad fp32; param_bf16 (optional) gets the
// rounded copy of the updated master weights.
TITB_API int titb_adam_flat(float* master, void* param_lp, const float* grad, float* m, float* v, long long n,
                            float lr, float beta1, float beta2, float eps, float weight_decay, float bc1,
                            float bc2, float grad_scale, int lp_dtype, const float* dev_state,
                            cudaStream_t stream);
// dev_state: optional device float[4] = {t, 1-beta1^t, 1-beta2^t, lr} overriding bc1/bc2/lr;
// titb_adam_tick advances it by one step on the device (graph-capturable step counter).
TITB_API int titb_adam_tick(float* state, float beta1, float beta2, cudaStream_t stream);
TITB_API int titb_axpy(float* y, const void* x, float a, long long n, int x_dtype, cudaStream_t stream);
TITB_API int titb_sgd_flat(float* master, void* param_lp, const float* grad, long long n, float lr, int lp_dtype,
                           cudaStream_t stream);

// ---- elementwise family ------------------------------------------------------------------------
enum TitbUnary {
  TITB_NEG = 0, TITB_RECIPROCAL, TITB_SIN, TITB_COS, TITB_TANH, TITB_POW_SCALAR_EXP, TITB_POW_SCALAR_BASE,
  TITB_RSQRT, TITB_EQUALS_SCALAR, TITB_ADD_SCALAR, TITB_MUL_SCALAR, TITB_SIGMOID, TITB_COPY,
};
TITB_API int titb_unary_fwd(int op, const void* x, void* y, long long n, float s, int dtype, cudaStream_t stream);
// dx = dy * f'(.) where the saved tensor is the input (or the output for tanh/sigmoid).
TITB_API int titb_unary_bwd(int op, const void* dy, const void* saved, void* dx, long long n, float s, int dtype,
                            cudaStream_t stream);
enum TitbBinary { TITB_ADD = 0, TITB_SUB, TITB_MUL, TITB_DIV };
// y = a (op) broadcast(b); b is right-aligned against a, b_numel divides a_numel and the
// broadcast is described by up to 8 (a_dim, b_stride) pairs passed by value.
struct TitbBroadcast {
  int ndim;
  long long a_dims[8];
  long long b_strides[8];  // 0 where b is broadcast
};
TITB_API int titb_binary_fwd(int op, const void* a, const void* b, void* y, long long n, TitbBroadcast bc,
                             int dtype, cudaStream_t stream);
TITB_API int titb_cast(const void* x, void* y, long long n, int src_dtype, int dst_dtype, cudaStream_t stream);
TITB_API int titb_fill(void* y, long long n, float value, int dtype, cudaStream_t stream);
// 2-D batched transpose: in [batch, R, C] -> out [batch, C, R].
TITB_API int titb_transpose(const void* x, void* y, long long batch, int R, int C, int dtype, cudaStream_t stream);
TITB_API int titb_tri(const void* x, void* y, int R, int C, int diagonal, int upper, int dtype,
                      cudaStream_t stream);
TITB_API int titb_colsum(const void* x, float* out, long long rows, int C, int dtype, int accumulate,
                         float* scratch, cudaStream_t stream);
TITB_API int titb_colsum_blocks(long long rows);
// ---- reductions and view-like transforms (dtype: 0 = fp32, 1 = bf16) ---------------------------------
// x viewed as [outer, n, inner] -> y [outer, inner].  op: 0 sum, 1 mean, 2 max, 3 min; for max / min `idx`
// (may be null) receives the position along n of the selected element (lowest index on ties).
TITB_API int titb_reduce(const void* x, void* y, long long* idx, long long outer, long long n, long long inner, int op,
                         int dtype, cudaStream_t stream);
// dx[o, i, in] = g[o, in] * scale when idx is null, else g[o, in] where i == idx[o, in] and 0 elsewhere.
TITB_API int titb_reduce_bwd(const void* g, const long long* idx, void* dx, long long outer, long long n,
                             long long inner, float scale, int dtype, cudaStream_t stream);
// out (contiguous, row-major over size[0..nd)) <- in[in_offset + sum_d i_d * in_stride[d]]; nd <= 6.
// Strides are in elements, 0 repeats an element; elem_bytes in {2, 4, 8}.
TITB_API int titb_gather_nd(const void* in, void* out, int nd, const long long* size, const long long* in_stride,
                            long long in_offset, int elem_bytes, cudaStream_t stream);
// out[out_offset + sum_d i_d * out_stride[d]] <- (or +=, with atomics) in (contiguous); nd <= 6.
TITB_API int titb_scatter_nd(const void* in, void* out, int nd, const long long* size, const long long* out_stride,
                             long long out_offset, int dtype, int accumulate, cudaStream_t stream);
// y = masked ? value : x, or with bit 0 of `backward` set y = masked ? 0 : x (gradient of the former).  An
// element is masked when its mask entry is non-zero, or, with bit 1 of `backward` set, when it equals 1 (the
// reference's rule).  The mask has mask_n elements and repeats by modulo over the flattened x.
// mask_dtype: 0 fp32, 1 bf16, 2 uint8/bool.
TITB_API int titb_mask_fill(const void* x, const void* mask, void* y, long long n, long long mask_n, float value,
                            int backward, int dtype, int mask_dtype, cudaStream_t stream);
TITB_API int titb_outer(const void* a, const void* b, void* y, long long M, long long N, int dtype, cudaStream_t stream);
TITB_API int titb_outer_bwd(const void* g, const void* a, const void* b, void* da, void* db, long long M, long long N,
                            int dtype, cudaStream_t stream);

// ---- attention --------------------------------------------------------------------------------------
// Causal self-attention over packed projections.  q: [B, T, Hq, hd], k/v: [B, T, Hkv, hd] with
// arbitrary (16-byte aligned) token strides so a fused QKV buffer can be addressed in place.
struct TitbAttnDesc {
  const void* q; const void* k; const void* v;   // bf16
  void* o;                                        // bf16 [B, T, Hq, hd]
  float* lse;                                     // fp32 [B, Hq, T]
  const void* d_o; void* dq; void* dk; void* dv;   // backward only
  float* delta;                                   // fp32 [B, Hq, T] scratch (backward)
  float* dq_accum;                                // fp32 [B, T, Hq, hd] scratch (backward)
  int B, T, Hq, Hkv, hd;
  long long q_stride_t, k_stride_t, v_stride_t, o_stride_t;   // elements between tokens
  long long dq_stride_t, dk_stride_t, dv_stride_t, do_stride_t;
  float scale;
};
TITB_API int titb_attn_fwd(const TitbAttnDesc* d, cudaStream_t stream);
TITB_API int titb_attn_bwd(const TitbAttnDesc* d, cudaStream_t stream);

// ---- gradient-norm clipping (device resident: graph-capturable) -------------------------------------------------
// Stage 1: per-block partial sums of squares of a flat fp32 buffer (16-byte aligned).  `partials` must hold
// titb_clip_max_partials() floats; *n_partials receives how many were written.
TITB_API int titb_clip_max_partials(void);
TITB_API int titb_sumsq_partials(const float* x, long long n, float* partials, int* n_partials, cudaStream_t stream);
// Same for this rank's shard [shard_off, shard_off + shard_n) of the SUM over ranks of the peer-mapped gradient
// buffers (multimem.ld_reduce through NVSwitch when grad_mc is given, plain peer loads otherwise).
TITB_API int titb_rs_sumsq_partials(const unsigned long long* grad_ptrs, const void* grad_mc, long long shard_off,
                                    long long shard_n, int world, int rank, float* partials, int* n_partials,
                                    cudaStream_t stream);
// Stage 2 (one block, fixed order).  max_norm > 0: out[0] = sqrt(sum) * pre_scale, out[1] = min(1, max_norm / (out[0] + 1e-6)).
// max_norm <= 0: out[0] = sum (to be combined with other ranks' sums first).
TITB_API int titb_clip_coef(const float* partials, int n_partials, float pre_scale, float max_norm, float* out,
                            cudaStream_t stream);
// x *= coef[0] with the coefficient read from device memory; returns without touching memory when it is exactly 1.
TITB_API int titb_scale_by_dev(float* x, long long n, const float* coef, cudaStream_t stream);

// ---- NVLink communication (peer-mapped symmetric memory) -------------------------------------------
// Pointer tables are host arrays of device addresses, one per rank, valid on the calling GPU.
// Cross-GPU barrier on signal pads: pad of rank r = uint32[8 channels][16]; `epoch` is a device
// counter advanced by the kernel (graph-replayable).  The wait gives up after timeout_s seconds and
// records kStatusPeerTimeout in the library status word.
TITB_API int titb_comm_barrier(const unsigned long long* pad_ptrs, int rank, int world, int channel,
                               unsigned int* epoch, double timeout_s, cudaStream_t stream);
// ZeRO-1 step in one kernel: reduce this rank's gradient shard over all ranks, Adam on the fp32
// shard state, write the bf16 parameters of the shard into every rank's parameter buffer.
struct TitbRsAdamDesc {
  const unsigned long long* grad_ptrs;   // fp32 flat gradient buffer per rank
  const unsigned long long* param_ptrs;  // bf16 flat parameter buffer per rank
  const void* grad_mc;                   // NVLS multicast address of the gradient buffer, or null
  void* param_mc;                        // NVLS multicast address of the parameter buffer, or null
  float* master; float* m; float* v;     // local shard state (length shard_n)
  long long shard_off, shard_n;          // shard position in the flat space (elements; n % 8 == 0)
  int world, rank;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
  const float* dev_state;                // optional device {t, bc1, bc2, lr}
  int max_blocks;                        // 0 = default
};
TITB_API int titb_rs_adam_ag(const TitbRsAdamDesc* d, cudaStream_t stream);
TITB_API int titb_allreduce_small(const unsigned long long* buf_ptrs, float* out, int n, int world, int op,
                                  cudaStream_t stream);

// Standalone in-place collectives over a symmetric buffer (collectives.cu).  dtype: 0 fp32, 1 bf16.  byte_off and
// nbytes / world are multiples of 16.  No waits inside: the caller runs titb_comm_barrier before and after.
TITB_API int titb_symm_allreduce(const unsigned long long* buf_ptrs, unsigned long long mc_ptr, long long byte_off,
                                 long long nbytes, int dtype, int world, int rank, float scale, int max_blocks,
                                 cudaStream_t stream);
TITB_API int titb_symm_allgather(const unsigned long long* buf_ptrs, unsigned long long mc_ptr, long long byte_off,
                                 long long nbytes, int world, int rank, int max_blocks, cudaStream_t stream);
// Point-to-point flag in symmetric memory: signal stores `value` with release semantics after all earlier work of
// the stream; wait blocks the stream until the word has reached `value` or `timeout_s` has passed (then the status
// word reads kStatusPeerTimeout and the stream continues).
TITB_API int titb_symm_signal(unsigned long long remote_word, unsigned int value, cudaStream_t stream);
TITB_API int titb_symm_wait(unsigned long long local_word, unsigned int value, double timeout_s, cudaStream_t stream);
