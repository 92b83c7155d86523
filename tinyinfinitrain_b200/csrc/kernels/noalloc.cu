// LayerNorm backward that brings its own scratch memory (see noalloc.h for who needs this and
// for the contract).  The scratch holds the per-CTA partial sums of dweight and dbias that the
// two-stage reduction of norm.cu writes in stage 1 and folds in stage 2.
#include "noalloc.h"

namespace {

constexpr int kParts = 592;  // partial rows per gradient: must match titb_layernorm_bwd_blocks()
constexpr long long kScratchFloats = 2LL * kParts * TITB_NOALLOC_LAYERNORM_MAX_C;

// File-scope device array.  In host code this name is only a handle for the runtime's symbol
// table -- it is NOT a device address and must never be passed to a kernel as one.
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];

float* g_scratch_addr[64] = {nullptr};  // device address of the array, per device ordinal

}  // namespace

TITB_API int titb_layernorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean,
                                        const float* rstd, void* dx, float* dw, float* db, long long rows, int C,
                                        int dtype, int accumulate_wgrad, cudaStream_t stream) {
  if (C <= 0 || rows < 0) return TITB_ERR_SHAPE;
  if (C > TITB_NOALLOC_LAYERNORM_MAX_C) return TITB_ERR_NOALLOC_TOO_LARGE;
  if (titb_layernorm_bwd_blocks(rows) != kParts) return TITB_ERR_NOALLOC_LAYOUT;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return TITB_ERR_NOALLOC_SYMBOL;
  if (g_scratch_addr[dev] == nullptr) {
    // One-time set-up for this device, with this device current: ask the runtime where the
    // array lives on it.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (p == nullptr) return TITB_ERR_NOALLOC_SYMBOL;
    g_scratch_addr[dev] = static_cast<float*>(p);
  }
  return titb_layernorm_bwd(dy, x, w, mean, rstd, dx, dw, db, g_scratch_addr[dev], rows, C, dtype, accumulate_wgrad,
                            nullptr, stream);
}

TITB_API const char* titb_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case TITB_ERR_ALIGNMENT: return "an operand base pointer or row stride is not 16-byte aligned";
    case TITB_ERR_TENSOR_MAP: return "the TMA tensor map for an operand could not be encoded";
    case TITB_ERR_SHAPE: return "unsupported shape";
    case TITB_ERR_NOALLOC_TOO_LARGE:
      return "row width exceeds TITB_NOALLOC_LAYERNORM_MAX_C, the largest the built-in scratch array can serve";
    case TITB_ERR_NOALLOC_SYMBOL: return "the built-in scratch array could not be located on this device";
    case TITB_ERR_NOALLOC_LAYOUT:
      return "the built-in scratch array was sized for another partial-row count than the LayerNorm backward kernel uses";
    default: return cudaGetErrorString(static_cast<cudaError_t>(code));
  }
}
