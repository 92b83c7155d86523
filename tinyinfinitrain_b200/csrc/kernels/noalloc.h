// Allocation-free entry point of the kernel library.
//
// This header has no counterpart in the reference project: TinyInfiniTrain allocates
// every temporary with cudaMallocAsync on each call (infini_train/src/tensor.cc:58-96)
// and offers no way around it.
//
// Who needs it: code that drives these kernels from a context where creating or freeing
// device memory is not possible or not allowed -- a thread inside a CUDA-graph stream
// capture (an allocation would invalidate the capture), a real-time or latency-bounded
// serving loop that may not take the allocator lock or trigger a device synchronisation,
// a plug-in that runs under a host framework owning all device memory and handing out
// only input and output buffers, or a process whose memory budget is fixed at start-up.
// The regular LayerNorm backward (titb_layernorm_bwd in api.h) asks its caller for a
// scratch buffer; such callers have nowhere to get one from.
#pragma once
#include <cuda_runtime.h>

#include "api.h"

// Largest row width (elements of the normalised dimension) the built-in scratch can serve.
#define TITB_NOALLOC_LAYERNORM_MAX_C 2048

// LayerNorm backward with the library's own scratch.  Same arguments and results as
// titb_layernorm_bwd minus the `scratch` pointer: dx gets the input gradient, dw/db (fp32
// [C]) the weight and bias gradients (added to their previous contents when
// accumulate_wgrad != 0).  dtype: 0 = fp32, 1 = bf16.
//
// * The scratch is a fixed array in device memory, part of the library image:
//   2 * 592 * TITB_NOALLOC_LAYERNORM_MAX_C floats (about 9.7 MB) on every GPU that loads the
//   library, held until the process exits.
// * C > TITB_NOALLOC_LAYERNORM_MAX_C is refused with TITB_ERR_NOALLOC_TOO_LARGE (nothing is
//   launched); titb_strerror() gives the text.
// * The function calls no cudaMalloc/cudaFree and no allocating library routine.  The first call
//   on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//   current) and remembers it; make that first call outside any stream capture.
// * All calls on one device share the one array.  Each call overwrites every scratch element it
//   later reads, so nothing has to be cleared between calls, but two calls whose kernels overlap
//   on the GPU (different streams, no dependency) race on it and give wrong dw/db.  Calls on the
//   same stream are ordered and safe.
TITB_API int titb_layernorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean,
                                        const float* rstd, void* dx, float* dw, float* db, long long rows, int C,
                                        int dtype, int accumulate_wgrad, cudaStream_t stream);

#define TITB_ERR_NOALLOC_TOO_LARGE 20010
#define TITB_ERR_NOALLOC_SYMBOL 20011
#define TITB_ERR_NOALLOC_LAYOUT 20012  /* library built inconsistently: scratch sized for another kernel layout */

// Text for the library's own error codes (>= 20000); cudaGetErrorString for anything else.
TITB_API const char* titb_strerror(int code);
