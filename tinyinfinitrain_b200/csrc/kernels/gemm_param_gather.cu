// Parameter all-gather fused into the consuming GEMM (ZeRO-style weight sharding over data-parallel ranks).
//
// Y[M, N] = X[M, K] . W[N, K]^T where rank r holds the authoritative rows [r N/W, (r+1) N/W) of W.  One kernel:
// helper CTAs pull the other ranks' rows over NVLink (plain peer loads, 128-row chunks, a flag per chunk) into
// this rank's full-size copy of W while the GEMM CTAs -- the tcgen05 / TMA pipeline of gemm_tcgen05.cu, with all
// its epilogues -- start on the n-blocks of the local shard and move on to the others as their chunks land.  No
// TMA load ever reads peer memory; every wait is bounded and reports through the library status word.  After the
// launch the local copy of W is complete, so dgrad and wgrad of the same step use it as an ordinary operand.
//
// The body is gemm_tcgen05.cu compiled a second time under another namespace with collective mode 3 switched on;
// the copy that serves every other GEMM of the framework is not affected by this file.
//
// The reference has no data parallelism and no sharded parameters (infini_train/src/device.cc:11-17 allows one
// device); its Linear is a cuBLAS call on a whole local weight (infini_train/src/kernels/cuda/linear.cu:58-128).
#define TITB_GEMM_PARAM_GATHER 1
#define titb titb_param_gather
#include "gemm_tcgen05.cu"
