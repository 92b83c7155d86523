// Optimizer steps over flat parameter ranges.
//
// Counterpart of infini_train/src/kernels/cuda/accumulate_grad.cu:6-23
// (AccumulateGrad, used for gradient accumulation and as the SGD step) and the
// AdamAccumulateGrad stub at :25-32 whose expected math is the closed form of
// test/optimizer/test_adam.cc:50-58.  One launch covers a whole flat buffer
// (every parameter of a model shard), reads and writes 128 bits per access,
// keeps fp32 master weights and moments, and emits the rounded bf16 copy of the
// weights in the same pass.
#include "api.h"
#include "common.cuh"

namespace titb {

template <typename LP>
__global__ void adam_flat_kernel(float* __restrict__ master, LP* __restrict__ lp, const float* __restrict__ grad,
                                 float* __restrict__ m, float* __restrict__ v, long long n, float lr, float b1,
                                 float b2, float eps, float wd, float bc1, float bc2, float gscale,
                                 const float* __restrict__ dev_state) {
  if (dev_state != nullptr) {  // step-dependent scalars kept on the device so a captured graph stays valid
    bc1 = dev_state[1];
    bc2 = dev_state[2];
    lr = dev_state[3];
  }
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n) {
      float4 g = *reinterpret_cast<const float4*>(grad + i);
      float4 mm = *reinterpret_cast<const float4*>(m + i);
      float4 vv = *reinterpret_cast<const float4*>(v + i);
      float4 w = *reinterpret_cast<const float4*>(master + i);
      float* gp = &g.x; float* mp = &mm.x; float* vp = &vv.x; float* wp = &w.x;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float ge = gp[e] * gscale;
        mp[e] = b1 * mp[e] + (1.f - b1) * ge;
        vp[e] = b2 * vp[e] + (1.f - b2) * ge * ge;
        const float mh = mp[e] / bc1, vh = vp[e] / bc2;
        wp[e] -= lr * (mh / (sqrtf(vh) + eps) + wd * wp[e]);
      }
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
      *reinterpret_cast<float4*>(master + i) = w;
      if (lp != nullptr) {
        if constexpr (sizeof(LP) == 2) {
          uint2 u = make_uint2(pack_bf16x2(wp[0], wp[1]), pack_bf16x2(wp[2], wp[3]));
          *reinterpret_cast<uint2*>(lp + i) = u;
        } else {
          *reinterpret_cast<float4*>(lp + i) = w;
        }
      }
    } else {
      for (long long j = i; j < n; ++j) {
        const float ge = grad[j] * gscale;
        const float mj = b1 * m[j] + (1.f - b1) * ge;
        const float vj = b2 * v[j] + (1.f - b2) * ge * ge;
        m[j] = mj; v[j] = vj;
        const float wj = master[j] - lr * ((mj / bc1) / (sqrtf(vj / bc2) + eps) + wd * master[j]);
        master[j] = wj;
        if (lp != nullptr) lp[j] = from_f32<LP>(wj);
      }
    }
  }
}

// state = {t, 1 - b1^t, 1 - b2^t, lr}; advances t by one.
__global__ void adam_tick_kernel(float* state, float b1, float b2) {
  const float t = state[0] + 1.f;
  state[0] = t;
  state[1] = 1.f - powf(b1, t);
  state[2] = 1.f - powf(b2, t);
}

template <typename LP>
__global__ void sgd_flat_kernel(float* __restrict__ master, LP* __restrict__ lp, const float* __restrict__ grad,
                                long long n, float lr) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float w = master[i] - lr * grad[i];
    master[i] = w;
    if (lp != nullptr) lp[i] = from_f32<LP>(w);
  }
}

template <typename X>
__global__ void axpy_kernel(float* __restrict__ y, const X* __restrict__ x, float a, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] += a * to_f32(x[i]);
}

static inline int blocks_for(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = device_sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace titb
using namespace titb;

TITB_API int titb_adam_flat(float* master, void* param_lp, const float* grad, float* m, float* v, long long n, float lr,
                            float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                            float grad_scale, int lp_dtype, const float* dev_state, cudaStream_t st) {
  if (n <= 0) return 0;
  const int blocks = blocks_for(n / 4 + 1);
  if (lp_dtype == 1)
    adam_flat_kernel<bf16><<<blocks, 256, 0, st>>>(master, (bf16*)param_lp, grad, m, v, n, lr, beta1, beta2, eps,
                                                   weight_decay, bc1, bc2, grad_scale, dev_state);
  else
    adam_flat_kernel<float><<<blocks, 256, 0, st>>>(master, (float*)param_lp, grad, m, v, n, lr, beta1, beta2, eps,
                                                    weight_decay, bc1, bc2, grad_scale, dev_state);
  return (int)cudaGetLastError();
}

TITB_API int titb_adam_tick(float* state, float beta1, float beta2, cudaStream_t st) {
  adam_tick_kernel<<<1, 1, 0, st>>>(state, beta1, beta2);
  return (int)cudaGetLastError();
}

TITB_API int titb_sgd_flat(float* master, void* param_lp, const float* grad, long long n, float lr, int lp_dtype,
                           cudaStream_t st) {
  if (n <= 0) return 0;
  if (lp_dtype == 1) sgd_flat_kernel<bf16><<<blocks_for(n), 256, 0, st>>>(master, (bf16*)param_lp, grad, n, lr);
  else sgd_flat_kernel<float><<<blocks_for(n), 256, 0, st>>>(master, (float*)param_lp, grad, n, lr);
  return (int)cudaGetLastError();
}

TITB_API int titb_axpy(float* y, const void* x, float a, long long n, int x_dtype, cudaStream_t st) {
  if (n <= 0) return 0;
  if (x_dtype == 1) axpy_kernel<bf16><<<blocks_for(n), 256, 0, st>>>(y, (const bf16*)x, a, n);
  else axpy_kernel<float><<<blocks_for(n), 256, 0, st>>>(y, (const float*)x, a, n);
  return (int)cudaGetLastError();
}
