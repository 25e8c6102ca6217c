// Fused AdamW update of a decoded bf16 weight: one pass over weight, gradient
// and the two moments.  It sits between the decode and the re-encode of the
// read -> update -> write cycle that the reference performs per layer inside
// backward (compressed_lomo_hook, neuzip/__init__.py:25-35, with plain SGD).
#include <cuda_bf16.h>

#include "nz_common.cuh"

namespace nz {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale;
};

__device__ __forceinline__ float load_state(const float *p, uint64_t i) { return p[i]; }
__device__ __forceinline__ float load_state(const __nv_bfloat16 *p, uint64_t i) {
  return __bfloat162float(p[i]);
}
__device__ __forceinline__ void store_state(float *p, uint64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void store_state(__nv_bfloat16 *p, uint64_t i, float v) {
  p[i] = __float2bfloat16_rn(v);
}

// 8 elements per thread: 128-bit loads of weight and gradient.
template <typename StateT>
__global__ void __launch_bounds__(256)
adamw_kernel(__nv_bfloat16 *__restrict__ w, const __nv_bfloat16 *__restrict__ g,
             StateT *__restrict__ m, StateT *__restrict__ v, uint64_t n, AdamArgs a) {
  const uint64_t n_vec = n / 8;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    uint4 wv = reinterpret_cast<const uint4 *>(w)[i];
    const uint4 gv = reinterpret_cast<const uint4 *>(g)[i];
    __nv_bfloat16 *wp = reinterpret_cast<__nv_bfloat16 *>(&wv);
    const __nv_bfloat16 *gp = reinterpret_cast<const __nv_bfloat16 *>(&gv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint64_t e = i * 8 + k;
      const float grad = __bfloat162float(gp[k]) * a.grad_scale;
      float mm = load_state(m, e), vv = load_state(v, e);
      mm = a.beta1 * mm + (1.0f - a.beta1) * grad;
      vv = a.beta2 * vv + (1.0f - a.beta2) * grad * grad;
      store_state(m, e, mm);
      store_state(v, e, vv);
      float x = __bfloat162float(wp[k]);
      x *= 1.0f - a.lr * a.weight_decay;
      x -= (a.lr / a.bias1) * mm / (sqrtf(vv / a.bias2) + a.eps);
      wp[k] = __float2bfloat16_rn(x);
    }
    reinterpret_cast<uint4 *>(w)[i] = wv;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (uint64_t e = n_vec * 8; e < n; ++e) {
      const float grad = __bfloat162float(g[e]) * a.grad_scale;
      float mm = load_state(m, e), vv = load_state(v, e);
      mm = a.beta1 * mm + (1.0f - a.beta1) * grad;
      vv = a.beta2 * vv + (1.0f - a.beta2) * grad * grad;
      store_state(m, e, mm);
      store_state(v, e, vv);
      float x = __bfloat162float(w[e]);
      x *= 1.0f - a.lr * a.weight_decay;
      x -= (a.lr / a.bias1) * mm / (sqrtf(vv / a.bias2) + a.eps);
      w[e] = __float2bfloat16_rn(x);
    }
  }
}

}  // namespace nz

extern "C" int nz_adamw_bf16(void *weight_bf16, const void *grad_bf16, void *exp_avg,
                             void *exp_avg_sq, uint64_t n, int state_is_bf16, float lr,
                             float beta1, float beta2, float eps, float weight_decay,
                             uint32_t step, float grad_scale, void *stream) {
  if (n == 0) return NZ_OK;
  if (!weight_bf16 || !grad_bf16 || !exp_avg || !exp_avg_sq || step == 0) {
    nz::set_error("nz_adamw_bf16: null pointer or step 0");
    return NZ_E_ARG;
  }
  if (((uintptr_t)weight_bf16 & 15) || ((uintptr_t)grad_bf16 & 15)) {
    nz::set_error("nz_adamw_bf16: weight and gradient must be 16-byte aligned");
    return NZ_E_ARG;
  }
  nz::AdamArgs a;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.weight_decay = weight_decay;
  a.bias1 = 1.0f - powf(beta1, (float)step);
  a.bias2 = 1.0f - powf(beta2, (float)step);
  a.grad_scale = grad_scale;
  uint64_t blocks = (n / 8 + 255) / 256;
  const uint64_t cap = (uint64_t)nz::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  cudaStream_t st = (cudaStream_t)stream;
  if (state_is_bf16)
    nz::adamw_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
        (__nv_bfloat16 *)weight_bf16, (const __nv_bfloat16 *)grad_bf16, (__nv_bfloat16 *)exp_avg,
        (__nv_bfloat16 *)exp_avg_sq, n, a);
  else
    nz::adamw_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(
        (__nv_bfloat16 *)weight_bf16, (const __nv_bfloat16 *)grad_bf16, (float *)exp_avg,
        (float *)exp_avg_sq, n, a);
  NZ_LAUNCH_CHECK("adamw_kernel");
  return NZ_OK;
}
