// Fused AdamW update of a decoded bf16 weight: one pass over weight, gradient
// and the two moments.  It sits between the decode and the re-encode of the
// read -> update -> write cycle that the reference performs per layer inside
// backward (compressed_lomo_hook, neuzip/__init__.py:25-35, with plain SGD).
#include <cuda_bf16.h>

#include "nz_common.cuh"

namespace nz {

__device__ __forceinline__ float load_state(const float *p, uint64_t i) { return p[i]; }
__device__ __forceinline__ float load_state(const __nv_bfloat16 *p, uint64_t i) {
  return __bfloat162float(p[i]);
}
__device__ __forceinline__ void store_state(float *p, uint64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void store_state(__nv_bfloat16 *p, uint64_t i, float v) {
  p[i] = __float2bfloat16_rn(v);
}

// The 8 moments a thread owns, as 128-bit accesses: one for bf16 moments, two for fp32.
struct State8 {
  float f[8];
};
__device__ __forceinline__ State8 load_state8(const float *p, uint64_t i) {
  State8 s;
  const float4 a = reinterpret_cast<const float4 *>(p)[2 * i];
  const float4 b = reinterpret_cast<const float4 *>(p)[2 * i + 1];
  s.f[0] = a.x; s.f[1] = a.y; s.f[2] = a.z; s.f[3] = a.w;
  s.f[4] = b.x; s.f[5] = b.y; s.f[6] = b.z; s.f[7] = b.w;
  return s;
}
__device__ __forceinline__ State8 load_state8(const __nv_bfloat16 *p, uint64_t i) {
  State8 s;
  const uint4 q = reinterpret_cast<const uint4 *>(p)[i];
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    s.f[2 * k] = __uint_as_float(w[k] << 16);
    s.f[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
  }
  return s;
}
__device__ __forceinline__ void store_state8(float *p, uint64_t i, const State8 &s) {
  reinterpret_cast<float4 *>(p)[2 * i] = make_float4(s.f[0], s.f[1], s.f[2], s.f[3]);
  reinterpret_cast<float4 *>(p)[2 * i + 1] = make_float4(s.f[4], s.f[5], s.f[6], s.f[7]);
}
__device__ __forceinline__ void store_state8(__nv_bfloat16 *p, uint64_t i, const State8 &s) {
  __nv_bfloat16 h[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) h[k] = __float2bfloat16_rn(s.f[k]);
  reinterpret_cast<uint4 *>(p)[i] = *reinterpret_cast<const uint4 *>(h);
}

// 8 elements per thread: 128-bit loads and stores of weight, gradient and both moments
// (moment arrays 16-byte aligned: the host checks).
template <typename StateT>
__global__ void __launch_bounds__(256)
adamw_kernel(__nv_bfloat16 *__restrict__ w, const __nv_bfloat16 *__restrict__ g,
             StateT *__restrict__ m, StateT *__restrict__ v, uint64_t n, AdamArgs a) {
  const uint64_t n_vec = n / 8;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    uint4 wv = reinterpret_cast<const uint4 *>(w)[i];
    const uint4 gv = reinterpret_cast<const uint4 *>(g)[i];
    State8 mm = load_state8(m, i), vv = load_state8(v, i);
    __nv_bfloat16 *wp = reinterpret_cast<__nv_bfloat16 *>(&wv);
    const __nv_bfloat16 *gp = reinterpret_cast<const __nv_bfloat16 *>(&gv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float x = adamw_element(__bfloat162float(wp[k]), __bfloat162float(gp[k]), mm.f[k],
                                    vv.f[k], a);
      wp[k] = __float2bfloat16_rn(x);
    }
    store_state8(m, i, mm);
    store_state8(v, i, vv);
    reinterpret_cast<uint4 *>(w)[i] = wv;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (uint64_t e = n_vec * 8; e < n; ++e) {
      float mm = load_state(m, e), vv = load_state(v, e);
      const float x = adamw_element(__bfloat162float(w[e]), __bfloat162float(g[e]), mm, vv, a);
      store_state(m, e, mm);
      store_state(v, e, vv);
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
  if (((uintptr_t)weight_bf16 & 15) || ((uintptr_t)grad_bf16 & 15) || ((uintptr_t)exp_avg & 15) ||
      ((uintptr_t)exp_avg_sq & 15)) {
    nz::set_error("nz_adamw_bf16: weight, gradient and moments must be 16-byte aligned");
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

namespace nz {
int decode_update(const void *container, uint64_t container_bytes, const void *frac, uint64_t n,
                  uint64_t operand_cols, int precision, uint32_t S, uint32_t max_unit_words,
                  int canon, const void *grad, void *exp_avg, void *exp_avg_sq, const AdamArgs &adam,
                  void *out_bf16, void *status, cudaStream_t st);
int compress_bf16_fused(const void *in, uint64_t n, int precision, uint32_t LS, uint32_t cols,
                        void *frac_out, void *container, uint64_t container_cap, void *scratch,
                        uint64_t scratch_bytes, cudaStream_t st);
uint64_t compress_fused_scratch_bytes(uint64_t n, uint32_t LS);
}  // namespace nz

extern "C" uint64_t nz_adamw_compressed_scratch_bytes(uint64_t n, uint32_t lane_symbols) {
  if (!nz::valid_lane_symbols(lane_symbols)) return 0;
  // the updated bf16 weights, then the compressor's own scratch
  return nz::align16(2 * n) + nz::compress_fused_scratch_bytes(n, lane_symbols);
}

extern "C" int nz_adamw_compressed_bf16(const void *container, uint64_t container_bytes,
                                        const void *frac_in, uint64_t n, uint64_t operand_cols,
                                        int precision, uint32_t lane_symbols,
                                        uint32_t max_unit_words, int canonical_nan,
                                        const void *grad_bf16, void *exp_avg_bf16,
                                        void *exp_avg_sq_bf16, float lr, float beta1, float beta2,
                                        float eps, float weight_decay, uint32_t step,
                                        float grad_scale, void *frac_out, void *container_out,
                                        uint64_t container_cap, void *scratch,
                                        uint64_t scratch_bytes, void *status, void *stream) {
  if (!nz::valid_precision(precision) || !nz::valid_lane_symbols(lane_symbols)) {
    nz::set_error("nz_adamw_compressed_bf16: bad precision %d or lane_symbols %u", precision,
                  lane_symbols);
    return NZ_E_ARG;
  }
  if (n == 0 || n >= (1ull << 32) || step == 0) {
    nz::set_error("nz_adamw_compressed_bf16: between 1 and 2^32 - 1 elements, step >= 1");
    return NZ_E_ARG;
  }
  if (operand_cols) {
    const uint64_t c = operand_cols;
    if (c % 64 || n % (4 * c) || (c / 64) % (lane_symbols / 8) || c >= (1ull << 31)) {
      nz::set_error("nz_adamw_compressed_bf16: %llu elements in rows of %llu are not in operand "
                    "order for lane_symbols %u", (unsigned long long)n, (unsigned long long)c,
                    lane_symbols);
      return NZ_E_ARG;
    }
  } else if (n % 8) {
    // the fused path moves 8 elements (16 bytes) of gradient and moments per lane
    nz::set_error("nz_adamw_compressed_bf16: the element count must be a multiple of 8");
    return NZ_E_ARG;
  }
  if (!container || ((uintptr_t)container & 15) || !frac_in || ((uintptr_t)frac_in & 7) ||
      !grad_bf16 || ((uintptr_t)grad_bf16 & 15) || !exp_avg_bf16 || ((uintptr_t)exp_avg_bf16 & 15) ||
      !exp_avg_sq_bf16 || ((uintptr_t)exp_avg_sq_bf16 & 15) || !frac_out || ((uintptr_t)frac_out & 7) ||
      !container_out || ((uintptr_t)container_out & 15) || !scratch || ((uintptr_t)scratch & 15)) {
    nz::set_error("nz_adamw_compressed_bf16: null or misaligned pointer (containers, gradient, "
                  "moments and scratch 16-byte, fractions 8-byte aligned)");
    return NZ_E_ARG;
  }
  const uint64_t need = nz_adamw_compressed_scratch_bytes(n, lane_symbols);
  if (scratch_bytes < need) {
    nz::set_error("nz_adamw_compressed_bf16: scratch of %llu bytes is smaller than the %llu required",
                  (unsigned long long)scratch_bytes, (unsigned long long)need);
    return NZ_E_CAPACITY;
  }
  if (container_bytes < nz::payload_offset(nz::unit_count(n, lane_symbols))) {
    nz::set_error("nz_adamw_compressed_bf16: container too short");
    return NZ_E_FORMAT;
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
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t *w_new = (uint8_t *)scratch;
  uint8_t *rest = w_new + nz::align16(2 * n);
  int rc = nz::decode_update(container, container_bytes, frac_in, n, operand_cols, precision,
                             lane_symbols, max_unit_words, canonical_nan, grad_bf16, exp_avg_bf16,
                             exp_avg_sq_bf16, a, w_new, status, st);
  if (rc) return rc;
  return nz::compress_bf16_fused(w_new, n, precision, lane_symbols, (uint32_t)operand_cols, frac_out,
                                 container_out, container_cap, rest, scratch_bytes - nz::align16(2 * n),
                                 st);
}
