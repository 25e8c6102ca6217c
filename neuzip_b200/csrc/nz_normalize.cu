// Block normaliser (normalizer_size > 0): per-group scaling of a bf16 tensor
// before the split and the inverse after the merge.
//
// Intended semantics of the normalized=true path of the reference kernels
// (cuda/kernels.cuh:94-118 in kernel_aligned_split, :188-191 and :208-216 in
// kernel_aligned_merge).  For every run of `group` consecutive elements:
//   absmax = max |float(v)|, elements past the end count as 0;
//   scale  = 1.<23 mantissa bits of absmax>, a float in [1, 2);
//   v'     = bf16(float(v) / scale)            (round to nearest even);
//   stored byte = top 8 bits of that mantissa.
// Reading rebuilds the scale from the stored byte only and returns
//   bf16(scale8 * float(v')).
// The reference reduces with a cub::BlockReduce sized for `group` threads inside a
// 1024-thread block, which only works for groups of up to 32 and of 1024 threads;
// this file implements what that code means, for every group size.
#include <cuda_bf16.h>

#include "nz_common.cuh"

namespace nz {

constexpr int kNormThreads = 128;          // x 8 elements = 1024 = the largest group

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ uint32_t float_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// One block = 1024 consecutive elements; thread t owns elements 8t..8t+7.
__global__ void __launch_bounds__(kNormThreads)
normalize_groups_kernel(const uint16_t *__restrict__ in, uint64_t n, uint32_t group,
                        uint16_t *__restrict__ out, uint8_t *__restrict__ normalizers) {
  __shared__ float warp_max[kNormThreads / 32];
  const uint64_t base = (uint64_t)blockIdx.x * 1024 + threadIdx.x * 8;
  uint32_t v[8];
  if (base + 8 <= n) {
    const uint4 q = *reinterpret_cast<const uint4 *>(in + base);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = (w[k >> 1] >> ((k & 1) * 16)) & 0xFFFFu;
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = (base + k < n) ? in[base + k] : 0u;
  }
  float a[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = bf16_bits_to_float(v[k] & 0x7FFFu);
  // absmax of the group each element belongs to
  float gmax[8];
  if (group < 8) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float m = 0.0f;
      const int first = k - (k % (int)group);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j >= first && j < first + (int)group && a[j] > m) m = a[j];
      gmax[k] = m;
    }
  } else {
    float m = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (a[k] > m) m = a[k];
    const uint32_t threads_per_group = group / 8;          // 1 .. 128
    // within a warp: butterfly over the lanes of the group
    for (uint32_t o = 1; o < threads_per_group && o < 32; o <<= 1) {
      const float other = __shfl_xor_sync(0xFFFFFFFFu, m, o);
      if (other > m) m = other;
    }
    if (threads_per_group > 32) {                           // groups of 512 or 1024 elements
      if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
      __syncthreads();
      const uint32_t warps_per_group = threads_per_group / 32;
      const uint32_t w0 = (threadIdx.x >> 5) / warps_per_group * warps_per_group;
      m = 0.0f;
      for (uint32_t w = 0; w < warps_per_group; ++w)
        if (warp_max[w0 + w] > m) m = warp_max[w0 + w];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) gmax[k] = m;
  }
  uint32_t o[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t frac = __float_as_uint(gmax[k]) & 0x007FFFFFu;
    const float scale = __uint_as_float(0x3F800000u | frac);
    o[k] = float_to_bf16_bits(__fdiv_rn(bf16_bits_to_float(v[k]), scale));
    const uint64_t e = base + k;
    if (e < n && e % group == 0) normalizers[e / group] = (uint8_t)(frac >> 15);
  }
  if (base + 8 <= n) {
    *reinterpret_cast<uint4 *>(out + base) =
        make_uint4(o[0] | (o[1] << 16), o[2] | (o[3] << 16), o[4] | (o[5] << 16), o[6] | (o[7] << 16));
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (base + k < n) out[base + k] = (uint16_t)o[k];
  }
}

__global__ void __launch_bounds__(256)
denormalize_groups_kernel(uint16_t *__restrict__ v, uint64_t n, uint32_t group,
                          const uint8_t *__restrict__ normalizers) {
  const uint64_t n_vec = n / 8;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    uint4 q = reinterpret_cast<uint4 *>(v)[i];
    uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint64_t e = i * 8 + k;
      const float scale = __uint_as_float(0x3F800000u | ((uint32_t)normalizers[e / group] << 15));
      const uint32_t b = (w[k >> 1] >> ((k & 1) * 16)) & 0xFFFFu;
      const uint32_t r = float_to_bf16_bits(scale * bf16_bits_to_float(b));
      w[k >> 1] = (k & 1) ? ((w[k >> 1] & 0x0000FFFFu) | (r << 16)) : ((w[k >> 1] & 0xFFFF0000u) | r);
    }
    reinterpret_cast<uint4 *>(v)[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (uint64_t e = n_vec * 8; e < n; ++e) {
      const float scale = __uint_as_float(0x3F800000u | ((uint32_t)normalizers[e / group] << 15));
      v[e] = (uint16_t)float_to_bf16_bits(scale * bf16_bits_to_float(v[e]));
    }
  }
}

static bool valid_group(uint32_t g) { return g >= 1 && g <= 1024 && (g & (g - 1)) == 0; }

}  // namespace nz

extern "C" uint64_t nz_normalizer_bytes(uint64_t n, uint32_t group) {
  if (!nz::valid_group(group)) return 0;
  return (n + group - 1) / group;
}

extern "C" int nz_normalize_bf16(const void *in_bf16, uint64_t n, uint32_t group, void *out_bf16,
                                 void *normalizers, void *stream) {
  if (!nz::valid_group(group)) {
    nz::set_error("nz_normalize_bf16: group must be a power of two in [1, 1024] (got %u)", group);
    return NZ_E_ARG;
  }
  if (n == 0) return NZ_OK;
  if (!in_bf16 || !out_bf16 || !normalizers || ((uintptr_t)in_bf16 & 15) || ((uintptr_t)out_bf16 & 15)) {
    nz::set_error("nz_normalize_bf16: null pointer or tensors not 16-byte aligned");
    return NZ_E_ARG;
  }
  const uint64_t blocks = (n + 1023) / 1024;
  if (blocks > 0x7FFFFFFFull) {
    nz::set_error("nz_normalize_bf16: tensor too large");
    return NZ_E_ARG;
  }
  nz::normalize_groups_kernel<<<(unsigned)blocks, nz::kNormThreads, 0, (cudaStream_t)stream>>>(
      (const uint16_t *)in_bf16, n, group, (uint16_t *)out_bf16, (uint8_t *)normalizers);
  NZ_LAUNCH_CHECK("normalize_groups_kernel");
  return NZ_OK;
}

extern "C" int nz_denormalize_bf16(void *inout_bf16, uint64_t n, uint32_t group,
                                   const void *normalizers, void *stream) {
  if (!nz::valid_group(group)) {
    nz::set_error("nz_denormalize_bf16: group must be a power of two in [1, 1024] (got %u)", group);
    return NZ_E_ARG;
  }
  if (n == 0) return NZ_OK;
  if (!inout_bf16 || !normalizers || ((uintptr_t)inout_bf16 & 15)) {
    nz::set_error("nz_denormalize_bf16: null pointer or tensor not 16-byte aligned");
    return NZ_E_ARG;
  }
  uint64_t blocks = (n / 8 + 255) / 256;
  const uint64_t cap = (uint64_t)nz::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  nz::denormalize_groups_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (uint16_t *)inout_bf16, n, group, (const uint8_t *)normalizers);
  NZ_LAUNCH_CHECK("denormalize_groups_kernel");
  return NZ_OK;
}
