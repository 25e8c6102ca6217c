// bf16 split / merge kernels: bf16 <-> exponent byte stream + packed
// (sign | top-s mantissa bits) stream.
//
// Semantics follow kernel_aligned_split / kernel_aligned_merge of the
// reference (cuda/kernels.cuh:120-155 and :197-216, normalized=false): the
// 15-bit magnitude is rounded half-up at bit (7-s), the carry may ripple into
// the exponent byte (255 wraps to 0), fields are (s+1) bits wide and packed
// MSB-first, padded with zero bits.  Unlike the reference, one thread handles
// 64/(s+1) consecutive elements with 128-bit loads and 64-bit stores, indices
// are 64-bit and the tail is guarded.
#include "nz_common.cuh"

namespace nz {

template <int S>
struct SplitGeom {
  static constexpr int kFieldBits = S + 1;
  static constexpr int kVecs = 8 / kFieldBits;     // 16-byte loads per thread
  static constexpr int kElems = 8 * kVecs;         // elements per thread
};

// One element: returns the (s+1)-bit field, stores the exponent byte.
template <int S>
__device__ __forceinline__ uint32_t split_one(uint32_t val, uint32_t &exp) {
  const uint32_t sign = (val >> 15) & 1u;
  const uint32_t mag = val & 0x7FFFu;
  uint32_t keep = mag >> (7 - S);
  if (S < 7) keep += (mag >> (6 - S)) & 1u;
  keep &= (1u << (8 + S)) - 1u;
  exp = keep >> S;
  return (sign << S) | (keep & ((1u << S) - 1u));
}

template <int S>
__global__ void __launch_bounds__(256)
split_kernel(const uint16_t *__restrict__ in, uint8_t *__restrict__ exp_out,
             uint8_t *__restrict__ frac_out, uint64_t n) {
  using G = SplitGeom<S>;
  const uint64_t n_groups = n / G::kElems;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
    const uint4 *src = reinterpret_cast<const uint4 *>(in + g * G::kElems);
    uint4 v[G::kVecs];
#pragma unroll
    for (int k = 0; k < G::kVecs; ++k) v[k] = __ldcs(src + k);
    uint64_t packed = 0;  // big-endian bit order: first element in the top bits
#pragma unroll
    for (int k = 0; k < G::kVecs; ++k) {
      const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
      uint32_t elo = 0, ehi = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t val = (w[j >> 1] >> ((j & 1) * 16)) & 0xFFFFu;
        uint32_t e;
        const uint32_t field = split_one<S>(val, e);
        packed = (packed << G::kFieldBits) | field;
        if (j < 4) elo |= e << (8 * j); else ehi |= e << (8 * (j - 4));
      }
      reinterpret_cast<uint2 *>(exp_out + g * G::kElems)[k] = make_uint2(elo, ehi);
    }
    // byte 0 of the output holds the first elements: store big-endian
    const uint32_t hi = (uint32_t)(packed >> 32), lo = (uint32_t)packed;
    reinterpret_cast<uint2 *>(frac_out)[g] =
        make_uint2(__byte_perm(hi, 0, 0x0123), __byte_perm(lo, 0, 0x0123));
  }
  // Tail: fewer than kElems elements, one thread, byte stores.
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const uint64_t first = n_groups * G::kElems;
    uint32_t acc = 0, bits = 0;
    uint64_t byte = first * G::kFieldBits / 8;
    for (uint64_t i = first; i < n; ++i) {
      uint32_t e;
      const uint32_t field = split_one<S>(in[i], e);
      exp_out[i] = (uint8_t)e;
      acc = (acc << G::kFieldBits) | field;
      bits += G::kFieldBits;
      if (bits == 8) {
        frac_out[byte++] = (uint8_t)acc;
        acc = 0;
        bits = 0;
      }
    }
    if (bits) frac_out[byte] = (uint8_t)(acc << (8 - bits));
  }
}

// One element of the merge: field -> bf16 bits.
template <int S>
__device__ __forceinline__ uint32_t merge_one(uint32_t field, uint32_t exp, bool canon) {
  const uint32_t frac = (field & ((1u << S) - 1u)) << (7 - S);
  const uint32_t sign = (field >> S) & 1u;
  uint32_t v = (exp << 7) | frac;
  if (canon && exp == 255u && frac != 0u) return 0x7FFFu;
  return v | (sign << 15);
}

template <int S>
__global__ void __launch_bounds__(256)
merge_kernel(const uint8_t *__restrict__ exp_in, const uint8_t *__restrict__ frac_in,
             uint16_t *__restrict__ out, uint64_t n, int canon) {
  using G = SplitGeom<S>;
  const uint64_t n_groups = n / G::kElems;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
    const uint2 f = __ldcs(reinterpret_cast<const uint2 *>(frac_in) + g);
    const uint64_t packed =
        ((uint64_t)__byte_perm(f.x, 0, 0x0123) << 32) | __byte_perm(f.y, 0, 0x0123);
#pragma unroll
    for (int k = 0; k < G::kVecs; ++k) {
      const uint2 e = __ldcs(reinterpret_cast<const uint2 *>(exp_in + g * G::kElems) + k);
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int idx = k * 8 + j;
        const uint32_t field =
            (uint32_t)(packed >> (64 - G::kFieldBits * (idx + 1))) & ((1u << G::kFieldBits) - 1u);
        const uint32_t ex = ((j < 4 ? e.x : e.y) >> (8 * (j & 3))) & 0xFFu;
        const uint32_t v = merge_one<S>(field, ex, canon != 0);
        if (j & 1) w[j >> 1] |= v << 16; else w[j >> 1] = v;
      }
      __stcs(reinterpret_cast<uint4 *>(out + g * G::kElems) + k, make_uint4(w[0], w[1], w[2], w[3]));
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (uint64_t i = n_groups * G::kElems; i < n; ++i) {
      const uint64_t bit = i * G::kFieldBits;
      const uint32_t shift = 7 - S - (uint32_t)(bit & 7);
      const uint32_t field = ((uint32_t)frac_in[bit >> 3] >> shift) & ((1u << G::kFieldBits) - 1u);
      out[i] = (uint16_t)merge_one<S>(field, exp_in[i], canon != 0);
    }
  }
}

template <int S>
static int launch_split(const void *in, uint64_t n, void *exp_out, void *frac_out, cudaStream_t st) {
  using G = SplitGeom<S>;
  const uint64_t groups = n / G::kElems;
  uint64_t blocks = (groups + 255) / 256;
  const uint64_t cap = (uint64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  split_kernel<S><<<(unsigned)blocks, 256, 0, st>>>((const uint16_t *)in, (uint8_t *)exp_out,
                                                     (uint8_t *)frac_out, n);
  NZ_LAUNCH_CHECK("split_kernel");
  return NZ_OK;
}

template <int S>
static int launch_merge(const void *exp_in, const void *frac_in, uint64_t n, int canon, void *out,
                        cudaStream_t st) {
  using G = SplitGeom<S>;
  const uint64_t groups = n / G::kElems;
  uint64_t blocks = (groups + 255) / 256;
  const uint64_t cap = (uint64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  merge_kernel<S><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t *)exp_in, (const uint8_t *)frac_in,
                                                     (uint16_t *)out, n, canon);
  NZ_LAUNCH_CHECK("merge_kernel");
  return NZ_OK;
}

int split_bf16(const void *in, uint64_t n, int precision, void *exp_out, void *frac_out,
               cudaStream_t st) {
  switch (precision) {
    case 0: return launch_split<0>(in, n, exp_out, frac_out, st);
    case 1: return launch_split<1>(in, n, exp_out, frac_out, st);
    case 3: return launch_split<3>(in, n, exp_out, frac_out, st);
    default: return launch_split<7>(in, n, exp_out, frac_out, st);
  }
}

}  // namespace nz

extern "C" int nz_split_bf16(const void *in_bf16, uint64_t n, int precision, void *exp_out,
                             void *frac_out, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_split_bf16: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  if (n == 0) return NZ_OK;
  if (!in_bf16 || !exp_out || !frac_out) {
    nz::set_error("nz_split_bf16: null pointer");
    return NZ_E_ARG;
  }
  if (((uintptr_t)in_bf16 & 15) || ((uintptr_t)exp_out & 7) || ((uintptr_t)frac_out & 7)) {
    nz::set_error("nz_split_bf16: input must be 16-byte and outputs 8-byte aligned");
    return NZ_E_ARG;
  }
  return nz::split_bf16(in_bf16, n, precision, exp_out, frac_out, (cudaStream_t)stream);
}

extern "C" int nz_merge_bf16(const void *exp_in, const void *frac_in, uint64_t n, int precision,
                             int canonical_nan, void *out_bf16, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_merge_bf16: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  if (n == 0) return NZ_OK;
  if (!exp_in || !frac_in || !out_bf16) {
    nz::set_error("nz_merge_bf16: null pointer");
    return NZ_E_ARG;
  }
  if (((uintptr_t)out_bf16 & 15) || ((uintptr_t)exp_in & 7) || ((uintptr_t)frac_in & 7)) {
    nz::set_error("nz_merge_bf16: output must be 16-byte and inputs 8-byte aligned");
    return NZ_E_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  switch (precision) {
    case 0: return nz::launch_merge<0>(exp_in, frac_in, n, canonical_nan, out_bf16, st);
    case 1: return nz::launch_merge<1>(exp_in, frac_in, n, canonical_nan, out_bf16, st);
    case 3: return nz::launch_merge<3>(exp_in, frac_in, n, canonical_nan, out_bf16, st);
    default: return nz::launch_merge<7>(exp_in, frac_in, n, canonical_nan, out_bf16, st);
  }
}
