// Operand order: storing a [rows, cols] bf16 matrix so that the decoder produces
// tensor-core operand tiles (see operand_index in nz_decode_core.cuh), and reading
// it back in the ordinary row-major order.
//
// The codec itself is unchanged: a matrix in operand order is the flat codec applied
// to a permutation of the matrix.  The reference never exposes its compressed bytes
// (they live inside its C++ cache, cuda/high_level.cu:35-43), so the order of the
// elements inside the stored streams is this library's to choose; what write / read
// return (cuda/high_level.cu:132-162, :223-250) is unchanged.
#include "nz_decode_core.cuh"

namespace nz {

int decode_operand(const void *container, uint64_t container_bytes, const void *frac, uint64_t rows,
                   uint64_t cols, int precision, uint32_t S, uint32_t max_unit_words, int canon,
                   void *out_bf16, void *status, cudaStream_t st);

// Stream order <- row-major: one 16-byte chunk (8 elements of one row) per thread.
__global__ void __launch_bounds__(256)
to_operand_order_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out, uint64_t n_chunks,
                        uint32_t cols) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_chunks) return;
  out[i] = __ldcs(in + operand_index(i * 8, cols) / 8);
}

static bool operand_shape_ok(uint64_t rows, uint64_t cols, uint32_t S) {
  if (rows == 0 || rows % 4 || cols == 0 || cols % 64 || !valid_lane_symbols(S)) return false;
  return (cols / 64) % (S / 8) == 0 && cols < (1ull << 31);
}

}  // namespace nz

extern "C" uint64_t nz_compress_operand_scratch_bytes(uint64_t rows, uint64_t cols,
                                                      uint32_t lane_symbols) {
  const uint64_t n = rows * cols;
  const uint64_t base = nz_compress_scratch_bytes(n, lane_symbols);
  if (base == 0) return 0;
  return nz::align16(base) + nz::align16(2 * n);     // + the permuted copy
}

extern "C" int nz_compress_bf16_operand(const void *in_bf16, uint64_t rows, uint64_t cols,
                                        int precision, uint32_t lane_symbols, void *frac_out,
                                        void *container, uint64_t container_cap, void *scratch,
                                        uint64_t scratch_bytes, void *stream) {
  if (!nz::operand_shape_ok(rows, cols, lane_symbols)) {
    nz::set_error("nz_compress_bf16_operand: a [%llu, %llu] matrix with lane_symbols %u cannot be "
                  "stored in operand order (rows must be a multiple of 4, columns of 64, "
                  "lane_symbols / 8 must divide columns / 64)",
                  (unsigned long long)rows, (unsigned long long)cols, lane_symbols);
    return NZ_E_ARG;
  }
  const uint64_t n = rows * cols;
  if (n >= (1ull << 32)) {
    nz::set_error("nz_compress_bf16_operand: tensors of 2^32 or more elements are not supported");
    return NZ_E_ARG;
  }
  if (!in_bf16 || ((uintptr_t)in_bf16 & 15) || !scratch || ((uintptr_t)scratch & 15)) {
    nz::set_error("nz_compress_bf16_operand: input and scratch must be 16-byte aligned device pointers");
    return NZ_E_ARG;
  }
  const uint64_t base = nz::align16(nz_compress_scratch_bytes(n, lane_symbols));
  if (scratch_bytes < base + nz::align16(2 * n)) {
    nz::set_error("nz_compress_bf16_operand: scratch of %llu bytes is smaller than the %llu required",
                  (unsigned long long)scratch_bytes,
                  (unsigned long long)(base + nz::align16(2 * n)));
    return NZ_E_CAPACITY;
  }
  uint8_t *permuted = (uint8_t *)scratch + base;
  const uint64_t chunks = n / 8;
  nz::to_operand_order_kernel<<<(unsigned)((chunks + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint4 *)in_bf16, (uint4 *)permuted, chunks, (uint32_t)cols);
  NZ_LAUNCH_CHECK("to_operand_order_kernel");
  return nz_compress_bf16(permuted, n, precision, lane_symbols, frac_out, container, container_cap,
                          scratch, base, stream);
}

extern "C" int nz_decompress_bf16_operand(const void *container, uint64_t container_bytes,
                                          const void *frac_in, uint64_t rows, uint64_t cols,
                                          int precision, uint32_t lane_symbols,
                                          uint32_t max_unit_words, int canonical_nan,
                                          void *out_bf16, void *status, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_decompress_bf16_operand: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  if (!nz::operand_shape_ok(rows, cols, lane_symbols) || rows * cols >= (1ull << 32)) {
    nz::set_error("nz_decompress_bf16_operand: a [%llu, %llu] matrix with lane_symbols %u is not "
                  "in operand order", (unsigned long long)rows, (unsigned long long)cols,
                  lane_symbols);
    return NZ_E_ARG;
  }
  if (!container || ((uintptr_t)container & 15) || !out_bf16 || !frac_in ||
      ((uintptr_t)out_bf16 & 15) || ((uintptr_t)frac_in & 7)) {
    nz::set_error("nz_decompress_bf16_operand: container and output must be 16-byte, fractions "
                  "8-byte aligned");
    return NZ_E_ARG;
  }
  return nz::decode_operand(container, container_bytes, frac_in, rows, cols, precision,
                            lane_symbols, max_unit_words, canonical_nan, out_bf16, status,
                            (cudaStream_t)stream);
}
