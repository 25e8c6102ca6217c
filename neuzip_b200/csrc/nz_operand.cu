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

int compress_bf16_fused(const void *in, uint64_t n, int precision, uint32_t LS, uint32_t cols,
                        void *frac_out, void *container, uint64_t container_cap, void *scratch,
                        uint64_t scratch_bytes, cudaStream_t st);

static bool operand_shape_ok(uint64_t rows, uint64_t cols, uint32_t S) {
  if (rows == 0 || rows % 4 || cols == 0 || cols % 64 || !valid_lane_symbols(S)) return false;
  return (cols / 64) % (S / 8) == 0 && cols < (1ull << 31);
}

}  // namespace nz

extern "C" uint64_t nz_compress_operand_scratch_bytes(uint64_t rows, uint64_t cols,
                                                      uint32_t lane_symbols) {
  return nz_compress_scratch_bytes(rows * cols, lane_symbols);
}

extern "C" int nz_compress_bf16_operand(const void *in_bf16, uint64_t rows, uint64_t cols,
                                        int precision, uint32_t lane_symbols, void *frac_out,
                                        void *container, uint64_t container_cap, void *scratch,
                                        uint64_t scratch_bytes, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_compress_bf16_operand: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
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
  if (!in_bf16 || ((uintptr_t)in_bf16 & 15) || !scratch || ((uintptr_t)scratch & 15) ||
      !container || ((uintptr_t)container & 15) || !frac_out || ((uintptr_t)frac_out & 7)) {
    nz::set_error("nz_compress_bf16_operand: input, container and scratch must be 16-byte aligned "
                  "device pointers, fractions 8-byte aligned");
    return NZ_E_ARG;
  }
  const uint64_t need = nz_compress_scratch_bytes(n, lane_symbols);
  if (scratch_bytes < need) {
    nz::set_error("nz_compress_bf16_operand: scratch of %llu bytes is smaller than the %llu required",
                  (unsigned long long)scratch_bytes, (unsigned long long)need);
    return NZ_E_CAPACITY;
  }
  // the element a coder lane handles is looked up through the operand order: no permuted copy
  return nz::compress_bf16_fused(in_bf16, n, precision, lane_symbols, (uint32_t)cols, frac_out,
                                 container, container_cap, scratch, scratch_bytes,
                                 (cudaStream_t)stream);
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
