// Library-level entry points: version, error text, device check, size
// helpers and the whole-tensor compress path.
#include <stdarg.h>
#include <string.h>

#include "nz_common.cuh"

namespace nz {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t err, const char *what) {
  set_error("CUDA error %d (%s) in %s", (int)err, cudaGetErrorString(err), what);
  return NZ_E_CUDA;
}

int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    cached = v;
    cached_dev = dev;
  }
  return cached;
}

int compress_bf16_fused(const void *in, uint64_t n, int precision, uint32_t LS, uint32_t cols,
                        void *frac_out, void *container, uint64_t container_cap, void *scratch,
                        uint64_t scratch_bytes, cudaStream_t st);
uint64_t compress_fused_scratch_bytes(uint64_t n, uint32_t LS);

}  // namespace nz

extern "C" int nz_version(void) { return 100; }

extern "C" const char *nz_last_error(void) { return nz::g_error; }

extern "C" int nz_device_check(void) {
  int dev = 0, major = 0;
  NZ_CUDA_TRY(cudaGetDevice(&dev));
  NZ_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) {
    nz::set_error("device %d has compute capability %d.x; this library is built for sm_100a only",
                  dev, major);
    return NZ_E_DEVICE;
  }
  return NZ_OK;
}

extern "C" uint64_t nz_frac_bytes(uint64_t n, int precision) {
  if (!nz::valid_precision(precision)) return 0;
  return (n * (uint64_t)(precision + 1) + 7) / 8;
}

extern "C" uint32_t nz_default_lane_symbols(int precision) {
  // Short lane streams decode with more parallelism (and leave a warp's units of the
  // compressor and the decoder more shared memory), long ones cost fewer bytes of per-lane
  // state.  Lossy modes store fewer bytes in total, so the same absolute overhead weighs
  // more there: the two coarsest get longer streams, as long as the decoder keeps its rate
  // (on a B200 it falls by a quarter from 512 to 640 symbols: fewer resident warps).
  switch (precision) {
    case 7: return 256;
    case 3: return 256;
    case 1: return 384;
    case 0: return 512;
    default: return 0;
  }
}

extern "C" uint64_t nz_compress_scratch_bytes(uint64_t n, uint32_t lane_symbols) {
  if (!nz::valid_lane_symbols(lane_symbols)) return 0;
  return nz::compress_fused_scratch_bytes(n, lane_symbols);
}

extern "C" int nz_compress_bf16(const void *in_bf16, uint64_t n, int precision,
                                uint32_t lane_symbols, void *frac_out, void *container,
                                uint64_t container_cap, void *scratch, uint64_t scratch_bytes,
                                void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_compress_bf16: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  if (!nz::valid_lane_symbols(lane_symbols)) {
    nz::set_error("nz_compress_bf16: lane_symbols must be a multiple of 8 in [8, %u] (got %u)",
                  nz::kMaxLaneSymbols, lane_symbols);
    return NZ_E_ARG;
  }
  if (n >= (1ull << 32)) {
    nz::set_error("nz_compress_bf16: tensors of 2^32 or more elements are not supported");
    return NZ_E_ARG;
  }
  if (!container || !scratch || (n && (!in_bf16 || !frac_out))) {
    nz::set_error("nz_compress_bf16: null pointer");
    return NZ_E_ARG;
  }
  if (((uintptr_t)in_bf16 & 15) || ((uintptr_t)frac_out & 7) || ((uintptr_t)container & 15) ||
      ((uintptr_t)scratch & 15)) {
    nz::set_error("nz_compress_bf16: input, container and scratch must be 16-byte aligned, "
                  "fractions 8-byte aligned");
    return NZ_E_ARG;
  }
  const uint64_t need = nz::compress_fused_scratch_bytes(n, lane_symbols);
  if (scratch_bytes < need) {
    nz::set_error("nz_compress_bf16: scratch of %llu bytes is smaller than the %llu required",
                  (unsigned long long)scratch_bytes, (unsigned long long)need);
    return NZ_E_CAPACITY;
  }
  return nz::compress_bf16_fused(in_bf16, n, precision, lane_symbols, 0, frac_out, container,
                                 container_cap, scratch, scratch_bytes, (cudaStream_t)stream);
}
