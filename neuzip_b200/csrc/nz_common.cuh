// Shared definitions of the neuzip_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/neuzip_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "neuzip_b200 kernels are written for sm_100a (B200) only"
#endif

namespace nz {

constexpr uint32_t kMinProbBits = 9;          // lowest resolution a container may carry
constexpr uint32_t kDefaultLowProbBits = 10;  // resolution for up to 32 distinct symbols
constexpr uint32_t kMaxProbBits = 12;
constexpr uint32_t kStateLow = 1u << 16;
constexpr uint32_t kMagic = 0x31525A4Eu;  // "NZR1"
constexpr uint32_t kHeaderBytes = 64;
constexpr uint32_t kFreqOffset = 64;
constexpr uint32_t kOffsetsOffset = 576;
constexpr uint32_t kRawFlag = 0x80000000u;
constexpr uint32_t kMaxLaneSymbols = 1024;
constexpr uint32_t kMaxDynamicSmem = 227u * 1024u;   // dynamic shared memory a CTA can opt in to
constexpr int kMaxDeviceOrdinals = 64;               // per-device bookkeeping tables

// Container header; must match struct nzo_header of the specification.
struct Header {
  uint32_t magic;
  uint32_t version;
  uint64_t n_symbols;
  uint32_t lane_symbols;
  uint32_t len_quantum;
  uint32_t n_units;
  uint32_t prob_bits;
  uint64_t payload_offset;
  uint64_t payload_words;
  uint64_t total_bytes;
  uint32_t n_raw_units;
  uint32_t max_coded_unit_words;
};
static_assert(sizeof(Header) == kHeaderBytes, "header layout");

__host__ __device__ inline uint64_t align16(uint64_t x) { return (x + 15) & ~uint64_t(15); }
__host__ __device__ inline uint32_t len_quantum(uint32_t S) { return (S + 767) / 768; }
__host__ __device__ inline uint32_t lane_cap_words(uint32_t S) {
  uint32_t a = 255u * len_quantum(S), b = S / 2;
  return a < b ? a : b;
}
__host__ __device__ inline uint64_t unit_count(uint64_t n, uint32_t S) {
  uint64_t U = 32ull * S;
  return (n + U - 1) / U;
}
__host__ __device__ inline uint64_t payload_offset(uint64_t n_units) {
  return align16(kOffsetsOffset + 4 * (n_units + 1));
}
inline bool valid_precision(int s) { return s == 0 || s == 1 || s == 3 || s == 7; }
inline bool valid_lane_symbols(uint32_t S) { return S != 0 && (S & 7) == 0 && S <= kMaxLaneSymbols; }

// Per-thread last-error text.
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t err, const char *what);

#define NZ_CUDA_TRY(expr)                                   \
  do {                                                      \
    cudaError_t nz_err__ = (expr);                          \
    if (nz_err__ != cudaSuccess) return ::nz::cuda_fail(nz_err__, #expr); \
  } while (0)

#define NZ_LAUNCH_CHECK(name)                               \
  do {                                                      \
    cudaError_t nz_err__ = cudaGetLastError();              \
    if (nz_err__ != cudaSuccess) return ::nz::cuda_fail(nz_err__, name); \
  } while (0)

int sm_count();

// Launch with programmatic stream serialisation: the grid may be set up while the kernel
// before it in the stream is still running, which hides the launch latency between the
// short kernels of a pipeline.  Every kernel launched this way starts with
// dependent_wait(), which waits for the preceding grid to complete (and its memory to be
// visible) before anything is read or written, so stream order is preserved; it calls
// dependent_trigger() where the next grid may come in: a long kernel near its end (blocks
// of the next grid that are resident early only wait, and hold registers and shared
// memory meanwhile), a single-block kernel at once.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), unsigned grid, unsigned block,
                                    size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
// Both are no-ops for an ordinary launch.
__device__ __forceinline__ void dependent_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void dependent_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// AdamW step on one element, in fp32: the one formula shared by the stand-alone update
// kernel and by the decoder's update mode, so that both give the same bits.
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale;
};
__device__ __forceinline__ float adamw_element(float w, float g, float &m, float &v,
                                               const AdamArgs &a) {
  // every operation is spelled out with its rounding, so that the compiler cannot contract
  // multiplies and adds differently in the kernels that share the formula
  const float grad = __fmul_rn(g, a.grad_scale);
  m = __fmaf_rn(a.beta1, m, __fmul_rn(__fsub_rn(1.0f, a.beta1), grad));
  v = __fmaf_rn(a.beta2, v, __fmul_rn(__fmul_rn(__fsub_rn(1.0f, a.beta2), grad), grad));
  w = __fmul_rn(w, __fsub_rn(1.0f, __fmul_rn(a.lr, a.weight_decay)));
  const float denom = __fadd_rn(__fsqrt_rn(__fdiv_rn(v, a.bias2)), a.eps);
  w = __fsub_rn(w, __fdiv_rn(__fmul_rn(__fdiv_rn(a.lr, a.bias1), m), denom));
  return w;
}

}  // namespace nz
