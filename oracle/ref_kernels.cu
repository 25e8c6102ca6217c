// TEST INFRASTRUCTURE ONLY: runs the reference's own split / merge kernels.
//
// This file holds no reference code.  It includes the reference's kernel
// header (cuda/kernels.cuh of BorealisAI/neuzip) from where the reference
// tree lies -- the build recipe (oracle/Makefile, target `ref`) puts that
// directory on the include path, together with a directory of empty
// nvcomp headers: the header includes nvcomp (cuda/kernels.cuh:13-17) but the two
// kernels use none of it.  The kernels are instantiated exactly as the
// reference's Manager does for bf16 tensors:
//   kernel_aligned_split<at::BFloat16, uint8_t, uint16_t, 7, 8, s, 1024, tpn, normalized>
//     (cuda/high_level.cu:95-101, type arguments :149-150)
//   kernel_aligned_merge<...same...>   (cuda/high_level.cu:194-201)
// with THREADS = 1024, grid = ceil(n / 1024), for s in {0, 1, 3, 7}.
// normalized=false uses tpn = 1024 (cuda/high_level.cu:97-98).  normalized=true
// is instantiated for the group sizes for which the reference's block reduction
// is well defined (up to one warp, and the whole block); groups of 64 to 512
// threads race inside the reference kernel and are left out.
//
// The resulting library (oracle/_ref/libnz_ref_kernels.so) is loaded only by
// the GPU parity tests, which require the CPU oracle and the product's kernels
// to reproduce its outputs bit for bit.  Callers must pass a size that is a
// multiple of 1024 and buffers sized as the reference sizes them
// (cuda/high_level.cu:81-93): the reference kernels do not guard their tail.
#include "kernels.cuh"

namespace {

constexpr int kThreads = 1024;   // THREADS of the reference build

template <int S, int TPN, bool NORM>
void run_split(void *in, uint8_t *exp, uint8_t *frac, uint8_t *norm, size_t n, cudaStream_t st) {
  const int blocks = (int)((n + kThreads - 1) / kThreads);
  kernel_aligned_split<at::BFloat16, uint8_t, uint16_t, 7, 8, S, kThreads, TPN, NORM>
      <<<blocks, kThreads, 0, st>>>((at::BFloat16 *)in, exp, frac, norm, n);
}

template <int S, int TPN, bool NORM>
void run_merge(void *out, uint8_t *exp, uint8_t *frac, uint8_t *norm, size_t n, cudaStream_t st) {
  const int blocks = (int)((n + kThreads - 1) / kThreads);
  kernel_aligned_merge<at::BFloat16, uint8_t, uint16_t, 7, 8, S, kThreads, TPN, NORM>
      <<<blocks, kThreads, 0, st>>>((at::BFloat16 *)out, exp, frac, norm, n);
}

template <int S>
int dispatch(bool split, int group, void *data, uint8_t *exp, uint8_t *frac, uint8_t *norm,
             size_t n, cudaStream_t st) {
#define NZREF_CASE(G, TPN, NORM)                                              \
  case G:                                                                     \
    if (split) run_split<S, TPN, NORM>(data, exp, frac, norm, n, st);         \
    else run_merge<S, TPN, NORM>(data, exp, frac, norm, n, st);               \
    return 0;
  switch (group) {
    NZREF_CASE(0, 1024, false)
    NZREF_CASE(1, 1, true)
    NZREF_CASE(2, 2, true)
    NZREF_CASE(4, 4, true)
    NZREF_CASE(8, 8, true)
    NZREF_CASE(16, 16, true)
    NZREF_CASE(32, 32, true)
    NZREF_CASE(1024, 1024, true)
    default: return -1;
  }
#undef NZREF_CASE
}

int run(bool split, int precision, int group, void *data, void *exp, void *frac, void *norm,
        size_t n, void *stream) {
  if (n == 0 || n % kThreads) return -2;          // the reference kernels do not guard the tail
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  switch (precision) {
    case 0: rc = dispatch<0>(split, group, data, (uint8_t *)exp, (uint8_t *)frac, (uint8_t *)norm, n, st); break;
    case 1: rc = dispatch<1>(split, group, data, (uint8_t *)exp, (uint8_t *)frac, (uint8_t *)norm, n, st); break;
    case 3: rc = dispatch<3>(split, group, data, (uint8_t *)exp, (uint8_t *)frac, (uint8_t *)norm, n, st); break;
    case 7: rc = dispatch<7>(split, group, data, (uint8_t *)exp, (uint8_t *)frac, (uint8_t *)norm, n, st); break;
    default: return -1;
  }
  if (rc) return rc;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

// group = 0: normalized=false (the Manager_f{s}_n0 classes); otherwise the
// normaliser group size.  All pointers are device pointers; `norm` must hold
// ceil(n / 1024) bytes for group 0 and ceil(n / group) bytes otherwise.
extern "C" int nzref_split(int precision, int group, void *in_bf16, void *exp_out, void *frac_out,
                           void *norm_out, size_t n, void *stream) {
  return run(true, precision, group, in_bf16, exp_out, frac_out, norm_out, n, stream);
}

extern "C" int nzref_merge(int precision, int group, void *out_bf16, void *exp_in, void *frac_in,
                           void *norm_in, size_t n, void *stream) {
  return run(false, precision, group, out_bf16, exp_in, frac_in, norm_in, n, stream);
}
