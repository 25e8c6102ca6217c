// rANS decoder of the NZR1 container, fused with the bf16 merge.
//
// Replaces nvcomp's ANS decompress followed by kernel_aligned_merge in the
// reference's read path (cuda/high_level.cu:184-201, cuda/kernels.cuh:158-217):
// the decoded exponent bytes stay in registers and are merged with the packed
// fractions straight into the bf16 output, so the exponent stream never makes
// the round trip through HBM.
//
// Work decomposition.  One warp decodes one unit (32 lane streams of S
// symbols).  The unit's coded bytes are staged into the warp's shared-memory
// slot with one bulk asynchronous copy (cp.async.bulk + mbarrier, no
// multicast); each lane then walks its own stream with a private read pointer,
// so a renormalisation costs one predicated 16-bit shared load and no
// warp-wide vote.  A lane produces 8 consecutive tensor elements per step and
// writes them with one 128-bit store; the warp's stores are 512 contiguous
// bytes.  The 4096-entry decode table (symbol | freq << 8 | bias << 20) is
// built once per CTA from the container's frequency table.
//
// Robustness.  Header, offset table and lane lengths are validated before
// use; a malformed container sets bits in the caller's status word and the
// affected units are skipped.  Reads of the coded stream are confined to the
// CTA's shared memory (a guard band behind the last slot absorbs run-away
// pointers), output and fraction addresses never depend on coded data, and
// the wait on the bulk copy is bounded.
#include "nz_common.cuh"

namespace nz {

constexpr uint32_t kLutBytes = kProbScale * 4;
constexpr uint32_t kMaxWaitIters = 1u << 20;

// ------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bulk asynchronous copy global -> this CTA's shared memory (no multicast).
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// ------------------------------------------------------------------ decode
struct LaneState {
  uint32_t x;     // rANS state
  uint32_t p;     // shared address of the next unread stream word
  uint32_t w;     // that word, already loaded
};

// One symbol.  Returns the table entry; the symbol is its low byte.
__device__ __forceinline__ uint32_t decode_step(LaneState &st, uint32_t lut) {
  const uint32_t ent = lds_u32(lut + ((st.x & (kProbScale - 1)) << 2));
  st.x = ((ent >> 8) & 0xFFFu) * (st.x >> kProbBits) + (ent >> 20);
  if (st.x < kStateLow) {
    st.x = (st.x << 16) | st.w;
    st.p += 2;
    st.w = lds_u16(st.p);
  }
  return ent;
}

// Merge two decoded symbols (low bytes of ea, eb) with their fields.
template <int S>
__device__ __forceinline__ uint32_t merge_pair_generic(uint32_t ea, uint32_t eb, uint32_t fa,
                                                       uint32_t fb, bool canon) {
  uint32_t out[2];
  const uint32_t e[2] = {ea & 0xFFu, eb & 0xFFu};
  const uint32_t f[2] = {fa, fb};
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const uint32_t frac = (f[k] & ((1u << S) - 1u)) << (7 - S);
    const uint32_t sign = (f[k] >> S) & 1u;
    uint32_t v = (e[k] << 7) | frac | (sign << 15);
    if (canon && e[k] == 255u && frac != 0u) v = 0x7FFFu;
    out[k] = v;
  }
  return out[0] | (out[1] << 16);
}

// Field of element j (0..7) of a lane's block; `bits` holds the lane's
// (s+1) bytes of packed fractions, first byte in the low bits.
template <int S>
__device__ __forceinline__ uint32_t field_of(uint64_t bits, int j) {
  constexpr int FB = S + 1;
  const int bit = j * FB;                 // MSB-first position inside the byte string
  const int byte = bit >> 3;
  const int shift = 7 - S - (bit & 7);
  return (uint32_t)(bits >> (8 * byte + shift)) & ((1u << FB) - 1u);
}

// Lossless fast path: two symbols + two fraction bytes -> one 32-bit word.
//   sel picks the two fraction bytes (a in both low bytes, b in both high).
__device__ __forceinline__ uint32_t merge_pair_s7(uint32_t ea, uint32_t eb, uint32_t fw,
                                                  uint32_t sel) {
  const uint32_t e = __byte_perm(ea, eb, 0x4400) << 7;   // exp_a<<7 | exp_b<<23 (+spill)
  const uint32_t g = __byte_perm(fw, 0, sel);            // fa fa fb fb
  return (e & 0x7F807F80u) | (g & 0x807F807Fu);
}

template <int S>
__device__ __forceinline__ uint64_t load_frac(const uint8_t *p) {
  if (S == 7) {
    const uint2 v = __ldcs(reinterpret_cast<const uint2 *>(p));
    return ((uint64_t)v.y << 32) | v.x;
  } else if (S == 3) {
    return __ldcs(reinterpret_cast<const uint32_t *>(p));
  } else if (S == 1) {
    return __ldcs(reinterpret_cast<const uint16_t *>(p));
  } else {
    return __ldcs(p);
  }
}

// Assemble and store one block of 8 elements of a lane.
template <int S, bool CANON>
__device__ __forceinline__ void store_block(const uint32_t (&ent)[8], uint64_t fbits,
                                            uint16_t *dst) {
  uint32_t w[4];
  if (S == 7 && !CANON) {
    const uint32_t lo = (uint32_t)fbits, hi = (uint32_t)(fbits >> 32);
    w[0] = merge_pair_s7(ent[0], ent[1], lo, 0x1100);
    w[1] = merge_pair_s7(ent[2], ent[3], lo, 0x3322);
    w[2] = merge_pair_s7(ent[4], ent[5], hi, 0x1100);
    w[3] = merge_pair_s7(ent[6], ent[7], hi, 0x3322);
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      w[k] = merge_pair_generic<S>(ent[2 * k], ent[2 * k + 1], field_of<S>(fbits, 2 * k),
                                   field_of<S>(fbits, 2 * k + 1), CANON);
  }
  __stcs(reinterpret_cast<uint4 *>(dst), make_uint4(w[0], w[1], w[2], w[3]));
}

struct DecodeArgs {
  const uint8_t *container;
  uint64_t container_bytes;
  const uint8_t *frac;
  uint64_t n;
  uint32_t S;
  uint32_t n_units;
  uint32_t slot_bytes;
  int canon;
  uint16_t *out_bf16;
  uint8_t *out_exp;
  uint32_t *status;
};

__device__ __forceinline__ void raise(uint32_t *status, uint32_t bits) {
  if (status) atomicOr(status, bits);
}

// Decode the `n_blocks` full blocks of one unit for this lane.
template <int S, bool MERGE, bool CANON>
__device__ __forceinline__ void decode_blocks(LaneState &st, uint32_t lut, uint32_t n_blocks,
                                              const uint8_t *frac_lane, uint16_t *out_lane,
                                              uint8_t *exp_lane) {
  constexpr uint32_t kFracStride = 32u * (S + 1);  // bytes of fractions per 256 elements
  uint64_t fnext = 0;
  if (MERGE && n_blocks) fnext = load_frac<S>(frac_lane);
  for (uint32_t b = 0; b < n_blocks; ++b) {
    const uint64_t fbits = fnext;
    if (MERGE && b + 1 < n_blocks) fnext = load_frac<S>(frac_lane + (uint64_t)(b + 1) * kFracStride);
    uint32_t ent[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) ent[t] = decode_step(st, lut);
    if (MERGE) {
      store_block<S, CANON>(ent, fbits, out_lane + (uint64_t)b * 256);
    } else {
      const uint32_t lo = __byte_perm(__byte_perm(ent[0], ent[1], 0x0040),
                                      __byte_perm(ent[2], ent[3], 0x0040), 0x5410);
      const uint32_t hi = __byte_perm(__byte_perm(ent[4], ent[5], 0x0040),
                                      __byte_perm(ent[6], ent[7], 0x0040), 0x5410);
      __stcs(reinterpret_cast<uint2 *>(exp_lane + (uint64_t)b * 256), make_uint2(lo, hi));
    }
  }
}

// One element with all guards, used for the partial block at the very end of
// the tensor and for raw units.
template <int S, bool MERGE>
__device__ __forceinline__ void emit_guarded(uint32_t sym, uint64_t e, const DecodeArgs &a) {
  if (e >= a.n) return;
  if (MERGE) {
    const uint64_t bit = e * (S + 1);
    const uint32_t shift = 7 - S - (uint32_t)(bit & 7);
    const uint32_t field = ((uint32_t)a.frac[bit >> 3] >> shift) & ((2u << S) - 1u);
    a.out_bf16[e] = (uint16_t)merge_pair_generic<S>(sym, 0, field, 0, a.canon != 0);
  } else {
    a.out_exp[e] = (uint8_t)sym;
  }
}

template <int S, bool MERGE>
__global__ void __launch_bounds__(512)
decode_kernel(const DecodeArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t n_warps = blockDim.x >> 5;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t *lut_p = reinterpret_cast<uint32_t *>(smem);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kLutBytes);
  uint16_t *cum_sh = reinterpret_cast<uint16_t *>(smem + kLutBytes + 8 * 32);  // 257 entries
  uint32_t *flag_sh = reinterpret_cast<uint32_t *>(smem + kLutBytes + 8 * 32 + 520);
  uint8_t *slots = smem + kLutBytes + 1024;
  const uint32_t lut = smem_u32(lut_p);

  // ---- header + table validation, decode-table build
  const Header *h = reinterpret_cast<const Header *>(a.container);
  const uint64_t pay_off = payload_offset(a.n_units);
  if (threadIdx.x == 0) {
    uint32_t bad = 0;
    if (h->magic != kMagic || h->version != 1 || h->n_symbols != a.n || h->lane_symbols != a.S ||
        h->n_units != a.n_units || h->len_quantum != len_quantum(a.S) ||
        h->payload_offset != pay_off || pay_off + h->payload_words * 2 > a.container_bytes ||
        h->payload_words >= kRawFlag)
      bad = NZ_STATUS_BAD_HEADER;
    *flag_sh = bad;
  }
  if (threadIdx.x < n_warps) mbar_init(smem_u32(&bars[threadIdx.x]), 1);
  const uint16_t *freq_g = reinterpret_cast<const uint16_t *>(a.container + kFreqOffset);
  if (warp == 0) {
    // inclusive scan of the 256 frequencies, 8 per lane
    uint32_t f[8], s = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      f[k] = freq_g[lane * 8 + k];
      s += f[k];
    }
    uint32_t incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= (uint32_t)o) incl += v;
    }
    uint32_t run = incl - s;
    if (lane == 0) cum_sh[0] = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      run += f[k];
      cum_sh[lane * 8 + k + 1] = (uint16_t)(run > 0xFFFF ? 0xFFFF : run);
    }
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && cum_sh[256] != kProbScale) *flag_sh |= NZ_STATUS_BAD_HEADER;
  __syncthreads();
  if (*flag_sh) {
    if (threadIdx.x == 0 && blockIdx.x == 0) raise(a.status, *flag_sh);
    return;
  }
  for (uint32_t slot = threadIdx.x; slot < kProbScale; slot += blockDim.x) {
    // largest symbol whose cumulative start is <= slot
    uint32_t lo = 0, hi = 256;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const uint32_t mid = (lo + hi) >> 1;
      if (cum_sh[mid] <= slot) lo = mid; else hi = mid;
    }
    const uint32_t start = cum_sh[lo];
    const uint32_t fr = cum_sh[lo + 1] - start;
    lut_p[slot] = lo | (fr << 8) | ((slot - start) << 20);
  }
  const bool canon = MERGE && a.canon && (freq_g[255] != 0);
  __syncthreads();

  // ---- units
  const uint32_t *offsets = reinterpret_cast<const uint32_t *>(a.container + kOffsetsOffset);
  const uint8_t *payload = a.container + pay_off;
  const uint64_t payload_words = h->payload_words;
  const uint32_t lenq = len_quantum(a.S);
  const uint64_t U = 32ull * a.S;
  const uint32_t bar = smem_u32(&bars[warp]);
  uint8_t *slot_p = slots + (uint64_t)warp * a.slot_bytes;
  const uint32_t slot = smem_u32(slot_p);
  uint32_t parity = 0;

  for (uint32_t u = blockIdx.x * n_warps + warp; u < a.n_units; u += gridDim.x * n_warps) {
    const uint32_t off0 = __ldg(offsets + u), off1 = __ldg(offsets + u + 1);
    const uint64_t w0 = off0 & ~kRawFlag, w1 = off1 & ~kRawFlag;
    const uint64_t first = (uint64_t)u * U;
    const uint64_t count = (a.n - first < U) ? (a.n - first) : U;
    if (w1 < w0 || w1 > payload_words) {
      if (lane == 0) raise(a.status, NZ_STATUS_BAD_OFFSETS);
      continue;
    }
    if (off0 & kRawFlag) {
      if ((w1 - w0) * 2 < count) {
        if (lane == 0) raise(a.status, NZ_STATUS_BAD_OFFSETS);
        continue;
      }
      const uint8_t *src = payload + w0 * 2;
      for (uint64_t i = lane; i < count; i += 32) emit_guarded<S, MERGE>(src[i], first + i, a);
      continue;
    }
    const uint64_t b0 = w0 * 2, b1 = w1 * 2;
    const uint64_t c0 = b0 & ~uint64_t(15), c1 = (b1 + 15) & ~uint64_t(15);
    const uint32_t bytes = (uint32_t)(c1 - c0);
    if (w1 - w0 < 16 + 2 * 32 || bytes > a.slot_bytes) {
      if (lane == 0) raise(a.status, NZ_STATUS_BAD_OFFSETS);
      continue;
    }
    // stage the unit: all lanes are done with the slot's previous contents
    __syncwarp();
    if (lane == 0) {
      mbar_expect_tx(bar, bytes);
      bulk_g2s(slot, payload + c0, bytes, bar);
    }
    bool arrived = false;
    for (uint32_t it = 0; it < kMaxWaitIters; ++it) {
      if (mbar_try_wait(bar, parity)) {
        arrived = true;
        break;
      }
    }
    parity ^= 1;
    if (!__all_sync(0xFFFFFFFFu, arrived)) {
      // Give the copy one more bounded chance to land, then give up on the
      // whole kernel: the slot cannot be reused while a copy may be in flight.
      if (!arrived)
        for (uint32_t it = 0; it < kMaxWaitIters && !mbar_try_wait(bar, parity ^ 1); ++it) {
        }
      if (lane == 0) raise(a.status, NZ_STATUS_TIMEOUT);
      return;
    }
    const uint32_t ub = slot + (uint32_t)(b0 - c0);  // shared address of the unit
    const uint32_t q = lds_u8(ub + lane) * lenq;     // my stream length in words
    uint32_t incl = q;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= (uint32_t)o) incl += v;
    }
    const uint32_t total = __shfl_sync(0xFFFFFFFFu, incl, 31);
    if (__any_sync(0xFFFFFFFFu, q < 2) || 16ull + total != w1 - w0) {
      if (lane == 0) raise(a.status, NZ_STATUS_BAD_LANES);
      continue;
    }
    LaneState st;
    const uint32_t sw = ub + 2 * (16 + incl - q);
    st.x = lds_u16(sw) | (lds_u16(sw + 2) << 16);
    st.p = sw + 4;
    st.w = lds_u16(st.p);

    const uint32_t full_blocks = (uint32_t)(count / 256);
    const uint64_t e_lane = first + lane * 8;
    const uint8_t *frac_lane = MERGE ? a.frac + e_lane * (S + 1) / 8 : nullptr;
    uint16_t *out_lane = MERGE ? a.out_bf16 + e_lane : nullptr;
    uint8_t *exp_lane = MERGE ? nullptr : a.out_exp + e_lane;
    if (canon)
      decode_blocks<S, MERGE, true>(st, lut, full_blocks, frac_lane, out_lane, exp_lane);
    else
      decode_blocks<S, MERGE, false>(st, lut, full_blocks, frac_lane, out_lane, exp_lane);
    if (count == U) {
      if (__any_sync(0xFFFFFFFFu, st.x != kStateLow) && lane == 0)
        raise(a.status, NZ_STATUS_BAD_STATE);
    } else if (count & 255) {
      // the partial block that ends the tensor
      const uint64_t e0 = e_lane + (uint64_t)full_blocks * 256;
      for (int t = 0; t < 8; ++t) {
        const uint32_t ent = decode_step(st, lut);
        emit_guarded<S, MERGE>(ent & 0xFFu, e0 + t, a);
      }
    }
  }
}

// ------------------------------------------------------------------- host
struct LaunchGeom {
  uint32_t warps, slot_bytes, smem_bytes, blocks;
};

static int decode_geometry(uint64_t n, uint32_t S, uint32_t max_unit_words, LaunchGeom &g) {
  const uint64_t U = 32ull * S;
  uint64_t unit_bytes = max_unit_words ? (uint64_t)max_unit_words * 2 : U;
  if (unit_bytes > U) unit_bytes = U;
  if (unit_bytes < 160) unit_bytes = 160;
  g.slot_bytes = (uint32_t)((unit_bytes + 32 + 127) & ~uint64_t(127));
  const uint32_t guard = ((S + 8) * 2 + 127) & ~127u;
  const uint32_t budget = 200 * 1024;
  uint32_t warps = 16;
  while (warps > 1 && kLutBytes + 1024 + warps * g.slot_bytes + guard > budget) warps >>= 1;
  g.warps = warps;
  g.smem_bytes = kLutBytes + 1024 + warps * g.slot_bytes + guard;
  if (g.smem_bytes > 227 * 1024) {
    set_error("decode: a unit of %u symbols does not fit in shared memory", (unsigned)U);
    return NZ_E_ARG;
  }
  const uint64_t nu = unit_count(n, S);
  uint64_t blocks = (nu + warps - 1) / warps;
  // resident CTAs per SM by shared memory and by threads (2048 per SM)
  uint32_t per_sm = (227u * 1024u) / (g.smem_bytes + 1024);
  const uint32_t by_threads = 2048 / (warps * 32);
  if (per_sm > by_threads) per_sm = by_threads;
  if (per_sm < 1) per_sm = 1;
  const uint64_t cap = (uint64_t)sm_count() * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  g.blocks = (uint32_t)blocks;
  return NZ_OK;
}

template <int S, bool MERGE>
static int launch_decode(const DecodeArgs &a, const LaunchGeom &g, cudaStream_t st) {
  auto kern = decode_kernel<S, MERGE>;
  NZ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)g.smem_bytes));
  kern<<<g.blocks, g.warps * 32, g.smem_bytes, st>>>(a);
  NZ_LAUNCH_CHECK("decode_kernel");
  return NZ_OK;
}

int decode_common(const void *container, uint64_t container_bytes, const void *frac, uint64_t n,
                  int precision, uint32_t S, uint32_t max_unit_words, int canon, void *out_bf16,
                  void *out_exp, void *status, cudaStream_t st) {
  if (n == 0) return NZ_OK;
  const uint64_t nu = unit_count(n, S);
  if (container_bytes < payload_offset(nu)) {
    set_error("decode: container of %llu bytes is too short for %llu units",
              (unsigned long long)container_bytes, (unsigned long long)nu);
    return NZ_E_FORMAT;
  }
  LaunchGeom g;
  int rc = decode_geometry(n, S, max_unit_words, g);
  if (rc) return rc;
  DecodeArgs a;
  a.container = (const uint8_t *)container;
  a.container_bytes = container_bytes;
  a.frac = (const uint8_t *)frac;
  a.n = n;
  a.S = S;
  a.n_units = (uint32_t)nu;
  a.slot_bytes = g.slot_bytes;
  a.canon = canon;
  a.out_bf16 = (uint16_t *)out_bf16;
  a.out_exp = (uint8_t *)out_exp;
  a.status = (uint32_t *)status;
  if (!out_bf16) return launch_decode<7, false>(a, g, st);
  switch (precision) {
    case 0: return launch_decode<0, true>(a, g, st);
    case 1: return launch_decode<1, true>(a, g, st);
    case 3: return launch_decode<3, true>(a, g, st);
    default: return launch_decode<7, true>(a, g, st);
  }
}

}  // namespace nz

static int check_decode_args(const char *who, const void *container, uint64_t n, uint32_t S) {
  if (!nz::valid_lane_symbols(S)) {
    nz::set_error("%s: lane_symbols must be a multiple of 8 in [8, %u] (got %u)", who,
                  nz::kMaxLaneSymbols, S);
    return NZ_E_ARG;
  }
  if (n >= (1ull << 32)) {
    nz::set_error("%s: tensors of 2^32 or more elements are not supported", who);
    return NZ_E_ARG;
  }
  if (n && (!container || ((uintptr_t)container & 15))) {
    nz::set_error("%s: container must be a 16-byte aligned device pointer", who);
    return NZ_E_ARG;
  }
  return NZ_OK;
}

extern "C" int nz_decode_exponents(const void *container, uint64_t container_bytes, uint64_t n,
                                   uint32_t lane_symbols, uint32_t max_unit_words, void *exp_out,
                                   void *status, void *stream) {
  int rc = check_decode_args("nz_decode_exponents", container, n, lane_symbols);
  if (rc) return rc;
  if (n && (!exp_out || ((uintptr_t)exp_out & 7))) {
    nz::set_error("nz_decode_exponents: output must be an 8-byte aligned device pointer");
    return NZ_E_ARG;
  }
  return nz::decode_common(container, container_bytes, nullptr, n, 7, lane_symbols,
                           max_unit_words, 0, nullptr, exp_out, status, (cudaStream_t)stream);
}

extern "C" int nz_decompress_bf16(const void *container, uint64_t container_bytes,
                                  const void *frac_in, uint64_t n, int precision,
                                  uint32_t lane_symbols, uint32_t max_unit_words,
                                  int canonical_nan, void *out_bf16, void *status, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_decompress_bf16: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  int rc = check_decode_args("nz_decompress_bf16", container, n, lane_symbols);
  if (rc) return rc;
  if (n && (!out_bf16 || !frac_in || ((uintptr_t)out_bf16 & 15) || ((uintptr_t)frac_in & 7))) {
    nz::set_error("nz_decompress_bf16: output must be 16-byte, fractions 8-byte aligned");
    return NZ_E_ARG;
  }
  return nz::decode_common(container, container_bytes, frac_in, n, precision, lane_symbols,
                           max_unit_words, canonical_nan, out_bf16, nullptr, status,
                           (cudaStream_t)stream);
}
