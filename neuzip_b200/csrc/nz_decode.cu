// rANS decoder of the NZR1 container, fused with the bf16 merge.
//
// Replaces nvcomp's ANS decompress followed by kernel_aligned_merge in the
// reference's read path (cuda/high_level.cu:184-201, cuda/kernels.cuh:158-217):
// the decoded exponent bytes stay in registers and are merged with the packed
// fractions straight into the bf16 output, so the exponent stream never makes
// the round trip through HBM.
//
// Work decomposition.  One CTA per SM; a warp decodes kChains units side by
// side (32 lane streams of S symbols each: the independent rANS chains hide one
// another's latency).  The units' coded bytes are staged into the warp's
// shared-memory slots with bulk asynchronous copies (cp.async.bulk + mbarrier,
// no multicast); each lane then walks its own stream with a private read
// pointer, so a renormalisation costs one predicated 16-bit shared load and no
// warp-wide vote.  A lane produces 8 consecutive tensor elements per block and
// writes them with one 128-bit store; the warp's stores are 512 contiguous
// bytes.  The same kernel, instantiated differently, decodes a list of units
// (gather) or feeds the decoded words to a dot product instead of a store.
//
// Decode table.  One 32-bit entry per slot (symbol << 23 | freq << 12 | offset
// inside the symbol's slot range), built once per CTA from the container's
// frequency table.  Random table lookups by 32 lanes would collide in the 32
// shared-memory banks (3.5 wavefronts per lookup on average, which made the
// shared-memory pipe the limiter), so the table is replicated across banks as
// far as the shared memory left by the slots allows (64 KB for lossless
// tensors: 32 copies of a 2^9-slot table, one per bank; 16 of a 2^10-slot one).
//
// Robustness.  Header, offset table and lane lengths are validated before
// use; a malformed container sets bits in the caller's status word and the
// affected units are skipped.  Reads of the coded stream are confined to the
// CTA's shared memory (a guard band behind the last slot absorbs run-away
// pointers), output and fraction addresses never depend on coded data, and
// the wait on the bulk copy is bounded.
#include <cuda_bf16.h>
#include <string.h>
#include <mutex>
#include <type_traits>

#include "nz_decode_core.cuh"

// Tuning constants (measured on B200, lossless config-2 stack): two units per warp
// and 20 warps per CTA beat three units with 14-16 warps by 3 %; unrolling the
// block loop 1, 2 or 4 times makes no difference.
#ifndef NZ_DECODE_ROLLED
#define NZ_DECODE_ROLLED 4
#endif
#ifndef NZ_DECODE_MAX_WARPS
#define NZ_DECODE_MAX_WARPS (NZ_DECODE_CHAINS == 2 ? 20 : 16)
#endif

namespace nz {

// One launch decodes up to kMaxBatch tensors; each tensor gets its own range of
// CTAs (one CTA per SM), sized in proportion to its unit count, so a small
// tensor does not leave most of the machine idle.
constexpr uint32_t kMaxBatch = 8;
struct BatchItem {
  const uint8_t *container;
  uint64_t container_bytes;
  const uint8_t *frac;
  uint64_t n;
  uint16_t *out_bf16;
  uint8_t *out_exp;
  uint32_t n_units;
  uint32_t cta_begin;     // first CTA of this tensor
  uint32_t tile_cols;     // operand order: row length (0 = stream order)
  uint32_t S;             // lane symbols of this tensor
  const uint8_t *norm;    // block normaliser bytes (null = none), log2 of the group size
  uint32_t norm_lg;
};
struct BatchArgs {
  BatchItem item[kMaxBatch];
  const uint32_t *unit_list;   // gather launches (count == 1): units of item[0] to decode
  uint32_t n_list;
  const float *gx;             // matrix-vector launches (count == 1), see DecodeArgs
  float *partial;
  uint32_t in, seg;
  const uint16_t *grad;        // update launches (count == 1): gradient, AdamW moments (bf16)
  uint16_t *exp_avg, *exp_avg_sq;
  AdamArgs adam;
  uint32_t inputs_stable;      // containers and fractions were complete before the previous kernel
  uint32_t count;
  uint32_t n_ctas;        // == gridDim.x
  uint32_t S, slot_bytes, lut_shift, lut_bytes, ring_offset;
  int canon;
  uint32_t *status;
};

// Exponent-only output: the 8 symbols of a lane's block as one 64-bit store.
__device__ __forceinline__ void store_exp_block(const uint32_t (&ent)[8], uint8_t *exp) {
  uint32_t b[8];                                          // symbol in the top byte
#pragma unroll
  for (int k = 0; k < 8; ++k) b[k] = ent[k] << (24 - kEntSymShift);
  const uint32_t lo = __byte_perm(__byte_perm(b[0], b[1], 0x0073),
                                  __byte_perm(b[2], b[3], 0x0073), 0x5410);
  const uint32_t hi = __byte_perm(__byte_perm(b[4], b[5], 0x0073),
                                  __byte_perm(b[6], b[7], 0x0073), 0x5410);
  __stcs(reinterpret_cast<uint2 *>(exp), make_uint2(lo, hi));
}

template <int S, bool MERGE, bool CANON>
__device__ __forceinline__ void decode_one_block(LaneState &st, const LutView &lut, uint64_t fbits,
                                                 uint16_t *out, uint8_t *exp) {
  uint32_t ent[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) ent[t] = decode_step<0>(st, lut);
  if (MERGE) {
    store_block<S, CANON>(ent, fbits, out);
  } else {
    store_exp_block(ent, exp);
  }
}

// Decode the `n_blocks` full blocks of one unit for this lane.  The packed
// fractions are fetched four blocks ahead of their use.
template <int S, bool MERGE, bool CANON>
__device__ __forceinline__ void decode_blocks(LaneState &st, const LutView &lut, uint32_t n_blocks,
                                              const uint8_t *frac_lane, uint16_t *out_lane,
                                              uint8_t *exp_lane, uint32_t adv = 256) {
  constexpr uint32_t kFracStride = 32u * (S + 1);  // bytes of fractions per 256 elements
  constexpr int kAhead = 4;
  uint64_t f[kAhead] = {0, 0, 0, 0};
  if (MERGE) {
#pragma unroll
    for (int k = 0; k < kAhead; ++k)
      if ((uint32_t)k < n_blocks) f[k] = load_frac<S>(frac_lane + k * kFracStride);
  }
  uint32_t b = 0;
  for (; b + kAhead <= n_blocks; b += kAhead) {
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      const uint64_t fbits = f[k];
      if (MERGE && b + kAhead + k < n_blocks)
        f[k] = load_frac<S>(frac_lane + (kAhead + k) * kFracStride);
      decode_one_block<S, MERGE, CANON>(st, lut, fbits, MERGE ? out_lane + k * adv : nullptr,
                                        MERGE ? nullptr : exp_lane + k * 256);
    }
    if (MERGE) {
      frac_lane += kAhead * kFracStride;
      out_lane += kAhead * adv;
    } else {
      exp_lane += kAhead * 256;
    }
  }
#pragma unroll
  for (int k = 0; k < kAhead - 1; ++k) {
    if (b + k < n_blocks)
      decode_one_block<S, MERGE, CANON>(st, lut, f[k], MERGE ? out_lane + k * adv : nullptr,
                                        MERGE ? nullptr : exp_lane + k * 256);
  }
}

// One element with all guards, used for the partial block at the very end of
// the tensor and for raw units.
// `delta` is the distance (in elements) from an element's place in the tensor
// to its place in the output: 0 except in gather launches.
template <int S, bool MERGE>
__device__ __forceinline__ void emit_guarded(uint32_t sym, uint64_t e, int64_t delta,
                                             const DecodeArgs &a) {
  if (e >= a.n) return;
  if (MERGE) {
    const uint64_t bit = e * (S + 1);
    const uint32_t shift = 7 - S - (uint32_t)(bit & 7);
    const uint32_t field = ((uint32_t)a.frac[bit >> 3] >> shift) & ((2u << S) - 1u);
    uint32_t v = merge_pair_generic<S>(sym << kEntSymShift, 0, field, 0, a.canon != 0) & 0xFFFFu;
    if (a.norm) v = scale_bf16_bits(v, norm_scale(a.norm[e >> a.norm_lg]));
    a.out_bf16[out_index(a, e) + delta] = (uint16_t)v;
  } else {
    a.out_exp[e + delta] = (uint8_t)sym;
  }
}

constexpr int kFastRow = 7;                      // 128-byte table rows: one copy per bank
constexpr int kRolled = NZ_DECODE_ROLLED;        // blocks per trip of the rolled decode loop
constexpr uint32_t kRingSlots = 4;               // blocks of fractions in flight per unit + 1
// Shared-memory ring of a warp for the packed fractions, by precision.  One unit's
// place holds, for precisions 7 and 3, one block (32 lanes x 8 or 4 bytes; four such
// slots) and, for precisions 1 and 0, a group of four blocks (32 lanes x 8 or 4
// bytes; two buffers).
__host__ __device__ constexpr uint32_t ring_unit_bytes(int precision) {
  return (precision == 7 || precision == 1) ? 256u : 128u;
}
__host__ __device__ constexpr uint32_t ring_warp_bytes(int precision) {
  return ((precision == 7 || precision == 3) ? kRingSlots : 2u) * kChains *
         ring_unit_bytes(precision);
}

// Where the four words (8 bf16) that a lane produces per block and chain go.
// StoreSink writes them to the output tensor.
// ADV = elements between a lane's consecutive blocks: 256, or 64 in operand order (a
// compile-time constant, so that the offsets fold into the store instructions).
template <int ADV>
struct StoreSinkT {
  uint16_t *out[kChains];
  __device__ __forceinline__ void begin(int) {}
  __device__ __forceinline__ void put(int c, int k, const uint32_t (&w)[4]) {
    __stcs(reinterpret_cast<uint4 *>(out[c] + k * ADV), make_uint4(w[0], w[1], w[2], w[3]));
  }
  __device__ __forceinline__ void advance(int blocks) {
#pragma unroll
    for (int c = 0; c < kChains; ++c) out[c] += blocks * ADV;
  }
};
using StoreSink = StoreSinkT<256>;

// One lane's running dot product of a weight row with the input vector.  The
// tensor is a row-major [out, in] matrix with `in` a multiple of 256, so the 256
// elements of a block lie in one row and the end of a row is the same event for
// all lanes of the warp.  At the end of a row (and of the unit) the warp's sum
// goes to the next partial-sum place of the unit; a finishing kernel adds the
// partial sums of each row in unit order, so results do not depend on timing.
struct DotLane {
  const float *x;      // input vector, fp32
  uint32_t in;         // row length
  uint32_t col;        // this lane's column of the next block (block start + lane * 8)
  float acc;
  float *part;         // next partial-sum place of the unit
  __device__ __forceinline__ void start(const float *xv, uint32_t in_features, uint64_t first_elem,
                                        float *unit_part, uint32_t lane) {
    x = xv;
    in = in_features;
    col = (uint32_t)(first_elem % in_features) + lane * 8;
    acc = 0.f;
    part = unit_part;
  }
  __device__ __forceinline__ void emit(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if ((threadIdx.x & 31) == 0) *part = v;
    ++part;
  }
  // The 8 input values of a block are requested before the block's symbols are
  // decoded and used after, so that their latency hides behind the decode steps.
  float4 xa, xb;
  __device__ __forceinline__ void begin() {
    xa = __ldg(reinterpret_cast<const float4 *>(x + col));
    xb = __ldg(reinterpret_cast<const float4 *>(x + col + 4));
  }
  __device__ __forceinline__ void put(const uint32_t (&w)[4]) {
    float a = acc;
    a = fmaf(__uint_as_float(w[0] << 16), xa.x, a);
    a = fmaf(__uint_as_float(w[0] & 0xFFFF0000u), xa.y, a);
    a = fmaf(__uint_as_float(w[1] << 16), xa.z, a);
    a = fmaf(__uint_as_float(w[1] & 0xFFFF0000u), xa.w, a);
    a = fmaf(__uint_as_float(w[2] << 16), xb.x, a);
    a = fmaf(__uint_as_float(w[2] & 0xFFFF0000u), xb.y, a);
    a = fmaf(__uint_as_float(w[3] << 16), xb.z, a);
    a = fmaf(__uint_as_float(w[3] & 0xFFFF0000u), xb.w, a);
    acc = a;
    col += 256;
    if (col >= in) {          // same verdict in every lane: in - (col - lane*8) is a multiple of 256
      emit(acc);
      acc = 0.f;
      col -= in;
    }
  }
  // end of the unit: a row that is still open gives its partial sum
  __device__ __forceinline__ void finish() {
    if (col & ~255u) emit(acc);
  }
};
struct DotSink {
  DotLane lane[kChains];
  __device__ __forceinline__ void begin(int c) { lane[c].begin(); }
  __device__ __forceinline__ void put(int c, int, const uint32_t (&w)[4]) { lane[c].put(w); }
  __device__ __forceinline__ void advance(int) {}
};

// A sink in front of another: tensors written with a block normaliser are multiplied by
// their group's scale as they are produced (8 elements of a lane share one stored byte for
// groups of 8 and more, else each run of `group` elements has its own).
template <class Inner>
struct NormSink {
  Inner inner;
  const uint8_t *norm;
  uint32_t lg;
  uint32_t e0[kChains];       // tensor index of the lane's first element of the unit
  int blk[kChains];
  uint64_t bytes[kChains];
  __device__ __forceinline__ void begin(int c) {
    inner.begin(c);
    const uint32_t e = e0[c] + ((uint32_t)blk[c] << 8);
    if (lg >= 3) {
      bytes[c] = __ldg(norm + (e >> lg));
    } else {
      const uint8_t *p = norm + (e >> lg);
      uint64_t b = 0;
      const int count = 8 >> lg;
      for (int i = 0; i < count; ++i) b |= (uint64_t)__ldg(p + i) << (8 * i);
      bytes[c] = b;
    }
  }
  __device__ __forceinline__ void put(int c, int k, const uint32_t (&w)[4]) {
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t i0 = 2 * j, i1 = 2 * j + 1;
      const float s0 = norm_scale((uint32_t)(bytes[c] >> (lg >= 3 ? 0 : 8 * (i0 >> lg))) & 0xFFu);
      const float s1 = norm_scale((uint32_t)(bytes[c] >> (lg >= 3 ? 0 : 8 * (i1 >> lg))) & 0xFFu);
      o[j] = scale_bf16_bits(w[j] & 0xFFFFu, s0) | (scale_bf16_bits(w[j] >> 16, s1) << 16);
    }
    inner.put(c, k, o);
    ++blk[c];
  }
  __device__ __forceinline__ void advance(int n) { inner.advance(n); }
};

// Update launches: the four decoded words of a block (8 weights of one row) take an
// AdamW step against the gradient and the moments at the same place of their (row-major)
// tensors and go, rounded to bf16 once, to the output tensor; the moments are updated in
// place.  Gradient and moments of a block are requested before its symbols are decoded.
__device__ __forceinline__ void adamw_words(const uint32_t (&w)[4], const uint4 &gv, uint4 &mv,
                                            uint4 &vv, const AdamArgs &a, uint4 &out) {
  const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
  uint32_t mw[4] = {mv.x, mv.y, mv.z, mv.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w}, ow[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    uint32_t res = 0, mres = 0, vres = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t sh = 16 * h;
      float m = __bfloat162float(__ushort_as_bfloat16((unsigned short)(mw[k] >> sh)));
      float v = __bfloat162float(__ushort_as_bfloat16((unsigned short)(vw[k] >> sh)));
      const float x = adamw_element(
          __bfloat162float(__ushort_as_bfloat16((unsigned short)(w[k] >> sh))),
          __bfloat162float(__ushort_as_bfloat16((unsigned short)(gw[k] >> sh))), m, v, a);
      res |= (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x)) << sh;
      mres |= (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(m)) << sh;
      vres |= (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v)) << sh;
    }
    ow[k] = res;
    mw[k] = mres;
    vw[k] = vres;
  }
  out = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  mv = make_uint4(mw[0], mw[1], mw[2], mw[3]);
  vv = make_uint4(vw[0], vw[1], vw[2], vw[3]);
}

template <int ADV>
struct UpdateSinkT {
  uint16_t *out[kChains];
  const uint16_t *g[kChains];
  uint16_t *m[kChains], *v[kChains];
  uint4 gv[kChains], mv[kChains], vv[kChains];
  int blk[kChains];
  AdamArgs adam;
  __device__ __forceinline__ void begin(int c) {
    const int o = blk[c] * ADV;
    gv[c] = __ldcs(reinterpret_cast<const uint4 *>(g[c] + o));
    mv[c] = __ldcs(reinterpret_cast<const uint4 *>(m[c] + o));
    vv[c] = __ldcs(reinterpret_cast<const uint4 *>(v[c] + o));
  }
  __device__ __forceinline__ void put(int c, int, const uint32_t (&w)[4]) {
    uint4 res;
    adamw_words(w, gv[c], mv[c], vv[c], adam, res);
    const int o = blk[c] * ADV;
    __stcs(reinterpret_cast<uint4 *>(out[c] + o), res);
    __stcs(reinterpret_cast<uint4 *>(m[c] + o), mv[c]);
    __stcs(reinterpret_cast<uint4 *>(v[c] + o), vv[c]);
    ++blk[c];
  }
  __device__ __forceinline__ void advance(int) {}
};

// kChains units interleaved in one lane: the rANS chains are independent, so
// each hides the shared-memory and multiply latency of the others.  For
// precisions 3 and 7 the packed fractions travel through a small ring in shared
// memory, fetched three blocks ahead with per-lane asynchronous copies; the
// narrower fractions of precisions 0 and 1 (1 and 2 bytes per lane and block)
// are fetched four blocks at a time by the whole warp.
template <int S, bool MERGE, bool CANON, int ROW, typename Sink>
__device__ __forceinline__ void decode_blocks_multi(LaneState (&st)[kChains], const LutView &lut,
                                                    uint32_t n_blocks,
                                                    const uint8_t *(&frac)[kChains], Sink &sink,
                                                    uint8_t *(&exp)[kChains], uint32_t ring) {
  constexpr uint32_t kFracStride = 32u * (S + 1);
  constexpr bool kAsync = MERGE && (S == 7 || S == 3);
  constexpr int kAhead = 4;
  constexpr uint32_t kRingUnitBytes = ring_unit_bytes(S);
  constexpr uint32_t kRingSlotBytes = kChains * kRingUnitBytes;
  if (MERGE && (S == 0 || S == 1) && (n_blocks & 3) == 0) {
    // Narrow fractions: four blocks of a unit are 128 (s=0) or 256 (s=1) contiguous
    // bytes, copied by the whole warp (4 or 8 bytes per lane) into a double-buffered
    // ring one group of four blocks ahead; lanes then read their own 1 or 2 bytes.
    constexpr uint32_t kLaneBytes = 4u * (S + 1);          // per lane and group
    constexpr uint32_t kGroupBytes = 32u * kLaneBytes;     // per unit and group
    constexpr uint32_t kBufBytes = kChains * kRingUnitBytes;
    const uint32_t lane_id = threadIdx.x & 31;
    const uint32_t ring0 = ring - lane_id * 4;             // `ring` carries lane*4 for s<7
    const uint32_t n_groups = n_blocks >> 2;
    const uint8_t *gbase[kChains];
#pragma unroll
    for (int c = 0; c < kChains; ++c) gbase[c] = frac[c] - (uint64_t)lane_id * (S + 1);
    auto issue = [&](uint32_t g) {
      const uint32_t dst = ring0 + (g & 1) * kBufBytes + lane_id * kLaneBytes;
#pragma unroll
      for (int c = 0; c < kChains; ++c) {
        const uint8_t *src = gbase[c] + (uint64_t)g * kGroupBytes + lane_id * kLaneBytes;
        if (S == 1)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + c * kRingUnitBytes),
                       "l"(src)
                       : "memory");
        else
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + c * kRingUnitBytes),
                       "l"(src)
                       : "memory");
      }
      frac_commit();
    };
    issue(0);
    for (uint32_t g = 0; g < n_groups; ++g) {
      __syncwarp();                       // everyone is done with the buffer about to be refilled
      if (g + 1 < n_groups) {
        issue(g + 1);
        frac_wait<1>();
      } else {
        frac_wait<0>();
      }
      __syncwarp();                       // all lanes' copies of group g have landed
      const uint32_t src = ring0 + (g & 1) * kBufBytes + lane_id * (S + 1);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint64_t bits[kChains];
#pragma unroll
        for (int c = 0; c < kChains; ++c)
          bits[c] = (S == 1) ? lds_u16(src + c * kRingUnitBytes + k * 64)
                             : lds_u8(src + c * kRingUnitBytes + k * 32);
#pragma unroll
        for (int c = 0; c < kChains; ++c) sink.begin(c);
        uint32_t w[kChains][4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint32_t e0[kChains], e1[kChains];
#pragma unroll
          for (int c = 0; c < kChains; ++c) e0[c] = decode_step<ROW>(st[c], lut);
#pragma unroll
          for (int c = 0; c < kChains; ++c) e1[c] = decode_step<ROW>(st[c], lut);
#pragma unroll
          for (int c = 0; c < kChains; ++c) w[c][t] = merge_word<S, CANON>(e0[c], e1[c], bits[c], t);
        }
#pragma unroll
        for (int c = 0; c < kChains; ++c) sink.put(c, k, w[c]);
      }
      sink.advance(4);
    }
    return;
  }
  if (kAsync && (n_blocks % kRolled) == 0) {
    // Rolled form: the loop body covers kRolled blocks, so that the instruction
    // working set of a CTA's warps stays small.  A trip starts at a multiple of
    // kRolled: when that is a multiple of the ring size, a block's ring slot is a
    // compile-time constant.
    auto ring_slot = [](uint32_t block, int in_trip) -> uint32_t {
      return (kRolled % kRingSlots == 0) ? (uint32_t)in_trip % kRingSlots : block % kRingSlots;
    };
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      if ((uint32_t)k < n_blocks) {
#pragma unroll
        for (int c = 0; c < kChains; ++c)
          frac_async<S>(ring + k * kRingSlotBytes + c * kRingUnitBytes, frac[c] + k * kFracStride);
      }
      frac_commit();
    }
#pragma unroll 1
    for (uint32_t b = 0; b < n_blocks; b += kRolled) {
#pragma unroll
      for (int k = 0; k < kRolled; ++k) {
        const uint32_t bk = b + k;
        if (bk + 3 < n_blocks) {
#pragma unroll
          for (int c = 0; c < kChains; ++c)
            frac_async<S>(ring + ring_slot(bk + 3, k + 3) * kRingSlotBytes + c * kRingUnitBytes,
                          frac[c] + (k + 3) * kFracStride);
        }
        frac_commit();
        frac_wait<3>();
        uint64_t bits[kChains];
#pragma unroll
        for (int c = 0; c < kChains; ++c)
          bits[c] = frac_from_ring<S>(ring + ring_slot(bk, k) * kRingSlotBytes + c * kRingUnitBytes);
#pragma unroll
        for (int c = 0; c < kChains; ++c) sink.begin(c);
        uint32_t w[kChains][4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint32_t e0[kChains], e1[kChains];
#pragma unroll
          for (int c = 0; c < kChains; ++c) e0[c] = decode_step<ROW>(st[c], lut);
#pragma unroll
          for (int c = 0; c < kChains; ++c) e1[c] = decode_step<ROW>(st[c], lut);
#pragma unroll
          for (int c = 0; c < kChains; ++c) w[c][t] = merge_word<S, CANON>(e0[c], e1[c], bits[c], t);
        }
#pragma unroll
        for (int c = 0; c < kChains; ++c) sink.put(c, k, w[c]);
      }
#pragma unroll
      for (int c = 0; c < kChains; ++c) frac[c] += kRolled * kFracStride;
      sink.advance(kRolled);
    }
    frac_wait<0>();
    return;
  }
  uint64_t fr[kChains][kAhead];
#pragma unroll
  for (int c = 0; c < kChains; ++c)
#pragma unroll
    for (int k = 0; k < kAhead; ++k) fr[c][k] = 0;
  if (kAsync) {
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      if ((uint32_t)k < n_blocks) {
#pragma unroll
        for (int c = 0; c < kChains; ++c)
          frac_async<S>(ring + k * kRingSlotBytes + c * kRingUnitBytes, frac[c] + k * kFracStride);
      }
      frac_commit();
    }
  } else if (MERGE) {
#pragma unroll
    for (int k = 0; k < kAhead; ++k)
      if ((uint32_t)k < n_blocks) {
#pragma unroll
        for (int c = 0; c < kChains; ++c) fr[c][k] = load_frac<S>(frac[c] + k * kFracStride);
      }
  }
  // One block of every unit: fetch the fractions of block b+k (and start the copy
  // for block b+k+3), decode 8 symbols of each chain, merge, store.  `guard`
  // is false when the block count is a multiple of four and nothing needs testing
  // except the end of the prefetch.
  auto one_block = [&](uint32_t b, int k, bool guard) {
    if (guard && !(b + k < n_blocks)) return;
    uint64_t bits[kChains];
#pragma unroll
    for (int c = 0; c < kChains; ++c) bits[c] = fr[c][k];
    if (kAsync) {
      // block b+k+3 goes into the ring slot that block b+k-1 has left
      if (b + k + 3 < n_blocks) {
#pragma unroll
        for (int c = 0; c < kChains; ++c)
          frac_async<S>(ring + ((k + 3) & 3) * kRingSlotBytes + c * kRingUnitBytes,
                        frac[c] + (k + 3) * kFracStride);
      }
      frac_commit();
      frac_wait<3>();
#pragma unroll
      for (int c = 0; c < kChains; ++c)
        bits[c] = frac_from_ring<S>(ring + k * kRingSlotBytes + c * kRingUnitBytes);
    } else if (MERGE && b + kAhead + k < n_blocks) {
#pragma unroll
      for (int c = 0; c < kChains; ++c) fr[c][k] = load_frac<S>(frac[c] + (kAhead + k) * kFracStride);
    }
    if (MERGE) {
      // two symbols of each chain, then their output words: the table entries do
      // not have to stay live for the whole block
#pragma unroll
      for (int c = 0; c < kChains; ++c) sink.begin(c);
      uint32_t w[kChains][4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        uint32_t e0[kChains], e1[kChains];
#pragma unroll
        for (int c = 0; c < kChains; ++c) e0[c] = decode_step<ROW>(st[c], lut);
#pragma unroll
        for (int c = 0; c < kChains; ++c) e1[c] = decode_step<ROW>(st[c], lut);
#pragma unroll
        for (int c = 0; c < kChains; ++c) w[c][t] = merge_word<S, CANON>(e0[c], e1[c], bits[c], t);
      }
#pragma unroll
      for (int c = 0; c < kChains; ++c) sink.put(c, k, w[c]);
    } else {
      uint32_t e[kChains][8];
#pragma unroll
      for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int c = 0; c < kChains; ++c) e[c][t] = decode_step<ROW>(st[c], lut);
#pragma unroll
      for (int c = 0; c < kChains; ++c) store_exp_block(e[c], exp[c] + k * 256);
    }
  };
  auto advance = [&]() {
#pragma unroll
    for (int c = 0; c < kChains; ++c) {
      if (MERGE) {
        frac[c] += kAhead * kFracStride;
      } else {
        exp[c] += kAhead * 256;
      }
    }
    if (MERGE) sink.advance(kAhead);
  };
  if ((n_blocks & 3) == 0) {
    for (uint32_t b = 0; b < n_blocks; b += kAhead) {
#pragma unroll
      for (int k = 0; k < kAhead; ++k) one_block(b, k, false);
      advance();
    }
  } else {
    for (uint32_t b = 0; b < n_blocks; b += kAhead) {
#pragma unroll
      for (int k = 0; k < kAhead; ++k) one_block(b, k, true);
      advance();
    }
  }
  if (kAsync) frac_wait<0>();
}

// Decode one unit on its own (raw units, the tensor's last unit, odd counts).
template <int S, bool MERGE>
__device__ __forceinline__ void decode_single(const DecodeArgs &a, const UnitPlan &pl, uint32_t u,
                                              int64_t delta, uint32_t slot, const LutView &lv, bool canon,
                                              const uint8_t *payload, uint32_t lenq,
                                              uint32_t lane) {
  const uint64_t U = 32ull * a.S;
  const uint64_t first = (uint64_t)u * U;
  const uint64_t count = (a.n - first < U) ? (a.n - first) : U;
  if (pl.kind == kUnitRaw) {
    const uint8_t *src = payload + pl.byte0;
    for (uint64_t i = lane; i < count; i += 32) emit_guarded<S, MERGE>(src[i], first + i, delta, a);
    return;
  }
  if (pl.kind != kUnitCoded) return;
  LaneState st;
  if (!open_unit(pl, slot, lenq, lane, st)) {
    if (lane == 0) raise(a.status, NZ_STATUS_BAD_LANES);
    return;
  }
  const uint64_t e_lane = first + lane * 8;
  if (MERGE && a.norm) {
    // a unit decoded on its own in a tensor with a block normaliser: element by element
    const uint32_t blocks = (uint32_t)((count + 255) / 256);
    for (uint32_t b = 0; b < blocks; ++b)
      for (int t = 0; t < 8; ++t) {
        const uint32_t ent = decode_step<0>(st, lv);
        emit_guarded<S, MERGE>(entry_symbol(ent), e_lane + (uint64_t)b * 256 + t, delta, a);
      }
    if (count == U && __any_sync(0xFFFFFFFFu, st.x != kStateLow) && lane == 0)
      raise(a.status, NZ_STATUS_BAD_STATE);
    return;
  }
  const uint32_t full_blocks = (uint32_t)(count / 256);
  const uint8_t *frac_lane = MERGE ? a.frac + e_lane * (S + 1) / 8 : nullptr;
  // in operand order a lane's blocks are 64 elements apart in its row (units never
  // straddle a row group); the exponent-only output is always in stream order
  uint16_t *out_lane = MERGE ? a.out_bf16 + (out_index(a, e_lane) + delta) : nullptr;
  uint8_t *exp_lane = MERGE ? nullptr : a.out_exp + (e_lane + delta);
  const uint32_t adv = (MERGE && a.tile_cols) ? 64u : 256u;
  if (canon)
    decode_blocks<S, MERGE, true>(st, lv, full_blocks, frac_lane, out_lane, exp_lane, adv);
  else
    decode_blocks<S, MERGE, false>(st, lv, full_blocks, frac_lane, out_lane, exp_lane, adv);
  if (count == U) {
    if (__any_sync(0xFFFFFFFFu, st.x != kStateLow) && lane == 0)
      raise(a.status, NZ_STATUS_BAD_STATE);
  } else if (count & 255) {
    // the partial block that ends the tensor
    const uint64_t e0 = e_lane + (uint64_t)full_blocks * 256;
    for (int t = 0; t < 8; ++t) {
      const uint32_t ent = decode_step<0>(st, lv);
      emit_guarded<S, MERGE>(entry_symbol(ent), e0 + t, delta, a);
    }
  }
}

template <int ADV>
__device__ __forceinline__ void init_sink(StoreSinkT<ADV> &sk, int c, const DecodeArgs &a, uint32_t,
                                          uint64_t out_elem, uint32_t) {
  // out_elem is the lane's first element of the unit in stream order (a multiple of 8)
  sk.out[c] = a.out_bf16 ? a.out_bf16 + out_index(a, out_elem) : nullptr;
}
__device__ __forceinline__ void init_sink(DotSink &sk, int c, const DecodeArgs &a, uint32_t unit,
                                          uint64_t, uint32_t lane) {
  sk.lane[c].start(a.gx, a.in, (uint64_t)unit * (32ull * a.S), a.partial + (uint64_t)unit * a.seg,
                   lane);
}
template <int ADV>
__device__ __forceinline__ void finish_sink(StoreSinkT<ADV> &) {}
template <int ADV>
__device__ __forceinline__ void init_sink(UpdateSinkT<ADV> &sk, int c, const DecodeArgs &a, uint32_t,
                                          uint64_t out_elem, uint32_t) {
  const uint64_t o = out_index(a, out_elem);
  sk.out[c] = a.out_bf16 + o;
  sk.g[c] = a.grad + o;
  sk.m[c] = a.exp_avg + o;
  sk.v[c] = a.exp_avg_sq + o;
  sk.blk[c] = 0;
  sk.adam = a.adam;
}
template <int ADV>
__device__ __forceinline__ void finish_sink(UpdateSinkT<ADV> &) {}
template <class Inner>
__device__ __forceinline__ void init_sink(NormSink<Inner> &sk, int c, const DecodeArgs &a,
                                          uint32_t unit, uint64_t out_elem, uint32_t lane) {
  init_sink(sk.inner, c, a, unit, out_elem, lane);
  sk.norm = a.norm;
  sk.lg = a.norm_lg;
  sk.e0[c] = unit * (32u * a.S) + lane * 8;
  sk.blk[c] = 0;
}
template <class Inner>
__device__ __forceinline__ void finish_sink(NormSink<Inner> &sk) { finish_sink(sk.inner); }

// Update launches, units that do not take the fast path: the unit has just been decoded
// into the output tensor the ordinary way; its elements take their step there.
__device__ __forceinline__ void update_decoded_unit(const DecodeArgs &a, uint32_t u, uint32_t lane) {
  if (u >= a.n_units) return;
  const uint64_t U = 32ull * a.S;
  const uint64_t first = (uint64_t)u * U;
  const uint64_t count = (a.n - first < U) ? (a.n - first) : U;
  __syncwarp();
  for (uint64_t i = lane; i < count; i += 32) {
    const uint64_t o = out_index(a, first + i);
    float m = __bfloat162float(__ushort_as_bfloat16(a.exp_avg[o]));
    float v = __bfloat162float(__ushort_as_bfloat16(a.exp_avg_sq[o]));
    const float x = adamw_element(__bfloat162float(__ushort_as_bfloat16(a.out_bf16[o])),
                                  __bfloat162float(__ushort_as_bfloat16(a.grad[o])), m, v, a.adam);
    a.out_bf16[o] = __bfloat16_as_ushort(__float2bfloat16_rn(x));
    a.exp_avg[o] = __bfloat16_as_ushort(__float2bfloat16_rn(m));
    a.exp_avg_sq[o] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
  }
}
__device__ __forceinline__ void finish_sink(DotSink &sk) {
#pragma unroll
  for (int c = 0; c < kChains; ++c) sk.lane[c].finish();
}

// Matrix-vector launches, units that do not take the fast path (raw units, the
// tensor's last unit, units whose neighbour in the group is one of those).  The
// partial sums of unit u go to partial[u * seg ...], one per row the unit
// touches, in row order -- the same places the fast path fills.
template <int S>
__device__ __forceinline__ void dot_single(const DecodeArgs &a, const UnitPlan &pl, uint32_t u,
                                           uint32_t slot, const LutView &lv, bool canon,
                                           const uint8_t *payload, uint32_t lenq, uint32_t lane) {
  if (u >= a.n_units) return;
  const uint64_t U = 32ull * a.S;
  const uint64_t first = (uint64_t)u * U;
  const uint64_t count = (a.n - first < U) ? (a.n - first) : U;
  float *part = a.partial + (uint64_t)u * a.seg;
  const uint64_t row0 = first / a.in, row1 = (first + count - 1) / a.in;
  bool filled = false;
  if (pl.kind == kUnitRaw) {
    const uint8_t *src = payload + pl.byte0;
    for (uint64_t r = row0; r <= row1; ++r) {
      const uint64_t lo = r * a.in > first ? r * a.in : first;
      const uint64_t hi = (r + 1) * a.in < first + count ? (r + 1) * a.in : first + count;
      float acc = 0.f;
      for (uint64_t e = lo + lane; e < hi; e += 32) {
        const uint64_t bit = e * (S + 1);
        const uint32_t shift = 7 - S - (uint32_t)(bit & 7);
        const uint32_t field = ((uint32_t)a.frac[bit >> 3] >> shift) & ((2u << S) - 1u);
        const uint32_t v = merge_pair_generic<S>((uint32_t)src[e - first] << kEntSymShift, 0, field,
                                                 0, a.canon != 0);
        acc = fmaf(__uint_as_float(v << 16), a.gx[e - r * a.in], acc);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
      if (lane == 0) part[r - row0] = acc;
    }
    filled = true;
  } else if (pl.kind == kUnitCoded) {
    LaneState st;
    if (open_unit(pl, slot, lenq, lane, st)) {
      // the row length is a multiple of 256, so is the element count: whole blocks only
      const uint32_t n_blocks = (uint32_t)(count / 256);
      const uint8_t *frac_lane = a.frac + (first + lane * 8) * (S + 1) / 8;
      DotLane d;
      d.start(a.gx, a.in, first, part, lane);
      for (uint32_t b = 0; b < n_blocks; ++b) {
        const uint64_t fbits = load_frac<S>(frac_lane + (uint64_t)b * 32u * (S + 1));
        uint32_t ent[8], w[4];
        d.begin();
#pragma unroll
        for (int t = 0; t < 8; ++t) ent[t] = decode_step<0>(st, lv);
#pragma unroll
        for (int t = 0; t < 4; ++t)
          w[t] = canon ? merge_word<S, true>(ent[2 * t], ent[2 * t + 1], fbits, t)
                       : merge_word<S, false>(ent[2 * t], ent[2 * t + 1], fbits, t);
        d.put(w);
      }
      d.finish();
      if (count == U && __any_sync(0xFFFFFFFFu, st.x != kStateLow) && lane == 0)
        raise(a.status, NZ_STATUS_BAD_STATE);
      filled = true;
    } else if (lane == 0) {
      raise(a.status, NZ_STATUS_BAD_LANES);
    }
  }
  if (!filled && lane == 0)          // a unit that could not be decoded contributes zeros
    for (uint64_t r = row0; r <= row1; ++r) part[r - row0] = 0.f;
}

// Adds the partial sums of each output row in unit order, adds the bias and
// rounds to bf16 (round to nearest even, like the library GEMM's epilogue).
__global__ void dot_finish_kernel(const float *__restrict__ partial, uint32_t seg, uint64_t U,
                                  uint32_t in, uint32_t out_features,
                                  const uint16_t *__restrict__ bias, uint16_t *__restrict__ y) {
  const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= out_features) return;
  const uint64_t e_lo = (uint64_t)r * in, e_hi = e_lo + in - 1;
  float sum = 0.f;
  for (uint64_t u = e_lo / U; u <= e_hi / U; ++u)
    sum += partial[u * seg + (r - (uint32_t)(u * U / in))];
  if (bias) sum += __uint_as_float((uint32_t)bias[r] << 16);
  uint32_t bits = __float_as_uint(sum);
  if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu))
    bits = 0x7FFF0000u;                                  // NaN
  else
    bits += 0x7FFFu + ((bits >> 16) & 1u);               // round to nearest even
  y[r] = (uint16_t)(bits >> 16);
}

// MODE kModeList: gather launch -- the launch decodes the units named in
// batch.unit_list (of the single tensor item[0]) and writes them one after the other.
// MODE kModeDot: matrix-vector launch -- nothing is written back; every unit's
// elements are multiplied with the input vector as they are decoded.
constexpr int kModeTensor = 0, kModeList = 1, kModeDot = 2, kModeUpdate = 3;
constexpr int kUpdateMaxWarps = 16;                 // the update's operands want registers
constexpr int kDotMaxWarps = NZ_DECODE_MAX_WARPS;   // 16 warps and 128 registers measured slower
template <int S, bool MERGE, int MODE>
__global__ void __launch_bounds__((MODE == kModeDot ? kDotMaxWarps : MODE == kModeUpdate ? kUpdateMaxWarps : NZ_DECODE_MAX_WARPS) * 32, 1)
decode_kernel(const BatchArgs batch) {
  constexpr bool LIST = MODE == kModeList;
  constexpr bool DOT = MODE == kModeDot;
  constexpr bool UPDATE = MODE == kModeUpdate;
  extern __shared__ __align__(128) uint8_t smem[];
  // which tensor this CTA works on, and its rank among that tensor's CTAs
  uint32_t ti = 0;
#pragma unroll
  for (uint32_t t = 1; t < kMaxBatch; ++t)
    if (t < batch.count && blockIdx.x >= batch.item[t].cta_begin) ti = t;
  const uint32_t cta_first = batch.item[ti].cta_begin;
  const uint32_t cta_end = (ti + 1 < batch.count) ? batch.item[ti + 1].cta_begin : batch.n_ctas;
  const uint32_t cta_rank = blockIdx.x - cta_first, cta_count = cta_end - cta_first;
  DecodeArgs a;
  a.container = batch.item[ti].container;
  a.container_bytes = batch.item[ti].container_bytes;
  a.frac = batch.item[ti].frac;
  a.n = batch.item[ti].n;
  a.S = batch.item[ti].S;
  a.n_units = batch.item[ti].n_units;
  a.slot_bytes = batch.slot_bytes;
  a.lut_shift = batch.lut_shift;
  a.lut_bytes = batch.lut_bytes;
  a.ring_offset = batch.ring_offset;
  a.canon = batch.canon;
  a.out_bf16 = batch.item[ti].out_bf16;
  a.out_exp = batch.item[ti].out_exp;
  a.status = batch.status;
  a.unit_list = LIST ? batch.unit_list : nullptr;
  a.n_work = LIST ? batch.n_list : a.n_units;
  a.gx = DOT ? batch.gx : nullptr;
  a.partial = DOT ? batch.partial : nullptr;
  a.in = DOT ? batch.in : 0;
  a.seg = DOT ? batch.seg : 0;
  a.tile_cols = ((MODE == kModeTensor || UPDATE) && MERGE) ? batch.item[ti].tile_cols : 0;
  a.norm = (MERGE && (MODE == kModeTensor || LIST)) ? batch.item[ti].norm : nullptr;
  a.norm_lg = batch.item[ti].norm_lg;
  a.grad = UPDATE ? batch.grad : nullptr;
  a.exp_avg = UPDATE ? batch.exp_avg : nullptr;
  a.exp_avg_sq = UPDATE ? batch.exp_avg_sq : nullptr;
  if (UPDATE) a.adam = batch.adam;
  const uint32_t n_warps = blockDim.x >> 5;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t lut_bytes = 4096u << a.lut_shift;           // 2^pb slots would need 4 << shift each
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + a.lut_bytes);
  uint16_t *cum_sh = reinterpret_cast<uint16_t *>(smem + a.lut_bytes + 8 * 32);  // 257 entries
  uint32_t *flag_sh = reinterpret_cast<uint32_t *>(smem + a.lut_bytes + 8 * 32 + 520);  // 3 words
  uint8_t *slots = smem + a.lut_bytes + 1024;
  (void)lut_bytes;
  const uint32_t bar = smem_u32(&bars[warp]);
  const uint32_t slot0 = smem_u32(slots + (uint64_t)(kChains * warp) * a.slot_bytes);
  // per-warp ring for the packed fractions, behind all slots and their guard band
  const uint32_t ring =
      smem_u32(smem) + a.ring_offset + warp * ring_warp_bytes(S) + lane * (S == 7 ? 8 : 4);

  // Each warp owns one mbarrier; its lane 0 initialises it and is the only
  // thread that ever arms it.
  if (lane == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  // Programmatic dependent launch: let the next kernel of the stream start its
  // own launch now, and do not touch global memory before the previous kernel
  // of the stream has completed.  When the caller vouches that the compressed
  // inputs were complete before that kernel was launched, only the outputs (and
  // the input vector of a matrix-vector launch) depend on it: the wait then
  // moves behind the table build, which overlaps the previous kernel's tail.
  // Both instructions are no-ops for an ordinary launch.
  const bool early = MODE != kModeList && batch.inputs_stable != 0;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!early) asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- start fetching the first group of units, build the decode table meanwhile
  const Header *h = reinterpret_cast<const Header *>(a.container);
  const uint64_t pay_off = payload_offset(a.n_units);
  const uint64_t max_words = (a.container_bytes - pay_off) / 2;   // host checked bytes >= pay_off
  const uint32_t stride = kChains * cta_count * n_warps;
  uint32_t u = kChains * (cta_rank * n_warps + warp);
  uint32_t parity = 0;
  UnitPlan pl[kChains];
  uint32_t real[kChains];      // the units behind work items u .. u+kChains-1
  auto plan_group = [&](uint32_t w) {
#pragma unroll
    for (int c = 0; c < kChains; ++c) {
      real[c] = w + c;
      if (LIST) {
        real[c] = a.n_units;                         // "no unit": plans as nothing to do
        if (w + c < a.n_work) {
          real[c] = __ldg(a.unit_list + w + c);
          if (real[c] >= a.n_units) {
            if (lane == 0) raise(a.status, NZ_STATUS_BAD_UNIT);
            real[c] = a.n_units;
          }
        }
      }
      pl[c] = plan_unit(a, real[c], pay_off, max_words, lane);
    }
  };
  plan_group(u);
  bool staged = stage_units(a, pl, pay_off, slot0, bar, lane);

  table_scan(a, h, pay_off, max_words, cum_sh, flag_sh, warp, lane, n_warps);
  __syncthreads();
  uint32_t pb;
  const uint32_t bad = table_verdict(cum_sh, flag_sh, pb);
  if (bad) {
    // Every exit path orders itself behind the previous kernel of the stream first: the
    // status word is shared with it, and a kernel that retired without waiting would let
    // the next programmatically serialised launch overtake that kernel's reads.
    if (early) asm volatile("griddepcontrol.wait;" ::: "memory");
    // copies may be in flight into this warp's slots: let them land before leaving
    if (staged) wait_staged(bar, parity);
    if (threadIdx.x == 0 && cta_rank == 0) raise(a.status, bad);
    return;
  }
  LutView lv;
  uint32_t row_shift;
  table_fill(a.lut_shift, a.S, pb, smem, cum_sh, warp, lane, n_warps, lv, row_shift);
  const bool canon = MERGE && a.canon && (cum_sh[256] != cum_sh[255]);
  __syncthreads();
  if (early) asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- units, kChains at a time
  const uint8_t *payload = a.container + pay_off;
  const uint32_t lenq = len_quantum(a.S);
  const uint64_t U = 32ull * a.S;

  for (; u < a.n_work; u += stride) {
    if (staged) {
      const bool arrived = wait_staged(bar, parity);
      parity ^= 1;
      if (!__all_sync(0xFFFFFFFFu, arrived)) {
        // The copies may still be in flight, so the slots cannot be reused: flag it,
        // give them one more bounded chance to land and leave.
        if (lane == 0) raise(a.status, NZ_STATUS_TIMEOUT);
        if (!arrived) wait_staged(bar, parity ^ 1);
        return;
      }
    }
    bool full_group = true;
#pragma unroll
    for (int c = 0; c < kChains; ++c)
      full_group = full_group && pl[c].kind == kUnitCoded && (uint64_t)(real[c] + 1) * U <= a.n;
    bool done = false;
    if (full_group) {
      LaneState st[kChains];
      bool ok = true;
#pragma unroll
      for (int c = 0; c < kChains; ++c)
        ok = open_unit(pl[c], slot0 + c * a.slot_bytes, lenq, lane, st[c]) && ok;
      if (ok) {
        done = true;
        const uint8_t *fr[kChains];
        uint8_t *xb[kChains];
        auto run = [&](auto &sink) {
#pragma unroll
          for (int c = 0; c < kChains; ++c) {
            const uint64_t e = (uint64_t)real[c] * U + lane * 8;                  // in the tensor
            const uint64_t o = LIST ? (uint64_t)(u + c) * U + lane * 8 : e;       // in the output
            fr[c] = MERGE ? a.frac + e * (S + 1) / 8 : nullptr;
            xb[c] = MERGE ? nullptr : a.out_exp + o;
            init_sink(sink, c, a, real[c], o, lane);
          }
          if (canon)
            decode_blocks_multi<S, MERGE, true, 0>(st, lv, a.S / 8, fr, sink, xb, ring);
          else if (row_shift == kFastRow)
            decode_blocks_multi<S, MERGE, false, kFastRow>(st, lv, a.S / 8, fr, sink, xb, ring);
          else
            decode_blocks_multi<S, MERGE, false, 0>(st, lv, a.S / 8, fr, sink, xb, ring);
          finish_sink(sink);
        };
        if (DOT) {
          typename std::conditional<DOT, DotSink, StoreSink>::type sink;
          run(sink);
        } else if (UPDATE) {
          if (a.tile_cols) {
            typename std::conditional<UPDATE, UpdateSinkT<64>, StoreSink>::type sink;
            run(sink);
          } else {
            typename std::conditional<UPDATE, UpdateSinkT<256>, StoreSink>::type sink;
            run(sink);
          }
        } else if (MODE == kModeTensor && MERGE && a.tile_cols) {
          typename std::conditional<DOT, DotSink, StoreSinkT<64>>::type sink;     // operand order
          run(sink);
        } else if (MERGE && !UPDATE && a.norm) {
          typename std::conditional<DOT || UPDATE || !MERGE, StoreSink, NormSink<StoreSink>>::type sink;
          run(sink);
        } else {
          typename std::conditional<DOT, DotSink, StoreSink>::type sink;
          run(sink);
        }
        bool low = true;
#pragma unroll
        for (int c = 0; c < kChains; ++c) low = low && st[c].x == kStateLow;
        if (__any_sync(0xFFFFFFFFu, !low) && lane == 0) raise(a.status, NZ_STATUS_BAD_STATE);
      }
    }
    if (!done) {
#pragma unroll
      for (int c = 0; c < kChains; ++c) {
        if (DOT) {
          dot_single<S>(a, pl[c], real[c], slot0 + c * a.slot_bytes, lv, canon, payload, lenq, lane);
        } else {
          const int64_t delta = LIST ? ((int64_t)(u + c) - (int64_t)real[c]) * (int64_t)U : 0;
          decode_single<S, MERGE>(a, pl[c], real[c], delta, slot0 + c * a.slot_bytes, lv, canon,
                                  payload, lenq, lane);
          if (UPDATE) update_decoded_unit(a, real[c], lane);
        }
      }
    }
    // every lane is done reading the slots: fetch this warp's next group
    __syncwarp();
    plan_group(u + stride);
    staged = stage_units(a, pl, pay_off, slot0, bar, lane);
  }
}

// ------------------------------------------------------------------- host
struct HostItem {
  const void *container;
  uint64_t container_bytes;
  const void *frac;
  uint64_t n;
  uint32_t max_unit_words;
  void *out_bf16;
  void *out_exp;
  const uint32_t *unit_list;   // gather: device array of unit numbers (else null)
  uint32_t n_list;
  const float *gx;             // matrix-vector: input vector (else null), partial sums,
  float *partial;              //   row length and partial-sum places per unit
  uint32_t in, seg;
  uint32_t flags;              // NZ_ITEM_* of the C interface
  uint32_t tile_cols;          // operand order: row length of the matrix (0 = stream order)
  uint32_t S;                  // lane symbols of this tensor
  const uint16_t *grad;        // update: gradient and AdamW moments (bf16, else null)
  uint16_t *exp_avg, *exp_avg_sq;
  AdamArgs adam;
  const uint8_t *norm;         // block normaliser bytes (else null) and log2 of the group size
  uint32_t norm_lg;
};

// Units a launch decodes for an item.
static inline uint64_t work_units(const HostItem &it) {
  return it.unit_list ? it.n_list : unit_count(it.n, it.S);
}

// Grid geometry of one launch over `count` tensors.  One CTA per SM.  Every
// warp decodes whole units, kChains at a time, so a tensor is only as fast as its
// busiest CTA: each tensor gets CTAs in proportion to its units, every CTA the
// same number of warps, every warp the same number of unit groups (within one).
// The decode table gets what shared memory the slots and rings leave (more
// copies = fewer bank conflicts), at most 128 KB.
static int decode_geometry(const HostItem *items, uint32_t count, uint32_t ring_bytes,
                           BatchArgs &b, uint32_t &warps, uint32_t &smem_bytes) {
  // tensors of one launch may differ in lane symbols: slots and guard band are sized for
  // the longest unit, and a tensor's share of the CTAs follows its symbols, not its units
  uint32_t S = 0;
  uint64_t unit_bytes = 0, total_units = 0;
  for (uint32_t t = 0; t < count; ++t) {
    const uint64_t U = 32ull * items[t].S;
    uint64_t ub = items[t].max_unit_words ? (uint64_t)items[t].max_unit_words * 2 : U;
    if (ub > U) ub = U;
    if (ub > unit_bytes) unit_bytes = ub;
    if (items[t].S > S) S = items[t].S;
    total_units += work_units(items[t]) * items[t].S;
  }
  const uint64_t U = 32ull * S;
  b.S = S;
  if (unit_bytes < 160) unit_bytes = 160;
  b.slot_bytes = (uint32_t)((unit_bytes + 32 + 15) & ~uint64_t(15));
  const uint32_t guard = ((S + 8) * 2 + 127) & ~127u;
  const uint32_t sm_smem = 227u * 1024u;
  const uint32_t kMaxWarps = items[0].gx ? (uint32_t)kDotMaxWarps
                             : items[0].grad ? (uint32_t)kUpdateMaxWarps : (uint32_t)NZ_DECODE_MAX_WARPS;
  const uint32_t per_warp = kChains * b.slot_bytes + ring_bytes;
  const uint32_t min_fixed = 16 * 1024 + 1024 + guard;
  if (min_fixed + per_warp > sm_smem) {
    set_error("decode: a warp's units of %u symbols do not fit in shared memory", (unsigned)U);
    return NZ_E_ARG;
  }
  uint32_t cap = (sm_smem - min_fixed) / per_warp;
  if (cap > kMaxWarps) cap = kMaxWarps;

  // CTAs per tensor: proportional to units, at least one, summing to the SM count
  // (or fewer when there is not enough work to give every SM a group of units)
  const uint32_t sms = (uint32_t)sm_count();
  uint64_t total_groups = 0;
  for (uint32_t t = 0; t < count; ++t) total_groups += (work_units(items[t]) + kChains - 1) / kChains;
  uint32_t n_ctas = sms;
  if (total_groups < n_ctas) n_ctas = (uint32_t)total_groups;
  if (n_ctas < count) n_ctas = count;
  uint32_t ctas[kMaxBatch], used = 0;
  for (uint32_t t = 0; t < count; ++t) {
    const uint64_t nu = work_units(items[t]);
    uint64_t c = total_units ? (nu * items[t].S * n_ctas + total_units / 2) / total_units : 1;
    const uint64_t groups = (nu + kChains - 1) / kChains;
    if (c > groups) c = groups;
    if (c < 1) c = 1;
    ctas[t] = (uint32_t)c;
    used += ctas[t];
  }
  // fix the rounding: take from / give to the tensor with the most / fewest groups per CTA
  auto load = [&](uint32_t t, uint32_t c) {
    return (double)((work_units(items[t]) + kChains - 1) / kChains) * items[t].S / (double)c;
  };
  while (used > n_ctas) {
    uint32_t best = kMaxBatch;
    for (uint32_t t = 0; t < count; ++t)
      if (ctas[t] > 1 && (best == kMaxBatch || load(t, ctas[t] - 1) < load(best, ctas[best] - 1)))
        best = t;
    if (best == kMaxBatch) break;
    --ctas[best];
    --used;
  }
  while (used < n_ctas) {
    uint32_t best = kMaxBatch;
    for (uint32_t t = 0; t < count; ++t) {
      const uint64_t groups = (work_units(items[t]) + kChains - 1) / kChains;
      if (ctas[t] < groups && (best == kMaxBatch || load(t, ctas[t]) > load(best, ctas[best])))
        best = t;
    }
    if (best == kMaxBatch) break;
    ++ctas[best];
    ++used;
  }
  // warps per CTA: enough for the busiest CTA's groups, spread over whole rounds
  uint32_t max_groups = 1;
  for (uint32_t t = 0; t < count; ++t) {
    const uint64_t groups = (work_units(items[t]) + kChains - 1) / kChains;
    const uint32_t per_cta = (uint32_t)((groups + ctas[t] - 1) / ctas[t]);
    if (per_cta > max_groups) max_groups = per_cta;
  }
  const uint32_t rounds = (max_groups + cap - 1) / cap;
  warps = (max_groups + rounds - 1) / rounds;
  if (warps < 1) warps = 1;
  // largest table that still leaves room for these warps
  b.lut_shift = 2;
  for (uint32_t sh = 5; sh > 2; --sh) {        // 2^12 slots x 2^(sh-2) copies
    if ((4096u << sh) + 1024 + guard + warps * per_warp <= sm_smem) {
      b.lut_shift = sh;
      break;
    }
  }
  b.lut_bytes = 4096u << b.lut_shift;
  b.ring_offset = b.lut_bytes + 1024 + guard + warps * kChains * b.slot_bytes;
  smem_bytes = b.ring_offset + warps * ring_bytes;
  uint32_t begin = 0;
  for (uint32_t t = 0; t < count; ++t) {
    b.item[t].cta_begin = begin;
    begin += ctas[t];
  }
  b.n_ctas = begin;
  return NZ_OK;
}

template <int S, bool MERGE, int MODE = kModeTensor>
static int launch_decode(const BatchArgs &b, uint32_t warps, uint32_t smem_bytes, cudaStream_t st) {
  auto kern = decode_kernel<S, MERGE, MODE>;
  // The opt-in to large dynamic shared memory is per kernel and device.  It is made once
  // per (instantiation, device), for the most a CTA can have, under a lock: concurrent
  // callers can then never leave the attribute below what a launch needs.
  {
    static std::mutex mu;
    static bool opted[kMaxDeviceOrdinals] = {};
    int dev = 0;
    NZ_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= kMaxDeviceOrdinals || !opted[dev]) {
      NZ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)kMaxDynamicSmem));
      if (dev >= 0 && dev < kMaxDeviceOrdinals) opted[dev] = true;
    }
  }
  // Programmatic stream serialisation: this launch may begin while the previous
  // kernel of the stream drains; the kernel itself waits (griddepcontrol.wait)
  // before it reads or writes global memory, so ordering is preserved.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(b.n_ctas);
  cfg.blockDim = dim3(warps * 32);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  NZ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, b));
  return NZ_OK;
}

// Decode `count` tensors (same precision and lane_symbols), kMaxBatch per launch.
int decode_many(const HostItem *items, uint32_t count, int precision, uint32_t S, int canon,
                bool merge, void *status, cudaStream_t st) {
  HostItem live[kMaxBatch];
  uint32_t n_live = 0;
  auto flush = [&]() -> int {
    if (n_live == 0) return NZ_OK;
    BatchArgs b;
    memset(&b, 0, sizeof(b));
    uint32_t warps = 0, smem_bytes = 0;
    // the exponent-only kernel is the precision-7 instantiation
    int rc = decode_geometry(live, n_live, ring_warp_bytes(merge ? precision : 7), b, warps,
                             smem_bytes);
    if (rc) return rc;
    b.count = n_live;
    b.canon = canon;
    b.status = (uint32_t *)status;
    for (uint32_t t = 0; t < n_live; ++t) {
      b.item[t].container = (const uint8_t *)live[t].container;
      b.item[t].container_bytes = live[t].container_bytes;
      b.item[t].frac = (const uint8_t *)live[t].frac;
      b.item[t].n = live[t].n;
      b.item[t].out_bf16 = (uint16_t *)live[t].out_bf16;
      b.item[t].out_exp = (uint8_t *)live[t].out_exp;
      b.item[t].n_units = (uint32_t)unit_count(live[t].n, live[t].S);
      b.item[t].tile_cols = live[t].tile_cols;
      b.item[t].S = live[t].S;
      b.item[t].norm = live[t].norm;
      b.item[t].norm_lg = live[t].norm_lg;
    }
    const bool gather = live[0].unit_list != nullptr;   // gather calls pass a single item
    b.unit_list = live[0].unit_list;
    b.n_list = live[0].n_list;
    const bool dot = live[0].gx != nullptr;             // so do matrix-vector calls
    b.gx = live[0].gx;
    b.partial = live[0].partial;
    b.in = live[0].in;
    b.seg = live[0].seg;
    const bool update = live[0].grad != nullptr;        // and update calls
    b.grad = live[0].grad;
    b.exp_avg = live[0].exp_avg;
    b.exp_avg_sq = live[0].exp_avg_sq;
    b.adam = live[0].adam;
    b.inputs_stable = 1;
    for (uint32_t t = 0; t < n_live; ++t)
      if (!(live[t].flags & NZ_ITEM_INPUTS_STABLE)) b.inputs_stable = 0;
    n_live = 0;
    if (gather) {
      switch (precision) {
        case 0: return launch_decode<0, true, kModeList>(b, warps, smem_bytes, st);
        case 1: return launch_decode<1, true, kModeList>(b, warps, smem_bytes, st);
        case 3: return launch_decode<3, true, kModeList>(b, warps, smem_bytes, st);
        default: return launch_decode<7, true, kModeList>(b, warps, smem_bytes, st);
      }
    }
    if (update) {
      switch (precision) {
        case 0: return launch_decode<0, true, kModeUpdate>(b, warps, smem_bytes, st);
        case 1: return launch_decode<1, true, kModeUpdate>(b, warps, smem_bytes, st);
        case 3: return launch_decode<3, true, kModeUpdate>(b, warps, smem_bytes, st);
        default: return launch_decode<7, true, kModeUpdate>(b, warps, smem_bytes, st);
      }
    }
    if (dot) {
      switch (precision) {
        case 0: return launch_decode<0, true, kModeDot>(b, warps, smem_bytes, st);
        case 1: return launch_decode<1, true, kModeDot>(b, warps, smem_bytes, st);
        case 3: return launch_decode<3, true, kModeDot>(b, warps, smem_bytes, st);
        default: return launch_decode<7, true, kModeDot>(b, warps, smem_bytes, st);
      }
    }
    if (!merge) return launch_decode<7, false>(b, warps, smem_bytes, st);
    switch (precision) {
      case 0: return launch_decode<0, true>(b, warps, smem_bytes, st);
      case 1: return launch_decode<1, true>(b, warps, smem_bytes, st);
      case 3: return launch_decode<3, true>(b, warps, smem_bytes, st);
      default: return launch_decode<7, true>(b, warps, smem_bytes, st);
    }
  };
  for (uint32_t i = 0; i < count; ++i) {
    if (items[i].n == 0) continue;
    const uint64_t nu = unit_count(items[i].n, items[i].S ? items[i].S : S);
    if (items[i].container_bytes < payload_offset(nu)) {
      set_error("decode: container %u of %llu bytes is too short for %llu units", i,
                (unsigned long long)items[i].container_bytes, (unsigned long long)nu);
      return NZ_E_FORMAT;
    }
    live[n_live] = items[i];
    if (!live[n_live].S) live[n_live].S = S;
    ++n_live;
    if (n_live == kMaxBatch) {
      int rc = flush();
      if (rc) return rc;
    }
  }
  return flush();
}

int decode_common(const void *container, uint64_t container_bytes, const void *frac, uint64_t n,
                  int precision, uint32_t S, uint32_t max_unit_words, int canon, void *out_bf16,
                  void *out_exp, void *status, cudaStream_t st) {
  HostItem it;
  it.container = container;
  it.container_bytes = container_bytes;
  it.frac = frac;
  it.n = n;
  it.max_unit_words = max_unit_words;
  it.out_bf16 = out_bf16;
  it.out_exp = out_exp;
  it.unit_list = nullptr;
  it.n_list = 0;
  it.gx = nullptr;
  it.partial = nullptr;
  it.in = it.seg = 0;
  it.flags = 0;
  it.tile_cols = 0;
  it.S = 0;
  it.grad = nullptr;
  it.exp_avg = it.exp_avg_sq = nullptr;
  it.norm = nullptr;
  it.norm_lg = 0;
  return decode_many(&it, 1, precision, S, canon, out_bf16 != nullptr, status, st);
}

// A [rows, cols] matrix stored in operand order, decoded to row-major.
int decode_operand(const void *container, uint64_t container_bytes, const void *frac, uint64_t rows,
                   uint64_t cols, int precision, uint32_t S, uint32_t max_unit_words, int canon,
                   void *out_bf16, void *status, cudaStream_t st) {
  HostItem it;
  memset(&it, 0, sizeof(it));
  it.container = container;
  it.container_bytes = container_bytes;
  it.frac = frac;
  it.n = rows * cols;
  it.max_unit_words = max_unit_words;
  it.out_bf16 = out_bf16;
  it.tile_cols = (uint32_t)cols;
  return decode_many(&it, 1, precision, S, canon, true, status, st);
}

// Decode a tensor and apply an AdamW step to it on the way out: out_bf16 receives the
// updated (row-major) weights, the moments (bf16) are updated in place.
int decode_update(const void *container, uint64_t container_bytes, const void *frac, uint64_t n,
                  uint64_t operand_cols, int precision, uint32_t S, uint32_t max_unit_words,
                  int canon, const void *grad, void *exp_avg, void *exp_avg_sq, const AdamArgs &adam,
                  void *out_bf16, void *status, cudaStream_t st) {
  HostItem it;
  memset(&it, 0, sizeof(it));
  it.container = container;
  it.container_bytes = container_bytes;
  it.frac = frac;
  it.n = n;
  it.max_unit_words = max_unit_words;
  it.out_bf16 = out_bf16;
  it.tile_cols = (uint32_t)operand_cols;
  it.grad = (const uint16_t *)grad;
  it.exp_avg = (uint16_t *)exp_avg;
  it.exp_avg_sq = (uint16_t *)exp_avg_sq;
  it.adam = adam;
  return decode_many(&it, 1, precision, S, canon, true, status, st);
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

extern "C" int nz_decompress_bf16_batch(const nz_decompress_item *items, uint32_t count,
                                        int precision, uint32_t lane_symbols, int canonical_nan,
                                        void *status, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_decompress_bf16_batch: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  if (count == 0) return NZ_OK;
  if (!items) {
    nz::set_error("nz_decompress_bf16_batch: null item array");
    return NZ_E_ARG;
  }
  constexpr uint32_t kChunk = 64;
  nz::HostItem host[kChunk];
  for (uint32_t base = 0; base < count; base += kChunk) {
    const uint32_t m = count - base < kChunk ? count - base : kChunk;
    for (uint32_t i = 0; i < m; ++i) {
      const nz_decompress_item &it = items[base + i];
      int rc = check_decode_args("nz_decompress_bf16_batch", it.container, it.n, lane_symbols);
      if (rc) return rc;
      if (it.n && (!it.out_bf16 || !it.frac_in || ((uintptr_t)it.out_bf16 & 15) ||
                   ((uintptr_t)it.frac_in & 7))) {
        nz::set_error("nz_decompress_bf16_batch: item %u: output must be 16-byte, fractions "
                      "8-byte aligned", base + i);
        return NZ_E_ARG;
      }
      host[i].container = it.container;
      host[i].container_bytes = it.container_bytes;
      host[i].frac = it.frac_in;
      host[i].n = it.n;
      host[i].max_unit_words = it.max_unit_words;
      host[i].out_bf16 = it.out_bf16;
      host[i].out_exp = nullptr;
      host[i].unit_list = nullptr;
      host[i].n_list = 0;
      host[i].gx = nullptr;
      host[i].partial = nullptr;
      host[i].in = host[i].seg = 0;
      host[i].flags = it.flags;
      host[i].tile_cols = 0;
      host[i].S = 0;
      host[i].grad = nullptr;
      host[i].exp_avg = host[i].exp_avg_sq = nullptr;
      host[i].norm = nullptr;
      host[i].norm_lg = 0;
      if (it.normalizers) {
        const uint32_t g = it.normalizer_group;
        if (g == 0 || g > 1024 || (g & (g - 1)) || it.operand_cols) {
          nz::set_error("nz_decompress_bf16_batch: item %u: the normaliser group must be a power "
                        "of two in [1, 1024] (got %u) and the tensor in stream order", base + i, g);
          return NZ_E_ARG;
        }
        host[i].norm = (const uint8_t *)it.normalizers;
        while ((1u << host[i].norm_lg) < g) ++host[i].norm_lg;
      }
      if (it.lane_symbols) {
        if (!nz::valid_lane_symbols(it.lane_symbols)) {
          nz::set_error("nz_decompress_bf16_batch: item %u: lane_symbols must be a multiple of 8 "
                        "in [8, %u] (got %u)", base + i, nz::kMaxLaneSymbols, it.lane_symbols);
          return NZ_E_ARG;
        }
        host[i].S = it.lane_symbols;
      }
      if (it.operand_cols) {
        const uint64_t c = it.operand_cols;
        const uint32_t item_s = it.lane_symbols ? it.lane_symbols : lane_symbols;
        if (c % 64 || it.n % (4 * c) || (c / 64) % (item_s / 8) || c >= (1ull << 31)) {
          nz::set_error("nz_decompress_bf16_batch: item %u: %llu elements in rows of %llu are not "
                        "in operand order for lane_symbols %u", base + i,
                        (unsigned long long)it.n, (unsigned long long)c, lane_symbols);
          return NZ_E_ARG;
        }
        host[i].tile_cols = (uint32_t)c;
      }
    }
    int rc = nz::decode_many(host, m, precision, lane_symbols, canonical_nan, true, status,
                             (cudaStream_t)stream);
    if (rc) return rc;
  }
  return NZ_OK;
}

static int decompress_units(const void *container, uint64_t container_bytes, const void *frac_in,
                            uint64_t n, int precision, uint32_t lane_symbols,
                            uint32_t max_unit_words, int canonical_nan, const void *unit_ids,
                            uint32_t n_ids, const void *normalizers, uint32_t group, void *out_bf16,
                            void *status, void *stream);

extern "C" int nz_decompress_bf16_units(const void *container, uint64_t container_bytes,
                                        const void *frac_in, uint64_t n, int precision,
                                        uint32_t lane_symbols, uint32_t max_unit_words,
                                        int canonical_nan, const void *unit_ids, uint32_t n_ids,
                                        void *out_bf16, void *status, void *stream) {
  return decompress_units(container, container_bytes, frac_in, n, precision, lane_symbols,
                          max_unit_words, canonical_nan, unit_ids, n_ids, nullptr, 0, out_bf16, status,
                          stream);
}

static int decompress_units(const void *container, uint64_t container_bytes, const void *frac_in,
                            uint64_t n, int precision, uint32_t lane_symbols,
                            uint32_t max_unit_words, int canonical_nan, const void *unit_ids,
                            uint32_t n_ids, const void *normalizers, uint32_t group, void *out_bf16,
                            void *status, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_decompress_bf16_units: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  int rc = check_decode_args("nz_decompress_bf16_units", container, n, lane_symbols);
  if (rc) return rc;
  if (n_ids == 0) return NZ_OK;
  if (n == 0) {
    nz::set_error("nz_decompress_bf16_units: an empty tensor has no units");
    return NZ_E_ARG;
  }
  if (!unit_ids || ((uintptr_t)unit_ids & 3) || !out_bf16 || !frac_in ||
      ((uintptr_t)out_bf16 & 15) || ((uintptr_t)frac_in & 7)) {
    nz::set_error("nz_decompress_bf16_units: unit list must be a 4-byte aligned device pointer, "
                  "output 16-byte, fractions 8-byte aligned");
    return NZ_E_ARG;
  }
  nz::HostItem it;
  it.container = container;
  it.container_bytes = container_bytes;
  it.frac = frac_in;
  it.n = n;
  it.max_unit_words = max_unit_words;
  it.out_bf16 = out_bf16;
  it.out_exp = nullptr;
  it.unit_list = (const uint32_t *)unit_ids;
  it.n_list = n_ids;
  it.gx = nullptr;
  it.partial = nullptr;
  it.in = it.seg = 0;
  it.flags = 0;
  it.tile_cols = 0;
  it.S = 0;
  it.grad = nullptr;
  it.exp_avg = it.exp_avg_sq = nullptr;
  it.norm = nullptr;
  it.norm_lg = 0;
  if (normalizers) {
    if (group == 0 || group > 1024 || (group & (group - 1))) {
      nz::set_error("gather: the normaliser group must be a power of two in [1, 1024] (got %u)", group);
      return NZ_E_ARG;
    }
    it.norm = (const uint8_t *)normalizers;
    while ((1u << it.norm_lg) < group) ++it.norm_lg;
  }
  return nz::decode_many(&it, 1, precision, lane_symbols, canonical_nan, true, status,
                         (cudaStream_t)stream);
}

namespace nz {

// Row gather, step 1: the units that hold each requested row.  Row r of a
// table with rows of `row_len` elements starts at element r * row_len; it is
// decoded as `per_row` consecutive units from the one that holds its first
// element (numbers past the last unit are clamped: their output is not used).
// Rows outside the table get unit n_units, which the decoder reports.
__global__ void gather_plan_kernel(const int64_t *__restrict__ rows, uint32_t k, uint64_t row_len,
                                   uint64_t n_rows, uint64_t U, uint32_t n_units, uint32_t per_row,
                                   uint32_t *__restrict__ units) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (uint64_t)k * per_row) return;
  const int64_t r = rows[i / per_row];
  uint32_t u = n_units;
  if (r >= 0 && (uint64_t)r < n_rows) {
    const uint64_t v = (uint64_t)r * row_len / U + i % per_row;
    u = v < n_units ? (uint32_t)v : n_units - 1;
  }
  units[i] = u;
}

// Row gather, step 3: copy each row out of the units decoded for it.  VEC = 8
// moves 16 bytes per thread (row length and so every offset a multiple of 8).
template <int VEC>
__global__ void gather_copy_kernel(const int64_t *__restrict__ rows, uint32_t k, uint64_t row_len,
                                   uint64_t n_rows, uint64_t U, uint32_t per_row,
                                   const uint16_t *__restrict__ staging,
                                   uint16_t *__restrict__ out) {
  const uint64_t per = row_len / VEC;
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (uint64_t)k * per) return;
  const uint64_t row = i / per, j = (i % per) * VEC;
  const int64_t r = rows[row];
  if (r < 0 || (uint64_t)r >= n_rows) return;        // flagged by the decoder; left untouched
  const uint64_t src = row * per_row * U + ((uint64_t)r * row_len) % U + j;
  if (VEC == 8)
    *reinterpret_cast<uint4 *>(out + row * row_len + j) =
        *reinterpret_cast<const uint4 *>(staging + src);
  else
    out[row * row_len + j] = staging[src];
}

static inline uint32_t gather_units_per_row(uint64_t row_len, uint64_t U) {
  if (U % row_len == 0) return 1;                            // a unit holds whole rows
  if (row_len % U == 0) return (uint32_t)(row_len / U);      // a row is whole units
  return (uint32_t)((row_len + U - 1) / U + 1);              // rows straddle unit boundaries
}

}  // namespace nz

extern "C" uint64_t nz_gather_scratch_bytes(uint32_t n_rows_out, uint64_t row_len,
                                            uint32_t lane_symbols) {
  if (!nz::valid_lane_symbols(lane_symbols) || row_len == 0) return 0;
  const uint64_t U = 32ull * lane_symbols;
  const uint64_t per_row = nz::gather_units_per_row(row_len, U);
  // unit list (4 bytes each, rounded to 16) + the decoded units
  return nz::align16((uint64_t)n_rows_out * per_row * 4) + (uint64_t)n_rows_out * per_row * U * 2;
}

extern "C" int nz_gather_rows_bf16(const void *container, uint64_t container_bytes,
                                   const void *frac_in, uint64_t n, int precision,
                                   uint32_t lane_symbols, uint32_t max_unit_words,
                                   int canonical_nan, uint64_t row_len, const void *rows_i64,
                                   uint32_t n_rows_out, void *out_bf16, void *scratch,
                                   uint64_t scratch_bytes, void *status, void *stream) {
  return nz_gather_rows_normalized_bf16(container, container_bytes, frac_in, n, precision,
                                        lane_symbols, max_unit_words, canonical_nan, row_len,
                                        rows_i64, n_rows_out, nullptr, 0, out_bf16, scratch,
                                        scratch_bytes, status, stream);
}

extern "C" int nz_gather_rows_normalized_bf16(const void *container, uint64_t container_bytes,
                                              const void *frac_in, uint64_t n, int precision,
                                              uint32_t lane_symbols, uint32_t max_unit_words,
                                              int canonical_nan, uint64_t row_len,
                                              const void *rows_i64, uint32_t n_rows_out,
                                              const void *normalizers, uint32_t normalizer_group,
                                              void *out_bf16, void *scratch, uint64_t scratch_bytes,
                                              void *status, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_gather_rows_bf16: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  int rc = check_decode_args("nz_gather_rows_bf16", container, n, lane_symbols);
  if (rc) return rc;
  if (row_len == 0 || n == 0 || n % row_len) {
    nz::set_error("nz_gather_rows_bf16: row length %llu does not divide the %llu elements",
                  (unsigned long long)row_len, (unsigned long long)n);
    return NZ_E_ARG;
  }
  if (n_rows_out == 0) return NZ_OK;
  if (!rows_i64 || ((uintptr_t)rows_i64 & 7) || !out_bf16 || !frac_in || !scratch ||
      ((uintptr_t)scratch & 15) || ((uintptr_t)frac_in & 7)) {
    nz::set_error("nz_gather_rows_bf16: null or misaligned pointer (rows and fractions 8-byte, "
                  "scratch 16-byte aligned)");
    return NZ_E_ARG;
  }
  const uint64_t need = nz_gather_scratch_bytes(n_rows_out, row_len, lane_symbols);
  if (scratch_bytes < need) {
    nz::set_error("nz_gather_rows_bf16: scratch of %llu bytes is smaller than the %llu required",
                  (unsigned long long)scratch_bytes, (unsigned long long)need);
    return NZ_E_CAPACITY;
  }
  const uint64_t U = 32ull * lane_symbols;
  const uint32_t per_row = nz::gather_units_per_row(row_len, U);
  const uint64_t n_list = (uint64_t)n_rows_out * per_row;
  if (n_list >= (1ull << 32)) {
    nz::set_error("nz_gather_rows_bf16: %u rows of %u units each are too many for one call",
                  n_rows_out, per_row);
    return NZ_E_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t *units = (uint32_t *)scratch;
  uint16_t *staging = (uint16_t *)((uint8_t *)scratch + nz::align16(n_list * 4));
  const uint32_t n_units = (uint32_t)nz::unit_count(n, lane_symbols);
  const uint64_t table_rows = n / row_len;
  nz::gather_plan_kernel<<<(unsigned)((n_list + 255) / 256), 256, 0, st>>>(
      (const int64_t *)rows_i64, n_rows_out, row_len, table_rows, U, n_units, per_row, units);
  NZ_LAUNCH_CHECK("gather_plan_kernel");
  rc = decompress_units(container, container_bytes, frac_in, n, precision, lane_symbols,
                        max_unit_words, canonical_nan, units, (uint32_t)n_list, normalizers,
                        normalizer_group, staging, status, stream);
  if (rc) return rc;
  const bool vec = row_len % 8 == 0 && ((uintptr_t)out_bf16 & 15) == 0;
  const uint64_t threads = vec ? (uint64_t)n_rows_out * (row_len / 8) : (uint64_t)n_rows_out * row_len;
  const uint64_t blocks = (threads + 255) / 256;
  if (blocks >= (1ull << 31)) {
    nz::set_error("nz_gather_rows_bf16: output too large for one call");
    return NZ_E_ARG;
  }
  if (vec)
    nz::gather_copy_kernel<8><<<(unsigned)blocks, 256, 0, st>>>(
        (const int64_t *)rows_i64, n_rows_out, row_len, table_rows, U, per_row, staging,
        (uint16_t *)out_bf16);
  else
    nz::gather_copy_kernel<1><<<(unsigned)blocks, 256, 0, st>>>(
        (const int64_t *)rows_i64, n_rows_out, row_len, table_rows, U, per_row, staging,
        (uint16_t *)out_bf16);
  NZ_LAUNCH_CHECK("gather_copy_kernel");
  return NZ_OK;
}

namespace nz {
// Rows of an [out, in] matrix that one unit of U elements can touch.
static inline uint32_t dot_segments(uint64_t in_features, uint64_t U) {
  return (uint32_t)((U - 1) / in_features + 2);
}
}  // namespace nz

extern "C" uint64_t nz_linear_vec_scratch_bytes(uint64_t n, uint64_t in_features,
                                                uint32_t lane_symbols) {
  if (!nz::valid_lane_symbols(lane_symbols) || in_features == 0) return 0;
  const uint64_t U = 32ull * lane_symbols;
  return nz::align16(nz::unit_count(n, lane_symbols) * nz::dot_segments(in_features, U) * 4);
}

extern "C" int nz_linear_vec_bf16(const void *container, uint64_t container_bytes,
                                  const void *frac_in, uint64_t n, int precision,
                                  uint32_t lane_symbols, uint32_t max_unit_words,
                                  int canonical_nan, uint64_t in_features, const void *x_f32,
                                  const void *bias_bf16, void *y_bf16, void *scratch,
                                  uint64_t scratch_bytes, void *status, void *stream) {
  if (!nz::valid_precision(precision)) {
    nz::set_error("nz_linear_vec_bf16: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  int rc = check_decode_args("nz_linear_vec_bf16", container, n, lane_symbols);
  if (rc) return rc;
  if (n == 0 || in_features == 0 || in_features % 256 || n % in_features ||
      in_features >= (1ull << 31) || n / in_features >= (1ull << 31)) {
    nz::set_error("nz_linear_vec_bf16: the matrix must have rows of a multiple of 256 elements "
                  "(got %llu elements, rows of %llu)", (unsigned long long)n,
                  (unsigned long long)in_features);
    return NZ_E_ARG;
  }
  if (!x_f32 || ((uintptr_t)x_f32 & 15) || !y_bf16 || !frac_in || ((uintptr_t)frac_in & 7) ||
      !scratch || ((uintptr_t)scratch & 15)) {
    nz::set_error("nz_linear_vec_bf16: null or misaligned pointer (input vector and scratch "
                  "16-byte, fractions 8-byte aligned)");
    return NZ_E_ARG;
  }
  const uint64_t need = nz_linear_vec_scratch_bytes(n, in_features, lane_symbols);
  if (scratch_bytes < need) {
    nz::set_error("nz_linear_vec_bf16: scratch of %llu bytes is smaller than the %llu required",
                  (unsigned long long)scratch_bytes, (unsigned long long)need);
    return NZ_E_CAPACITY;
  }
  const uint64_t U = 32ull * lane_symbols;
  nz::HostItem it;
  it.container = container;
  it.container_bytes = container_bytes;
  it.frac = frac_in;
  it.n = n;
  it.max_unit_words = max_unit_words;
  it.out_bf16 = nullptr;
  it.out_exp = nullptr;
  it.unit_list = nullptr;
  it.n_list = 0;
  it.gx = (const float *)x_f32;
  it.partial = (float *)scratch;
  it.in = (uint32_t)in_features;
  it.seg = nz::dot_segments(in_features, U);
  it.flags = 0;
  it.tile_cols = 0;
  it.S = 0;
  it.grad = nullptr;
  it.exp_avg = it.exp_avg_sq = nullptr;
  it.norm = nullptr;
  it.norm_lg = 0;
  rc = nz::decode_many(&it, 1, precision, lane_symbols, canonical_nan, true, status,
                       (cudaStream_t)stream);
  if (rc) return rc;
  const uint32_t out_features = (uint32_t)(n / in_features);
  nz::dot_finish_kernel<<<(out_features + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      (const float *)scratch, it.seg, U, it.in, out_features, (const uint16_t *)bias_bf16,
      (uint16_t *)y_bf16);
  NZ_LAUNCH_CHECK("dot_finish_kernel");
  return NZ_OK;
}
