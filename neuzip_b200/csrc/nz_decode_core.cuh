// Device-side building blocks of the NZR1 rANS decoder, shared by the decode
// kernels (nz_decode.cu) and the fused decode -> tensor-core GEMM (nz_linear.cu):
// PTX helpers, the per-symbol decode step, the merge of decoded exponents with the
// packed fractions, unit planning / staging / opening, and the decode-table build.
#pragma once

#include "nz_common.cuh"

#ifndef NZ_DECODE_CHAINS
#define NZ_DECODE_CHAINS 2
#endif

namespace nz {

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

// Per-lane constants of the replicated decode table.
struct LutView {
  uint32_t base;    // shared address of this lane's copy (table base + bank offset)
  uint32_t mask;    // 2^pb - 1
  uint32_t stride;  // bytes between slots (4 x copies)
  uint32_t pb;      // probability bits
  uint32_t k64k;    // 65536 in a register: keeps the shift-in an integer multiply-add
};

// Table entry: symbol << 23 | freq << 12 | (slot - first slot of the symbol).
// Frequencies never exceed 2047 (the encoder's choice of resolution sees to
// that, the table build checks it), so bit 31 is clear.  The symbol sits where
// the exponent of the upper bf16 of an output word goes, and 16 bits above
// where the exponent of the lower one goes.
constexpr uint32_t kEntSymShift = 23;
constexpr uint32_t kEntFreqShift = 12;
constexpr uint32_t kEntLowMask = (1u << kEntSymShift) - 1u;   // freq << 12 | offset
__device__ __forceinline__ uint32_t entry_symbol(uint32_t ent) { return ent >> kEntSymShift; }

// One symbol.  Returns the table entry.  Written in PTX so that the
// renormalisation stays predicated (no divergent branch) and the 16-bit stream
// word is loaded straight into a 32-bit register.  ROW is log2 of the bytes
// between table slots when the caller knows it at compile time (0 = use
// lv.stride): a constant shift folds into the address add, which shortens the
// dependent chain x -> slot -> entry -> x that bounds a lane's rate.
// The state update uses f*(q - 4096) + (f*4096 + offset) = f*q + offset
// (mod 2^32), so that the entry's low 23 bits serve as the addend unshifted.
template <int ROW>
__device__ __forceinline__ uint32_t decode_step(LaneState &st, const LutView &lv) {
  uint32_t ent;
  if (ROW > 0) {
    asm volatile(
        "{\n\t"
        ".reg .b32 a, q, f, b;\n\t"
        ".reg .pred r;\n\t"
        "and.b32 a, %1, %5;\n\t"
        "shl.b32 a, a, %8;\n\t"
        "add.u32 a, a, %4;\n\t"                // slot * 2^ROW + lane's table base
        "ld.shared.u32 %0, [a];\n\t"
        "shr.u32 q, %1, %6;\n\t"
        "add.s32 q, q, -4096;\n\t"
        "and.b32 b, %0, 0x7FFFFF;\n\t"         // freq << 12 | offset
        "shr.u32 f, b, 12;\n\t"
        "mad.lo.u32 %1, f, q, b;\n\t"
        "setp.lt.u32 r, %1, 65536;\n\t"
        "@r mad.lo.u32 %1, %1, %7, %3;\n\t"    // x = x * 65536 + w
        "@r add.u32 %2, %2, 2;\n\t"
        "@r ld.shared.u16 %3, [%2];\n\t"
        "}"
        : "=&r"(ent), "+r"(st.x), "+r"(st.p), "+r"(st.w)
        : "r"(lv.base), "r"(lv.mask), "r"(lv.pb), "r"(lv.k64k), "n"(ROW));
  } else {
    asm volatile(
        "{\n\t"
        ".reg .b32 a, q, f, b;\n\t"
        ".reg .pred r;\n\t"
        "and.b32 a, %1, %5;\n\t"
        "mad.lo.u32 a, a, %6, %4;\n\t"         // slot * stride + lane's table base
        "ld.shared.u32 %0, [a];\n\t"
        "shr.u32 q, %1, %7;\n\t"
        "add.s32 q, q, -4096;\n\t"
        "and.b32 b, %0, 0x7FFFFF;\n\t"         // freq << 12 | offset
        "shr.u32 f, b, 12;\n\t"
        "mad.lo.u32 %1, f, q, b;\n\t"
        "setp.lt.u32 r, %1, 65536;\n\t"
        "@r mad.lo.u32 %1, %1, %8, %3;\n\t"    // x = x * 65536 + w
        "@r add.u32 %2, %2, 2;\n\t"
        "@r ld.shared.u16 %3, [%2];\n\t"
        "}"
        : "=&r"(ent), "+r"(st.x), "+r"(st.p), "+r"(st.w)
        : "r"(lv.base), "r"(lv.mask), "r"(lv.stride), "r"(lv.pb), "r"(lv.k64k));
  }
  return ent;
}

// Merge two decoded symbols (table entries ea, eb) with their fields.
template <int S>
__device__ __forceinline__ uint32_t merge_pair_generic(uint32_t ea, uint32_t eb, uint32_t fa,
                                                       uint32_t fb, bool canon) {
  uint32_t out[2];
  const uint32_t e[2] = {entry_symbol(ea), entry_symbol(eb)};
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

// Lossless fast path: two entries + two fraction bytes -> one 32-bit word.
//   sel picks the two fraction bytes (a in both low bytes, b in both high).
// The upper halves of the two entries already hold the exponents in place.
__device__ __forceinline__ uint32_t merge_pair_s7(uint32_t ea, uint32_t eb, uint32_t fw,
                                                  uint32_t sel) {
  const uint32_t e = __byte_perm(ea, eb, 0x7632);        // ea >> 16 | eb & 0xFFFF0000
  const uint32_t g = __byte_perm(fw, 0, sel);            // fa fa fb fb
  return (e & 0x7F807F80u) | (g & 0x807F807Fu);
}

// A lane's packed fractions for one block (8 elements = s+1 bytes), streaming
// (evict-first) and volatile so that the loads stay where the code puts them:
// several blocks ahead of their use.
template <int S>
__device__ __forceinline__ uint64_t load_frac(const uint8_t *p) {
  if (S == 7) {
    uint32_t lo, hi;
    asm volatile("ld.global.cs.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "l"(p));
    return ((uint64_t)hi << 32) | lo;
  } else if (S == 3) {
    uint32_t v;
    asm volatile("ld.global.cs.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
  } else if (S == 1) {
    uint32_t v;
    asm volatile("ld.global.cs.u16 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
  } else {
    uint32_t v;
    asm volatile("ld.global.cs.u8 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
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

// One output word (two elements) from two table entries and the lane's packed
// fractions of the block; `pair` is 0..3.
template <int S, bool CANON>
__device__ __forceinline__ uint32_t merge_word(uint32_t ea, uint32_t eb, uint64_t fbits, int pair) {
  if (S == 7 && !CANON) {
    const uint32_t half = (pair < 2) ? (uint32_t)fbits : (uint32_t)(fbits >> 32);
    return merge_pair_s7(ea, eb, half, (pair & 1) ? 0x3322 : 0x1100);
  }
  if (!CANON) {
    // Lossy precisions: the pair's (s+1)-bit fields share one byte B of the packed
    // fractions.  One multiplication lays copies of B side by side (the shifts are
    // far enough apart that the copies never overlap, so nothing carries) such that
    // every sign and mantissa bit has a copy at its place in the output word; a mask
    // keeps those places.  The exponents come in place from the two entries' upper
    // halves, as in the lossless path.
    const uint32_t e = __byte_perm(ea, eb, 0x7632) & 0x7F807F80u;
    const uint32_t f = (uint32_t)fbits;
    if (S == 3) {
      // B = [sa ma2 ma1 ma0 sb mb2 mb1 mb0]: ma -> bits 4..6 (shift 0), sa -> 15 (8),
      // mb -> 20..22 (20), sb -> 31 (28)
      const uint32_t B = __byte_perm(f, 0, 0x4440 | pair);
      return e | ((B * 0x10100101u) & 0x80708070u);
    }
    if (S == 1) {
      // B holds four 2-bit fields [s m]; the pair is the upper or the lower two of them
      const uint32_t B = __byte_perm(f, 0, 0x4440 | (pair >> 1));
      // upper two: sa bit 7 -> 15 (8), ma bit 6 -> 6 (0), sb bit 5 -> 31 (26), mb bit 4 -> 22 (18)
      // lower two: sa bit 3 -> 15 (12), ma bit 2 -> 6 (4), sb bit 1 -> 31 (30), mb bit 0 -> 22 (22)
      const uint32_t m = (pair & 1) ? 0x40401010u : 0x04040101u;
      return e | ((B * m) & 0x80408040u);
    }
    if (S == 0) {
      // B holds the block's eight sign bits, first element in bit 7:
      // sa bit 7-2p -> 15 (8+2p), sb bit 6-2p -> 31 (25+2p)
      const uint32_t B = f & 0xFFu;
      return e | ((B * ((1u << (8 + 2 * pair)) + (1u << (25 + 2 * pair)))) & 0x80008000u);
    }
  }
  return merge_pair_generic<S>(ea, eb, field_of<S>(fbits, 2 * pair), field_of<S>(fbits, 2 * pair + 1),
                               CANON);
}

struct DecodeArgs {
  const uint8_t *container;
  uint64_t container_bytes;
  const uint8_t *frac;
  uint64_t n;
  uint32_t S;
  uint32_t n_units;
  uint32_t slot_bytes;
  uint32_t lut_shift;   // log2 of the bytes per slot row for a 2^12-slot table (2..5)
  uint32_t lut_bytes;   // 4096 << lut_shift
  uint32_t ring_offset; // byte offset of the fraction rings in shared memory
  int canon;
  uint16_t *out_bf16;
  uint8_t *out_exp;
  uint32_t *status;
  const uint32_t *unit_list;   // units to decode, in output order (gather launches only)
  uint32_t n_work;             // units this launch decodes: n_units, or the length of the list
  const float *gx;             // matrix-vector launches: input vector (fp32, `in` entries)
  float *partial;              //   partial sums, `seg` places per unit
  uint32_t in;                 //   row length of the [out, in] matrix, a multiple of 256
  uint32_t seg;                //   rows a unit can touch
  uint32_t tile_cols;          // operand order: row length of the matrix (0 = the stream is the tensor)
  // block normaliser: one stored byte per group of 2^norm_lg elements (null = none)
  const uint8_t *norm;
  uint32_t norm_lg;
  // update launches: gradient (bf16) and AdamW moments (bf16), indexed like the output tensor
  const uint16_t *grad;
  uint16_t *exp_avg, *exp_avg_sq;
  AdamArgs adam;
};

// Operand order.  A [rows, cols] matrix (rows % 4 == 0, cols % 64 == 0) may be stored
// with its elements permuted so that one 256-element block of the stream is a
// 4-row x 64-column patch of the matrix: stream element
//   e = ((g * (cols / 64) + kb) * 4 + r) * 64 + c
// is matrix element (4 g + r, 64 kb + c).  A lane's 8 consecutive stream elements
// are still 8 consecutive elements of one row (16 contiguous bytes), a quarter warp's
// 64 are 128 contiguous bytes; 32 consecutive row groups at one kb form the 128 x 64
// tensor-core operand tile.  Units hold whole blocks and never straddle a row group
// (lane_symbols / 8 divides cols / 64).
__device__ __forceinline__ uint64_t operand_index(uint64_t e, uint32_t cols) {
  const uint64_t block = e >> 8;
  const uint32_t w = (uint32_t)e & 255u;
  const uint32_t spr = cols >> 6;                       // blocks per row group
  const uint64_t g = block / spr;
  const uint32_t kb = (uint32_t)(block - g * spr);
  return (4 * g + (w >> 6)) * cols + kb * 64u + (w & 63u);
}
// Block normaliser on the way out (cuda/kernels.cuh:208-216 of the reference): a decoded
// bf16 value times the scale 1.<8 stored mantissa bits> of its group, rounded to bf16
// (nearest even) -- the arithmetic of nz_denormalize_bf16.
__device__ __forceinline__ float norm_scale(uint32_t stored_byte) {
  return __uint_as_float(0x3F800000u | (stored_byte << 15));
}
__device__ __forceinline__ uint32_t scale_bf16_bits(uint32_t bits16, float scale) {
  const float f = scale * __uint_as_float(bits16 << 16);
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return 0x7FFFu;    // NaN
  u += 0x7FFFu + ((u >> 16) & 1u);
  return u >> 16;
}
// Where stream element e goes in the output tensor.
__device__ __forceinline__ uint64_t out_index(const DecodeArgs &a, uint64_t e) {
  return a.tile_cols ? operand_index(e, a.tile_cols) : e;
}

__device__ __forceinline__ void raise(uint32_t *status, uint32_t bits) {
  if (status) atomicOr(status, bits);
}

// Asynchronous per-lane copy of one block's packed fractions (4 or 8 bytes)
// from global to this lane's place in the warp's shared-memory ring.  Unlike a
// register load this occupies no register scoreboard while in flight, so the
// table and stream loads of the decode chain never wait behind it.
template <int S>
__device__ __forceinline__ void frac_async(uint32_t dst, const uint8_t *src) {
  if (S == 7)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void frac_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void frac_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
template <int S>
__device__ __forceinline__ uint64_t frac_from_ring(uint32_t addr) {
  if (S == 7) {
    uint32_t lo, hi;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(addr));
    return ((uint64_t)hi << 32) | lo;
  }
  return lds_u32(addr);
}

constexpr int kChains = NZ_DECODE_CHAINS;        // units a warp decodes side by side

// What a warp knows about a unit it has planned.
struct UnitPlan {
  uint32_t kind;       // 0 = nothing to do, 1 = raw, 2 = coded
  uint32_t head;       // byte offset of the unit inside its slot (coded)
  uint32_t words;      // unit length in words
  uint32_t copy_bytes; // size of the widened bulk copy (coded)
  uint64_t byte0;      // byte offset of the unit inside the payload
};
constexpr uint32_t kUnitSkip = 0, kUnitRaw = 1, kUnitCoded = 2;

// Look up unit u in the offset table and validate it against the buffer limits
// the host passed (not against anything read from the container).  All lanes
// return the same plan.
__device__ __forceinline__ UnitPlan plan_unit(const DecodeArgs &a, uint32_t u, uint64_t pay_off,
                                              uint64_t max_words, uint32_t lane) {
  UnitPlan pl;
  pl.kind = kUnitSkip;
  pl.head = 0;
  pl.words = 0;
  pl.copy_bytes = 0;
  pl.byte0 = 0;
  if (u >= a.n_units) return pl;
  const uint32_t *offsets = reinterpret_cast<const uint32_t *>(a.container + kOffsetsOffset);
  const uint32_t off0 = __ldg(offsets + u), off1 = __ldg(offsets + u + 1);
  const uint64_t w0 = off0 & ~kRawFlag, w1 = off1 & ~kRawFlag;
  const uint64_t U = 32ull * a.S;
  const uint64_t first = (uint64_t)u * U;
  const uint64_t count = (a.n - first < U) ? (a.n - first) : U;
  if (w1 < w0 || w1 > max_words) {
    if (lane == 0) raise(a.status, NZ_STATUS_BAD_OFFSETS);
    return pl;
  }
  pl.words = (uint32_t)(w1 - w0);
  pl.byte0 = w0 * 2;
  if (off0 & kRawFlag) {
    if ((w1 - w0) * 2 < count) {
      if (lane == 0) raise(a.status, NZ_STATUS_BAD_OFFSETS);
      return pl;
    }
    pl.kind = kUnitRaw;
    return pl;
  }
  const uint64_t b0 = w0 * 2, b1 = w1 * 2;
  const uint64_t c0 = b0 & ~uint64_t(15), c1 = (b1 + 15) & ~uint64_t(15);
  const uint32_t bytes = (uint32_t)(c1 - c0);
  // the copy is widened to 16-byte boundaries: it must still end inside the buffer
  if (w1 - w0 < 16 + 2 * 32 || bytes > a.slot_bytes ||
      pay_off + c1 > (a.container_bytes & ~uint64_t(15))) {
    if (lane == 0) raise(a.status, NZ_STATUS_BAD_OFFSETS);
    return pl;
  }
  pl.head = (uint32_t)(b0 - c0);
  pl.copy_bytes = bytes;
  pl.kind = kUnitCoded;
  return pl;
}

// Lane 0 arms the warp's mbarrier with the bytes of all copies and starts them.
// Returns true when at least one copy was issued.
__device__ __forceinline__ bool stage_units(const DecodeArgs &a, const UnitPlan (&pl)[kChains],
                                            uint64_t pay_off, uint32_t slot0, uint32_t bar,
                                            uint32_t lane) {
  uint32_t bytes = 0;
#pragma unroll
  for (int c = 0; c < kChains; ++c) bytes += pl[c].copy_bytes;
  if (bytes == 0) return false;
  if (lane == 0) {
    mbar_expect_tx(bar, bytes);
#pragma unroll
    for (int c = 0; c < kChains; ++c)
      if (pl[c].copy_bytes)
        bulk_g2s(slot0 + c * a.slot_bytes, a.container + pay_off + (pl[c].byte0 & ~uint64_t(15)),
                 pl[c].copy_bytes, bar);
  }
  return true;
}

// Bounded wait for the warp's bulk copies.  Returns false when it ran out.
__device__ __forceinline__ bool wait_staged(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kMaxWaitIters; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// Read the 32 lane lengths of a staged unit, check them against the unit
// length and set up this lane's state.  Returns false (same for all lanes)
// when the lengths are inconsistent.
__device__ __forceinline__ bool open_unit(const UnitPlan &pl, uint32_t slot, uint32_t lenq,
                                          uint32_t lane, LaneState &st) {
  const uint32_t ub = slot + pl.head;            // shared address of the unit
  const uint32_t q = lds_u8(ub + lane) * lenq;   // my stream length in words
  uint32_t incl = q;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= (uint32_t)o) incl += v;
  }
  const uint32_t total = __shfl_sync(0xFFFFFFFFu, incl, 31);
  if (__any_sync(0xFFFFFFFFu, q < 2) || 16u + total != pl.words) return false;
  const uint32_t sw = ub + 2 * (16 + incl - q);
  st.x = lds_u16(sw) | (lds_u16(sw + 2) << 16);
  st.p = sw + 4;
  st.w = lds_u16(st.p);
  return true;
}

// ---------------------------------------------------------------- decode table
// The table is built by all warps of a CTA in three steps with a __syncthreads()
// between them (the caller places the barriers):
//   table_scan     warp 0 scans the container's 256 frequencies into cum_sh[257]; one
//                  other thread checks the header against what the host passed
//   table_verdict  (after a barrier) every thread computes the same verdict
//   table_fill     warps take 32 slots in turn, look their symbols up and write the rows
// flag_sh points at three words: header verdict, probability bits, "a frequency does
// not fit the table entry".
__device__ __forceinline__ void table_scan(const DecodeArgs &a, const Header *h, uint64_t pay_off,
                                           uint64_t max_words, uint16_t *cum_sh, uint32_t *flag_sh,
                                           uint32_t warp, uint32_t lane, uint32_t n_warps) {
  uint32_t *pb_sh = flag_sh + 1;
  uint32_t *wide_sh = flag_sh + 2;
  const uint16_t *freq_g = reinterpret_cast<const uint16_t *>(a.container + kFreqOffset);
  if (warp == 0) {
    // inclusive scan of the 256 frequencies, 8 per lane
    const uint4 fv = __ldg(reinterpret_cast<const uint4 *>(freq_g) + lane);
    const uint32_t fw[4] = {fv.x, fv.y, fv.z, fv.w};
    uint32_t f[8], sum = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      f[k] = (fw[k >> 1] >> ((k & 1) * 16)) & 0xFFFFu;
      sum += f[k];
    }
    uint32_t incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= (uint32_t)o) incl += v;
    }
    uint32_t run = incl - sum;
    uint32_t widest = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) widest = max(widest, f[k]);
    const bool too_wide = __any_sync(0xFFFFFFFFu, widest >> (kEntSymShift - kEntFreqShift));
    if (lane == 0) {
      cum_sh[0] = 0;
      *wide_sh = too_wide ? 1u : 0u;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      run += f[k];
      cum_sh[lane * 8 + k + 1] = (uint16_t)(run > 0xFFFF ? 0xFFFF : run);
    }
  }
  if (threadIdx.x == (n_warps > 1 ? 32u : 0u)) {
    const bool ok = h->magic == kMagic && h->version == 1 && h->n_symbols == a.n &&
                    h->lane_symbols == a.S && h->n_units == a.n_units &&
                    h->len_quantum == len_quantum(a.S) && h->payload_offset == pay_off &&
                    h->payload_words <= max_words && h->prob_bits >= kMinProbBits &&
                    h->prob_bits <= kMaxProbBits;
    *flag_sh = ok ? 0u : (uint32_t)NZ_STATUS_BAD_HEADER;
    *pb_sh = h->prob_bits;
  }
}

// Nothing writes the flags or cum_sh after the barrier that follows table_scan, so
// every thread computes the same verdict.  Returns status bits (0 = go on).
__device__ __forceinline__ uint32_t table_verdict(const uint16_t *cum_sh, const uint32_t *flag_sh,
                                                  uint32_t &pb) {
  pb = flag_sh[1];
  uint32_t bad = flag_sh[0];
  if (pb < kMinProbBits || pb > kMaxProbBits || cum_sh[256] != (1u << (pb & 15)) || flag_sh[2])
    bad |= NZ_STATUS_BAD_HEADER;
  return bad;
}

// Decode table at `smem`: warps take symbols in turn; a symbol's slot range is a run
// of rows (all copies of a slot hold the same word).  The host sized the table for
// 2^12 slots x 2^(lut_shift-2) copies; with fewer probability bits the spare room
// becomes more copies.
__device__ __forceinline__ void table_fill(uint32_t lut_shift, uint32_t S, uint32_t pb,
                                           uint8_t *smem, const uint16_t *cum_sh, uint32_t warp,
                                           uint32_t lane, uint32_t n_warps, LutView &lv,
                                           uint32_t &row_shift) {
  lv.pb = pb;
  lv.mask = (1u << pb) - 1u;
  row_shift = lut_shift + (kMaxProbBits - pb);              // log2 of the bytes per slot row
  if (row_shift > 7) row_shift = 7;                         // 32 copies are enough
  lv.stride = 1u << row_shift;
  lv.base = smem_u32(smem) + ((lane << 2) & (lv.stride - 1u));
  lv.k64k = S ? 65536u : 0u;        // S is never 0; the compiler cannot know
  uint32_t *lut_w = reinterpret_cast<uint32_t *>(smem);
  const uint32_t wsh = row_shift - 2;                     // log2 of the words per slot row
  // A warp takes 32 slots at a time: lane l finds the symbol that owns slot s0 + l (the
  // largest symbol whose cumulative count is not above the slot; symbols that do not occur
  // share their successor's count and are skipped by "largest"), then the warp writes the
  // 32 rows with whole-warp stores.  The cost does not depend on how the counts are spread
  // over the symbols, and a CTA of few warps is not held up by the 256-symbol walk.
  const uint32_t n_slots = 1u << pb;
  for (uint32_t s0 = warp * 32; s0 < n_slots; s0 += n_warps * 32) {
    const uint32_t slot = s0 + lane;
    uint32_t sym = 0;
#pragma unroll
    for (uint32_t step = 128; step >= 1; step >>= 1)
      if (cum_sh[sym + step] <= slot) sym += step;
    const uint32_t start = cum_sh[sym];
    const uint32_t entry = (sym << kEntSymShift) | ((cum_sh[sym + 1] - start) << kEntFreqShift) |
                           (slot - start);
    uint32_t *dst = lut_w + (s0 << wsh);
    if (wsh == 5) {
#pragma unroll 8
      for (uint32_t j = 0; j < 32; ++j) dst[j * 32 + lane] = __shfl_sync(0xFFFFFFFFu, entry, j);
    } else {
      for (uint32_t k = lane; k < (32u << wsh); k += 32)
        dst[k] = __shfl_sync(0xFFFFFFFFu, entry, k >> wsh);
    }
  }
}

}  // namespace nz
