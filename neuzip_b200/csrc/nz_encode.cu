// Entropy-encoder side of the codec: histogram of the exponent bytes, integer
// normalisation to 12-bit frequencies, lane-interleaved rANS encoding, and
// compaction of the coded units into the NZR1 container.
//
// Replaces the nvcomp ANS manager calls of the reference's write path
// (cuda/high_level.cu:103-124: configure_compression, compress,
// get_compressed_output_size, right-sizing copy).  The byte format and the
// arithmetic are specified by the CPU oracle; containers produced here are
// byte-identical to the oracle's.
//
// Scratch layout (device, caller-provided):
//   [0, 1024)            u32 hist[256]
//   [1024, 1536)         u16 freq[256]
//   [1536, 2560)         u32 enc_tab[256]   (freq | cum << 16)
//   [2560, 2576)         u32 misc[4]        (pad symbol, probability bits, -, -)
//   [4096, 4096+4*(nu+1))           u32 unit_words[nu]  (bit 31 = raw)
//   [.., + 64*nu)                   u16 lane_len[nu][32]   (words; 0 = unit raw)
//   [.., + nu*32*cap*2)             u16 lane_words[nu][32][cap]   cap = lane_cap_words(S)
#include <string.h>

#include <mutex>

#include "nz_common.cuh"

namespace nz {

constexpr uint32_t kScratchHist = 0;
constexpr uint32_t kScratchFreq = 1024;
constexpr uint32_t kScratchTab = 1536;
constexpr uint32_t kScratchMisc = 2560;
constexpr uint32_t kScratchUnits = 4096;

struct ScratchLayout {
  uint64_t unit_words, lane_len, lane_words, total;
};

__host__ __device__ inline ScratchLayout scratch_layout(uint64_t n, uint32_t S) {
  const uint64_t nu = unit_count(n, S);
  ScratchLayout L;
  L.unit_words = kScratchUnits;
  L.lane_len = align16(L.unit_words + 4 * (nu + 1));
  L.lane_words = align16(L.lane_len + 64 * nu);
  L.total = align16(L.lane_words + nu * 32ull * lane_cap_words(S) * 2) + 16;
  return L;
}

// ---------------------------------------------------------------- histogram
// One 256-bin histogram per warp in shared memory (the exponent distribution
// is so peaked that a block-wide histogram would serialise on two bins), folded
// into the global histogram with one atomic per non-empty bin.
constexpr int kHistThreads = 256;
constexpr int kHistWarps = kHistThreads / 32;

__global__ void __launch_bounds__(kHistThreads)
histogram_kernel(const uint8_t *__restrict__ sym, uint64_t n, uint32_t *__restrict__ hist) {
  __shared__ uint32_t sh[kHistWarps][256];
  for (int i = threadIdx.x; i < kHistWarps * 256; i += kHistThreads) (&sh[0][0])[i] = 0;
  __syncthreads();
  uint32_t *mine = sh[threadIdx.x >> 5];
  const uint64_t n_vec = n / 16;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint4 *v = reinterpret_cast<const uint4 *>(sym);
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    const uint4 q = __ldcs(v + i);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      // runs of equal bytes inside a word are common: count them locally
      const uint32_t b0 = w[k] & 0xFF, b1 = (w[k] >> 8) & 0xFF, b2 = (w[k] >> 16) & 0xFF,
                     b3 = w[k] >> 24;
      if (b0 == b1 && b1 == b2 && b2 == b3) {
        atomicAdd(&mine[b0], 4u);
      } else {
        atomicAdd(&mine[b0], 1u);
        atomicAdd(&mine[b1], 1u);
        atomicAdd(&mine[b2], 1u);
        atomicAdd(&mine[b3], 1u);
      }
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (uint64_t i = n_vec * 16; i < n; ++i) atomicAdd(&mine[sym[i]], 1u);
  __syncthreads();
  for (int b = threadIdx.x; b < 256; b += kHistThreads) {
    uint32_t s = 0;
#pragma unroll
    for (int w = 0; w < kHistWarps; ++w) s += sh[w][b];
    if (s) atomicAdd(&hist[b], s);
  }
}

// ------------------------------------------------------------ normalisation
// Integer-only, identical to nzo_choose_prob_bits + nzo_normalize of the
// specification.  The counts are 32-bit here (a tensor of 2^32 or more
// elements is rejected by the host code), the products 64-bit.
__global__ void normalize_kernel(const uint32_t *__restrict__ hist, uint16_t *__restrict__ freq,
                                 uint32_t *__restrict__ enc_tab, uint32_t *__restrict__ misc,
                                 uint16_t *__restrict__ container_freq, uint32_t low_pb) {
  __shared__ int32_t f[256];
  __shared__ uint64_t red64[8];
  __shared__ uint32_t red32[8];
  __shared__ uint32_t redmx[8];
  __shared__ int32_t top_sh[8];
  dependent_trigger();
  dependent_wait();
  const int t = threadIdx.x;  // 256 threads
  const int lane = t & 31, wid = t >> 5;
  const uint64_t h = hist[t];
  // total count and number of distinct symbols
  uint64_t tot = h;
  uint32_t dis = h != 0;
  uint32_t mx = (uint32_t)h;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    tot += __shfl_xor_sync(0xFFFFFFFFu, tot, o);
    dis += __shfl_xor_sync(0xFFFFFFFFu, dis, o);
    mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  }
  if (lane == 0) {
    red64[wid] = tot;
    red32[wid] = dis;
    redmx[wid] = mx;
  }
  __syncthreads();
  uint64_t total = 0;
  uint32_t distinct = 0, top_count = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    total += red64[w];
    distinct += red32[w];
    top_count = max(top_count, redmx[w]);
  }
  // 12 bits only while the largest frequency is sure to stay below 2048
  const uint32_t wide_pb = ((uint64_t)top_count * 4096u < total * 1900u) ? 12u : 11u;
  const uint32_t pb = distinct <= 32 ? low_pb : (distinct <= 64 ? 11u : wide_pb);
  const uint32_t M = 1u << pb;
  int32_t v = 0;
  if (total == 0) {
    v = (t == 0) ? (int32_t)M : 0;
  } else if (h) {
    const uint64_t q = (h * M + total / 2) / total;
    v = q ? (int32_t)q : 1;
  }
  f[t] = v;
  __syncthreads();
  // block-wide helpers over f[]: sum, and arg-max with the lowest index on ties
  auto block_sum = [&]() {
    int32_t x = f[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, o);
    __syncthreads();
    if (lane == 0) top_sh[wid] = x;
    __syncthreads();
    int32_t sum = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += top_sh[w];
    return sum;
  };
  auto block_argmax = [&]() {
    int32_t bv = f[t], bi = t;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const int32_t ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
      const int32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    __syncthreads();
    if (lane == 0) top_sh[wid] = bi;
    __syncthreads();
    int32_t best = top_sh[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      const int32_t c = top_sh[w];
      if (f[c] > f[best]) best = c;   // ascending w keeps the lowest index on ties
    }
    return best;
  };
  int32_t d = (int32_t)M - block_sum();
  while (d != 0) {            // same verdict in every thread: all values come from shared memory
    const int32_t top = block_argmax();
    __syncthreads();
    if (d > 0) {
      if (t == 0) f[top] += d;
      d = 0;
    } else {
      const int32_t room = f[top] - 1;
      const int32_t take = (-d < room) ? -d : room;
      __syncthreads();
      if (t == 0) f[top] -= take;
      d += take;
    }
    __syncthreads();
  }
  // an alphabet of one symbol: M-1 for it, 1 for its successor
  const bool full = f[t] == (int32_t)M;
  __syncthreads();
  if (full) {
    f[t] = (int32_t)M - 1;
    f[(t + 1) & 255] = 1;
  }
  __syncthreads();
  // cumulative starts by a two-level warp scan
  const int32_t mine = f[t];
  int32_t incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int32_t u = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += u;
  }
  if (lane == 31) top_sh[wid] = incl;
  __syncthreads();
  int32_t base = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w)
    if (w < wid) base += top_sh[w];
  const uint32_t cum = (uint32_t)(base + incl - mine);
  enc_tab[t] = (uint32_t)mine | (cum << 16);
  freq[t] = (uint16_t)mine;
  container_freq[t] = (uint16_t)mine;
  const int32_t pad = block_argmax();
  if (t == 0) {
    misc[0] = (uint32_t)pad;
    misc[1] = pb;
  }
}

// ------------------------------------------------------------------ encoder
// One warp per unit, one lane per lane stream.  A lane walks its S symbols
// backwards (8 consecutive exponent bytes per 64-bit load), emits 16-bit
// renormalisation words backwards into its slice of the scratch area and
// finally its 32-bit state, so that the slice read forwards is the stream in
// decoder order.
constexpr int kEncWarps = 4;

// One symbol of one lane, in PTX to keep it short: the symbol is byte `sel & 3`
// of `src`; its 16-byte table entry holds {threshold, reciprocal, -freq, cum}.
//   if (x >= threshold) { slice[max(idx, 1)] = low16(x); --idx; x >>= 16; }
//   q = umulhi(x, rcp); rem = x - q*freq; if (rem >= freq) { ++q; rem -= freq; }
//   x = q*M + rem + cum
// idx is signed and simply keeps counting down: once it is below 2 the lane has
// used the two places kept for its final state, the writes pile up harmlessly on
// place 1 and the count of emitted words (cap - 1 - idx) stays exact, which is how
// the caller sees the overflow.  The quotient estimate is exact or one short
// because rcp = floor(2^32 / freq).
__device__ __forceinline__ void encode_step(uint32_t &x, int32_t &idx, uint32_t src, uint32_t sel,
                                            uint32_t tab_addr, uint16_t *slice, uint32_t pow_m) {
  asm volatile(
      "{\n\t"
      ".reg .b32 s, a, xm, rc, nf, cm, q, r0, r1, j;\n\t"
      ".reg .b64 ad;\n\t"
      ".reg .pred p, g;\n\t"
      "prmt.b32 s, %2, 0, %3;\n\t"
      "mad.lo.u32 a, s, 16, %4;\n\t"
      "ld.shared.v4.u32 {xm, rc, nf, cm}, [a];\n\t"
      "setp.ge.u32 p, %0, xm;\n\t"
      "max.s32 j, %1, 1;\n\t"
      "@p mad.wide.u32 ad, j, 2, %5;\n\t"
      "@p st.global.u16 [ad], %0;\n\t"
      "@p shr.u32 %0, %0, 16;\n\t"
      "@p sub.s32 %1, %1, 1;\n\t"
      "mul.hi.u32 q, %0, rc;\n\t"
      "mad.lo.u32 r0, q, nf, %0;\n\t"         // x - q*freq
      "add.u32 r1, r0, nf;\n\t"               // ... - freq
      "setp.ge.s32 g, r1, 0;\n\t"             // estimate one short?
      "@g add.u32 q, q, 1;\n\t"
      "@g mov.b32 r0, r1;\n\t"
      "add.u32 r0, r0, cm;\n\t"
      "mad.lo.u32 %0, q, %6, r0;\n\t"
      "}"
      : "+r"(x), "+r"(idx)
      : "r"(src), "r"(sel), "r"(tab_addr), "l"(slice), "r"(pow_m));
}

__global__ void __launch_bounds__(kEncWarps * 32)
encode_kernel(const uint8_t *__restrict__ sym, uint64_t n, uint32_t S, uint32_t n_units,
              const uint32_t *__restrict__ enc_tab_g, const uint32_t *__restrict__ misc,
              uint32_t *__restrict__ unit_words, uint16_t *__restrict__ lane_len,
              uint16_t *__restrict__ lane_words) {
  // per symbol: renormalisation threshold, reciprocal, minus frequency, cumulative start
  __shared__ uint4 tab[256];
  const uint32_t pb = misc[1];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    const uint32_t e = enc_tab_g[i];
    const uint32_t fr = e & 0xFFFFu;
    // floor(2^32 / freq): the quotient estimate it gives is exact or one short
    const uint32_t rc = fr > 1 ? (uint32_t)((1ull << 32) / fr) : 0xFFFFFFFFu;
    tab[i] = make_uint4(fr << (32 - pb), rc, 0u - fr, e >> 16);
  }
  __syncthreads();
  const uint32_t pad = misc[0];
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t lenq = len_quantum(S);
  const uint32_t cap = lane_cap_words(S);
  const uint64_t U = 32ull * S;
  const uint32_t tab_addr = (uint32_t)__cvta_generic_to_shared(tab);
  const uint32_t pow_m = 1u << pb;
  for (uint32_t u = blockIdx.x * kEncWarps + (threadIdx.x >> 5); u < n_units;
       u += gridDim.x * kEncWarps) {
    const uint64_t first = (uint64_t)u * U;
    const uint64_t count = (n - first < U) ? (n - first) : U;
    uint16_t *mine = lane_words + ((uint64_t)u * 32 + lane) * cap;
    // Words are written downwards from the end of the slice; the two lowest places
    // are for the final state.
    int32_t idx = (int32_t)cap - 1;   // next write position in the slice, counts down
    uint32_t x = kStateLow;
    for (int32_t blk = (int32_t)(S / 8) - 1; blk >= 0; --blk) {
      const uint64_t e0 = first + (uint64_t)blk * 256 + lane * 8;
      uint32_t lo, hi;
      if (e0 + 8 <= n) {
        const uint2 q = *reinterpret_cast<const uint2 *>(sym + e0);
        lo = q.x;
        hi = q.y;
      } else {
        lo = hi = 0;
        for (int t = 0; t < 8; ++t) {
          const uint32_t s = (e0 + t < n) ? sym[e0 + t] : pad;
          if (t < 4) lo |= s << (8 * t); else hi |= s << (8 * (t - 4));
        }
      }
#pragma unroll
      for (int t = 7; t >= 0; --t)
        encode_step(x, idx, t < 4 ? lo : hi, 0x4440u | (uint32_t)(t & 3), tab_addr, mine, pow_m);
    }
    const uint32_t emitted = (uint32_t)((int32_t)cap - 1 - idx);
    const bool overflow = emitted + 2 > cap;
    const uint32_t words = emitted + 2;
    const uint32_t q = (words + lenq - 1) / lenq;
    if (!overflow) {
      // state in front of the emitted words
      mine[cap - emitted - 2] = (uint16_t)(x & 0xFFFFu);
      mine[cap - emitted - 1] = (uint16_t)(x >> 16);
    }
    const bool any_overflow = __any_sync(0xFFFFFFFFu, overflow);
    uint32_t tot = q * lenq;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xFFFFFFFFu, tot, o);
    const uint64_t coded = 16ull + tot;
    const uint64_t raw_words = (count + 1) / 2;
    const bool raw = any_overflow || coded >= raw_words;
    lane_len[(uint64_t)u * 32 + lane] = raw ? 0 : (uint16_t)words;
    if (lane == 0) unit_words[u] = raw ? ((uint32_t)raw_words | kRawFlag) : (uint32_t)coded;
  }
}

// Exclusive scan of the unit sizes -> offset table in the container, plus the
// header.  One block; the unit count is small (N / (32 S)).
__global__ void __launch_bounds__(1024)
scan_kernel(const uint32_t *__restrict__ unit_words, uint32_t n_units, uint64_t n, uint32_t S,
            const uint32_t *__restrict__ misc, uint8_t *__restrict__ container) {
  __shared__ uint64_t part[1024];
  __shared__ uint32_t raw_cnt[1024];
  __shared__ uint32_t max_w[1024];
  dependent_trigger();
  dependent_wait();
  const uint32_t t = threadIdx.x;
  const uint32_t per = (n_units + 1023) / 1024;
  const uint32_t lo = t * per < n_units ? t * per : n_units;
  const uint32_t hi = lo + per < n_units ? lo + per : n_units;
  uint64_t s = 0;
  uint32_t r = 0, m = 0;
  for (uint32_t u = lo; u < hi; ++u) {
    const uint32_t w = unit_words[u];
    s += w & ~kRawFlag;
    if (w & kRawFlag) ++r; else if (w > m) m = w;
  }
  // block-wide exclusive scan of s (and totals of r, max of m): warp scans, then
  // one warp scans the 32 warp totals
  const uint32_t lane = t & 31, wid = t >> 5;
  uint64_t incl = s;
  uint32_t rsum = r, mmax = m;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint64_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= (uint32_t)o) incl += v;
    rsum += __shfl_xor_sync(0xFFFFFFFFu, rsum, o);
    const uint32_t mo = __shfl_xor_sync(0xFFFFFFFFu, mmax, o);
    if (mo > mmax) mmax = mo;
  }
  if (lane == 31) part[wid] = incl;
  if (lane == 0) {
    raw_cnt[wid] = rsum;
    max_w[wid] = mmax;
  }
  __syncthreads();
  if (wid == 0) {
    uint64_t wt = part[lane], winc = wt;
    uint32_t rr = raw_cnt[lane], mm = max_w[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint64_t v = __shfl_up_sync(0xFFFFFFFFu, winc, o);
      if (lane >= (uint32_t)o) winc += v;
      rr += __shfl_xor_sync(0xFFFFFFFFu, rr, o);
      const uint32_t mo = __shfl_xor_sync(0xFFFFFFFFu, mm, o);
      if (mo > mm) mm = mo;
    }
    part[lane] = winc - wt;                // exclusive warp offsets
    if (lane == 31) part[32] = winc;       // grand total
    if (lane == 0) {
      raw_cnt[0] = rr;
      max_w[0] = mm;
    }
  }
  __syncthreads();
  const uint64_t my_start = part[wid] + incl - s;
  if (t == 0) {
    const uint64_t run = part[32];
    const uint32_t rr = raw_cnt[0], mm = max_w[0];
    const uint64_t pay_off = payload_offset(n_units);
    Header h;
    h.magic = kMagic;
    h.version = 1;
    h.n_symbols = n;
    h.lane_symbols = S;
    h.len_quantum = len_quantum(S);
    h.n_units = n_units;
    h.prob_bits = misc[1];
    h.payload_offset = pay_off;
    h.payload_words = run;
    h.total_bytes = align16(pay_off + run * 2);
    h.n_raw_units = rr;
    h.max_coded_unit_words = mm;
    *reinterpret_cast<Header *>(container) = h;
    uint32_t *offsets = reinterpret_cast<uint32_t *>(container + kOffsetsOffset);
    offsets[n_units] = (uint32_t)run;
    // zero the gaps: after the offset table and after the payload
    for (uint64_t b = kOffsetsOffset + 4ull * (n_units + 1); b < pay_off; ++b) container[b] = 0;
    for (uint64_t b = pay_off + run * 2; b < h.total_bytes; ++b) container[b] = 0;
  }
  uint64_t run = my_start;
  uint32_t *offsets = reinterpret_cast<uint32_t *>(container + kOffsetsOffset);
  for (uint32_t u = lo; u < hi; ++u) {
    const uint32_t w = unit_words[u];
    offsets[u] = (uint32_t)run | (w & kRawFlag);
    run += w & ~kRawFlag;
  }
}

// Copy each unit to its place in the payload: one warp per unit.  The unit's
// 32 scratch slices (one fixed-size slice per lane, the stream at its end) are
// brought into shared memory with 16-byte loads that are all in flight together,
// squeezed there into the unit's final layout, and written out with consecutive
// lanes on consecutive words.
constexpr int kCompactWarps = 4;

__global__ void __launch_bounds__(kCompactWarps * 32)
compact_kernel(const uint8_t *__restrict__ sym, uint64_t n, uint32_t S, uint32_t n_units,
               const uint16_t *__restrict__ lane_len, const uint16_t *__restrict__ lane_words,
               uint8_t *__restrict__ container) {
  extern __shared__ __align__(16) uint8_t cmp_smem[];
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t lenq = len_quantum(S);
  const uint32_t cap = lane_cap_words(S);
  const uint64_t U = 32ull * S;
  const uint32_t *offsets = reinterpret_cast<const uint32_t *>(container + kOffsetsOffset);
  uint16_t *payload = reinterpret_cast<uint16_t *>(container + payload_offset(n_units));
  // per warp: 16 words for the length bytes, then the 32 slices
  const uint32_t cell_words = 16 + 32 * cap;
  uint16_t *cell = reinterpret_cast<uint16_t *>(cmp_smem) + (uint64_t)warp * ((cell_words + 7) & ~7u);
  for (uint32_t u = blockIdx.x * kCompactWarps + warp; u < n_units;
       u += gridDim.x * kCompactWarps) {
    const uint32_t off = offsets[u];
    const uint32_t w0 = off & ~kRawFlag;
    uint16_t *dst = payload + w0;
    if (off & kRawFlag) {
      const uint64_t first = (uint64_t)u * U;
      const uint64_t count = (n - first < U) ? (n - first) : U;
      uint8_t *d8 = reinterpret_cast<uint8_t *>(dst);
      for (uint64_t i = lane; i < count; i += 32) d8[i] = sym[first + i];
      if ((count & 1) && lane == 0) d8[count] = 0;
      continue;
    }
    const uint32_t words_total = (offsets[u + 1] & ~kRawFlag) - w0;
    // 1. slices -> shared memory: the 32 slices of a unit are one run of 64*cap bytes
    //    that starts on a 64-byte boundary, whatever cap is
    {
      const uint4 *s4 = reinterpret_cast<const uint4 *>(lane_words + (uint64_t)u * 32 * cap);
      uint4 *c4 = reinterpret_cast<uint4 *>(cell + 16);
      for (uint32_t k = lane; k < 4 * cap; k += 32) c4[k] = s4[k];
    }
    const uint32_t my_words = lane_len[(uint64_t)u * 32 + lane];
    const uint32_t my_q = (my_words + lenq - 1) / lenq;
    __syncwarp();
    reinterpret_cast<uint8_t *>(cell)[lane] = (uint8_t)my_q;
    // 2. squeeze: lane streams move down, in lane order, to sit back to back.  A
    //    stream never moves up, and it ends before the next lane's slice begins, so
    //    going lane by lane and chunk by chunk (read, sync, write) is safe in place.
    uint32_t p = 16;
    for (uint32_t j = 0; j < 32; ++j) {
      const uint32_t words = __shfl_sync(0xFFFFFFFFu, my_words, j);
      const uint32_t padded = __shfl_sync(0xFFFFFFFFu, my_q, j) * lenq;
      const uint32_t from = 16 + (j + 1) * cap - words;
      for (uint32_t k0 = 0; k0 < padded; k0 += 32) {
        const uint32_t k = k0 + lane;
        const uint16_t v = (k < words) ? cell[from + k] : (uint16_t)0;
        __syncwarp();
        if (k < padded) cell[p + k] = v;
        __syncwarp();
      }
      p += padded;
    }
    // 3. out: p == words_total
    if ((w0 & 1) == 0) {
      const uint32_t *c32 = reinterpret_cast<const uint32_t *>(cell);
      uint32_t *d32 = reinterpret_cast<uint32_t *>(dst);
      for (uint32_t k = lane; k < words_total / 2; k += 32) d32[k] = c32[k];
      if ((words_total & 1) && lane == 0) dst[words_total - 1] = cell[words_total - 1];
    } else {
      for (uint32_t k = lane; k < words_total; k += 32) dst[k] = cell[k];
    }
    __syncwarp();
  }
}

// ------------------------------------------------------------------- host
int histogram_u8(const void *sym, uint64_t n, void *hist, cudaStream_t st) {
  NZ_CUDA_TRY(cudaMemsetAsync(hist, 0, 1024, st));
  if (n == 0) return NZ_OK;
  uint64_t blocks = (n / 16 + kHistThreads - 1) / kHistThreads;
  const uint64_t cap = (uint64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  histogram_kernel<<<(unsigned)blocks, kHistThreads, 0, st>>>((const uint8_t *)sym, n, (uint32_t *)hist);
  NZ_LAUNCH_CHECK("histogram_kernel");
  return NZ_OK;
}

uint64_t container_bound(uint64_t n, uint32_t S) {
  const uint64_t U = 32ull * S;
  const uint64_t nu = unit_count(n, S);
  return align16(kOffsetsOffset + 4 * (nu + 1)) + align16(nu * U + 2 * nu) + 16;
}

int encode_exponents(const void *exp_in, uint64_t n, uint32_t S, void *container,
                     uint64_t container_cap, void *scratch, uint64_t scratch_bytes,
                     cudaStream_t st, uint32_t low_prob_bits) {
  const ScratchLayout L = scratch_layout(n, S);
  if (scratch_bytes < L.total) {
    set_error("encode: scratch of %llu bytes is smaller than the %llu required",
              (unsigned long long)scratch_bytes, (unsigned long long)L.total);
    return NZ_E_CAPACITY;
  }
  if (container_cap < container_bound(n, S)) {
    set_error("encode: container capacity %llu is below the bound %llu",
              (unsigned long long)container_cap, (unsigned long long)container_bound(n, S));
    return NZ_E_CAPACITY;
  }
  uint8_t *sc = (uint8_t *)scratch;
  uint8_t *cont = (uint8_t *)container;
  const uint32_t nu = (uint32_t)unit_count(n, S);
  int rc = histogram_u8(exp_in, n, sc + kScratchHist, st);
  if (rc) return rc;
  normalize_kernel<<<1, 256, 0, st>>>((const uint32_t *)(sc + kScratchHist),
                                      (uint16_t *)(sc + kScratchFreq),
                                      (uint32_t *)(sc + kScratchTab),
                                      (uint32_t *)(sc + kScratchMisc),
                                      (uint16_t *)(cont + kFreqOffset), low_prob_bits);
  NZ_LAUNCH_CHECK("normalize_kernel");
  if (nu) {
    uint32_t blocks = (nu + kEncWarps - 1) / kEncWarps;
    encode_kernel<<<blocks, kEncWarps * 32, 0, st>>>(
        (const uint8_t *)exp_in, n, S, nu, (const uint32_t *)(sc + kScratchTab),
        (const uint32_t *)(sc + kScratchMisc), (uint32_t *)(sc + L.unit_words),
        (uint16_t *)(sc + L.lane_len), (uint16_t *)(sc + L.lane_words));
    NZ_LAUNCH_CHECK("encode_kernel");
  }
  scan_kernel<<<1, 1024, 0, st>>>((const uint32_t *)(sc + L.unit_words), nu, n, S,
                                  (const uint32_t *)(sc + kScratchMisc), cont);
  NZ_LAUNCH_CHECK("scan_kernel");
  if (nu) {
    const uint32_t cell_bytes = ((16 + 32 * lane_cap_words(S) + 7) & ~7u) * 2;
    const uint32_t cmp_smem_bytes = kCompactWarps * cell_bytes;
    {
      // once per device, under a lock, for the most a CTA can have
      static std::mutex mu;
      static bool opted[kMaxDeviceOrdinals] = {};
      int dev = 0;
      NZ_CUDA_TRY(cudaGetDevice(&dev));
      std::lock_guard<std::mutex> lock(mu);
      if (dev < 0 || dev >= kMaxDeviceOrdinals || !opted[dev]) {
        NZ_CUDA_TRY(cudaFuncSetAttribute(compact_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kMaxDynamicSmem));
        if (dev >= 0 && dev < kMaxDeviceOrdinals) opted[dev] = true;
      }
    }
    uint32_t blocks = (nu + kCompactWarps - 1) / kCompactWarps;
    const uint32_t capb = (uint32_t)sm_count() * 16;
    if (blocks > capb) blocks = capb;
    compact_kernel<<<blocks, kCompactWarps * 32, cmp_smem_bytes, st>>>((const uint8_t *)exp_in, n, S, nu,
                                           (const uint16_t *)(sc + L.lane_len),
                                           (const uint16_t *)(sc + L.lane_words), cont);
    NZ_LAUNCH_CHECK("compact_kernel");
  }
  return NZ_OK;
}


// ===========================================================================
// Whole-tensor compressor: bf16 in, fractions + container out, with no exponent
// stream in global memory.
//
// Replaces split + nvcomp compress + right-sizing of the reference's write path
// (cuda/high_level.cu:81-124) in two sweeps over the bf16 input:
//   1. bf16_histogram_kernel  counts the exponent bytes (after the rounding of the
//      lossy precisions, exactly as the split computes them);
//   2. bf16_encode_kernel     reads the input again (largely from L2 for tensors of
//      the usual size), writes the packed fractions and rANS-codes the exponents.
//      A warp codes one unit at a time (kFusedChains; two side by side measured slower:
//      the hardware interleaves warps better than the compiler interleaves the chains of
//      one warp, and a warp's cells then take half the shared memory); each lane's 16-bit
//      words go into its slice of a shared-memory cell, the
//      cell is then squeezed into the unit's final layout and written with
//      coalesced stores into the unit's slot of the scratch area.
// scan_kernel then fixes the offsets and place_units_kernel copies every slot to
// its place in the payload.  The input may be a matrix to be stored in operand
// order: the element a lane handles is then found through operand_index().
// The results are byte-identical to split + nz_encode_exponents.
//
// A lane's slice holds `cap_s` words (4 bits per symbol on average; real weights
// need about 2.6).  A unit in which some lane needs more is coded again, words
// placed straight into the slot in global memory: slower, same bytes.
constexpr int kFusedWarps = 8;
constexpr int kFusedChains = 1;      // units a warp codes side by side (1 or 2)

template <int S>
__device__ __forceinline__ uint32_t exp_of(uint32_t val) {
  const uint32_t mag = val & 0x7FFFu;
  uint32_t keep = mag >> (7 - S);
  if (S < 7) keep += (mag >> (6 - S)) & 1u;
  return (keep >> S) & 0xFFu;
}

// The 8 elements of a 16-byte load, two per 32-bit word, split with half-word
// arithmetic: exponent bytes (lo: elements 0-3, hi: 4-7) and the S+1 bytes of packed
// fields in memory order (f0: first four bytes, f1: the rest at precision 7).
template <int S>
__device__ __forceinline__ void split8(const uint32_t (&w)[4], uint32_t &lo, uint32_t &hi,
                                       uint32_t &f0, uint32_t &f1) {
  constexpr uint32_t kOnes = 0x00010001u;
  constexpr uint32_t kKeep = ((1u << (8 + S)) - 1u) * kOnes;
  uint32_t ex[4], fd[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t m = w[j] & 0x7FFF7FFFu;
    uint32_t k = (m >> (7 - S)) & kKeep;
    if (S < 7) k = (k + ((m >> (6 - S)) & kOnes)) & kKeep;   // the carry stays inside its half
    ex[j] = (k >> S) & 0x00FF00FFu;
    fd[j] = ((w[j] >> (15 - S)) & ((1u << S) * kOnes)) | (k & (((1u << S) - 1u) * kOnes));
  }
  lo = __byte_perm(ex[0], ex[1], 0x6420);
  hi = __byte_perm(ex[2], ex[3], 0x6420);
  f1 = 0;
  if (S == 7) {
    f0 = __byte_perm(fd[0], fd[1], 0x6420);
    f1 = __byte_perm(fd[2], fd[3], 0x6420);
  } else if (S == 3) {
    uint32_t b[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = ((fd[j] << 4) | (fd[j] >> 16)) & 0xFFu;
    f0 = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
  } else if (S == 1) {
    uint32_t nib[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) nib[j] = ((fd[j] & 3u) << 2) | ((fd[j] >> 16) & 3u);
    f0 = ((nib[0] << 4) | nib[1]) | (((nib[2] << 4) | nib[3]) << 8);
  } else {
    uint32_t pr[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) pr[j] = ((fd[j] & 1u) << 1) | ((fd[j] >> 16) & 1u);
    f0 = (pr[0] << 6) | (pr[1] << 4) | (pr[2] << 2) | pr[3];
  }
}

template <int S>
__device__ __forceinline__ void store_fields(uint8_t *dst, uint32_t f0, uint32_t f1) {
  if (S == 7) *reinterpret_cast<uint2 *>(dst) = make_uint2(f0, f1);
  else if (S == 3) *reinterpret_cast<uint32_t *>(dst) = f0;
  else if (S == 1) *reinterpret_cast<uint16_t *>(dst) = (uint16_t)f0;
  else *dst = (uint8_t)f0;
}

template <int S>
__global__ void __launch_bounds__(kHistThreads)
bf16_histogram_kernel(const uint16_t *__restrict__ in, uint64_t n, uint32_t *__restrict__ hist) {
  __shared__ uint32_t sh[kHistWarps][256];
  dependent_wait();
  for (int i = threadIdx.x; i < kHistWarps * 256; i += kHistThreads) (&sh[0][0])[i] = 0;
  __syncthreads();
  uint32_t *mine = sh[threadIdx.x >> 5];
  const uint64_t n_vec = n / 8;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint4 *v = reinterpret_cast<const uint4 *>(in);
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    const uint4 q = __ldg(v + i);          // read again by the encode kernel: keep it in L2
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t lo, hi, f0, f1;
    split8<S>(w, lo, hi, f0, f1);
    // one shared-memory atomic per element (a shortcut for four equal exponents in a row
    // fires for 1.5 % of the quads of a weight matrix and costs more than it saves)
    const uint32_t quad[2] = {lo, hi};
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      atomicAdd(&mine[quad[k] & 0xFF], 1u);
      atomicAdd(&mine[(quad[k] >> 8) & 0xFF], 1u);
      atomicAdd(&mine[(quad[k] >> 16) & 0xFF], 1u);
      atomicAdd(&mine[quad[k] >> 24], 1u);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (uint64_t i = n_vec * 8; i < n; ++i) atomicAdd(&mine[exp_of<S>(in[i])], 1u);
  dependent_trigger();
  __syncthreads();
  for (int b = threadIdx.x; b < 256; b += kHistThreads) {
    uint32_t t = 0;
#pragma unroll
    for (int w = 0; w < kHistWarps; ++w) t += sh[w][b];
    if (t) atomicAdd(&hist[b], t);
  }
}

// Matrix element behind stream element e (see the operand order in the decoder).
__device__ __forceinline__ uint64_t source_index(uint64_t e, uint32_t cols) {
  if (!cols) return e;
  const uint64_t block = e >> 8;
  const uint32_t w = (uint32_t)e & 255u;
  const uint32_t spr = cols >> 6;
  const uint64_t g = block / spr;
  const uint32_t kb = (uint32_t)(block - g * spr);
  return (4 * g + (w >> 6)) * cols + kb * 64u + (w & 63u);
}

// The 8 stream elements from e0 (a multiple of 8) as exponent bytes (lo: elements
// 0-3, hi: 4-7, first element in the low byte) and packed fields; elements past n
// give the pad symbol and zero fields.  `store` writes the (S+1) bytes of fields
// (or as many as hold elements that exist).
template <int S>
__device__ __forceinline__ void load_group(const uint16_t *__restrict__ in, uint64_t e0, uint64_t n,
                                           uint32_t cols, uint32_t pad, uint8_t *__restrict__ frac_out,
                                           bool store, uint32_t &lo, uint32_t &hi) {
  constexpr int FB = S + 1;
  uint32_t val[8];
  const uint32_t valid = e0 + 8 <= n ? 8u : (e0 < n ? (uint32_t)(n - e0) : 0u);
  if (valid == 8) {
    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(in + source_index(e0, cols)));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      val[2 * k] = w[k] & 0xFFFFu;
      val[2 * k + 1] = w[k] >> 16;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) val[k] = (uint32_t)k < valid ? in[source_index(e0 + k, cols)] : 0u;
  }
  uint64_t packed = 0;        // first element in the top bits
  lo = hi = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    uint32_t ex;
    uint32_t field;
    {
      const uint32_t sign = (val[k] >> 15) & 1u;
      const uint32_t mag = val[k] & 0x7FFFu;
      uint32_t keep = mag >> (7 - S);
      if (S < 7) keep += (mag >> (6 - S)) & 1u;
      keep &= (1u << (8 + S)) - 1u;
      ex = keep >> S;
      field = (sign << S) | (keep & ((1u << S) - 1u));
    }
    if ((uint32_t)k >= valid) {
      ex = pad;
      field = 0;
    }
    packed = (packed << FB) | field;
    if (k < 4) lo |= ex << (8 * k); else hi |= ex << (8 * (k - 4));
  }
  if (store && valid) {
    uint8_t *dst = frac_out + e0 * FB / 8;
    if (valid == 8) {
      if (S == 7) {
        const uint32_t a = (uint32_t)(packed >> 32), b = (uint32_t)packed;
        *reinterpret_cast<uint2 *>(dst) = make_uint2(__byte_perm(a, 0, 0x0123), __byte_perm(b, 0, 0x0123));
      } else if (S == 3) {
        *reinterpret_cast<uint32_t *>(dst) = __byte_perm((uint32_t)packed, 0, 0x0123);
      } else if (S == 1) {
        *reinterpret_cast<uint16_t *>(dst) = (uint16_t)__byte_perm((uint32_t)packed, 0, 0x3301);
      } else {
        *dst = (uint8_t)packed;
      }
    } else {
      const uint32_t bytes = (valid * FB + 7) / 8;
      for (uint32_t b = 0; b < bytes; ++b) dst[b] = (uint8_t)(packed >> (8 * (FB - 1 - b)));
    }
  }
}

// encode_step with the word going to shared memory (16-bit places from `slice`).
__device__ __forceinline__ void encode_step_sh(uint32_t &x, int32_t &idx, uint32_t src, uint32_t sel,
                                               uint32_t tab_addr, uint32_t slice, uint32_t pow_m) {
  asm volatile(
      "{\n\t"
      ".reg .b32 s, a, xm, rc, nf, cm, q, r0, r1, j;\n\t"
      ".reg .pred p, g;\n\t"
      "prmt.b32 s, %2, 0, %3;\n\t"
      "mad.lo.u32 a, s, 16, %4;\n\t"
      "ld.shared.v4.u32 {xm, rc, nf, cm}, [a];\n\t"
      "setp.ge.u32 p, %0, xm;\n\t"
      "max.s32 j, %1, 1;\n\t"
      "@p mad.lo.u32 j, j, 2, %5;\n\t"
      "@p st.shared.u16 [j], %0;\n\t"
      "@p shr.u32 %0, %0, 16;\n\t"
      "@p sub.s32 %1, %1, 1;\n\t"
      "mul.hi.u32 q, %0, rc;\n\t"
      "mad.lo.u32 r0, q, nf, %0;\n\t"
      "add.u32 r1, r0, nf;\n\t"
      "setp.ge.s32 g, r1, 0;\n\t"
      "@g add.u32 q, q, 1;\n\t"
      "@g mov.b32 r0, r1;\n\t"
      "add.u32 r0, r0, cm;\n\t"
      "mad.lo.u32 %0, q, %6, r0;\n\t"
      "}"
      : "+r"(x), "+r"(idx)
      : "r"(src), "r"(sel), "r"(tab_addr), "r"(slice), "r"(pow_m)
      : "memory");
}

// One encoder step with the symbol's table entry already in registers: the entry only
// depends on the symbol, so the caller fetches it a step ahead and the shared-memory
// latency stays off the chain state -> state.  `e` = (renormalisation bound, reciprocal,
// minus frequency, cumulative count), as bf16_encode_kernel lays the table out.
__device__ __forceinline__ void encode_apply(uint32_t &x, int32_t &idx, const uint4 e,
                                             uint32_t slice, uint32_t pow_m) {
  // renormalisation without a branch: the store is predicated, shift and count are selects
  const uint32_t full = x >= e.x;
  const uint32_t at = slice + 2u * (uint32_t)max(idx, 1);
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.u32 p, %2, 0;\n\t"
      "@p st.shared.u16 [%0], %1;\n\t"
      "}" ::"r"(at), "h"((uint16_t)x), "r"(full)
      : "memory");
  x = full ? x >> 16 : x;
  idx -= (int32_t)full;
  uint32_t q = __umulhi(x, e.y);
  uint32_t r0 = q * e.z + x;                 // x - q * freq
  const uint32_t r1 = r0 + e.z;
  if ((int32_t)r1 >= 0) {
    ++q;
    r0 = r1;
  }
  x = q * pow_m + (r0 + e.w);
}


// Second coding of a unit whose words did not fit the shared-memory slices: the
// lengths are known from the first attempt, so every word goes straight to its
// final place in the slot (global memory).
template <int S>
__device__ __noinline__ void encode_unit_in_place(const uint16_t *__restrict__ in, uint64_t n,
                                                  uint32_t LS, uint32_t cols, uint64_t first,
                                                  uint32_t pad, uint32_t tab_addr, uint32_t pow_m,
                                                  uint16_t *slot, uint32_t offset, uint32_t words,
                                                  uint32_t padded, uint32_t lane) {
  // the lane's stream occupies slot[offset .. offset + padded); words are emitted
  // backwards from offset + words - 1, the state ends up in the first two places
  uint16_t *mine = slot + offset;
  int32_t idx = (int32_t)words - 1;
  uint32_t x = kStateLow;
  for (int32_t blk = (int32_t)(LS / 8) - 1; blk >= 0; --blk) {
    uint32_t lo, hi;
    load_group<S>(in, first + (uint64_t)blk * 256 + lane * 8, n, cols, pad, nullptr, false, lo, hi);
#pragma unroll
    for (int t = 7; t >= 0; --t)
      encode_step(x, idx, t < 4 ? lo : hi, 0x4440u | (uint32_t)(t & 3), tab_addr, mine, pow_m);
  }
  mine[0] = (uint16_t)(x & 0xFFFFu);
  mine[1] = (uint16_t)(x >> 16);
  for (uint32_t k = words; k < padded; ++k) mine[k] = 0;
}

template <int S, int C>
__global__ void __launch_bounds__(kFusedWarps * 32)
bf16_encode_kernel(const uint16_t *__restrict__ in, uint64_t n, uint32_t LS, uint32_t n_units,
                   uint32_t cols, const uint32_t *__restrict__ enc_tab_g,
                   const uint32_t *__restrict__ misc, uint32_t cap_s,
                   uint8_t *__restrict__ frac_out, uint32_t *__restrict__ unit_words,
                   uint8_t *__restrict__ slots, uint32_t slot_stride) {
  extern __shared__ __align__(16) uint8_t enc_smem[];
  uint4 *tab = reinterpret_cast<uint4 *>(enc_smem);
  dependent_wait();
  const uint32_t pb = misc[1];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    const uint32_t e = enc_tab_g[i];
    const uint32_t fr = e & 0xFFFFu;
    const uint32_t rc = fr > 1 ? (uint32_t)((1ull << 32) / fr) : 0xFFFFFFFFu;
    tab[i] = make_uint4(fr << (32 - pb), rc, 0u - fr, e >> 16);
  }
  __syncthreads();
  const uint32_t pad = misc[0];
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t lenq = len_quantum(LS);
  const uint32_t cap = lane_cap_words(LS);
  const uint64_t U = 32ull * LS;
  const uint32_t tab_addr = (uint32_t)__cvta_generic_to_shared(tab);
  const uint32_t pow_m = 1u << pb;
  // a chain's cell: 16 words of lane lengths, then 32 slices of cap_s words one word apart
  const uint32_t sstride = cap_s + 1;
  const uint32_t cell_words = (16 + 32 * sstride + 7) & ~7u;
  uint16_t *cell0 = reinterpret_cast<uint16_t *>(enc_smem + 4096) +
                    (uint64_t)(warp * C) * cell_words;
  const uint32_t n_warps = blockDim.x >> 5;
  const uint32_t n_blocks = LS / 8;
  const uint32_t groups = (n_units + C - 1) / C;
  for (uint32_t gq = blockIdx.x * n_warps + warp; gq < groups; gq += gridDim.x * n_warps) {
    // the next kernel of the pipeline may be set up while the last units are coded
    if (gq + gridDim.x * n_warps >= groups) dependent_trigger();
    uint32_t u[C];
    uint64_t first[C];
    bool live[C];
    uint32_t x[C], slice[C];
    int32_t idx[C];
#pragma unroll
    for (int c = 0; c < C; ++c) {
      u[c] = gq * C + c;
      live[c] = u[c] < n_units;
      first[c] = (uint64_t)u[c] * U;
      x[c] = kStateLow;
      idx[c] = (int32_t)cap_s - 1;
      slice[c] = (uint32_t)__cvta_generic_to_shared(cell0 + c * cell_words + 16 + lane * sstride);
    }
    // Whole units walk two pointers down, block by block (in operand order a unit's
    // blocks are 64 elements apart in the lane's row; otherwise 256); only the tensor's
    // last unit can be ragged and takes the guarded loads.
    bool whole = true;
    const uint16_t *src[C];
    uint8_t *fdst[C];
#pragma unroll
    for (int c = 0; c < C; ++c) {
      if (live[c] && first[c] + U > n) whole = false;
      const uint64_t e_last = first[c] + (uint64_t)(n_blocks - 1) * 256 + lane * 8;
      src[c] = in + (live[c] && first[c] + U <= n ? source_index(e_last, cols) : 0);
      fdst[c] = frac_out + (live[c] ? e_last * (S + 1) / 8 : 0);
    }
    const uint32_t step = cols ? 64u : 256u;
    if (whole) {
      // Software pipeline, two stages deep: the 16 bytes of block b - 2 are requested and
      // block b - 1 is split into exponent bytes and fractions while the 8 symbols of block
      // b are coded; inside a block, the table entry of the next symbol (of either chain)
      // is fetched before the current one is applied.
      uint4 nxt[C];
      uint32_t lo[C], hi[C];
      uint4 ent[C];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        uint4 cur = make_uint4(0, 0, 0, 0);
        nxt[c] = cur;
        if (live[c]) cur = __ldg(reinterpret_cast<const uint4 *>(src[c]));
        src[c] -= step;
        if (live[c] && n_blocks > 1) nxt[c] = __ldg(reinterpret_cast<const uint4 *>(src[c]));
        const uint32_t w[4] = {cur.x, cur.y, cur.z, cur.w};
        uint32_t f0, f1;
        split8<S>(w, lo[c], hi[c], f0, f1);
        if (live[c]) store_fields<S>(fdst[c], f0, f1);
        fdst[c] -= 32 * (S + 1);
        ent[c] = tab[hi[c] >> 24];
      }
      for (int32_t blk = (int32_t)n_blocks - 1; blk >= 0; --blk) {
        // the block after this one: its bytes are here, the one after that is requested
        uint32_t lo_n[C], hi_n[C];
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const uint32_t w[4] = {nxt[c].x, nxt[c].y, nxt[c].z, nxt[c].w};
          src[c] -= step;
          if (live[c] && blk > 1) nxt[c] = __ldg(reinterpret_cast<const uint4 *>(src[c]));
          uint32_t f0, f1;
          split8<S>(w, lo_n[c], hi_n[c], f0, f1);
          if (live[c] && blk > 0) store_fields<S>(fdst[c], f0, f1);
          fdst[c] -= 32 * (S + 1);
        }
#pragma unroll
        for (int t = 7; t >= 0; --t) {
          uint4 ahead[C];
#pragma unroll
          for (int c = 0; c < C; ++c) {
            const uint32_t word = t > 4 ? hi[c] : (t > 0 ? lo[c] : hi_n[c]);   // holds symbol t - 1
            const int byte = (t + 7) & 3;                                      // (t - 1) mod 4
            ahead[c] = tab[(word >> (8 * byte)) & 0xFFu];
          }
#pragma unroll
          for (int c = 0; c < C; ++c) encode_apply(x[c], idx[c], ent[c], slice[c], pow_m);
#pragma unroll
          for (int c = 0; c < C; ++c) ent[c] = ahead[c];
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
          lo[c] = lo_n[c];
          hi[c] = hi_n[c];
        }
      }
    } else {
      for (int32_t blk = (int32_t)n_blocks - 1; blk >= 0; --blk) {
        uint32_t lo[C], hi[C];
#pragma unroll
        for (int c = 0; c < C; ++c) {
          lo[c] = hi[c] = 0;
          if (live[c])
            load_group<S>(in, first[c] + (uint64_t)blk * 256 + lane * 8, n, cols, pad, frac_out,
                          true, lo[c], hi[c]);
        }
#pragma unroll
        for (int t = 7; t >= 0; --t) {
#pragma unroll
          for (int c = 0; c < C; ++c)
            encode_step_sh(x[c], idx[c], t < 4 ? lo[c] : hi[c], 0x4440u | (uint32_t)(t & 3),
                           tab_addr, slice[c], pow_m);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < C; ++c) {
      if (!live[c]) continue;             // same verdict in every lane
      uint16_t *cell = cell0 + c * cell_words;
      const uint64_t count = (n - first[c] < U) ? (n - first[c]) : U;
      const uint32_t emitted = (uint32_t)((int32_t)cap_s - 1 - idx[c]);
      const uint32_t words = emitted + 2;
      const uint32_t q = (words + lenq - 1) / lenq;
      const uint32_t padded = q * lenq;
      uint32_t incl = padded;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= (uint32_t)o) incl += v;
      }
      const uint32_t total = 16u + __shfl_sync(0xFFFFFFFFu, incl, 31);
      const uint64_t raw_words = (count + 1) / 2;
      const bool too_long = __any_sync(0xFFFFFFFFu, words > cap);       // the format's own limit
      const bool raw = too_long || total >= raw_words;
      if (lane == 0) unit_words[u[c]] = raw ? ((uint32_t)raw_words | kRawFlag) : total;
      if (raw) continue;                  // placed from the input by place_units_kernel
      uint16_t *slot = reinterpret_cast<uint16_t *>(slots + (uint64_t)u[c] * slot_stride);
      if (__any_sync(0xFFFFFFFFu, words > cap_s)) {
        // did not fit the slices: code it again, straight into the slot
        reinterpret_cast<uint8_t *>(slot)[lane] = (uint8_t)q;
        encode_unit_in_place<S>(in, n, LS, cols, first[c], pad, tab_addr, pow_m, slot,
                                16 + incl - padded, words, padded, lane);
        continue;
      }
      // state in front of the emitted words, then squeeze the 32 streams together
      uint16_t *mine = cell + 16 + lane * sstride;
      mine[cap_s - emitted - 2] = (uint16_t)(x[c] & 0xFFFFu);
      mine[cap_s - emitted - 1] = (uint16_t)(x[c] >> 16);
      __syncwarp();
      reinterpret_cast<uint8_t *>(cell)[lane] = (uint8_t)q;
      uint32_t p = 16;
      for (uint32_t j = 0; j < 32; ++j) {
        const uint32_t wj = __shfl_sync(0xFFFFFFFFu, words, j);
        const uint32_t pj = __shfl_sync(0xFFFFFFFFu, padded, j);
        const uint32_t from = 16 + j * sstride + cap_s - wj;
        for (uint32_t k0 = 0; k0 < pj; k0 += 32) {
          const uint32_t k = k0 + lane;
          const uint16_t v = (k < wj) ? cell[from + k] : (uint16_t)0;
          __syncwarp();
          if (k < pj) cell[p + k] = v;
          __syncwarp();
        }
        p += pj;
      }
      // p == total; the cell and the slot are 16-byte aligned
      const uint4 *c4 = reinterpret_cast<const uint4 *>(cell);
      uint4 *d4 = reinterpret_cast<uint4 *>(slot);
      for (uint32_t k = lane; k < (total + 7) / 8; k += 32) d4[k] = c4[k];
      __syncwarp();
    }
  }
}

// Every unit to its place in the payload: coded units from their slots, raw units
// (exponent bytes as they are) from the input.
template <int S>
__global__ void __launch_bounds__(128)
place_units_kernel(const uint16_t *__restrict__ in, uint64_t n, uint32_t LS, uint32_t n_units,
                   uint32_t cols, const uint8_t *__restrict__ slots, uint32_t slot_stride,
                   uint8_t *__restrict__ container) {
  dependent_wait();
  const uint32_t lane = threadIdx.x & 31;
  const uint64_t U = 32ull * LS;
  const uint32_t *offsets = reinterpret_cast<const uint32_t *>(container + kOffsetsOffset);
  uint16_t *payload = reinterpret_cast<uint16_t *>(container + payload_offset(n_units));
  for (uint32_t u = blockIdx.x * 4 + (threadIdx.x >> 5); u < n_units; u += gridDim.x * 4) {
    const uint32_t off = offsets[u];
    const uint32_t w0 = off & ~kRawFlag;
    uint16_t *dst = payload + w0;
    if (off & kRawFlag) {
      const uint64_t first = (uint64_t)u * U;
      const uint64_t count = (n - first < U) ? (n - first) : U;
      uint8_t *d8 = reinterpret_cast<uint8_t *>(dst);
      for (uint64_t i = lane; i < count; i += 32)
        d8[i] = (uint8_t)exp_of<S>(in[source_index(first + i, cols)]);
      if ((count & 1) && lane == 0) d8[count] = 0;
      continue;
    }
    const uint32_t words = (offsets[u + 1] & ~kRawFlag) - w0;
    const uint32_t *src = reinterpret_cast<const uint32_t *>(slots + (uint64_t)u * slot_stride);
    if ((w0 & 1) == 0) {
      // four independent loads in flight per lane: the copy is latency-bound otherwise
      uint32_t *d32 = reinterpret_cast<uint32_t *>(dst);
      const uint32_t n32 = words / 2;
      for (uint32_t k0 = 0; k0 < n32; k0 += 128) {
        uint32_t v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t k = k0 + 32 * i + lane;
          v[i] = k < n32 ? __ldcs(src + k) : 0u;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t k = k0 + 32 * i + lane;
          if (k < n32) d32[k] = v[i];
        }
      }
      if ((words & 1) && lane == 0)
        dst[words - 1] = reinterpret_cast<const uint16_t *>(src)[words - 1];
    } else {
      // the destination starts on an odd word: one 16-bit store, then 32-bit stores of
      // source words shifted by half a word
      if (lane == 0) dst[0] = reinterpret_cast<const uint16_t *>(src)[0];
      uint32_t *d32 = reinterpret_cast<uint32_t *>(dst + 1);
      const uint32_t pairs = (words - 1) / 2;
      for (uint32_t k0 = 0; k0 < pairs; k0 += 128) {
        uint32_t a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t k = k0 + 32 * i + lane;
          a[i] = k < pairs ? __ldcs(src + k) : 0u;
          b[i] = k < pairs ? __ldcs(src + k + 1) : 0u;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t k = k0 + 32 * i + lane;
          if (k < pairs) d32[k] = __funnelshift_r(a[i], b[i], 16);
        }
      }
      if (((words - 1) & 1) && lane == 0)
        dst[words - 1] = reinterpret_cast<const uint16_t *>(src)[words - 1];
    }
  }
}

struct FusedLayout {
  uint64_t unit_words, slots, total;
  uint32_t slot_stride, cap_s;
};

__host__ __device__ inline FusedLayout fused_layout(uint64_t n, uint32_t LS) {
  const uint64_t nu = unit_count(n, LS);
  const uint32_t cap = lane_cap_words(LS);
  FusedLayout L;
  L.unit_words = kScratchUnits;
  // a slot holds a coded unit of any admissible length (one word past the end may be read
  // by the half-word-shifted copy)
  L.slot_stride = (uint32_t)align16((16ull + 32ull * cap) * 2 + 4);
  L.slots = align16(L.unit_words + 4 * (nu + 1));
  L.total = align16(L.slots + nu * (uint64_t)L.slot_stride) + 16;
  uint32_t cs = LS / 4 + 2;              // 4 bits per symbol and the state
  L.cap_s = cs < cap ? cs : cap;
  return L;
}

template <int S>
static int compress_fused(const void *in, uint64_t n, uint32_t LS, uint32_t cols, void *frac_out,
                          void *container, uint64_t container_cap, void *scratch,
                          uint64_t scratch_bytes, cudaStream_t st, uint32_t low_pb) {
  const FusedLayout L = fused_layout(n, LS);
  if (scratch_bytes < L.total) {
    set_error("compress: scratch of %llu bytes is smaller than the %llu required",
              (unsigned long long)scratch_bytes, (unsigned long long)L.total);
    return NZ_E_CAPACITY;
  }
  if (container_cap < container_bound(n, LS)) {
    set_error("compress: container capacity %llu is below the bound %llu",
              (unsigned long long)container_cap, (unsigned long long)container_bound(n, LS));
    return NZ_E_CAPACITY;
  }
  uint8_t *sc = (uint8_t *)scratch;
  uint8_t *cont = (uint8_t *)container;
  const uint32_t nu = (uint32_t)unit_count(n, LS);
  NZ_CUDA_TRY(cudaMemsetAsync(sc + kScratchHist, 0, 1024, st));
  if (n) {
    uint64_t blocks = (n / 8 + kHistThreads - 1) / kHistThreads;
    const uint64_t capb = (uint64_t)sm_count() * 8;
    if (blocks > capb) blocks = capb;
    if (blocks == 0) blocks = 1;
    NZ_CUDA_TRY(launch_dependent(bf16_histogram_kernel<S>, (unsigned)blocks, kHistThreads, 0, st,
                                 (const uint16_t *)in, n, (uint32_t *)(sc + kScratchHist)));
  }
  NZ_CUDA_TRY(launch_dependent(normalize_kernel, 1, 256, 0, st,
                               (const uint32_t *)(sc + kScratchHist),
                               (uint16_t *)(sc + kScratchFreq), (uint32_t *)(sc + kScratchTab),
                               (uint32_t *)(sc + kScratchMisc), (uint16_t *)(cont + kFreqOffset),
                               low_pb));
  if (nu) {
    const uint32_t cell_words = (16 + 32 * (L.cap_s + 1) + 7) & ~7u;
    // Units per warp: one, unless the tensor has more units than the GPU can keep resident
    // that way -- the hardware interleaves warps better than the compiler interleaves the
    // two chains of one warp.
    const uint32_t chains = kFusedChains;
    // up to 8 warps per block; long lane streams get fewer so that a block still fits
    uint32_t warps = (kMaxDynamicSmem - 4096) / (chains * cell_words * 2);
    if (warps > (uint32_t)kFusedWarps) warps = kFusedWarps;
    if (warps == 0) warps = 1;
    const uint32_t smem = 4096 + warps * chains * cell_words * 2;
    auto kern = bf16_encode_kernel<S, kFusedChains>;
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
    if (smem > kMaxDynamicSmem) {
      set_error("compress: lane_symbols %u needs %u bytes of shared memory per block", LS, smem);
      return NZ_E_ARG;
    }
    const uint32_t groups = (nu + chains - 1) / chains;
    uint32_t blocks = (groups + warps - 1) / warps;
    const uint32_t per_sm = kMaxDynamicSmem / (smem + 1024) ? kMaxDynamicSmem / (smem + 1024) : 1;
    const uint32_t capb = (uint32_t)sm_count() * per_sm;
    if (blocks > capb) blocks = capb;
    NZ_CUDA_TRY(launch_dependent(kern, blocks, warps * 32, smem, st, (const uint16_t *)in, n, LS, nu,
                                 cols, (const uint32_t *)(sc + kScratchTab),
                                 (const uint32_t *)(sc + kScratchMisc), L.cap_s,
                                 (uint8_t *)frac_out, (uint32_t *)(sc + L.unit_words),
                                 sc + L.slots, L.slot_stride));
  }
  NZ_CUDA_TRY(launch_dependent(scan_kernel, 1, 1024, 0, st, (const uint32_t *)(sc + L.unit_words),
                               nu, n, LS, (const uint32_t *)(sc + kScratchMisc), cont));
  if (nu) {
    uint32_t blocks = (nu + 3) / 4;
    const uint32_t capb = (uint32_t)sm_count() * 16;
    if (blocks > capb) blocks = capb;
    NZ_CUDA_TRY(launch_dependent(place_units_kernel<S>, blocks, 128, 0, st, (const uint16_t *)in,
                                 n, LS, nu, cols, (const uint8_t *)(sc + L.slots), L.slot_stride,
                                 cont));
  }
  return NZ_OK;
}

uint64_t compress_fused_scratch_bytes(uint64_t n, uint32_t LS) { return fused_layout(n, LS).total; }

// bf16[n] (a [n / cols, cols] matrix to be stored in operand order when cols != 0)
// -> fractions + container.
int compress_bf16_fused(const void *in, uint64_t n, int precision, uint32_t LS, uint32_t cols,
                        void *frac_out, void *container, uint64_t container_cap, void *scratch,
                        uint64_t scratch_bytes, cudaStream_t st) {
  // Lossless tensors keep 8 fraction bits per element, so the exponent stream is
  // a quarter of what is stored: 9-bit probabilities cost 0.2 % of the stored
  // size there and let the decoder keep one table copy per shared-memory bank.
  const uint32_t low_pb = precision == 7 ? kMinProbBits : kDefaultLowProbBits;
  switch (precision) {
    case 0: return compress_fused<0>(in, n, LS, cols, frac_out, container, container_cap, scratch, scratch_bytes, st, low_pb);
    case 1: return compress_fused<1>(in, n, LS, cols, frac_out, container, container_cap, scratch, scratch_bytes, st, low_pb);
    case 3: return compress_fused<3>(in, n, LS, cols, frac_out, container, container_cap, scratch, scratch_bytes, st, low_pb);
    default: return compress_fused<7>(in, n, LS, cols, frac_out, container, container_cap, scratch, scratch_bytes, st, low_pb);
  }
}

}  // namespace nz

static int check_encode_args(const char *who, uint64_t n, uint32_t S) {
  if (!nz::valid_lane_symbols(S)) {
    nz::set_error("%s: lane_symbols must be a multiple of 8 in [8, %u] (got %u)", who,
                  nz::kMaxLaneSymbols, S);
    return NZ_E_ARG;
  }
  if (n >= (1ull << 32)) {
    nz::set_error("%s: tensors of 2^32 or more elements are not supported", who);
    return NZ_E_ARG;
  }
  return NZ_OK;
}

extern "C" uint64_t nz_container_bound(uint64_t n, uint32_t lane_symbols) {
  if (!nz::valid_lane_symbols(lane_symbols)) return 0;
  return nz::container_bound(n, lane_symbols);
}

extern "C" uint64_t nz_encode_scratch_bytes(uint64_t n, uint32_t lane_symbols) {
  if (!nz::valid_lane_symbols(lane_symbols)) return 0;
  return nz::scratch_layout(n, lane_symbols).total;
}

extern "C" int nz_histogram_u8(const void *sym, uint64_t n, void *hist_u32, void *stream) {
  if (!hist_u32 || (n && !sym) || ((uintptr_t)sym & 15)) {
    nz::set_error("nz_histogram_u8: null or misaligned pointer (input must be 16-byte aligned)");
    return NZ_E_ARG;
  }
  if (n >= (1ull << 32)) {
    nz::set_error("nz_histogram_u8: 2^32 or more symbols are not supported");
    return NZ_E_ARG;
  }
  return nz::histogram_u8(sym, n, hist_u32, (cudaStream_t)stream);
}

extern "C" int nz_encode_exponents(const void *exp_in, uint64_t n, uint32_t lane_symbols,
                                   void *container, uint64_t container_cap, void *scratch,
                                   uint64_t scratch_bytes, void *stream) {
  int rc = check_encode_args("nz_encode_exponents", n, lane_symbols);
  if (rc) return rc;
  if (!container || !scratch || (n && !exp_in)) {
    nz::set_error("nz_encode_exponents: null pointer");
    return NZ_E_ARG;
  }
  if (((uintptr_t)exp_in & 15) || ((uintptr_t)container & 15) || ((uintptr_t)scratch & 15)) {
    nz::set_error("nz_encode_exponents: buffers must be 16-byte aligned");
    return NZ_E_ARG;
  }
  return nz::encode_exponents(exp_in, n, lane_symbols, container, container_cap, scratch,
                              scratch_bytes, (cudaStream_t)stream, nz::kDefaultLowProbBits);
}

// ---------------------------------------------------------------------------
// Encoding without any device allocation.
//
// Some hosts of this library are not allowed to allocate device memory at the
// point where they need to compress a tensor: a serving process that handed the
// whole GPU to its own arena at start-up and gives plugins no allocator, or a
// framework that bans cudaMalloc / cudaFree on its hot path because both
// synchronise the device and would stall every other stream.  For them the
// scratch area of the encoder lives in the library image itself: one fixed array
// in device memory, present on every GPU that loads the library until the
// process exits.
//
// The array below is a *host-side handle* as far as host code is concerned: its
// name is not a device address and must never be handed to a kernel.  The real
// address on the current device is looked up once per device with
// cudaGetSymbolAddress (here, in the same translation unit as the array) and
// that pointer is what the kernels receive.
constexpr size_t kStaticScratchBytes = 6u << 20;   // 6 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static void *g_static_ptr[kMaxDevices];            // resolved address per device ordinal

// Device address of g_static_scratch on the current device.  The first call on
// a device performs the lookup; later calls return the cached pointer.
static int static_scratch_ptr(void **out) {
  int dev = 0;
  NZ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    nz::set_error("static scratch: device ordinal %d is outside the supported range", dev);
    return NZ_E_ARG;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void *p = nullptr;
    NZ_CUDA_TRY(cudaGetSymbolAddress((void **)&p, g_static_scratch));
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return NZ_OK;
}

extern "C" uint64_t nz_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int nz_encode_exponents_static_scratch(const void *exp_in, uint64_t n,
                                                  uint32_t lane_symbols, void *container,
                                                  uint64_t container_cap, void *stream) {
  int rc = check_encode_args("nz_encode_exponents_static_scratch", n, lane_symbols);
  if (rc) return rc;
  if (!container || (n && !exp_in)) {
    nz::set_error("nz_encode_exponents_static_scratch: null pointer");
    return NZ_E_ARG;
  }
  if (((uintptr_t)exp_in & 15) || ((uintptr_t)container & 15)) {
    nz::set_error("nz_encode_exponents_static_scratch: buffers must be 16-byte aligned");
    return NZ_E_ARG;
  }
  const uint64_t need = nz::scratch_layout(n, lane_symbols).total;
  if (need > kStaticScratchBytes) {
    nz::set_error("nz_encode_exponents_static_scratch: %llu symbols with lane_symbols %u need %llu "
                  "bytes of scratch, the built-in area holds %llu; use nz_encode_exponents with "
                  "caller-provided scratch for tensors this large",
                  (unsigned long long)n, lane_symbols, (unsigned long long)need,
                  (unsigned long long)kStaticScratchBytes);
    return NZ_E_CAPACITY;
  }
  void *scratch = nullptr;
  rc = static_scratch_ptr(&scratch);
  if (rc) return rc;
  // The area still holds whatever the previous call left there.  The only part
  // that must start from zero is the histogram, and the pipeline clears it itself
  // (a memset on the stream) before counting; every other region is written in
  // full for the units of this call before it is read.
  return nz::encode_exponents(exp_in, n, lane_symbols, container, container_cap, scratch,
                              kStaticScratchBytes, (cudaStream_t)stream, nz::kDefaultLowProbBits);
}

extern "C" int nz_container_bytes(const void *container, uint64_t *total_bytes,
                                  uint32_t *max_unit_words, void *stream) {
  if (!container || !total_bytes) {
    nz::set_error("nz_container_bytes: null pointer");
    return NZ_E_ARG;
  }
  nz::Header h;
  NZ_CUDA_TRY(cudaMemcpyAsync(&h, container, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  NZ_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  if (h.magic != nz::kMagic || h.version != 1) {
    nz::set_error("nz_container_bytes: not an NZR1 container");
    return NZ_E_FORMAT;
  }
  *total_bytes = h.total_bytes;
  if (max_unit_words) *max_unit_words = h.max_coded_unit_words;
  return NZ_OK;
}

extern "C" int nz_container_header_async(const void *container, void *host_header64, void *stream) {
  if (!container || !host_header64) {
    nz::set_error("nz_container_header_async: null pointer");
    return NZ_E_ARG;
  }
  static_assert(sizeof(nz::Header) == 64, "header size");
  NZ_CUDA_TRY(cudaMemcpyAsync(host_header64, container, sizeof(nz::Header), cudaMemcpyDeviceToHost,
                              (cudaStream_t)stream));
  return NZ_OK;
}

extern "C" int nz_parse_header(const void *host_header64, uint64_t *total_bytes,
                               uint32_t *max_unit_words) {
  if (!host_header64 || !total_bytes) {
    nz::set_error("nz_parse_header: null pointer");
    return NZ_E_ARG;
  }
  nz::Header h;
  memcpy(&h, host_header64, sizeof(h));
  if (h.magic != nz::kMagic || h.version != 1) {
    nz::set_error("nz_parse_header: not an NZR1 header");
    return NZ_E_FORMAT;
  }
  *total_bytes = h.total_bytes;
  if (max_unit_words) *max_unit_words = h.max_coded_unit_words;
  return NZ_OK;
}
