/*
 * CPU oracle for the NeuZip bf16 codec hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA library is compared against.  Nothing in
 * the shipped package may call it; only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark load it.
 *
 * PARITY STATUS: pinned to reference-run split / merge.  The reference ships no
 * tests, no golden vectors and no CPU path, and its entropy stage is the
 * closed-source nvcomp library; but its two kernels, kernel_aligned_split and
 * kernel_aligned_merge (cuda/kernels.cuh:53-217), compile from the reference
 * tree without nvcomp (oracle/ref_kernels.cu, `make -C oracle ref`) and were run
 * on a B200.  What pins this file:
 *   - the GPU tests (tests/test_gpu_reference_pin.py) require nzo_split_literal(),
 *     nzo_split(), nzo_merge() with NaN canonicalisation and, for the group
 *     sizes whose reduction is well defined in the reference (1..32 and 1024),
 *     nzo_normalize_groups() / nzo_denormalize_groups() to equal the reference
 *     kernels' outputs bit for bit on all 65 536 bf16 patterns, on the seed-0
 *     4096x4096 matrix and on seeded weights;
 *   - CRC-32s of those reference-run outputs are committed
 *     (tests/golden/reference_pin.json) and checked on the CPU too;
 *   - nzo_split_literal() follows cuda/kernels.cuh:120-155 one statement at a
 *     time (including the 8-bit truncations of the C types used there),
 *     nzo_split() is the closed form of the same arithmetic, nzo_merge()
 *     follows cuda/kernels.cuh:197-216.
 *
 * The entropy stage (cuda/high_level.cu:103-115 compress, :184-192 decompress
 * call nvcomp's ANS manager) has no observable byte format in the reference:
 * the compressed bytes live only inside the C++ cache.  The rANS container
 * below is therefore this project's own format and this file is its
 * specification; the CUDA encoder must emit byte-identical containers and the
 * CUDA decoder must accept the containers produced here.
 *
 * ---------------------------------------------------------------------------
 * Container layout ("NZR1"), all little-endian:
 *
 *   [0,64)      header   (struct nzo_header)
 *   [64,576)    freq     u16[256], sum = M = 2^prob_bits, every present symbol
 *                        >= 1, no entry above M-1
 *   [576, ...)  offsets  u32[n_units+1]; entry u = word offset (16-bit words)
 *                        of unit u inside the payload, bit 31 set when the
 *                        unit is stored raw; last entry = total payload words
 *   pad to 16   payload  units back to back, each 2-byte aligned
 *   pad to 16   (end of container)
 *
 * A unit covers U = 32*S consecutive exponent bytes (S = lane_symbols, a
 * multiple of 8).  Inside a unit, lane j (0..31) owns the symbols
 *     element(i) = unit*U + (i/8)*256 + j*8 + (i%8),   i = 0..S-1
 * so that 8 consecutive symbols of a lane are 8 consecutive tensor elements.
 * Elements past N in the last unit are coded as the most frequent symbol.
 *
 * Coded unit:  32 length bytes len[j], then the 32 lane streams in lane
 * order.  Lane stream j holds len[j]*lenq 16-bit words: the final encoder
 * state (low word, high word), then the renormalisation words in the order
 * the decoder consumes them, then zero padding up to a multiple of lenq.
 * Raw unit: the unit's exponent bytes in element order, padded to even.
 * A unit is stored raw when any lane needs more than min(255*lenq, S/2) words
 * (S/2 words is the lane's share of the raw unit) or when the coded form is
 * not smaller than the raw form.
 *
 * rANS: 32-bit state x in [2^16, 2^32), prob_bits-bit probabilities (9 to
 * 12), 16-bit renormalisation.  Decoding one symbol, with M = 2^prob_bits:
 *     slot = x & (M-1); s = symbol whose [cum, cum+freq) holds slot;
 *     x = freq[s]*(x >> prob_bits) + slot - cum[s];
 *     if (x < 2^16) x = (x << 16) | next_word;
 * The encoder runs the lane's symbols backwards from state 2^16.
 *
 * prob_bits is chosen from the number of distinct symbols d of the tensor:
 * 10 for d <= 32, 11 for d <= 64, else 12 (11 if one symbol has 46 % of the
 * counts or more: no frequency may exceed 2047).  Exponent streams of network
 * weights have about 30 distinct values, and a 1024-slot decode table can be
 * replicated across the shared-memory banks of the GPU decoder.  The
 * whole-tensor compressor lowers the first step to 9 bits at precision 7
 * (nzo_choose_prob_bits_for): with 8 fraction bits stored per element the
 * exponent stream is a quarter of the stored bytes, the coarser table costs
 * 0.2 % of them, and 512 slots leave one table copy per bank.
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define NZO_MIN_PROB_BITS 9
#define NZO_MAX_PROB_BITS 12
#define NZO_MAX_PROB_SCALE (1u << NZO_MAX_PROB_BITS)
#define NZO_STATE_LOW (1u << 16)
#define NZO_MAGIC 0x31525A4Eu /* "NZR1" */

typedef struct nzo_header {
  uint32_t magic;
  uint32_t version;        /* 1 */
  uint64_t n_symbols;      /* N */
  uint32_t lane_symbols;   /* S */
  uint32_t len_quantum;    /* lenq: words per length-byte step */
  uint32_t n_units;
  uint32_t prob_bits;      /* 9 .. 12 */
  uint64_t payload_offset; /* byte offset of the payload in the container */
  uint64_t payload_words;  /* payload length in 16-bit words */
  uint64_t total_bytes;    /* container length, multiple of 16 */
  uint32_t n_raw_units;
  uint32_t max_coded_unit_words; /* largest coded (non-raw) unit, in words */
} nzo_header;

/* ------------------------------------------------------------------ split */

/* Statement-by-statement restatement of kernel_aligned_split for bf16 with
 * normalized=false (cuda/kernels.cuh:120-155; packing :86-89,:140-149).
 * The reference computes in uint8_t, so every intermediate is truncated to
 * 8 bits here as well.  The cub::WarpReduce Sum over the 8/(s+1) lanes of a
 * byte is a sum of fields shifted to disjoint bit positions, i.e. an OR.
 * Threads past `size` load the scalar 0 (kernels.cuh:92): tail bits are 0. */
void nzo_split_literal(const uint16_t *v, size_t n, int s, uint8_t *exp_out,
                       uint8_t *frac_out) {
  const int f_bits = 7, e_bits = 8;
  size_t frac_bytes = (n * (size_t)(s + 1) + 7) / 8;
  memset(frac_out, 0, frac_bytes);
  for (size_t idx = 0; idx < n; ++idx) {
    uint16_t value = v[idx];
    uint8_t sign = (uint8_t)((value >> (f_bits + e_bits)) & 0x1);      /* :122 */
    uint8_t repr = (uint8_t)(value & ((1 << f_bits) - 1));             /* :123 */
    uint8_t carry =
        (f_bits > s) ? (uint8_t)((repr >> (f_bits - s - 1)) & 1) : 0;  /* :126 */
    uint8_t exponent = (uint8_t)((value >> f_bits) & ((1 << e_bits) - 1)); /* :129 */
    repr = (uint8_t)(repr >> (f_bits - s));                            /* :132 */
    uint8_t overflow =
        (uint8_t)((__builtin_popcount(repr) == s) & carry);            /* :134 */
    repr = (uint8_t)((sign << s) |
                     (((1 << s) - 1) & (repr + carry)));               /* :137 */
    size_t bit = idx * (size_t)(s + 1);
    unsigned bit_in_byte = (unsigned)(bit & 7);                        /* :87 */
    unsigned shift = 7 - s - bit_in_byte;                              /* :89 */
    frac_out[bit >> 3] |= (uint8_t)(repr << shift);                    /* :140-149 */
    exp_out[idx] = (uint8_t)(exponent + overflow);                     /* :154 */
  }
}

/* Closed form of the same arithmetic: round the 15-bit magnitude half-up at
 * bit (7-s); the carry may ripple into the exponent; an exponent of 255 that
 * overflows wraps to 0 exactly as the uint8 store at kernels.cuh:154 does. */
void nzo_split(const uint16_t *v, size_t n, int s, uint8_t *exp_out,
               uint8_t *frac_out) {
  size_t frac_bytes = (n * (size_t)(s + 1) + 7) / 8;
  memset(frac_out, 0, frac_bytes);
  const uint32_t keep_mask = (1u << (8 + s)) - 1;
  const size_t blk = 1 << 16; /* multiple of 8: blocks never share a byte */
  const int64_t n_blk = (int64_t)((n + blk - 1) / blk);
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < n_blk; ++b) {
    size_t lo = (size_t)b * blk, hi = lo + blk < n ? lo + blk : n;
    for (size_t idx = lo; idx < hi; ++idx) {
      uint32_t val = v[idx];
      uint32_t sign = val >> 15;
      uint32_t mag = val & 0x7FFF;
      uint32_t round = (s < 7) ? ((mag >> (6 - s)) & 1u) : 0u;
      uint32_t keep = ((mag >> (7 - s)) + round) & keep_mask;
      uint32_t field = (sign << s) | (keep & ((1u << s) - 1));
      size_t bit = idx * (size_t)(s + 1);
      frac_out[bit >> 3] |= (uint8_t)(field << (7 - s - (bit & 7)));
      exp_out[idx] = (uint8_t)(keep >> s);
    }
  }
}

/* kernel_aligned_merge for bf16, normalized=false (cuda/kernels.cuh:197-216).
 * canonical_nan != 0 reproduces the float -> bf16 conversion of the store at
 * :214-216, which turns every NaN pattern into 0x7FFF. */
void nzo_merge(const uint8_t *exp_in, const uint8_t *frac_in, size_t n, int s,
               int canonical_nan, uint16_t *out) {
#pragma omp parallel for schedule(static)
  for (int64_t i64 = 0; i64 < (int64_t)n; ++i64) {
    size_t idx = (size_t)i64;
    size_t bit = idx * (size_t)(s + 1);
    unsigned shift = 7 - s - (unsigned)(bit & 7);
    uint32_t repr = (uint32_t)(frac_in[bit >> 3] >> shift);            /* :200 */
    uint32_t fraction = (repr & ((1u << s) - 1)) << (7 - s);           /* :202 */
    uint32_t sign = (repr >> s) & 1u;                                  /* :204 */
    uint32_t value = ((uint32_t)exp_in[idx] << 7) | fraction;          /* :197,:206 */
    uint32_t res = value | (sign << 15);
    if (canonical_nan && (value & 0x7F80) == 0x7F80 && (value & 0x7F))
      res = 0x7FFF;
    out[idx] = (uint16_t)res;
  }
}

/* ------------------------------------------------------- frequency table */

/* 256-bin histogram of the exponent bytes. */
void nzo_histogram(const uint8_t *sym, size_t n, uint64_t *hist) {
  memset(hist, 0, 256 * sizeof(uint64_t));
  for (size_t i = 0; i < n; ++i) hist[sym[i]]++;
}

/* Probability resolution for a histogram: 10 bits up to 32 distinct symbols,
 * 11 up to 64, else 12 -- but 11 when the most frequent symbol holds
 * 1900/4096 of the counts or more, so that no normalised frequency ever
 * needs more than 11 bits (rounding and the fix-up of nzo_normalize add at
 * most 128 to the largest entry).  The GPU decoder packs symbol, frequency
 * and slot offset into one 32-bit table entry and relies on that bound. */
uint32_t nzo_choose_prob_bits(const uint64_t *hist) {
  uint32_t d = 0;
  uint64_t total = 0, top = 0;
  for (int i = 0; i < 256; ++i) {
    d += hist[i] != 0;
    total += hist[i];
    if (hist[i] > top) top = hist[i];
  }
  if (d <= 32) return 10u;
  if (d <= 64) return 11u;
  return (top * 4096u < total * 1900u) ? 12u : 11u;
}

/* The same for a tensor compressed at precision s (0, 1, 3 or 7). */
uint32_t nzo_choose_prob_bits_for(const uint64_t *hist, int s) {
  const uint32_t pb = nzo_choose_prob_bits(hist);
  return (s == 7 && pb == 10u) ? NZO_MIN_PROB_BITS : pb;
}

/* Integer-only normalisation of a histogram to prob_bits-bit frequencies
 * (M = 2^prob_bits).  Pure integer arithmetic so that the CUDA encoder can
 * reproduce it bit for bit.
 *   1. f = round(h * M / T), at least 1 for every present symbol;
 *   2. the difference to M is taken from / given to the currently largest
 *      entry (lowest index on ties), never pushing an entry below 1;
 *   3. an alphabet of one symbol gets M-1 and its successor (mod 256) 1, so
 *      that no frequency needs prob_bits+1 bits.
 * An empty histogram yields freq[0] = M-1, freq[1] = 1.
 * Returns the most frequent symbol of the histogram. */
uint32_t nzo_normalize(const uint64_t *hist, uint32_t prob_bits, uint16_t *freq) {
  const uint32_t M = 1u << prob_bits;
  uint64_t total = 0;
  for (int i = 0; i < 256; ++i) total += hist[i];
  int32_t f[256];
  memset(f, 0, sizeof(f));
  uint32_t best = 0;
  if (total == 0) {
    f[0] = (int32_t)M;
  } else {
    for (int i = 0; i < 256; ++i) {
      if (hist[i] > hist[best]) best = (uint32_t)i;
      if (hist[i] == 0) continue;
      uint64_t q = (hist[i] * M + total / 2) / total;
      f[i] = q ? (int32_t)q : 1;
    }
  }
  int32_t sum = 0;
  for (int i = 0; i < 256; ++i) sum += f[i];
  int32_t d = (int32_t)M - sum;
  while (d != 0) {
    int top = 0;
    for (int i = 1; i < 256; ++i)
      if (f[i] > f[top]) top = i;
    if (d > 0) {
      f[top] += d;
      d = 0;
    } else {
      int32_t take = (-d < f[top] - 1) ? -d : f[top] - 1;
      f[top] -= take;
      d += take;
    }
  }
  for (int i = 0; i < 256; ++i) {
    if (f[i] == (int32_t)M) {
      f[i] = (int32_t)M - 1;
      f[(i + 1) & 255] = 1;
      break;
    }
  }
  for (int i = 0; i < 256; ++i) freq[i] = (uint16_t)f[i];
  return best;
}

/* ------------------------------------------------------------ container */

static size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

uint32_t nzo_len_quantum(uint32_t lane_symbols) {
  return (lane_symbols + 767) / 768;
}

/* Upper bound of the container size for n symbols. */
uint64_t nzo_container_bound(uint64_t n, uint32_t lane_symbols) {
  uint64_t U = 32ull * lane_symbols;
  uint64_t n_units = (n + U - 1) / U;
  uint64_t head = align16(64 + 512 + 4 * (n_units + 1));
  return head + align16(n_units * U + 2 * n_units) + 16;
}

static inline uint64_t unit_element(uint64_t unit, uint32_t S, uint32_t lane,
                                    uint32_t i) {
  return unit * 32ull * S + (uint64_t)(i >> 3) * 256 + lane * 8u + (i & 7);
}

/* Encode one lane of one unit.  Writes the lane stream (decoder order) to
 * `words` (capacity cap words) and returns its length in words, or 0 when the
 * capacity would be exceeded. */
static uint32_t encode_lane(const uint8_t *sym, uint64_t n, uint64_t unit,
                            uint32_t S, uint32_t lane, uint32_t pad,
                            uint32_t pb, const uint16_t *freq, const uint16_t *cum,
                            uint16_t *words, uint32_t cap, uint16_t *scratch) {
  uint32_t x = NZO_STATE_LOW;
  uint32_t emitted = 0; /* scratch[0..emitted) in emission order */
  for (int32_t i = (int32_t)S - 1; i >= 0; --i) {
    uint64_t e = unit_element(unit, S, lane, (uint32_t)i);
    uint32_t s = (e < n) ? sym[e] : pad;
    uint32_t fr = freq[s];
    uint32_t x_max = fr << (32 - pb);
    if (x >= x_max) {
      scratch[emitted++] = (uint16_t)(x & 0xFFFF);
      x >>= 16;
    }
    x = ((x / fr) << pb) + (x % fr) + cum[s];
  }
  uint32_t total = emitted + 2;
  if (total > cap) return 0;
  words[0] = (uint16_t)(x & 0xFFFF);
  words[1] = (uint16_t)(x >> 16);
  for (uint32_t k = 0; k < emitted; ++k) words[2 + k] = scratch[emitted - 1 - k];
  return total;
}

/* Encode one unit into `dst` (capacity U/2 + 1 words).  Returns the unit's
 * length in words; *raw is set when the unit had to be stored raw. */
static uint64_t encode_unit(const uint8_t *sym, uint64_t n, uint64_t u,
                            uint32_t S, uint32_t lenq, uint32_t pad, uint32_t pb,
                            const uint16_t *freq, const uint16_t *cum,
                            uint16_t *dst, int *raw) {
  const uint64_t U = 32ull * S;
  const uint32_t lane_cap = (255u * lenq < S / 2) ? 255u * lenq : S / 2;
  uint64_t first = u * U;
  uint64_t count = (n - first < U) ? (n - first) : U;
  uint64_t raw_words = (count + 1) / 2;
  uint16_t *lane_words = (uint16_t *)malloc((size_t)lane_cap * 2);
  uint16_t *scratch = (uint16_t *)malloc((size_t)(S + 8) * 2);
  uint8_t *lb = (uint8_t *)dst;
  uint64_t p = 16;
  int ok = 1;
  for (uint32_t j = 0; j < 32; ++j) {
    uint32_t l = encode_lane(sym, n, u, S, j, pad, pb, freq, cum, lane_words,
                             lane_cap, scratch);
    if (l == 0) {
      ok = 0;
      break;
    }
    uint32_t q = (l + lenq - 1) / lenq;
    if (p + (uint64_t)q * lenq >= raw_words) {
      ok = 0;
      break;
    }
    lb[j] = (uint8_t)q;
    memcpy(dst + p, lane_words, (size_t)l * 2);
    for (uint32_t k = l; k < q * lenq; ++k) dst[p + k] = 0;
    p += (uint64_t)q * lenq;
  }
  free(lane_words);
  free(scratch);
  if (ok) {
    *raw = 0;
    return p;
  }
  *raw = 1;
  uint8_t *d8 = (uint8_t *)dst;
  memcpy(d8, sym + first, count);
  if (count & 1) d8[count] = 0;
  return raw_words;
}

/* Encode n exponent bytes into an NZR1 container.  If `freq_in` is NULL the
 * table and its resolution are derived from the data (histogram,
 * nzo_choose_prob_bits, nzo_normalize); otherwise `prob_bits` gives the
 * resolution of `freq_in` (pass 0 to derive everything).  The pad symbol
 * is the most frequent entry of the table (lowest index on ties).  Returns
 * the container size in bytes, or 0 if `cap` is too small / arguments are
 * invalid.  Units are coded independently (OpenMP over units when built with
 * -fopenmp). */
uint64_t nzo_encode(const uint8_t *sym, uint64_t n, uint32_t lane_symbols,
                    const uint16_t *freq_in, uint32_t prob_bits, uint8_t *out,
                    uint64_t cap) {
  const uint32_t S = lane_symbols;
  if (S == 0 || (S & 7) || S > 8192) return 0;
  const uint32_t lenq = nzo_len_quantum(S);
  const uint64_t U = 32ull * S;
  const uint64_t n_units = (n + U - 1) / U;
  if (cap < nzo_container_bound(n, S)) return 0;

  uint16_t freq[256], cum[257];
  uint32_t pb = prob_bits;
  if (freq_in && pb >= NZO_MIN_PROB_BITS && pb <= NZO_MAX_PROB_BITS) {
    memcpy(freq, freq_in, sizeof(freq));
  } else {
    uint64_t hist[256];
    nzo_histogram(sym, n, hist);
    if (pb < NZO_MIN_PROB_BITS || pb > NZO_MAX_PROB_BITS) pb = nzo_choose_prob_bits(hist);
    nzo_normalize(hist, pb, freq);
  }
  uint32_t pad = 0;
  for (int i = 1; i < 256; ++i)
    if (freq[i] > freq[pad]) pad = (uint32_t)i;
  cum[0] = 0;
  for (int i = 0; i < 256; ++i) cum[i + 1] = (uint16_t)(cum[i] + freq[i]);

  nzo_header *h = (nzo_header *)out;
  memset(h, 0, sizeof(*h));
  memcpy(out + 64, freq, 512);
  uint32_t *offsets = (uint32_t *)(out + 576);
  const uint64_t payload_off = align16(576 + 4 * (n_units + 1));
  uint16_t *payload = (uint16_t *)(out + payload_off);

  const uint64_t slot_words = U / 2 + 1;
  uint16_t *tmp = (uint16_t *)malloc((size_t)(n_units ? n_units : 1) * slot_words * 2);
  uint64_t *ulen = (uint64_t *)malloc((size_t)(n_units + 1) * sizeof(uint64_t));
  uint8_t *uraw = (uint8_t *)malloc((size_t)n_units + 1);
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t u = 0; u < (int64_t)n_units; ++u) {
    int raw = 0;
    ulen[u] = encode_unit(sym, n, (uint64_t)u, S, lenq, pad, pb, freq, cum,
                          tmp + (size_t)u * slot_words, &raw);
    uraw[u] = (uint8_t)raw;
  }
  uint64_t w = 0;
  uint32_t n_raw = 0;
  uint64_t max_coded = 0;
  for (uint64_t u = 0; u < n_units; ++u) {
    offsets[u] = (uint32_t)w | (uraw[u] ? 0x80000000u : 0u);
    n_raw += uraw[u];
    uint64_t l = ulen[u];
    if (!uraw[u] && l > max_coded) max_coded = l;
    ulen[u] = w;
    w += l;
  }
  offsets[n_units] = (uint32_t)w;
  ulen[n_units] = w;
#pragma omp parallel for schedule(static)
  for (int64_t u = 0; u < (int64_t)n_units; ++u)
    memcpy(payload + ulen[u], tmp + (size_t)u * slot_words,
           (size_t)(ulen[u + 1] - ulen[u]) * 2);
  free(tmp);
  free(ulen);
  free(uraw);

  uint64_t end = payload_off + w * 2;
  uint64_t total = align16(end);
  memset(out + end, 0, total - end);
  {
    uint64_t tab_end = 576 + 4 * (n_units + 1);
    memset(out + tab_end, 0, payload_off - tab_end);
  }
  h->magic = NZO_MAGIC;
  h->version = 1;
  h->n_symbols = n;
  h->lane_symbols = S;
  h->len_quantum = lenq;
  h->n_units = (uint32_t)n_units;
  h->prob_bits = pb;
  h->payload_offset = payload_off;
  h->payload_words = w;
  h->total_bytes = total;
  h->n_raw_units = n_raw;
  h->max_coded_unit_words = (uint32_t)max_coded;
  return total;
}

static int decode_unit(const uint32_t *offsets, const uint16_t *payload,
                       uint64_t pw, uint64_t u, uint64_t n, uint32_t S,
                       uint32_t lenq, uint32_t pb, const uint16_t *freq,
                       const uint16_t *cum, const uint8_t *slot_sym,
                       uint8_t *sym_out) {
  const uint64_t U = 32ull * S;
  uint64_t w0 = offsets[u] & 0x7FFFFFFFu;
  uint64_t w1 = offsets[u + 1] & 0x7FFFFFFFu;
  int raw = (offsets[u] >> 31) & 1;
  if (w1 < w0 || w1 > pw) return -9;
  uint64_t first = u * U;
  uint64_t count = (n - first < U) ? (n - first) : U;
  if (raw) {
    if ((w1 - w0) * 2 < count) return -10;
    memcpy(sym_out + first, payload + w0, count);
    return 0;
  }
  if (w1 - w0 < 16) return -10;
  const uint8_t *lb = (const uint8_t *)(payload + w0);
  uint64_t p = w0 + 16;
  for (uint32_t j = 0; j < 32; ++j) {
    uint64_t lw = (uint64_t)lb[j] * lenq;
    if (lw < 2 || p + lw > w1) return -11;
    const uint16_t *ws = payload + p;
    uint64_t q = 2;
    uint32_t x = (uint32_t)ws[0] | ((uint32_t)ws[1] << 16);
    for (uint32_t i = 0; i < S; ++i) {
      uint32_t slot = x & ((1u << pb) - 1);
      uint32_t s = slot_sym[slot];
      x = (uint32_t)freq[s] * (x >> pb) + slot - cum[s];
      if (x < NZO_STATE_LOW) {
        if (q >= lw) return -12;
        x = (x << 16) | ws[q++];
      }
      uint64_t e = unit_element(u, S, j, i);
      if (e < n) sym_out[e] = (uint8_t)s;
    }
    if (x != NZO_STATE_LOW) return -13;
    p += lw;
  }
  if (p != w1) return -14;
  return 0;
}

/* Decode an NZR1 container into n exponent bytes.  Returns 0 on success, a
 * negative code when the container is malformed (never reads outside
 * [in, in+in_bytes)). */
int nzo_decode(const uint8_t *in, uint64_t in_bytes, uint8_t *sym_out,
               uint64_t n_expected) {
  if (in_bytes < 576 + 4) return -1;
  const nzo_header *h = (const nzo_header *)in;
  if (h->magic != NZO_MAGIC || h->version != 1) return -2;
  if (h->n_symbols != n_expected) return -3;
  const uint32_t S = h->lane_symbols;
  if (S == 0 || (S & 7) || S > 8192) return -4;
  const uint32_t lenq = h->len_quantum;
  if (lenq != nzo_len_quantum(S)) return -4;
  const uint64_t U = 32ull * S;
  const uint64_t n = h->n_symbols;
  const uint64_t n_units = (n + U - 1) / U;
  if (h->n_units != n_units) return -5;
  if (h->payload_offset != align16(576 + 4 * (n_units + 1))) return -6;
  if (h->payload_offset + h->payload_words * 2 > in_bytes) return -7;
  if (h->total_bytes > in_bytes) return -7;

  const uint32_t pb = h->prob_bits;
  if (pb < NZO_MIN_PROB_BITS || pb > NZO_MAX_PROB_BITS) return -4;
  const uint32_t M = 1u << pb;
  const uint16_t *freq = (const uint16_t *)(in + 64);
  uint16_t cum[257];
  uint32_t total = 0;
  cum[0] = 0;
  for (int i = 0; i < 256; ++i) {
    if (freq[i] > M - 1) return -8;
    total += freq[i];
    cum[i + 1] = (uint16_t)total;
  }
  if (total != M) return -8;
  uint8_t slot_sym[NZO_MAX_PROB_SCALE];
  for (int s = 0; s < 256; ++s)
    for (uint32_t k = cum[s]; k < cum[s + 1]; ++k) slot_sym[k] = (uint8_t)s;

  const uint32_t *offsets = (const uint32_t *)(in + 576);
  const uint16_t *payload = (const uint16_t *)(in + h->payload_offset);
  const uint64_t pw = h->payload_words;
  if ((offsets[n_units] & 0x7FFFFFFFu) != pw) return -9;

  int err = 0;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t u = 0; u < (int64_t)n_units; ++u) {
    int rc = decode_unit(offsets, payload, pw, (uint64_t)u, n, S, lenq, pb, freq,
                         cum, slot_sym, sym_out);
    if (rc) {
#pragma omp critical
      if (err == 0 || rc > err) err = rc;
    }
  }
  return err;
}

/* ---------------------------------------------------- whole-tensor helpers */

/* compress = split + encode; used by the CPU-baseline timing leg */
uint64_t nzo_compress_bf16(const uint16_t *v, uint64_t n, int s,
                           uint32_t lane_symbols, uint8_t *exp_scratch,
                           uint8_t *frac_out, uint8_t *cont_out, uint64_t cap) {
  uint64_t hist[256];
  nzo_split(v, n, s, exp_scratch, frac_out);
  nzo_histogram(exp_scratch, n, hist);
  return nzo_encode(exp_scratch, n, lane_symbols, NULL, nzo_choose_prob_bits_for(hist, s),
                    cont_out, cap);
}

/* decompress = decode + merge */
int nzo_decompress_bf16(const uint8_t *cont, uint64_t cont_bytes,
                        const uint8_t *frac, uint64_t n, int s,
                        int canonical_nan, uint8_t *exp_scratch,
                        uint16_t *out) {
  int rc = nzo_decode(cont, cont_bytes, exp_scratch, n);
  if (rc) return rc;
  nzo_merge(exp_scratch, frac, n, s, canonical_nan, out);
  return 0;
}

/* CRC-32 (IEEE, reflected) for the golden-vector checks. */
uint32_t nzo_crc32(const uint8_t *p, uint64_t n) {
  static uint32_t table[256];
  static int init = 0;
  if (!init) {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
      table[i] = c;
    }
    init = 1;
  }
  uint32_t c = 0xFFFFFFFFu;
  for (uint64_t i = 0; i < n; ++i) c = table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}

/* ------------------------------------------------------- block normaliser */

/* float -> bf16 bits, round to nearest even, NaN -> 0x7FFF: the conversion the
 * reference's stores perform (c10::BFloat16 from float on sm_80+). */
static uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return 0x7FFF;
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Per-group scaling before the split, the *intended* semantics of the
 * normalized=true path of kernel_aligned_split (cuda/kernels.cuh:94-118; the
 * reference's own BlockReduce misbehaves for groups of 64..512 threads, so its
 * bits are not reproducible there): for every run of `group` consecutive
 * elements, absmax of |float(v)| (missing tail elements count as 0), scale =
 * 1.<23 mantissa bits of absmax> in [1, 2), v' = bf16(float(v) / scale); the
 * stored normaliser byte is the top 8 mantissa bits (:103-116). */
void nzo_normalize_groups(const uint16_t *v, uint64_t n, uint32_t group, uint16_t *out,
                          uint8_t *normalizers) {
  const uint64_t n_groups = (n + group - 1) / group;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < (int64_t)n_groups; ++g) {
    uint64_t lo = (uint64_t)g * group, hi = lo + group < n ? lo + group : n;
    float amax = 0.0f;
    for (uint64_t i = lo; i < hi; ++i) {
      float a = bf16_to_f32((uint16_t)(v[i] & 0x7FFF));
      if (a > amax) amax = a; /* NaN never wins, like fmaxf-free cub::Max on floats */
    }
    uint32_t bits;
    memcpy(&bits, &amax, 4);
    uint32_t frac = bits & 0x007FFFFFu;
    uint32_t sbits = 0x3F800000u | frac;
    float scale;
    memcpy(&scale, &sbits, 4);
    normalizers[g] = (uint8_t)(frac >> 15);
    for (uint64_t i = lo; i < hi; ++i) out[i] = f32_to_bf16_rne(bf16_to_f32(v[i]) / scale);
  }
}

/* Inverse scaling after the merge (cuda/kernels.cuh:208-216): the scale is
 * rebuilt from the stored byte only, out = bf16(scale8 * float(v)). */
void nzo_denormalize_groups(uint16_t *v, uint64_t n, uint32_t group, const uint8_t *normalizers) {
#pragma omp parallel for schedule(static)
  for (int64_t i64 = 0; i64 < (int64_t)n; ++i64) {
    uint64_t i = (uint64_t)i64;
    uint32_t sbits = 0x3F800000u | ((uint32_t)normalizers[i / group] << 15);
    float scale;
    memcpy(&scale, &sbits, 4);
    v[i] = f32_to_bf16_rne(scale * bf16_to_f32(v[i]));
  }
}
