// y = x W^T (+ bias) with W decoded from its compressed form straight into the
// tensor cores' shared-memory operand tiles: the bf16 weight is never written to
// global memory and never read back by a library GEMM.
//
// Replaces, for inputs of up to a few hundred rows, the reference's
// Manager::linear / linear_without_bias (cuda/high_level.cu:252-263), which
// decompress the whole weight into a fresh tensor and hand it to a cuBLAS GEMM.
//
// Layout.  W is stored in operand order (see operand_index in nz_decode_core.cuh):
// one 256-element block of the coded stream is a 4-row x 64-column patch of W and
// a unit is a run of such blocks along a row group.  32 consecutive row groups at
// the same column block are exactly one 128 x 64 bf16 operand tile.
//
// Work decomposition.  One CTA per (128-row tile, column segment of one unit
// length).  16 decoder warps walk 2 units each (the 32 row groups of the tile),
// one block per step; a lane's 8 decoded elements are one 16-byte chunk of the
// tile, stored where the 128-byte-swizzled K-major layout of the tensor-core
// operand wants it.  Two more warps feed the tensor cores: one thread fetches the
// matching 64-column slab of x with a tiled bulk tensor copy (TMA, no multicast);
// another, when both the weight tile and the x slab of a step are complete, issues
// four tcgen05.mma (128 x N x 16, bf16 x bf16 -> fp32) that accumulate in tensor
// memory.  Tiles and slabs cycle through a small ring guarded by mbarriers:
//   full[s]   16 arrivals: every decoder warp has written its rows of tile s
//   xfull[s]  transaction barrier of the TMA copy into slab s
//   empty[s]  tcgen05.commit: the MMAs that read tile s / slab s have completed
// After the last step the accumulator (128 rows x N tokens, fp32) is read back
// from tensor memory by the decoder warps and written either to y (rounded to
// bf16, bias added) or, when the row is split over several column segments, to a
// per-segment fp32 buffer that a small kernel adds up in a fixed order.
//
// Every wait is bounded; a wait that runs out sets NZ_STATUS_TIMEOUT, raises a
// CTA-wide abort flag that all other waits watch, and the CTA leaves through the
// common exit, which frees its tensor memory.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "nz_decode_core.cuh"

namespace nz {

constexpr int kLinDecWarps = 16;                    // 2 units each: 32 row groups = 128 rows
constexpr int kLinWarps = kLinDecWarps + 2;         // + the tensor-core warp and the TMA warp
constexpr int kLinThreads = kLinWarps * 32;
constexpr uint32_t kTileRows = 128;
constexpr uint32_t kTileBytes = kTileRows * 128;    // 128 rows x 64 bf16
constexpr uint32_t kMaxTokensPerLaunch = 256;       // MMA N and tensor-memory columns
constexpr uint32_t kLinMaxStages = 4;
constexpr uint32_t kMaxPeers = 8;                   // ranks of a tensor-parallel group
constexpr uint32_t kTileCounterBytes = 4096;        // head of a peer workspace: u32 per row tile

struct LinearArgs {
  const uint8_t *container;
  uint64_t container_bytes;
  const uint8_t *frac;
  uint32_t rows, cols;        // W is [rows, cols] = [out_features, in_features]
  uint32_t S;                 // lane_symbols; a unit is S / 8 blocks of 4 x 64 elements
  uint32_t n_units;
  uint32_t segs;              // units per row group = column segments
  uint32_t slot_bytes;
  uint32_t lut_shift, lut_bytes;
  uint32_t stages;            // ring depth
  uint32_t n_pad;             // MMA N: tokens of this launch, padded to a multiple of 16
  uint32_t n_tok;             // tokens of this launch that exist
  uint32_t tok0;              // first token of this launch
  uint32_t m_total;           // tokens of the whole call (rows of x and y)
  uint32_t tmem_cols;         // power of two >= max(32, n_pad)
  int canon;
  const uint16_t *bias;       // bf16[rows] or null
  uint16_t *y;                // bf16[m_total, rows]
  float *partial;             // fp32[segs, m_total, rows] when segs > 1
  uint32_t *status;
  // tensor-parallel all-reduce fused into the epilogue (tp_world > 1): the rank's sums over
  // its columns go, by plain peer stores, into plane `tp_rank` of every rank's exchange area
  // [src rank][token][row]; every CTA then adds 1 (system scope) to counter `tp_rank` of every
  // rank's arrival counters.  With several column segments the CTAs of a row tile first put
  // their partial sums into `partial` (local); the one that arrives last at the tile's
  // counter adds them in segment order and does the peer stores.
  uint32_t tp_world, tp_rank;
  float *peer_partial[kMaxPeers];
  uint32_t *peer_arrivals[kMaxPeers];
  uint32_t *tile_counters;    // u32[row tiles], zero between launches
};

// ------------------------------------------------------------------ PTX
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// 2-D tiled bulk tensor copy global -> this CTA's shared memory (no multicast).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t c0,
                                            int32_t c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile of 128-byte
// rows (8-row groups 1024 bytes apart): start address >> 4 in bits 0-13, leading
// byte offset (unused for this layout) 1 in bits 16-29, stride byte offset
// 1024 >> 4 in bits 32-45, descriptor version 1 in bits 46-47, layout type
// "128-byte swizzle" = 2 in bits 61-63.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}
// D[tmem] (+)= A[smem] * B[smem]^T, one 128 x N x 16 step.
__device__ __forceinline__ void mma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// 16 consecutive fp32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Bounded wait on an mbarrier phase that also watches the CTA's abort flag.
// Returns false when the wait was abandoned.
__device__ __forceinline__ bool wait_phase(uint32_t bar, uint32_t parity,
                                           const volatile uint32_t *abort_flag) {
  for (uint32_t it = 0; it < kMaxWaitIters; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 63u && *abort_flag) return false;
  }
  return false;
}
// The same for a whole (converged) warp: every lane gets the same verdict.
__device__ __forceinline__ bool wait_phase_warp(uint32_t bar, uint32_t parity,
                                                const volatile uint32_t *abort_flag) {
  return __all_sync(0xFFFFFFFFu, wait_phase(bar, parity, abort_flag));
}

__device__ __forceinline__ uint16_t f32_to_bf16_rn(float f) {
  uint32_t bits = __float_as_uint(f);
  if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu)) return 0x7FFFu;   // NaN
  bits += 0x7FFFu + ((bits >> 16) & 1u);
  return (uint16_t)(bits >> 16);
}

// One chain = one unit = one row group (4 rows) of the tile over the CTA's column
// segment.  A coded chain walks its rANS stream; a raw chain reads the exponent
// bytes as they are.
struct LinChain {
  uint32_t kind;            // kUnitSkip / kUnitRaw / kUnitCoded
  LaneState st;
  const uint8_t *raw;       // raw chains: this lane's next 8 exponent bytes
  const uint8_t *frac;      // this lane's packed fractions of the next block
  uint32_t dst;             // offset of this lane's 16-byte chunk inside a tile
};

// 8 symbols of one chain as table entries (symbol in bits 23-30).
template <int ROW>
__device__ __forceinline__ void chain_symbols(LinChain &ch, const LutView &lv, uint32_t (&ent)[8]) {
  if (ch.kind == kUnitCoded) {
#pragma unroll
    for (int t = 0; t < 8; ++t) ent[t] = decode_step<ROW>(ch.st, lv);
  } else {
    const uint2 q = __ldg(reinterpret_cast<const uint2 *>(ch.raw));
    ch.raw += 256;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      ent[t] = ((q.x >> (8 * t)) & 0xFFu) << kEntSymShift;
      ent[t + 4] = ((q.y >> (8 * t)) & 0xFFu) << kEntSymShift;
    }
  }
}

template <int S, bool CANON, int ROW, bool BOTH_CODED>
__device__ __forceinline__ bool linear_decode_loop(LinChain (&ch)[2], const LutView &lv,
                                                   uint32_t n_blocks, uint32_t stages,
                                                   uint32_t tiles0, uint32_t bar_full0,
                                                   uint32_t bar_empty0, uint32_t lane,
                                                   const volatile uint32_t *abort_flag) {
  constexpr uint32_t kFracStride = 32u * (S + 1);
  constexpr int kAhead = 4;
  uint64_t fr[2][kAhead];
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int k = 0; k < kAhead; ++k)
      fr[c][k] = (ch[c].kind != kUnitSkip && (uint32_t)k < n_blocks)
                     ? load_frac<S>(ch[c].frac + k * kFracStride) : 0;
  uint32_t stage = 0, phase = 0;
#pragma unroll 1
  for (uint32_t b0 = 0; b0 < n_blocks; b0 += kAhead) {
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      const uint32_t b = b0 + k;
      if (b >= n_blocks) break;
      uint64_t bits[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        bits[c] = fr[c][k];
        if (ch[c].kind != kUnitSkip && b + kAhead < n_blocks)
          fr[c][k] = load_frac<S>(ch[c].frac + (kAhead + k) * kFracStride);
      }
      uint32_t w[2][4];
      if (BOTH_CODED) {
        // the two chains' steps alternate: each hides the other's table and multiply latency
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint32_t e0[2], e1[2];
#pragma unroll
          for (int c = 0; c < 2; ++c) e0[c] = decode_step<ROW>(ch[c].st, lv);
#pragma unroll
          for (int c = 0; c < 2; ++c) e1[c] = decode_step<ROW>(ch[c].st, lv);
#pragma unroll
          for (int c = 0; c < 2; ++c) w[c][t] = merge_word<S, CANON>(e0[c], e1[c], bits[c], t);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (ch[c].kind == kUnitSkip) continue;
          uint32_t ent[8];
          chain_symbols<ROW>(ch[c], lv, ent);
#pragma unroll
          for (int t = 0; t < 4; ++t)
            w[c][t] = merge_word<S, CANON>(ent[2 * t], ent[2 * t + 1], bits[c], t);
        }
      }
      // the tensor cores must be done with the tile this step overwrites
      if (b >= stages && !wait_phase_warp(bar_empty0 + 8 * stage, phase ^ 1, abort_flag)) return false;
      const uint32_t tile = tiles0 + stage * kTileBytes;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (!BOTH_CODED && ch[c].kind == kUnitSkip) continue;
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(tile + ch[c].dst),
                     "r"(w[c][0]), "r"(w[c][1]), "r"(w[c][2]), "r"(w[c][3])
                     : "memory");
      }
      // make this lane's stores visible to the tensor cores' (asynchronous proxy) reads,
      // then one arrival per warp
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_full0 + 8 * stage);
      if (++stage == stages) {
        stage = 0;
        phase ^= 1;
      }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) ch[c].frac += kAhead * kFracStride;
  }
  return true;
}

// Shared-memory map (offsets from the 1024-byte aligned base):
//   [0, lut_bytes)                      decode table
//   [lut_bytes, +1024)                  mbarriers, scan scratch, flags
//   [.., + 32 * slot_bytes + guard)     staged units
//   (1024-aligned) stages x 16 KB       weight tiles
//   (1024-aligned) stages x n_pad*128   x slabs
constexpr uint32_t kBarWarp = 0;         // 16 x 8 bytes: per-warp staging barriers
constexpr uint32_t kBarFull = 128;       // kLinMaxStages x 8
constexpr uint32_t kBarXFull = 160;
constexpr uint32_t kBarEmpty = 192;
constexpr uint32_t kBarDone = 224;
constexpr uint32_t kTmemSlot = 232;      // u32: tensor-memory base address
constexpr uint32_t kAbortSlot = 236;     // u32: abort flag
constexpr uint32_t kLastSlot = 240;      // u32: this CTA arrived last at its row tile's counter
constexpr uint32_t kCumOff = 256;        // u16[257]
constexpr uint32_t kFlagOff = 256 + 520; // u32[3]

template <int S>
__global__ void __launch_bounds__(kLinThreads, 1)
linear_kernel(const LinearArgs p, const __grid_constant__ CUtensorMap x_map) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t base = smem_u32(smem);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tile_id = blockIdx.x / p.segs, seg = blockIdx.x % p.segs;

  DecodeArgs a;
  a.container = p.container;
  a.container_bytes = p.container_bytes;
  a.frac = p.frac;
  a.n = (uint64_t)p.rows * p.cols;
  a.S = p.S;
  a.n_units = p.n_units;
  a.slot_bytes = p.slot_bytes;
  a.lut_shift = p.lut_shift;
  a.lut_bytes = p.lut_bytes;
  a.ring_offset = 0;
  a.canon = p.canon;
  a.out_bf16 = nullptr;
  a.out_exp = nullptr;
  a.status = p.status;
  a.unit_list = nullptr;
  a.n_work = p.n_units;
  a.gx = nullptr;
  a.partial = nullptr;
  a.in = 0;
  a.seg = 0;
  a.tile_cols = p.cols;

  uint8_t *misc = smem + p.lut_bytes;
  const uint32_t misc_a = base + p.lut_bytes;
  uint16_t *cum_sh = reinterpret_cast<uint16_t *>(misc + kCumOff);
  uint32_t *flag_sh = reinterpret_cast<uint32_t *>(misc + kFlagOff);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(misc + kAbortSlot);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc + kTmemSlot);
  const uint32_t guard = ((p.S + 8) * 2 + 127) & ~127u;
  const uint32_t slots_a = misc_a + 1024;
  const uint32_t tiles_a = (slots_a + 2 * kLinDecWarps * p.slot_bytes + guard + 1023u) & ~1023u;
  const uint32_t xslab_bytes = p.n_pad * 128u;
  const uint32_t xs_a = tiles_a + p.stages * kTileBytes;     // 16 KB tiles keep this 1024-aligned
  const uint32_t n_blocks = p.S / 8;
  const bool is_dec = warp < (uint32_t)kLinDecWarps;
  const bool is_mma = warp == (uint32_t)kLinDecWarps;

  // a dependent launch (the kernel that adds up the column segments) may be set up now; it
  // waits for this grid to complete before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // ---- barriers and tensor memory
  if (threadIdx.x == 0) *abort_flag = 0;
  if (is_dec) {
    if (lane == 0) mbar_init(misc_a + kBarWarp + 8 * warp, 1);
  } else if (is_mma) {
    if (lane == 0) {
      for (uint32_t s = 0; s < p.stages; ++s) {
        mbar_init(misc_a + kBarFull + 8 * s, kLinDecWarps);
        mbar_init(misc_a + kBarXFull + 8 * s, 1);
        mbar_init(misc_a + kBarEmpty + 8 * s, 1);
      }
      mbar_init(misc_a + kBarDone, 1);
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     misc_a + kTmemSlot),
                 "r"(p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (lane == 0) {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  __syncwarp();

  // ---- plan and stage this warp's two units, build the decode table meanwhile
  const Header *h = reinterpret_cast<const Header *>(a.container);
  const uint64_t pay_off = payload_offset(a.n_units);
  const uint64_t max_words = (a.container_bytes - pay_off) / 2;
  const uint32_t bar_w = misc_a + kBarWarp + 8 * (is_dec ? warp : 0);
  const uint32_t slot0 = slots_a + 2 * (is_dec ? warp : 0) * p.slot_bytes;
  UnitPlan pl[2];
  uint32_t unit[2] = {p.n_units, p.n_units};
  bool staged = false;
  if (is_dec) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint32_t group = tile_id * 32 + 2 * warp + c;        // row group = 4 rows of W
      if (group < p.rows / 4) unit[c] = group * p.segs + seg;
      pl[c] = plan_unit(a, unit[c], pay_off, max_words, lane);
    }
    staged = stage_units(a, pl, pay_off, slot0, bar_w, lane);
  }
  table_scan(a, h, pay_off, max_words, cum_sh, flag_sh, warp, lane, kLinWarps);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t pb;
  const uint32_t bad = table_verdict(cum_sh, flag_sh, pb);
  const uint32_t tmem = *tmem_slot;
  bool ok = bad == 0;
  LutView lv;
  uint32_t row_shift = 0;
  if (ok) table_fill(a.lut_shift, a.S, pb, smem, cum_sh, warp, lane, kLinWarps, lv, row_shift);
  else if (threadIdx.x == 0 && blockIdx.x == 0) raise(a.status, bad);
  const bool canon = a.canon && (cum_sh[256] != cum_sh[255]);
  __syncthreads();

  if (is_dec) {
    // ---------------------------------------------------------------- decoder warps
    if (staged && !__all_sync(0xFFFFFFFFu, wait_staged(bar_w, 0))) {
      if (lane == 0) raise(a.status, NZ_STATUS_TIMEOUT);
      *abort_flag = 1;
      ok = false;
    }
    if (ok) {
      LinChain ch[2];
      const uint64_t U = 32ull * a.S;
      const uint32_t lenq = len_quantum(a.S);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        ch[c].kind = pl[c].kind;
        ch[c].raw = nullptr;
        ch[c].st.x = kStateLow;
        ch[c].st.p = slot0;
        ch[c].st.w = 0;
        if (pl[c].kind == kUnitCoded) {
          if (!open_unit(pl[c], slot0 + c * a.slot_bytes, lenq, lane, ch[c].st)) {
            if (lane == 0) raise(a.status, NZ_STATUS_BAD_LANES);
            ch[c].kind = kUnitSkip;
          }
        } else if (pl[c].kind == kUnitRaw) {
          ch[c].raw = a.container + pay_off + pl[c].byte0 + lane * 8;
        }
        const uint64_t e = (uint64_t)unit[c] * U + lane * 8;        // stream order
        ch[c].frac = a.frac + e * (S + 1) / 8;
        const uint32_t r = 4 * (2 * warp + c) + (lane >> 3);        // row inside the tile
        ch[c].dst = r * 128u + (((lane & 7u) ^ (r & 7u)) << 4);
      }
      // Units that cannot be decoded leave their rows of the tile as they are: a row of
      // the operand only ever reaches the same row of the result, which is not stored
      // for rows outside the matrix and is flagged in the status word otherwise.
      const uint32_t bar_full0 = misc_a + kBarFull, bar_empty0 = misc_a + kBarEmpty;
      const bool both = ch[0].kind == kUnitCoded && ch[1].kind == kUnitCoded;
      bool fine;
#define NZ_LIN_LOOP(CANON, ROW, BOTH)                                                          \
  linear_decode_loop<S, CANON, ROW, BOTH>(ch, lv, n_blocks, p.stages, tiles_a, bar_full0,      \
                                          bar_empty0, lane, abort_flag)
      if (!both)
        fine = canon ? NZ_LIN_LOOP(true, 0, false) : NZ_LIN_LOOP(false, 0, false);
      else if (canon)
        fine = NZ_LIN_LOOP(true, 0, true);
      else if (row_shift == 7)
        fine = NZ_LIN_LOOP(false, 7, true);
      else
        fine = NZ_LIN_LOOP(false, 0, true);
#undef NZ_LIN_LOOP
      if (!fine) {
        if (lane == 0) raise(a.status, NZ_STATUS_TIMEOUT);
        *abort_flag = 1;
        ok = false;
      } else {
        bool low = true;
#pragma unroll
        for (int c = 0; c < 2; ++c) low = low && (ch[c].kind != kUnitCoded || ch[c].st.x == kStateLow);
        if (__any_sync(0xFFFFFFFFu, !low) && lane == 0) raise(a.status, NZ_STATUS_BAD_STATE);
      }
    }
    // ---- epilogue: the accumulator is complete when the last commit arrives
    if (ok && !wait_phase_warp(misc_a + kBarDone, 0, abort_flag)) {
      if (lane == 0) raise(a.status, NZ_STATUS_TIMEOUT);
      *abort_flag = 1;
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      const uint32_t sub = warp & 3;                       // tensor-memory lanes 32 sub .. +31
      const uint32_t r = tile_id * kTileRows + 32 * sub + lane;
      // the bias rides on the direct store, or (tensor parallel: on the one rank that was
      // given it) on the partial sums of segment 0
      const float bias = (p.bias && r < p.rows && p.segs == 1)
                             ? __uint_as_float((uint32_t)p.bias[r] << 16) : 0.f;
      for (uint32_t c0 = (warp >> 2) * 16; c0 < p.n_pad; c0 += 64) {
        uint32_t v[16];
        tmem_ld16(tmem + ((32 * sub) << 16) + c0, v);
        tmem_ld_wait();
        if (r < p.rows) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint32_t t = c0 + i;
            if (t >= p.n_tok) break;
            const uint64_t tok = p.tok0 + t;
            if (p.segs > 1) {
              p.partial[((uint64_t)seg * p.m_total + tok) * p.rows + r] = __uint_as_float(v[i]);
            } else if (p.tp_world > 1) {
              const uint64_t at = ((uint64_t)p.tp_rank * p.m_total + tok) * p.rows + r;
              const float part = __uint_as_float(v[i]) + bias;
              for (uint32_t q = 0; q < p.tp_world; ++q) p.peer_partial[q][at] = part;
            } else if (p.segs == 1) {
              p.y[tok * p.rows + r] = f32_to_bf16_rn(__uint_as_float(v[i]) + bias);
            } else {
              p.partial[((uint64_t)seg * p.m_total + tok) * p.rows + r] = __uint_as_float(v[i]);
            }
          }
        }
      }
    }
  } else if (is_mma) {
    // ---------------------------------------------------------- tensor-core thread
    if (ok && lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((p.n_pad >> 3) << 17) |
                             ((kTileRows >> 4) << 24);     // fp32 accumulate, bf16 x bf16, K-major
      uint32_t stage = 0, phase = 0;
      for (uint32_t b = 0; b < n_blocks; ++b) {
        ok = wait_phase(misc_a + kBarFull + 8 * stage, phase, abort_flag) &&
             wait_phase(misc_a + kBarXFull + 8 * stage, phase, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint64_t ad = smem_desc_sw128(tiles_a + stage * kTileBytes);
        const uint64_t bd = smem_desc_sw128(xs_a + stage * xslab_bytes);
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k)      // 4 x 16 columns; 32 bytes = 2 descriptor units each
          mma_bf16_ss(tmem, ad + 2 * k, bd + 2 * k, idesc, (b | k) != 0);
        // arrives when these MMAs are complete: tile and slab `stage` are free again
        mma_commit(misc_a + kBarEmpty + 8 * stage);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) {
        mma_commit(misc_a + kBarDone);
      } else {
        raise(a.status, NZ_STATUS_TIMEOUT);
        *abort_flag = 1;
      }
    }
  } else if (lane == 0) {
    // ------------------------------------------------------------------ TMA thread
    // the x slab of step b: columns [seg * S / 8 + b] * 64 .. + 63 of the launch's tokens
    if (ok) {
      const int32_t k_first = (int32_t)(seg * n_blocks * 64);
      uint32_t stage = 0, phase = 0;
      for (uint32_t b = 0; b < n_blocks; ++b) {
        if (b >= p.stages && !wait_phase(misc_a + kBarEmpty + 8 * stage, phase ^ 1, abort_flag)) {
          raise(a.status, NZ_STATUS_TIMEOUT);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(misc_a + kBarXFull + 8 * stage, xslab_bytes);
        tma_load_2d(xs_a + stage * xslab_bytes, &x_map, k_first + (int32_t)(b * 64), (int32_t)p.tok0,
                    misc_a + kBarXFull + 8 * stage);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  }

  // ---- common exit: everybody is done with tensor memory, then it is freed
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (is_mma) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(p.tmem_cols)
                 : "memory");
  }
  if (p.tp_world > 1) {
    if (p.segs > 1) {
      // the last of the row tile's CTAs adds the segments' partial sums, in segment order
      // whoever it is, and hands the sums to every rank
      volatile uint32_t *last_sh = reinterpret_cast<volatile uint32_t *>(misc + kLastSlot);
      if (threadIdx.x == 0) {
        __threadfence();                     // cumulative: the CTA's partial sums, then the count
        const uint32_t before = atomicAdd(p.tile_counters + tile_id, 1u);
        const bool last = before == p.segs - 1;
        if (last) atomicExch(p.tile_counters + tile_id, 0u);     // ready for the next launch
        *last_sh = last;
      }
      __syncthreads();
      if (*last_sh && is_dec) {
        __threadfence();
        const uint32_t r = tile_id * kTileRows + 32 * (warp & 3) + lane;
        if (r < p.rows) {
          const float bias = p.bias ? __uint_as_float((uint32_t)p.bias[r] << 16) : 0.f;
          // 8 tokens at a time: the loads of a pass are independent, only the adds are in order
          constexpr uint32_t kStep = kLinDecWarps / 4, kBatch = 8;
          for (uint32_t t0 = warp >> 2; t0 < p.n_tok; t0 += kStep * kBatch) {
            float sum[kBatch];
#pragma unroll
            for (uint32_t k = 0; k < kBatch; ++k) sum[k] = 0.f;
            for (uint32_t s = 0; s < p.segs; ++s) {
              const float *plane = p.partial + ((uint64_t)s * p.m_total + p.tok0) * p.rows + r;
              float part[kBatch];
#pragma unroll
              for (uint32_t k = 0; k < kBatch; ++k) {
                const uint32_t t = t0 + k * kStep;
                part[k] = t < p.n_tok ? __ldcg(plane + (uint64_t)t * p.rows) : 0.f;
              }
#pragma unroll
              for (uint32_t k = 0; k < kBatch; ++k) sum[k] += part[k];
            }
#pragma unroll
            for (uint32_t k = 0; k < kBatch; ++k) {
              const uint32_t t = t0 + k * kStep;
              if (t >= p.n_tok) break;
              const uint64_t at = ((uint64_t)p.tp_rank * p.m_total + p.tok0 + t) * p.rows + r;
              const float total = sum[k] + bias;
              for (uint32_t q = 0; q < p.tp_world; ++q) p.peer_partial[q][at] = total;
            }
          }
        }
      }
      __syncthreads();
    }
    if (threadIdx.x == 0 && (p.segs == 1 || *reinterpret_cast<volatile uint32_t *>(misc + kLastSlot))) {
      // one arrival per row tile and rank, from the CTA that did the tile's peer stores, also
      // when a CTA gave up: the peers' waits are bounded either way, and their status words
      // tell them when the sums cannot be trusted.  The fence is cumulative over the CTA's
      // stores that the barrier made visible to this thread.
      __threadfence_system();
      for (uint32_t q = 0; q < p.tp_world; ++q) atomicAdd_system(p.peer_arrivals[q] + p.tp_rank, 1u);
    }
  }
}

// y[t, r] = bf16(sum over segments of partial[seg, t, r] + bias[r]), segments in order.
__global__ void linear_finish_kernel(const float *__restrict__ partial, uint32_t segs,
                                     uint64_t plane, uint32_t rows,
                                     const uint16_t *__restrict__ bias, uint16_t *__restrict__ y) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // launched with programmatic stream serialisation: wait for the kernel that wrote the
  // partial sums (a no-op for an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (i >= plane) return;
  float sum = 0.f;
  for (uint32_t s = 0; s < segs; ++s) sum += partial[(uint64_t)s * plane + i];
  if (bias) sum += __uint_as_float((uint32_t)bias[i % rows] << 16);
  y[i] = f32_to_bf16_rn(sum);
}

// The last step for a tensor-parallel group: every rank's sums lie in this rank's exchange
// area [src rank][token][row]; wait (bounded) until every rank's CTAs of this call have
// arrived, then add rank by rank -- the same order on every rank, so all ranks get the same
// bits.  `expected` = arrivals per rank up to and including this call.
__global__ void linear_allreduce_finish_kernel(const float *__restrict__ partial,
                                               const uint32_t *arrivals, uint32_t expected,
                                               uint32_t world, uint64_t plane,
                                               uint16_t *__restrict__ y, uint32_t *status) {
  __shared__ uint32_t ok_sh;
  // launched with programmatic stream serialisation: this rank's linear kernel first
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    uint32_t ok = 1;
    for (uint32_t q = 0; q < world && ok; ++q) {
      uint32_t it = 0;
      for (;;) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(arrivals + q) : "memory");
        if ((int32_t)(seen - expected) >= 0) break;
        if (++it > (1u << 21)) {            // about a second
          ok = 0;
          break;
        }
        __nanosleep(400);
      }
    }
    if (!ok && status) atomicOr(status, NZ_STATUS_TIMEOUT);
    ok_sh = ok;
  }
  __syncthreads();
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= plane) return;
  float sum = 0.f;
  for (uint32_t k = 0; k < world; ++k) sum += __ldcv(partial + (uint64_t)k * plane + i);
  y[i] = f32_to_bf16_rn(sum);
  (void)ok_sh;
}

// --------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!fn) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// Units per row group for a matrix with `cols` columns stored with lane_symbols S,
// or 0 when S does not fit the operand order.
static uint32_t operand_segments(uint64_t cols, uint32_t S) {
  if (cols == 0 || cols % 64 || !valid_lane_symbols(S)) return 0;
  const uint64_t spr = cols / 64, beta = S / 8;
  return (spr % beta == 0) ? (uint32_t)(spr / beta) : 0;
}

struct LinearGeometry {
  uint32_t slot_bytes, lut_shift, stages, smem_bytes;
};

static bool linear_geometry(uint32_t S, uint32_t max_unit_words, uint32_t n_pad, LinearGeometry &g) {
  const uint64_t U = 32ull * S;
  uint64_t unit_bytes = max_unit_words ? (uint64_t)max_unit_words * 2 : U;
  if (unit_bytes > U) unit_bytes = U;
  if (unit_bytes < 160) unit_bytes = 160;
  g.slot_bytes = (uint32_t)((unit_bytes + 32 + 15) & ~uint64_t(15));
  const uint32_t guard = ((S + 8) * 2 + 127) & ~127u;
  const uint32_t fixed = 1024 /* alignment slack */ + 1024 /* misc */ +
                         2 * kLinDecWarps * g.slot_bytes + guard + 1024 /* tile alignment */;
  const uint32_t per_stage = kTileBytes + n_pad * 128u;
  // Ring depth first (decoder warps that run ahead of the slowest one need somewhere to
  // write), then table copies (fewer shared-memory bank conflicts per lookup).
  const char *force = getenv("NZ_LINEAR_GEOMETRY");      // "<lut_shift>,<stages>": tuning aid
  if (force) {
    unsigned sh = 0, st = 0;
    if (sscanf(force, "%u,%u", &sh, &st) == 2 && sh >= 2 && sh <= 4 && st >= 2 && st <= kLinMaxStages) {
      const uint64_t need = (uint64_t)fixed + (4096u << sh) + (uint64_t)st * per_stage;
      if (need <= kMaxDynamicSmem) {
        g.lut_shift = sh;
        g.stages = st;
        g.smem_bytes = (uint32_t)need;
        return true;
      }
    }
  }
  static const uint32_t order[][2] = {{4, 3}, {3, 3}, {4, 2}, {3, 2}, {2, 3}, {2, 2}};
  for (const auto &o : order) {
    const uint64_t need = (uint64_t)fixed + (4096u << o[0]) + (uint64_t)o[1] * per_stage;
    if (need <= kMaxDynamicSmem) {
      g.lut_shift = o[0];
      g.stages = o[1];
      g.smem_bytes = (uint32_t)need;
      return true;
    }
  }
  return false;
}

}  // namespace nz

extern "C" uint32_t nz_operand_lane_symbols(uint64_t cols, int precision) {
  if (!nz::valid_precision(precision) || cols == 0 || cols % 64) return 0;
  const uint32_t spr = (uint32_t)(cols / 64);
  const uint32_t want = nz_default_lane_symbols(precision) / 8;
  // the divisor of cols / 64 closest (in ratio) to the default unit length, within a
  // factor of two of it and between 16 and 128 blocks
  uint32_t best = 0;
  double best_cost = 0;
  for (uint32_t beta = 16; beta <= 128 && beta <= spr; ++beta) {
    if (spr % beta) continue;
    const double ratio = beta > want ? (double)beta / want : (double)want / beta;
    if (ratio > 2.0) continue;
    if (!best || ratio < best_cost) {
      best = beta;
      best_cost = ratio;
    }
  }
  return best * 8;
}

extern "C" uint32_t nz_operand_lane_symbols_for(uint64_t rows, uint64_t cols, int precision) {
  if (rows == 0) return nz_operand_lane_symbols(cols, precision);
  if (!nz::valid_precision(precision) || cols == 0 || cols % 64 || rows % 4) return 0;
  // The fused linear has one work item per (128-row tile, unit-long column segment) and a
  // B200 runs one per SM at a time; an item costs its unit's blocks in decode steps plus
  // about six steps of set-up.  Take the unit length (16 to 48 blocks: shorter units cost
  // more than 1 % of the stored bytes, longer ones do not fit beside the operand tiles) with
  // the fewest steps in sequence, the longer one on a tie.
  constexpr uint64_t kSMs = 148, kSetupSteps = 6;
  const uint64_t spr = cols / 64, tiles = (rows + nz::kTileRows - 1) / nz::kTileRows;
  uint32_t best = 0;
  uint64_t best_cost = 0;
  for (uint32_t beta = 16; beta <= 48 && beta <= spr; ++beta) {
    if (spr % beta) continue;
    const uint64_t items = tiles * (spr / beta);
    const uint64_t cost = ((items + kSMs - 1) / kSMs) * (beta + kSetupSteps);
    if (!best || cost <= best_cost) {
      best = beta;
      best_cost = cost;
    }
  }
  return best ? best * 8 : nz_operand_lane_symbols(cols, precision);
}

extern "C" uint64_t nz_linear_workspace_bytes(uint64_t rows, uint64_t cols, uint32_t lane_symbols,
                                              uint64_t m_tokens) {
  const uint32_t segs = nz::operand_segments(cols, lane_symbols);
  if (segs <= 1) return 16;
  return nz::align16((uint64_t)segs * m_tokens * rows * 4);
}

static int linear_impl(const void *container, uint64_t container_bytes, const void *frac_in,
                       uint64_t rows, uint64_t cols, int precision, uint32_t lane_symbols,
                       uint32_t max_unit_words, int canonical_nan, const void *x_bf16,
                       uint64_t m_tokens, const void *bias_bf16, void *y_bf16, void *workspace,
                       uint64_t workspace_bytes, void *status, void *stream,
                       const nz_peer_group *peers, uint32_t arrivals_before, uint32_t *arrivals_after) {
  using namespace nz;
  const uint32_t world = peers ? peers->world : 1;
  if (peers) {
    if (world < 2 || world > kMaxPeers || peers->rank >= world) {
      set_error("nz_linear_allreduce_bf16: a peer group has 2 to %u ranks (got %u, rank %u)",
                kMaxPeers, world, peers->rank);
      return NZ_E_ARG;
    }
    for (uint32_t q = 0; q < world; ++q)
      if (!peers->workspace[q] || ((uintptr_t)peers->workspace[q] & 15) || !peers->arrivals[q]) {
        set_error("nz_linear_allreduce_bf16: null or misaligned peer pointer for rank %u", q);
        return NZ_E_ARG;
      }
    workspace = peers->workspace[peers->rank];
    workspace_bytes = peers->workspace_bytes;
  }
  if (!valid_precision(precision)) {
    set_error("nz_linear_bf16: precision must be 0, 1, 3 or 7 (got %d)", precision);
    return NZ_E_ARG;
  }
  const uint32_t segs = operand_segments(cols, lane_symbols);
  if (rows == 0 || rows % 4 || segs == 0 || rows * cols >= (1ull << 32)) {
    set_error("nz_linear_bf16: a [%llu, %llu] matrix with lane_symbols %u is not in operand order "
              "(rows must be a multiple of 4, columns of 64, lane_symbols / 8 must divide columns / 64)",
              (unsigned long long)rows, (unsigned long long)cols, lane_symbols);
    return NZ_E_ARG;
  }
  if (m_tokens == 0) return NZ_OK;
  if (m_tokens >= (1ull << 31)) {
    set_error("nz_linear_bf16: too many input rows");
    return NZ_E_ARG;
  }
  if (!container || ((uintptr_t)container & 15) || !frac_in || ((uintptr_t)frac_in & 7) ||
      !x_bf16 || ((uintptr_t)x_bf16 & 15) || !y_bf16 || ((uintptr_t)y_bf16 & 1) ||
      ((uintptr_t)bias_bf16 & 1)) {
    set_error("nz_linear_bf16: null or misaligned pointer (container and x 16-byte, fractions "
              "8-byte aligned)");
    return NZ_E_ARG;
  }
  const uint64_t n = rows * cols;
  const uint64_t nu = unit_count(n, lane_symbols);
  if (container_bytes < payload_offset(nu)) {
    set_error("nz_linear_bf16: container of %llu bytes is too short for %llu units",
              (unsigned long long)container_bytes, (unsigned long long)nu);
    return NZ_E_FORMAT;
  }
  if (segs > 1 || peers) {
    const uint64_t need = peers ? nz_linear_allreduce_workspace_bytes(rows, cols, lane_symbols,
                                                                      m_tokens, world)
                                : nz_linear_workspace_bytes(rows, cols, lane_symbols, m_tokens);
    if (peers && (rows + kTileRows - 1) / kTileRows > kTileCounterBytes / 4) {
      set_error("nz_linear_allreduce_bf16: more than %u row tiles", kTileCounterBytes / 4);
      return NZ_E_ARG;
    }
    if (!workspace || ((uintptr_t)workspace & 15) || workspace_bytes < need) {
      set_error("nz_linear_bf16: workspace of %llu bytes is smaller than the %llu required "
                "(or misaligned)", (unsigned long long)workspace_bytes, (unsigned long long)need);
      return NZ_E_CAPACITY;
    }
  }
  // tokens per launch: all of them up to 256, padded to the MMA's multiple of 16
  const uint32_t per_launch =
      (uint32_t)(m_tokens < kMaxTokensPerLaunch ? m_tokens : kMaxTokensPerLaunch);
  const uint32_t n_pad = (per_launch + 15u) & ~15u;
  LinearGeometry g;
  if (!linear_geometry(lane_symbols, max_unit_words, n_pad, g)) {
    set_error("nz_linear_bf16: units of lane_symbols %u do not fit in shared memory next to the "
              "operand tiles", lane_symbols);
    return NZ_E_CAPACITY;
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) {
    set_error("nz_linear_bf16: the driver does not provide cuTensorMapEncodeTiled");
    return NZ_E_CUDA;
  }
  CUtensorMap x_map;
  const cuuint64_t gdim[2] = {cols, m_tokens};
  const cuuint64_t gstride[1] = {cols * 2};
  const cuuint32_t box[2] = {64, n_pad};
  const cuuint32_t estride[2] = {1, 1};
  const CUresult cr = encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)x_bf16, gdim,
                             gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) {
    set_error("nz_linear_bf16: cuTensorMapEncodeTiled failed with code %d", (int)cr);
    return NZ_E_CUDA;
  }
  LinearArgs p;
  memset(&p, 0, sizeof(p));
  p.container = (const uint8_t *)container;
  p.container_bytes = container_bytes;
  p.frac = (const uint8_t *)frac_in;
  p.rows = (uint32_t)rows;
  p.cols = (uint32_t)cols;
  p.S = lane_symbols;
  p.n_units = (uint32_t)nu;
  p.segs = segs;
  p.slot_bytes = g.slot_bytes;
  p.lut_shift = g.lut_shift;
  p.lut_bytes = 4096u << g.lut_shift;
  p.stages = g.stages;
  p.n_pad = n_pad;
  p.m_total = (uint32_t)m_tokens;
  p.tmem_cols = 32;
  while (p.tmem_cols < n_pad) p.tmem_cols <<= 1;
  p.canon = canonical_nan;
  p.bias = (const uint16_t *)bias_bf16;
  p.y = (uint16_t *)y_bf16;
  p.partial = (float *)workspace;
  p.status = (uint32_t *)status;
  if (peers) {
    p.tp_world = world;
    p.tp_rank = peers->rank;
    for (uint32_t q = 0; q < world; ++q) {
      p.peer_partial[q] = (float *)((uint8_t *)peers->workspace[q] + kTileCounterBytes);
      p.peer_arrivals[q] = (uint32_t *)peers->arrivals[q];
    }
    // this rank's workspace: tile counters, the exchange planes, the segments' partial sums
    p.tile_counters = (uint32_t *)workspace;
    p.partial = p.peer_partial[peers->rank] + (uint64_t)world * m_tokens * rows;
  }

  void (*kern)(const LinearArgs, const CUtensorMap) = nullptr;
  switch (precision) {
    case 0: kern = linear_kernel<0>; break;
    case 1: kern = linear_kernel<1>; break;
    case 3: kern = linear_kernel<3>; break;
    default: kern = linear_kernel<7>; break;
  }
  {
    static std::mutex mu;
    static bool opted[4][kMaxDeviceOrdinals] = {};
    const int which = precision == 0 ? 0 : precision == 1 ? 1 : precision == 3 ? 2 : 3;
    int dev = 0;
    NZ_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= kMaxDeviceOrdinals || !opted[which][dev]) {
      NZ_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)kMaxDynamicSmem));
      if (dev >= 0 && dev < kMaxDeviceOrdinals) opted[which][dev] = true;
    }
  }
  cudaStream_t st = (cudaStream_t)stream;
  const uint32_t tiles = (uint32_t)((rows + kTileRows - 1) / kTileRows);
  uint32_t launches = 0;
  for (uint64_t tok0 = 0; tok0 < m_tokens; tok0 += per_launch) {
    ++launches;
    p.tok0 = (uint32_t)tok0;
    p.n_tok = (uint32_t)(m_tokens - tok0 < per_launch ? m_tokens - tok0 : per_launch);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * segs);
    cfg.blockDim = dim3(kLinThreads);
    cfg.dynamicSmemBytes = g.smem_bytes;
    cfg.stream = st;
    NZ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p, x_map));
  }
  if (peers) {
    // every row tile of every rank's launches adds one arrival per rank
    const uint32_t expected = arrivals_before + launches * tiles;
    if (arrivals_after) *arrivals_after = expected;
    const uint64_t plane = m_tokens * rows;
    const uint64_t blocks = (plane + 255) / 256;
    if (blocks >= (1ull << 31)) {
      set_error("nz_linear_allreduce_bf16: output too large for one call");
      return NZ_E_ARG;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NZ_CUDA_TRY(cudaLaunchKernelEx(&cfg, linear_allreduce_finish_kernel,
                                   (const float *)p.peer_partial[peers->rank],
                                   (const uint32_t *)peers->arrivals[peers->rank], expected, world,
                                   plane, (uint16_t *)y_bf16, (uint32_t *)status));
    return NZ_OK;
  }
  if (segs > 1) {
    const uint64_t plane = m_tokens * rows;
    const uint64_t blocks = (plane + 255) / 256;
    if (blocks >= (1ull << 31)) {
      set_error("nz_linear_bf16: output too large for one call");
      return NZ_E_ARG;
    }
    // the launch itself may overlap the tail of the kernel before it; the kernel waits
    // (griddepcontrol.wait) before it reads the partial sums
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NZ_CUDA_TRY(cudaLaunchKernelEx(&cfg, linear_finish_kernel, (const float *)workspace, segs, plane,
                                   (uint32_t)rows, (const uint16_t *)bias_bf16,
                                   (uint16_t *)y_bf16));
  }
  return NZ_OK;
}

extern "C" int nz_linear_bf16(const void *container, uint64_t container_bytes, const void *frac_in,
                              uint64_t rows, uint64_t cols, int precision, uint32_t lane_symbols,
                              uint32_t max_unit_words, int canonical_nan, const void *x_bf16,
                              uint64_t m_tokens, const void *bias_bf16, void *y_bf16,
                              void *workspace, uint64_t workspace_bytes, void *status,
                              void *stream) {
  return linear_impl(container, container_bytes, frac_in, rows, cols, precision, lane_symbols,
                     max_unit_words, canonical_nan, x_bf16, m_tokens, bias_bf16, y_bf16, workspace,
                     workspace_bytes, status, stream, nullptr, 0, nullptr);
}

extern "C" uint64_t nz_linear_allreduce_workspace_bytes(uint64_t rows, uint64_t cols,
                                                        uint32_t lane_symbols, uint64_t m_tokens,
                                                        uint32_t world) {
  const uint32_t segs = nz::operand_segments(cols, lane_symbols);
  if (segs == 0 || world < 2) return 0;
  return nz::kTileCounterBytes + nz::align16((uint64_t)(world + (segs > 1 ? segs : 0)) * m_tokens * rows * 4);
}

extern "C" int nz_linear_allreduce_bf16(const void *container, uint64_t container_bytes,
                                        const void *frac_in, uint64_t rows, uint64_t cols,
                                        int precision, uint32_t lane_symbols,
                                        uint32_t max_unit_words, int canonical_nan,
                                        const void *x_bf16, uint64_t m_tokens,
                                        const void *bias_bf16, void *y_bf16,
                                        const nz_peer_group *peers, uint32_t arrivals_before,
                                        uint32_t *arrivals_after, void *status, void *stream) {
  if (!peers) {
    nz::set_error("nz_linear_allreduce_bf16: null peer group");
    return NZ_E_ARG;
  }
  return linear_impl(container, container_bytes, frac_in, rows, cols, precision, lane_symbols,
                     max_unit_words, canonical_nan, x_bf16, m_tokens, bias_bf16, y_bf16, nullptr, 0,
                     status, stream, peers, arrivals_before, arrivals_after);
}
