// Warp-specialised, persistent sm_100a omni-attention forward kernel.
//
// One CTA per SM stays resident and works through a list of UNITS; a unit is a PAIR of adjacent 128-row
// Q tiles (tile A = rows 256j .., tile B = rows 256j + 128 ..) of one (batch, head). For a unit the CTA
// walks the union of the two tiles' KV block lists once, so every K/V tile staged in shared memory
// feeds up to two Q tiles. Roles (384 threads = 3 warpgroups):
//   warps 0-3    softmax group of tile A   (thread = one query row, TMEM lane = row)
//   warps 4-7    softmax group of tile B
//   warp  8      TMA producer: Q tiles of a unit, then K,V tiles through a ring of shared-memory stages
//   warp  9      MMA issuer: tcgen05.mma for S = Q K^T (smem x smem) and O += P V (TMEM x smem)
//   warp  10     idle (completes the third warpgroup, which hands its registers to the softmax groups
//                with setmaxnreg: 208 registers per softmax thread, 88 elsewhere)
//   warp  11     unit scheduler: takes the next unit (atomic counter in caller-provided scratch, or a
//                fixed boustrophedon assignment without scratch), resolves the block lists into
//                per-KV-block code tables and one ascending schedule, double buffered, one unit ahead
// A separate output warpgroup (a fourth group of 128 threads that reads O out of TMEM, normalises and
// stores while the softmax groups go on to the next unit) was built and measured: 0.555 ms against
// 0.537 ms on the 8K-token workload, because 512 threads leave the softmax groups 192 registers instead
// of 208 and put a third warp on every scheduler; the softmax groups therefore write the output themselves.
// TMEM (512 columns): S_A [0,128) S_B [128,256) O_A [256,256+D) O_B [256+D,256+2D). P (16-bit) is
// written over the first 64 columns of its S.
//
// Everything that is per-unit overhead in a one-unit-per-CTA kernel overlaps here with the
// neighbouring units: table building (scheduler warp), the Q/K/V loads of the next unit (the ring never
// drains; Q is reloaded as soon as the last S of the unit has been issued), and the first S MMAs of
// the next unit run while the softmax groups still normalise and store the previous output.
//
// Per tile the MMA order is PV(e), S(e+1), PV(e+1) ...; the two tiles' batches alternate in the
// tensor pipe, so while one tile's softmax runs on the CUDA cores the pipe works on the other tile.
// An S tile becomes visible to its softmax group through an mbarrier armed by tcgen05.commit, which
// also implies that every earlier MMA (in particular the previous P*V of the same tile) has
// finished; that is what lets the softmax group itself rescale O in TMEM on the rare occasions when
// the (lazily moved) running maximum moves.
//
// Block types: FULL tiles take a path with no mask arithmetic; CAUSAL (diagonal) and PARTIAL tiles
// build four 32-bit allow words per row (PARTIAL: one 16-byte load of the bit-packed row, or eight
// for the reference's byte-per-element format) before the scores arrive; blocks that are not listed
// are never loaded. Lists in 64x64 blocks (B64) are walked as they are: a 128x128 tile is then a 2x2
// of sub-blocks with a code each, and a row's allow words are put together from its two sub-blocks.
// head_dim 32 runs as 64 with the upper 32 columns of Q, K and V read as zeros by the TMA unit.
// The behaviour replaced is the reference's KV loop
// (omni-attn-mma/mma/omni_attn_shared_kv.cu:148-559) and epilogue (:560-646).
//
// Barrier phases are counted per barrier by both sides over the events that really happen (units
// that load Q, units in which a tile has work), never derived from the unit number: an empty unit
// completes nothing, so it cannot make a phase slip past a waiter.
#include <type_traits>

#include "omni_common.cuh"
#include "omni_launch.h"

namespace omni {

// Header of a unit-table slot. The slot holds, in this order: the two code tables (tile A, tile B;
// one word per KV block, four with lists in 64-blocks), the schedule (KV blocks visited by either
// tile, ascending, 16-bit: block | kSchedA | kSchedB) and this header.
struct UnitHeader {
  int n_sched;   // entries in the schedule; -1 = no more units
  int cnt[2];    // blocks visited by tile A / tile B
  int bh;        // batch * H + head
  int pair;      // tile A = 128-row tile 2 * pair, tile B = 2 * pair + 1
  int pad[3];
};
static_assert(sizeof(UnitHeader) == 32, "slot layout");

struct UnitSlot {
  uint32_t* tab[2];
  uint16_t* sched;
  UnitHeader* hdr;
};

__host__ __device__ constexpr int ws_words_per_block(bool b64) { return b64 ? 4 : 1; }
__host__ __device__ inline int ws_slot_bytes(int nq, bool b64) {
  const int tab = nq * ws_words_per_block(b64) * 4;
  const int sched = nq * 2;
  return (2 * tab + sched + 15) / 16 * 16 + static_cast<int>(sizeof(UnitHeader));   // a multiple of 16
}

template <int D>
struct WsCfg {
  static constexpr int kTileBytes = kBlock * D * 2;
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = kBlock * 128;
  static constexpr int kStages = (D == 128) ? 4 : 8;  // ring entries, each one K or one V tile
  static constexpr int kTmemCols = 512;
  // Softmax shape, chosen by measurement (8K-token workload for D=128, 4K-token one for D=64):
  //  * D=128: two passes over S in TMEM (row maximum over the whole row, then exponentials 64 columns at
  //    a time), so that the scores and the packed P are never live together and nothing spills.
  //  * D=64: one pass with the whole row in registers, a quarter of the exponentials evaluated by a
  //    polynomial on the FMA pipe (the MMAs are half as long, MUFU is the scarcer unit).
  static constexpr bool kTwoPass = (D == 128);
  static constexpr int kPolyNum = (D == 128) ? 0 : 1;   // element pairs per group of kPolyDen on the FMA pipe
  static constexpr int kPolyDen = (D == 128) ? 1 : 4;
  // q_full[2] q_free ring_full[S] ring_empty[S] s_full[2] p_ready[2] done[2] o_free[2] tab_full[2]
  // tab_empty[2] near_end drained
  static constexpr int kNumBars = 3 + 2 * kStages + 13 + 1;
  static constexpr int kBarBytes = (8 * kNumBars + 64 + 15) & ~15;   // barriers + a few control words; the table slots
                                                                     // behind them stay 16-byte aligned
  static constexpr int kFixedBytes = (2 + kStages) * kTileBytes + kBarBytes + 1024;   // + alignment slack
};

constexpr int kWsThreads = 384;
// Register split made with setmaxnreg. The kernel is compiled for 168 registers per thread (the most
// 384 threads can have); the increase of the two softmax warpgroups must be covered by the decrease
// of the third one, or setmaxnreg.inc waits forever.
constexpr int kLaunchRegs = 168;
constexpr int kSoftmaxRegs = 208;   // warps 0-7
constexpr int kOtherRegs = 88;      // warps 8-11
static_assert(2 * kSoftmaxRegs + kOtherRegs <= 3 * kLaunchRegs, "setmaxnreg split exceeds the launch allocation");
static_assert(kSoftmaxRegs % 8 == 0 && kOtherRegs % 8 == 0, "setmaxnreg counts are multiples of 8");

// A schedule entry: KV block (128 keys) in the low bits, and which of the two tiles visit it.
constexpr int kSchedBlockMask = 0x3FFF;
constexpr int kSchedA = 0x4000;
constexpr int kSchedB = 0x8000;
static_assert(kMaxKvBlocks <= kSchedBlockMask + 1, "schedule entries are 16 bits");

constexpr float kLazyRescaleLog2 = 8.f;
// The scheduler warp takes the next unit only when the producer is this many KV blocks from the end
// of the current one: early enough for the next unit's tables to be ready before the loads run dry,
// late enough that a CTA does not sit on a unit while other CTAs have already run out of work
// (measured: 4 against 12 is 5 % on the 4 K-token workload, 0.5 % on the 8 K one; 2 and 6 are the same).
constexpr int kNearEndBlocks = 4;
// Cycle budget of the waits a CTA that gives up makes for its own copies and MMAs in flight.
constexpr long long kDrainCycles = 20000000LL;

// Unit index -> (batch*head, Q pair). The order is chosen for two things at once.
//  * The first quarter of the Q pairs (for causal-like masks: the shortest lists) of ALL heads comes
//    last, so that the tail of the grid is filled with short units; everything else comes first.
//  * Inside the first band, heads are taken in groups of `group_heads` (sized on the host so that
//    the K and V of one group fit in L2 together); inside a group the Q pairs run from last to first
//    with the group's heads adjacent, so that long units start early and CTAs working at the same
//    time keep re-reading the same few heads' K/V. The last band does the same with groups four
//    times as large (all heads at once when they fit).
__device__ __forceinline__ void decode_unit(const FwdParams& p, int unit, int npairs, int& bh, int& pair) {
  const int light = npairs / 4;                 // pairs [0, light) form the last band
  const int heavy = npairs - light;
  int top, pairs_here, rem;
  if (unit < heavy * p.BH) {
    top = npairs - 1;
    pairs_here = heavy;
    rem = unit;
  } else {
    top = light - 1;
    pairs_here = light;
    rem = unit - heavy * p.BH;
  }
  // The last band touches only the first quarter of every head's K/V, so four times as many heads
  // fit in L2 together; the wider its groups, the closer its order is to "descending over all heads",
  // which is what leaves the smallest units for the very end.
  const int G = unit < heavy * p.BH ? p.group_heads : min(p.BH, 4 * p.group_heads);
  const int grp = rem / (pairs_here * G);
  rem -= grp * pairs_here * G;
  const int heads_here = min(G, p.BH - grp * G);
  pair = top - rem / heads_here;
  bh = grp * G + rem % heads_here;
}

template <int D, bool BF16, bool SOFTCAP, bool B64>
__global__ void __launch_bounds__(kWsThreads, 1)
omni_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using Cfg = WsCfg<D>;
  // The swizzled tiles need 1024-byte alignment: the launch asks for 1 KB more than the layout takes and
  // the base is rounded up here. (Declaring the array 1024-byte aligned instead, which saves the spare
  // kilobyte, was measured 8 % slower on the 8K-token workload with an otherwise identical kernel.)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  // ---- shared memory carve-up ----------------------------------------------------------------
  const uint32_t sQ0 = smem_u32(smem);                          // Q tile A, then Q tile B
  const uint32_t sRing = sQ0 + 2 * Cfg::kTileBytes;             // kStages K/V tiles
  uint8_t* after_tiles = smem + (2 + Cfg::kStages) * Cfg::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(after_tiles);
  const uint32_t bar_q = smem_u32(bars + 0);                    // [2] Q tile landed
  const uint32_t bar_qfree = smem_u32(bars + 2);                // every S of the unit has been issued and is done
  const uint32_t bar_full = smem_u32(bars + 3);                 // [kStages] ring entry landed
  const uint32_t bar_empty = bar_full + 8 * Cfg::kStages;       // [kStages] ring entry consumed
  const uint32_t bar_s = bar_empty + 8 * Cfg::kStages;          // [2] S tile complete
  const uint32_t bar_p = bar_s + 16;                            // [2] P tile written (128 arrivals)
  const uint32_t bar_done = bar_p + 16;                         // [2] all MMAs of the tile in this unit complete
  const uint32_t bar_ofree = bar_done + 16;                     // [2] O of the unit read out of TMEM (128 arrivals)
  const uint32_t bar_tfull = bar_ofree + 16;                    // [2] unit table written
  const uint32_t bar_tempty = bar_tfull + 16;                   // [2] unit table no longer needed (10 arrivals)
  const uint32_t bar_near = bar_tempty + 16;                    // the producer is within a few blocks of the unit's end
  const uint32_t bar_drain = bar_near + 8;                      // every MMA issued by this CTA has retired
  int* misc = reinterpret_cast<int*>(bars + Cfg::kNumBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 0);
  volatile int* abort_flag = misc + 1;
  uint8_t* slot_base = after_tiles + Cfg::kBarBytes;
  const int slot_bytes = ws_slot_bytes(p.nq, B64);
  auto slot = [&](int k) -> UnitSlot {
    uint8_t* b = slot_base + (k & 1) * slot_bytes;
    const int tab_words = p.nq * ws_words_per_block(B64);
    UnitSlot s;
    s.tab[0] = reinterpret_cast<uint32_t*>(b);
    s.tab[1] = s.tab[0] + tab_words;
    s.sched = reinterpret_cast<uint16_t*>(s.tab[1] + tab_words);
    s.hdr = reinterpret_cast<UnitHeader*>(b + slot_bytes - sizeof(UnitHeader));
    return s;
  };

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int npairs = (p.nq + 1) >> 1;
  const long long wait_lim = p.wait_cycles;

  // ---- one-time set-up: barriers, tables, TMEM ---------------------------------------------------
  if (tid == 256) {
    mbar_init(bar_q, 1);
    mbar_init(bar_q + 8, 1);
    mbar_init(bar_qfree, 1);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(bar_s + 8 * g, 1);
      mbar_init(bar_p + 8 * g, 128);
      mbar_init(bar_done + 8 * g, 1);
      mbar_init(bar_ofree + 8 * g, 128);
      mbar_init(bar_tfull + 8 * g, 1);
      mbar_init(bar_tempty + 8 * g, 10);
    }
    mbar_init(bar_near, 1);
    mbar_init(bar_drain, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  // Both table slots start out as "no unit, nothing listed": a role that falls through a wait while
  // the CTA is giving up then finds a slot that ends its loop, never stale or unwritten entries.
  for (int i = tid; i < 2 * slot_bytes / 4; i += kWsThreads) reinterpret_cast<uint32_t*>(slot_base)[i] = 0u;
  __syncthreads();
  if (tid < 2) slot(tid).hdr->n_sched = -1;
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr int fmt = BF16 ? 1 : 0;
  constexpr uint32_t idesc_qk = umma_idesc_f16(128, 128, fmt, 0);
  constexpr uint32_t idesc_pv = umma_idesc_f16(128, D, fmt, 1);

  // Every consumer of the unit tables runs the same outer loop: wait for table k, stop on the
  // sentinel, work, hand the table slot back.
  auto wait_table = [&](int k, int where) -> UnitSlot {
    mbar_wait_lim(bar_tfull + 8 * (k & 1), (k >> 1) & 1, abort_flag, p.status, where, wait_lim);
    return slot(k);
  };
  if (warp < 8) {
    // =========================== softmax groups =================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int g = warp >> 2;                       // 0 = tile A, 1 = tile B
    const int r = tid & 127;                       // row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + 128 * g + lane_base;
    const uint32_t tO = tmem_base + 256 + D * g + lane_base;
    const uint32_t my_bar_s = bar_s + 8 * g;
    const uint32_t my_bar_p = bar_p + 8 * g;
    int n_tiles = 0;   // S tiles consumed so far over all units = phase count of the S and P barriers
    int n_units = 0;   // units in which this tile had work = phase count of its done barrier

    for (int k = 0;; ++k) {
      const UnitSlot T = wait_table(k, 10 + g);
      const int n_sched = T.hdr->n_sched;
      if (n_sched < 0) break;
      const uint32_t tab = smem_u32(T.tab[g]);
      const uint32_t sched = smem_u32(T.sched);
      const int my_cnt = T.hdr->cnt[g];
      const int unit_bh = T.hdr->bh, unit_pair = T.hdr->pair;

      RowState st{-INFINITY, 0.f};
      int cnt = 0;
      for (int e = 0; e < n_sched && cnt < my_cnt; ++e) {
        const int entry = lds_u16(sched + 2 * e);
        if ((entry & (g == 0 ? kSchedA : kSchedB)) == 0) continue;
        const int kvb = entry & kSchedBlockMask;
        uint32_t allow[4];
        const bool masked = tile_row_allow<B64>(p, tab, kvb, r, allow) == 2;

        mbar_wait_lim(my_bar_s, n_tiles & 1, abort_flag, p.status, 12 + g, wait_lim);
        tc_fence_after();

        if constexpr (Cfg::kTwoPass) {
        // pass 1: row maximum over the whole row (the scores are dropped again right away; with a
        // soft-cap the capped scores go back to TMEM first, so that pass 2 finds them there)
        float mx;
        {
          float s[128];
          load_scores(tS, s);
          if constexpr (SOFTCAP) {
            soft_cap_scores(s, p.cap_in, p.cap_out);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t rr[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) rr[j] = __float_as_uint(s[32 * c + j]);
              tmem_st32(tS + 32 * c, rr);
            }
          }
          if (masked) apply_allow(allow, s);
          mx = row_max(s);
          if constexpr (SOFTCAP) tc_wait_st();
        }
        const float alpha = softmax_update(st, mx, p.scale_log2, kLazyRescaleLog2);
        if (cnt > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.f)) rescale_o<D>(tO, alpha);
        // pass 2: exponentials; P half h (32 words) lands on columns that were read in pass 2 already
        float sum = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float s[64];
          load_scores64(tS + 64 * h, s);
          if (masked) apply_allow64(allow[2 * h], allow[2 * h + 1], s);
          uint32_t pk[32];
          sum += exp_and_pack_n<BF16, Cfg::kPolyNum, Cfg::kPolyDen>(s, st.M, p.scale_log2, p.inv_scale_log2, pk);
          tmem_st32(tS + 32 * h, pk);
        }
        st.l = st.l * alpha + sum;
        } else {
        // one pass with the whole row in registers
        float s[128];
        load_scores(tS, s);
        if constexpr (SOFTCAP) soft_cap_scores(s, p.cap_in, p.cap_out);
        if (masked) apply_allow(allow, s);
        const float alpha = softmax_update(st, row_max(s), p.scale_log2, kLazyRescaleLog2);
        if (cnt > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.f)) rescale_o<D>(tO, alpha);
        uint32_t pk[64];
        const float sum = exp_and_pack_n<BF16, Cfg::kPolyNum, Cfg::kPolyDen>(s, st.M, p.scale_log2, p.inv_scale_log2, pk);
        st.l = st.l * alpha + sum;
        store_p(tS, pk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(my_bar_p);
        ++cnt;
        ++n_tiles;
      }

      {
        // ---- output of the unit by the softmax group itself: O out of TMEM chunk by chunk, normalise,
        // store; O is handed back to the MMA issuer as soon as the last chunk has been read ----------
        if (my_cnt > 0) {
          mbar_wait_lim(bar_done + 8 * g, n_units & 1, abort_flag, p.status, 14 + g, wait_lim);
          tc_fence_after();
          ++n_units;
        }
        const int q_abs = (2 * unit_pair + g) * kBlock + r;
        const bool have_row = q_abs < p.N;
        const bool empty = my_cnt == 0 || q_abs >= p.seqlen_orig || st.M == -INFINITY || !(st.l > 0.f);
        const float inv = empty ? 0.f : 1.f / st.l;
        const long long row = static_cast<long long>(unit_bh) * p.N + q_abs;
        char* dst = static_cast<char*>(p.o) + row * (p.d_real * 2);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t rr[32];
          if (my_cnt > 0) {   // uniform over the group
            tmem_ld32(tO + 32 * c, rr);
            tc_wait_ld();
            if (c == D / 32 - 1) {
              tc_fence_before();
              mbar_arrive(bar_ofree + 8 * g);   // the next unit may overwrite O now
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) rr[j] = 0u;
          }
          if (have_row && 32 * c < p.d_real) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {   // 16 elements = 32 bytes = one full sector per store
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float a = empty ? 0.f : __uint_as_float(rr[16 * h + 2 * j]) * inv;
                const float b = empty ? 0.f : __uint_as_float(rr[16 * h + 2 * j + 1]) * inv;
                w[j] = pack2<BF16>(a, b);
              }
              char* d32 = dst + 64 * c + 32 * h;
              if (p.o_aligned32) {
                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(d32), "r"(w[0]), "r"(w[1]),
                             "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                             : "memory");
              } else {
                reinterpret_cast<uint4*>(d32)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                reinterpret_cast<uint4*>(d32)[1] = make_uint4(w[4], w[5], w[6], w[7]);
              }
            }
          }
        }
        if (have_row && p.lse != nullptr) {
          p.lse[row] = empty ? -INFINITY : fmaf(st.M, 0.6931471805599453f, __logf(st.l));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * (k & 1));
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
    if (warp == 8) {
      // =========================== TMA producer ===================================================
      if (lane == 0) {
        int fill = 0;              // ring entries filled so far, over all units
        int n_qunits = 0;          // units whose Q tiles were loaded = phase count of the Q-free barrier
        int n_qloads[2] = {0, 0};  // Q tile loads issued per tile
        for (int k = 0;; ++k) {
          const UnitSlot T = wait_table(k, 20);
          const int n_sched = T.hdr->n_sched;
          if (n_sched < 0) break;
          const int bh = T.hdr->bh;
          const int qbA = 2 * T.hdr->pair;
          if (*abort_flag) break;   // giving up: issue no further copies
          if (n_sched > 0) {
            // Q buffers are free once every S of the previous unit that used them is done.
            if (n_qunits > 0 && !mbar_wait_lim(bar_qfree, (n_qunits - 1) & 1, abort_flag, p.status, 21, wait_lim)) break;
            ++n_qunits;
            for (int g = 0; g < 2; ++g) {
              if (T.hdr->cnt[g] > 0) {
                mbar_expect_tx(bar_q + 8 * g, Cfg::kTileBytes);
                ++n_qloads[g];
#pragma unroll
                for (int c = 0; c < Cfg::kChunks; ++c) {
                  tma_load_3d(sQ0 + g * Cfg::kTileBytes + c * Cfg::kChunkBytes, &tmQ, bar_q + 8 * g, c * 64,
                              (qbA + g) * kBlock, bh);
                }
              }
            }
          }
          const int near_at = n_sched > kNearEndBlocks ? n_sched - kNearEndBlocks : 0;
          if (n_sched == 0) mbar_arrive(bar_near);
          bool alive = true;
          for (int e = 0; e < n_sched && alive; ++e) {
            if (e == near_at) mbar_arrive(bar_near);
            const int y = (static_cast<int>(T.sched[e]) & kSchedBlockMask) * kBlock;
#pragma unroll
            for (int kv = 0; kv < 2; ++kv, ++fill) {
              const int s = fill % Cfg::kStages;
              if (fill >= Cfg::kStages &&
                  !mbar_wait_lim(bar_empty + 8 * s, ((fill / Cfg::kStages) - 1) & 1, abort_flag, p.status, 22, wait_lim)) {
                alive = false;
                break;
              }
              const uint32_t dst = sRing + s * Cfg::kTileBytes;
              const uint32_t full = bar_full + 8 * s;
              mbar_expect_tx(full, Cfg::kTileBytes);
#pragma unroll
              for (int c = 0; c < Cfg::kChunks; ++c) {
                tma_load_3d(dst + c * Cfg::kChunkBytes, kv == 0 ? &tmK : &tmV, full, c * 64, y, bh);
              }
            }
          }
          if (!alive) break;
          mbar_arrive(bar_tempty + 8 * (k & 1));
        }
        if (*abort_flag) {
          // The CTA is giving up: wait, with a budget of its own, for every copy this thread issued,
          // so that nothing is still being written into shared memory when the CTA exits.
          for (int s = 0; s < Cfg::kStages && s < fill; ++s) {
            const int last = ((fill - 1 - s) / Cfg::kStages) * Cfg::kStages + s;   // last fill that used entry s
            mbar_wait_drain(bar_full + 8 * s, (last / Cfg::kStages) & 1, kDrainCycles);
          }
          for (int g = 0; g < 2; ++g) {
            if (n_qloads[g] > 0) mbar_wait_drain(bar_q + 8 * g, (n_qloads[g] - 1) & 1, kDrainCycles);
          }
        }
      }
    } else if (warp == 9) {
      // =========================== MMA issuer =====================================================
      // One thread feeds the tensor pipe, and it shares its scheduler with two softmax warps: every
      // instruction it does not need is pipe time. Descriptors are advanced as 32-bit low words (the
      // high word is one constant), accumulate flags are compile-time constants, what a schedule entry
      // means for the two tiles is in the entry itself, and a look ahead at a barrier is a
      // non-blocking test.
      if (lane == 0) {
        const uint32_t tS[2] = {tmem_base, tmem_base + 128};
        const uint32_t tO[2] = {tmem_base + 256, tmem_base + 256 + D};
        constexpr uint32_t desc_hi = umma_desc_hi_sw128(1024);
        const uint32_t k_lo0 = umma_desc_lo(sRing, 16);                 // K-major view of ring entry 0
        const uint32_t v_lo0 = umma_desc_lo(sRing, Cfg::kChunkBytes);   // MN-major view (V)
        const uint32_t q_lo[2] = {umma_desc_lo(sQ0, 16), umma_desc_lo(sQ0 + Cfg::kTileBytes, 16)};
        constexpr uint32_t kSlotStep = Cfg::kTileBytes >> 4;
        constexpr uint32_t kChunkStep = Cfg::kChunkBytes >> 4;
        uint32_t fbase = 0;             // ring index of K(0) of the current unit
        uint32_t n_p[2] = {0, 0};       // P tiles consumed so far over all units = phase count of the P barriers
        uint32_t n_q[2] = {0, 0};       // Q tile loads consumed so far
        uint32_t n_units[2] = {0, 0};   // units in which the tile had work = phase count of its done / O-free barriers
        bool issued_any = false;
        bool alive = true;              // false once a wait has given up: issue no further MMAs

        for (int k = 0;; ++k) {
          mbar_wait_lim(bar_tfull + 8 * (k & 1), (k >> 1) & 1, abort_flag, p.status, 30, wait_lim);
          const UnitSlot T = slot(k);
          const int n_sched = T.hdr->n_sched;
          if (n_sched < 0 || !alive) break;
          const int cnt_g[2] = {T.hdr->cnt[0], T.hdr->cnt[1]};
          const uint32_t sched = smem_u32(T.sched);
          bool q_ready[2] = {false, false};
          int n_pv[2] = {0, 0};    // P*V batches issued in this unit

          auto full_bar = [&](uint32_t f) { return bar_full + 8 * ((fbase + f) % Cfg::kStages); };
          auto full_par = [&](uint32_t f) { return ((fbase + f) / Cfg::kStages) & 1u; };
          auto wait_full = [&](uint32_t f) {
            alive &= mbar_wait_lim(full_bar(f), full_par(f), abort_flag, p.status, 31, wait_lim);
          };
          auto release = [&](uint32_t f) { tc_commit(bar_empty + 8 * ((fbase + f) % Cfg::kStages)); };
          // The tile index is a compile-time constant (std::integral_constant argument) so that the
          // per-tile state arrays are indexed statically and stay in registers.
          auto issue_s = [&](auto gc, uint32_t e, auto&& peek) {   // S_g = Q_g * K(e)^T
            constexpr int g = decltype(gc)::value;
            if (!q_ready[g]) {
              alive &= mbar_wait_lim(bar_q + 8 * g, n_q[g] & 1, abort_flag, p.status, 32, wait_lim);
              tc_fence_after();
              q_ready[g] = true;
              ++n_q[g];
            }
            const uint32_t kd = k_lo0 + ((fbase + 2 * e) % Cfg::kStages) * kSlotStep;
            const uint32_t qd = q_lo[g];
            const uint32_t d_tmem = tS[g];
            // 16 head-dim columns per step: 32 bytes inside a 64-column chunk, chunks kChunkBytes apart
            umma_ss_lo<false>(d_tmem, qd, kd, desc_hi, idesc_qk);
#pragma unroll
            for (int ks = 1; ks < D / 16; ++ks) {
              const uint32_t off = (ks / 4) * kChunkStep + (ks % 4) * 2;
              umma_ss_lo<true>(d_tmem, qd + off, kd + off, desc_hi, idesc_qk);
              if (ks == D / 16 - 4) peek();
            }
            tc_commit(bar_s + 8 * g);
          };
          auto issue_pv = [&](auto gc, uint32_t e, bool p_ready) {  // O_g += P_g * V(e)
            constexpr int g = decltype(gc)::value;
            // 16 keys per step = 16 rows of 128 bytes = 2048 bytes; P advances 8 TMEM columns
            const uint32_t vd = v_lo0 + ((fbase + 2 * e + 1) % Cfg::kStages) * kSlotStep;
            const uint32_t a_tmem = tS[g];
            const uint32_t d_tmem = tO[g];
            if (n_pv[g] == 0 && n_units[g] > 0) {
              // first write to O_g in this unit: whoever writes the output must have read out the previous one
              alive &= mbar_wait_lim(bar_ofree + 8 * g, (n_units[g] - 1) & 1, abort_flag, p.status, 33, wait_lim);
            }
            if (!p_ready) alive &= mbar_wait_lim(bar_p + 8 * g, n_p[g] & 1, abort_flag, p.status, 34 + g, wait_lim);
            tc_fence_after();
            umma_ts_lo(d_tmem, a_tmem, vd, desc_hi, idesc_pv, n_pv[g] > 0 ? 1u : 0u);
#pragma unroll
            for (int ks = 1; ks < kBlock / 16; ++ks) {
              umma_ts_lo_acc(d_tmem, a_tmem + 8 * ks, vd + ks * 128, desc_hi, idesc_pv);
            }
            ++n_pv[g];
            ++n_p[g];
            // last P*V of this tile in the unit: O may be read as soon as these MMAs retire, without
            // waiting for the other tile
            if (n_pv[g] == cnt_g[g]) {
              tc_commit(bar_done + 8 * g);
              ++n_units[g];
            }
          };
          auto no_peek = [] {};
          constexpr std::integral_constant<int, 0> tile_a{};
          constexpr std::integral_constant<int, 1> tile_b{};

          if (n_sched > 0) {
            issued_any = true;
            uint32_t cur = lds_u16(sched);
            {  // prologue: scores of the first visited block
              wait_full(0);
              tc_fence_after();
              if (cur & kSchedA) issue_s(tile_a, 0, no_peek);
              if (cur & kSchedB) issue_s(tile_b, 0, no_peek);
              release(0);
              if (n_sched == 1) tc_commit(bar_qfree);
            }
            bool ring_ok = false;   // V(e) and K(e+1) already seen complete
            bool pa_ok = false;     // P_A(e) already seen complete
            const uint32_t n = static_cast<uint32_t>(n_sched);
            for (uint32_t e = 0; e < n; ++e) {
              if (!alive) break;
              const bool has_next = e + 1 < n;
              const uint32_t nxt = has_next ? lds_u16(sched + 2 * (e + 1)) : 0u;
              const bool use_a = (cur & kSchedA) != 0, use_b = (cur & kSchedB) != 0;
              const bool next_a = (nxt & kSchedA) != 0, next_b = (nxt & kSchedB) != 0;
              if (!ring_ok) {
                wait_full(2 * e + 1);                 // V(e)
                if (has_next) wait_full(2 * e + 2);   // K(e+1)
              }
              tc_fence_after();
              bool pb_ok = false;
              if (use_a) issue_pv(tile_a, e, pa_ok);
              if (next_a) {
                issue_s(tile_a, e + 1, [&] { if (use_b) pb_ok = mbar_test_wait(bar_p + 8, n_p[1] & 1) != 0; });
              }
              if (use_b) issue_pv(tile_b, e, pb_ok);
              ring_ok = false;
              pa_ok = false;
              if (next_b) {
                issue_s(tile_b, e + 1, [&] {
                  bool ok = mbar_test_wait(full_bar(2 * e + 3), full_par(2 * e + 3)) != 0;                  // V(e+1)
                  if (e + 2 < n) ok = (mbar_test_wait(full_bar(2 * e + 4), full_par(2 * e + 4)) != 0) && ok; // K(e+2)
                  ring_ok = ok;
                  if (next_a) pa_ok = mbar_test_wait(bar_p, n_p[0] & 1) != 0;
                });
              }
              if (e + 2 == n) tc_commit(bar_qfree);   // the last S of the unit has been issued
              release(2 * e + 1);
              if (has_next) release(2 * e + 2);
              cur = nxt;
            }
          }
          if (!alive) break;
          fbase += 2 * static_cast<uint32_t>(n_sched);
          mbar_arrive(bar_tempty + 8 * (k & 1));
        }
        // Keep this thread (and with it the CTA's shared memory and TMEM) alive until every MMA it
        // issued has retired, whatever the other roles do (this wait has a budget of its own).
        if (issued_any) {
          tc_commit(bar_drain);
          if (!mbar_wait_drain(bar_drain, 0, *abort_flag ? kDrainCycles : wait_lim) && p.status != nullptr) {
            atomicExch(p.status, kStatusWaitTimeout | (36 << 8));
          }
        }
      }
    } else if (warp == 11) {
      // =========================== unit scheduler =================================================
      const int grid = static_cast<int>(gridDim.x);
      for (int k = 0;; ++k) {
        const UnitSlot T = slot(k);
        if (k >= 2) {
          if (lane == 0) {
            mbar_wait_lim(bar_tempty + 8 * (k & 1), ((k >> 1) - 1) & 1, abort_flag, p.status, 40, wait_lim);
          }
          __syncwarp();
        }
        int unit = 0;
        if (lane == 0) {
          if (k >= 1) mbar_wait_lim(bar_near, (k - 1) & 1, abort_flag, p.status, 41, wait_lim);
          if (*abort_flag) {
            unit = p.num_units;   // stop handing out work once a wait has timed out in this CTA
          } else if (p.unit_counter != nullptr) {
            unit = k == 0 ? static_cast<int>(blockIdx.x) : grid + atomicAdd(p.unit_counter, 1);
          } else {
            // no scratch: round k of a fixed assignment that reverses direction every round, which
            // evens out a list sorted from long to short
            unit = k * grid + ((k & 1) ? grid - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x));
          }
        }
        unit = __shfl_sync(0xFFFFFFFFu, unit, 0);
        if (unit >= p.num_units) {
          if (lane == 0) {
            T.hdr->n_sched = -1;
            mbar_arrive(bar_tfull + 8 * (k & 1));
          }
          break;
        }
        int bh, pair;
        decode_unit(p, unit, npairs, bh, pair);
        const int tab_words = p.nq * ws_words_per_block(B64);
        for (int i = lane; i < 2 * tab_words; i += 32) T.tab[0][i] = 0u;   // tile A's table, then tile B's
        __syncwarp();
        build_tile_table<B64>(p, bh, 2 * pair, T.tab[0]);
        build_tile_table<B64>(p, bh, 2 * pair + 1, T.tab[1]);
        __syncwarp();
        int n = 0, ca = 0, cb = 0;   // compact the visited KV blocks into an ascending list
        for (int base = 0; base < p.nq; base += 32) {
          const int kvb = base + lane;
          bool a = false, b = false;
          if (kvb < p.nq) {
            a = tile_visits<B64>(smem_u32(T.tab[0]), kvb);
            b = tile_visits<B64>(smem_u32(T.tab[1]), kvb);
          }
          const uint32_t any = __ballot_sync(0xFFFFFFFFu, a || b);
          ca += __popc(__ballot_sync(0xFFFFFFFFu, a));
          cb += __popc(__ballot_sync(0xFFFFFFFFu, b));
          if (a || b) {
            T.sched[n + __popc(any & ((1u << lane) - 1u))] =
                static_cast<uint16_t>(kvb | (a ? kSchedA : 0) | (b ? kSchedB : 0));
          }
          n += __popc(any);
        }
        if (lane == 0) {
          T.hdr->n_sched = n;
          T.hdr->cnt[0] = ca;
          T.hdr->cnt[1] = cb;
          T.hdr->bh = bh;
          T.hdr->pair = pair;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tfull + 8 * (k & 1));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// Dynamic shared memory of one CTA for sequences of nq 128-row tiles.
template <int D>
static int ws_smem_bytes(int nq, bool b64) {
  return WsCfg<D>::kFixedBytes + 2 * ws_slot_bytes(nq, b64);
}

constexpr int kMaxSmemPerCta = 232448;   // 227 KB, the most one CTA can have on sm_100

template <int D, bool BF16, bool SOFTCAP, bool B64>
static cudaError_t launch_ws_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                               FwdParams p, cudaStream_t stream) {
  auto kern = omni_fwd_ws_kernel<D, BF16, SOFTCAP, B64>;
  const int smem = ws_smem_bytes<D>(p.nq, B64);
  if (smem > kMaxSmemPerCta) return cudaErrorInvalidValue;   // the C-ABI layer refuses such lengths first
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  // Per-device facts, looked up once (any host thread may be the first).
  struct PerDevice {
    std::once_flag once;
    cudaError_t err = cudaSuccess;
    int num_sms = 0;
  };
  static PerDevice per_device[kMaxDevices];
  PerDevice& pd = per_device[dev];
  std::call_once(pd.once, [&] {
    pd.err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemPerCta);
    if (pd.err != cudaSuccess) return;
    // The setmaxnreg split inside the kernel is only safe if the kernel was really compiled for
    // kLaunchRegs registers per thread (an unsatisfiable increase would wait forever).
    cudaFuncAttributes fa;
    pd.err = cudaFuncGetAttributes(&fa, kern);
    if (pd.err != cudaSuccess) return;
    if (2 * kSoftmaxRegs + kOtherRegs > 3 * fa.numRegs) {
      pd.err = cudaErrorLaunchOutOfResources;
      return;
    }
    pd.err = cudaDeviceGetAttribute(&pd.num_sms, cudaDevAttrMultiProcessorCount, dev);
  });
  if (pd.err != cudaSuccess) return pd.err;
  const int npairs = (p.nq + 1) / 2;
  const long long units = static_cast<long long>(npairs) * p.BH;
  p.num_units = static_cast<int>(units);
  const int grid = static_cast<int>(units < pd.num_sms ? units : pd.num_sms);
  if (p.unit_counter != nullptr) {
    e = cudaMemsetAsync(p.unit_counter, 0, sizeof(int32_t), stream);
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, kWsThreads, smem, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError();
}

template <int D, bool BF16>
static cudaError_t launch_ws_d(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                               const FwdParams& p, cudaStream_t stream) {
  const bool cap = p.cap_out != 0.f;
  if (p.blk64) {
    return cap ? launch_ws_t<D, BF16, true, true>(tmQ, tmK, tmV, p, stream)
               : launch_ws_t<D, BF16, false, true>(tmQ, tmK, tmV, p, stream);
  }
  return cap ? launch_ws_t<D, BF16, true, false>(tmQ, tmK, tmV, p, stream)
             : launch_ws_t<D, BF16, false, false>(tmQ, tmK, tmV, p, stream);
}

// Longest sequence (in 128-row tiles) whose unit tables still fit beside the tiles in shared memory.
int ws_max_tiles(int head_dim, bool b64) {
  const int fixed = head_dim == 128 ? WsCfg<128>::kFixedBytes : WsCfg<64>::kFixedBytes;
  int nq = kMaxKvBlocks;
  while (nq > 0 && fixed + 2 * ws_slot_bytes(nq, b64) > kMaxSmemPerCta) nq -= 8;
  return nq;
}

// head_dim is the width the kernel computes with: 64 (also for tensors of head_dim 32) or 128.
cudaError_t launch_ws(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                      const CUtensorMap& tmV, const FwdParams& p, cudaStream_t stream) {
  if (head_dim == 64) {
    return bf16 ? launch_ws_d<64, true>(tmQ, tmK, tmV, p, stream) : launch_ws_d<64, false>(tmQ, tmK, tmV, p, stream);
  }
  return bf16 ? launch_ws_d<128, true>(tmQ, tmK, tmV, p, stream) : launch_ws_d<128, false>(tmQ, tmK, tmV, p, stream);
}

}  // namespace omni
