// Warp-specialised, persistent sm_100a omni-attention forward kernel.
//
// One CTA per SM stays resident and works through a list of UNITS; a unit is a PAIR of adjacent 128-row
// Q tiles (tile A = rows 256j .., tile B = rows 256j + 128 ..) of one (batch, head). For a unit the CTA
// walks the union of the two tiles' KV block lists once, so every K/V tile staged in shared memory
// feeds up to two Q tiles. Roles (512 threads = 4 warpgroups):
//   warps 0-3    softmax group of tile A   (thread = one query row, TMEM lane = row)
//   warps 4-7    softmax group of tile B
//   warp  8      TMA producer: Q tiles of a unit, then K,V tiles through a ring of shared-memory stages
//   warp  9      MMA issuer: tcgen05.mma for S = Q K^T (smem x smem) and O += P V (TMEM x smem)
//   warp  10     idle
//   warp  11     unit scheduler: takes the next unit (atomic counter in caller-provided scratch, or a
//                fixed boustrophedon assignment without scratch), resolves the block lists into
//                per-KV-block code tables and one ascending schedule, double buffered, one unit ahead
//   warps 12-15  output group: when a tile's last P*V of a unit has retired it reads O out of TMEM,
//                normalises, casts and stores it (and the log-sum-exp), while the softmax groups are
//                already at work on the next unit
// setmaxnreg moves registers from warps 8-15 to the softmax groups.
// TMEM (512 columns): S_A [0,128) S_B [128,256) O_A [256,256+D) O_B [256+D,256+2D). P (16-bit) is
// written over the first 64 columns of its S.
//
// Everything that is per-unit overhead in a one-unit-per-CTA kernel overlaps here with the
// neighbouring units: table building (scheduler warp), the Q/K/V loads of the next unit (the ring never
// drains; Q is reloaded as soon as the last S of the unit has been issued), the output of the previous
// unit (output group).
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
// tile, ascending, 16-bit) and this header.
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
#ifdef OMNI_WS_TWOPASS64
  static constexpr bool kTwoPass = true;
#else
  static constexpr bool kTwoPass = (D == 128);
#endif
#ifdef OMNI_WS_POLY_NUM128
  static constexpr int kPolyNum = (D == 128) ? OMNI_WS_POLY_NUM128 : 1;
  static constexpr int kPolyDen = (D == 128) ? OMNI_WS_POLY_DEN128 : 4;
#else
  static constexpr int kPolyNum = (D == 128) ? 0 : 1;   // element pairs per group of kPolyDen on the FMA pipe
  static constexpr int kPolyDen = (D == 128) ? 1 : 4;
#endif
  // q_full[2] q_free ring_full[S] ring_empty[S] s_full[2] p_ready[2] done[2] o_free[2] tab_full[2]
  // tab_empty[2] near_end row_state[2] row_state_free[2] drained
  static constexpr int kNumBars = 3 + 2 * kStages + 13 + 5;
  static constexpr int kRowStateBytes = 2 * kBlock * 8;   // (M, l) of every row of the two tiles
  static constexpr int kBarBytes = (8 * kNumBars + 64 + 15) & ~15;   // barriers + a few control words; the table slots
                                                                     // behind them stay 16-byte aligned
  static constexpr int kFixedBytes = (2 + kStages) * kTileBytes + kRowStateBytes + kBarBytes;
};

constexpr int kWsThreads = 512;
// Register split made with setmaxnreg. The kernel is compiled for 128 registers per thread (the most
// 512 threads can have); the increase of the two softmax warpgroups must be covered by the decrease
// of the other two, or setmaxnreg.inc waits forever.
constexpr int kLaunchRegs = 128;
#ifndef OMNI_WS_REGS128_S
#define OMNI_WS_REGS128_S 192
#define OMNI_WS_REGS128_R 88
#endif
#ifndef OMNI_WS_REGS64_S
#define OMNI_WS_REGS64_S 208
#define OMNI_WS_REGS64_R 64
#endif
template <int D>
struct WsRegs {
  static constexpr int kSoftmax = D == 128 ? OMNI_WS_REGS128_S : OMNI_WS_REGS64_S;   // warps 0-7
  static constexpr int kRole = D == 128 ? OMNI_WS_REGS128_R : OMNI_WS_REGS64_R;      // warps 8-11
  static constexpr int kOutput = 4 * kLaunchRegs - 2 * kSoftmax - kRole;              // warps 12-15
  static_assert(kSoftmax % 8 == 0 && kRole % 8 == 0 && kOutput % 8 == 0 && kRole >= 24 && kOutput >= 24,
                "setmaxnreg counts are multiples of 8, at least 24, and add up to the launch allocation");
};

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
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {   // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kStatusWaitTimeout | (1 << 8));
    return;
  }

  // ---- shared memory carve-up ----------------------------------------------------------------
  const uint32_t sQ0 = smem_u32(smem);                          // Q tile A, then Q tile B
  const uint32_t sRing = sQ0 + 2 * Cfg::kTileBytes;             // kStages K/V tiles
  uint8_t* after_tiles = smem + (2 + Cfg::kStages) * Cfg::kTileBytes;
  float2* row_state = reinterpret_cast<float2*>(after_tiles);   // [2][128] (M, l) handed to the output group
  uint64_t* bars = reinterpret_cast<uint64_t*>(after_tiles + Cfg::kRowStateBytes);
  const uint32_t bar_q = smem_u32(bars + 0);                    // [2] Q tile landed
  const uint32_t bar_qfree = smem_u32(bars + 2);                // every S of the unit has been issued and is done
  const uint32_t bar_full = smem_u32(bars + 3);                 // [kStages] ring entry landed
  const uint32_t bar_empty = bar_full + 8 * Cfg::kStages;       // [kStages] ring entry consumed
  const uint32_t bar_s = bar_empty + 8 * Cfg::kStages;          // [2] S tile complete
  const uint32_t bar_p = bar_s + 16;                            // [2] P tile written (128 arrivals)
  const uint32_t bar_done = bar_p + 16;                         // [2] all MMAs of the tile in this unit complete
  const uint32_t bar_ofree = bar_done + 16;                     // [2] O of the unit read out of TMEM (128 arrivals)
  const uint32_t bar_tfull = bar_ofree + 16;                    // [2] unit table written
  const uint32_t bar_tempty = bar_tfull + 16;                   // [2] unit table no longer needed (14 arrivals)
  const uint32_t bar_near = bar_tempty + 16;                    // the producer is within a few blocks of the unit's end
  const uint32_t bar_rs = bar_near + 8;                         // [2] row states of the tile written (128 arrivals)
  const uint32_t bar_rsfree = bar_rs + 16;                      // [2] row states read (128 arrivals)
  const uint32_t bar_drain = bar_rsfree + 16;                   // every MMA issued by this CTA has retired
  int* misc = reinterpret_cast<int*>(bars + Cfg::kNumBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 0);
  volatile int* abort_flag = misc + 1;
  uint8_t* slot_base = after_tiles + Cfg::kRowStateBytes + Cfg::kBarBytes;
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
      mbar_init(bar_tempty + 8 * g, 14);
      mbar_init(bar_rs + 8 * g, 128);
      mbar_init(bar_rsfree + 8 * g, 128);
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
  // Warp-collective form for the 128-thread groups: one lane polls (32 lanes polling the same
  // mbarrier cost shared-memory bandwidth that the tensor pipe's operand reads need).
  auto wait_warp = [&](uint32_t bar, uint32_t parity, int where) {
    if (lane == 0) mbar_wait_lim(bar, parity, abort_flag, p.status, where, wait_lim);
    __syncwarp();
  };

  if (warp < 8) {
    // =========================== softmax groups =================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(WsRegs<D>::kSoftmax));
    const int g = warp >> 2;                       // 0 = tile A, 1 = tile B
    const int r = tid & 127;                       // row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + 128 * g + lane_base;
    const uint32_t tO = tmem_base + 256 + D * g + lane_base;
    const uint32_t my_bar_s = bar_s + 8 * g;
    const uint32_t my_bar_p = bar_p + 8 * g;
    int n_tiles = 0;   // S tiles consumed so far over all units = phase count of the S and P barriers
    int n_units = 0;   // units in which this tile had work = phase count of the row-state barriers

    for (int k = 0;; ++k) {
      const UnitSlot T = wait_table(k, 10 + g);
      const int n_sched = T.hdr->n_sched;
      if (n_sched < 0) break;
      const uint32_t* tab = T.tab[g];
      const int my_cnt = T.hdr->cnt[g];

      RowState st{-INFINITY, 0.f};
      int cnt = 0;
      for (int e = 0; e < n_sched && cnt < my_cnt; ++e) {
        const int kvb = T.sched[e];
        uint32_t allow[4];
        const int kind = tile_row_allow<B64>(p, tab, kvb, r, allow);
        if (kind == 0) continue;
        const bool masked = kind == 2;

        wait_warp(my_bar_s, n_tiles & 1, 12 + g);
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

      // ---- hand the row's softmax state to the output group and go on to the next unit -----------
      if (my_cnt > 0) {
        if (n_units > 0) wait_warp(bar_rsfree + 8 * g, (n_units - 1) & 1, 14 + g);
        row_state[g * kBlock + r] = make_float2(st.M, st.l);
        mbar_arrive(bar_rs + 8 * g);
        ++n_units;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * (k & 1));
    }
  } else if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WsRegs<D>::kOutput));
    {
      // =========================== output group ===================================================
      const int r = tid & 127;
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      int n_units[2] = {0, 0};   // units in which the tile had work = phase count of its done / row-state barriers
      for (int k = 0;; ++k) {
        const UnitSlot T = wait_table(k, 50);
        if (T.hdr->n_sched < 0) break;
        const int bh = T.hdr->bh;
        const int pair = T.hdr->pair;
        const int cnt_g[2] = {T.hdr->cnt[0], T.hdr->cnt[1]};
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * (k & 1));   // everything needed from the table is in registers
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const int q_abs = (2 * pair + g) * kBlock + r;
          const bool have_row = q_abs < p.N;
          const bool have_acc = cnt_g[g] > 0;
          float2 ml = make_float2(-INFINITY, 0.f);
          if (have_acc) {
            const uint32_t ph = n_units[g] & 1;
            wait_warp(bar_rs + 8 * g, ph, 51 + g);
            ml = row_state[g * kBlock + r];
            mbar_arrive(bar_rsfree + 8 * g);
            wait_warp(bar_done + 8 * g, ph, 53 + g);
            tc_fence_after();
            ++n_units[g];
          }
          const bool empty = !have_acc || q_abs >= p.seqlen_orig || ml.x == -INFINITY || !(ml.y > 0.f);
          const float inv = empty ? 0.f : 1.f / ml.y;
          const long long row = static_cast<long long>(bh) * p.N + q_abs;
          char* dst = static_cast<char*>(p.o) + row * (p.d_real * 2);
          const uint32_t tO = tmem_base + 256 + D * g + lane_base;
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            uint32_t rr[16];
            if (have_acc) {   // uniform over the group
              tmem_ld16(tO + 16 * c, rr);
              tc_wait_ld();
              if (c == D / 16 - 1) {
                tc_fence_before();
                mbar_arrive(bar_ofree + 8 * g);   // the next unit may overwrite O now
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) rr[j] = 0u;
            }
            if (have_row && 16 * c < p.d_real) {   // 16 elements = 32 bytes = one full sector per store
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float a = empty ? 0.f : __uint_as_float(rr[2 * j]) * inv;
                const float b = empty ? 0.f : __uint_as_float(rr[2 * j + 1]) * inv;
                w[j] = pack2<BF16>(a, b);
              }
              char* d32 = dst + 32 * c;
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
          if (have_row && p.lse != nullptr) {
            p.lse[row] = empty ? -INFINITY : fmaf(ml.x, 0.6931471805599453f, __logf(ml.y));
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WsRegs<D>::kRole));
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
            const int y = static_cast<int>(T.sched[e]) * kBlock;
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
      if (lane == 0) {
        const uint32_t tS[2] = {tmem_base, tmem_base + 128};
        const uint32_t tO[2] = {tmem_base + 256, tmem_base + 256 + D};
        // UMMA descriptors: "base + constant" in the start-address field (16-byte units).
        const uint64_t k_desc0 = umma_smem_desc_sw128(sRing, 16, 1024);                 // K-major view of a ring slot
        const uint64_t v_desc0 = umma_smem_desc_sw128(sRing, Cfg::kChunkBytes, 1024);   // MN-major view (V)
        constexpr uint32_t kSlotStep = Cfg::kTileBytes >> 4;
        constexpr uint32_t kChunkStep = Cfg::kChunkBytes >> 4;
        const uint64_t q_desc[2] = {umma_smem_desc_sw128(sQ0, 16, 1024),
                                    umma_smem_desc_sw128(sQ0 + Cfg::kTileBytes, 16, 1024)};
        int fbase = 0;             // ring index of K(0) of the current unit
        int n_p[2] = {0, 0};       // P tiles consumed so far over all units = phase count of the P barriers
        int n_q[2] = {0, 0};       // Q tile loads consumed so far
        int n_units[2] = {0, 0};   // units in which the tile had work = phase count of its done / O-free barriers
        bool issued_any = false;
        bool alive = true;         // false once a wait has given up: issue no further MMAs

        for (int k = 0;; ++k) {
          const UnitSlot T = wait_table(k, 30);
          const int n_sched = T.hdr->n_sched;
          if (n_sched < 0 || !alive) break;
          const int cnt_g[2] = {T.hdr->cnt[0], T.hdr->cnt[1]};
          const uint32_t* tabA = T.tab[0];
          const uint32_t* tabB = T.tab[1];
          bool q_ready[2] = {false, false};
          int n_pv[2] = {0, 0};    // P*V batches issued in this unit

          auto slot_of = [&](int f) { return static_cast<uint32_t>((fbase + f) % Cfg::kStages); };
          auto wait_full = [&](int f) {
            alive &= mbar_wait_lim(bar_full + 8 * ((fbase + f) % Cfg::kStages), ((fbase + f) / Cfg::kStages) & 1,
                                   abort_flag, p.status, 31, wait_lim);
          };
          auto peek_full = [&](int f) -> bool {
            return mbar_try_wait(bar_full + 8 * ((fbase + f) % Cfg::kStages), ((fbase + f) / Cfg::kStages) & 1) != 0;
          };
          auto release = [&](int f) { tc_commit(bar_empty + 8 * ((fbase + f) % Cfg::kStages)); };
          // The tensor pipe accepts a tcgen05.mma only about as fast as it executes them, so this
          // thread is busy for the whole execution time of a batch and every cycle it then spends
          // finding out whether the next batch may start is a cycle the pipe idles. Polls for the
          // NEXT batch are therefore started in the middle of the current one (`peek`, non-blocking)
          // and only fall back to a blocking wait when they failed.
          // The tile index is a compile-time constant (std::integral_constant argument) so that the
          // per-tile state arrays are indexed statically and stay in registers.
          auto issue_s = [&](auto gc, int e, auto&& peek) {   // S_g = Q_g * K(e)^T
            constexpr int g = decltype(gc)::value;
            if (!q_ready[g]) {
              alive &= mbar_wait_lim(bar_q + 8 * g, n_q[g] & 1, abort_flag, p.status, 32, wait_lim);
              tc_fence_after();
              q_ready[g] = true;
              ++n_q[g];
            }
            const uint64_t kd = k_desc0 + slot_of(2 * e) * kSlotStep;
            const uint64_t qd = q_desc[g];
            const uint32_t d_tmem = tS[g];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              // 16 head-dim columns per step: 32 bytes inside a 64-column chunk, chunks kChunkBytes apart
              const uint32_t off = (ks / 4) * kChunkStep + (ks % 4) * 2;
              umma_ss(d_tmem, qd + off, kd + off, idesc_qk, ks > 0 ? 1u : 0u);
              if (ks == D / 16 - 4) peek();
            }
            tc_commit(bar_s + 8 * g);
          };
          auto issue_pv = [&](auto gc, int e, bool p_ready) {  // O_g += P_g * V(e)
            constexpr int g = decltype(gc)::value;
            // 16 keys per step = 16 rows of 128 bytes = 2048 bytes; P advances 8 TMEM columns
            const uint64_t vd = v_desc0 + slot_of(2 * e + 1) * kSlotStep;
            const uint32_t a_tmem = tS[g];
            const uint32_t d_tmem = tO[g];
            const uint32_t first = n_pv[g] > 0 ? 1u : 0u;
            if (n_pv[g] == 0 && n_units[g] > 0) {
              // first write to O_g in this unit: the output group must have read out the previous one
              alive &= mbar_wait_lim(bar_ofree + 8 * g, (n_units[g] - 1) & 1, abort_flag, p.status, 33, wait_lim);
            }
            if (!p_ready) alive &= mbar_wait_lim(bar_p + 8 * g, n_p[g] & 1, abort_flag, p.status, 34 + g, wait_lim);
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < kBlock / 16; ++ks) {
              umma_ts(d_tmem, a_tmem + 8 * ks, vd + ks * 128, idesc_pv, ks > 0 ? 1u : first);
            }
            ++n_pv[g];
            ++n_p[g];
            // last P*V of this tile in the unit: the output group may read O as soon as these MMAs
            // retire, without waiting for the other tile
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
            {  // prologue: scores of the first visited block
              const int kvb = T.sched[0];
              wait_full(0);
              tc_fence_after();
              if (tile_visits<B64>(tabA, kvb)) issue_s(tile_a, 0, no_peek);
              if (tile_visits<B64>(tabB, kvb)) issue_s(tile_b, 0, no_peek);
              release(0);
              if (n_sched == 1) tc_commit(bar_qfree);
            }
            bool ring_ok = false;   // V(e) and K(e+1) already seen complete
            bool pa_ok = false;     // P_A(e) already seen complete
            for (int e = 0; e < n_sched; ++e) {
              if (!alive) break;
              const int kvb = T.sched[e];
              const bool has_next = e + 1 < n_sched;
              const int kvb_next = has_next ? T.sched[e + 1] : 0;
              const bool use_a = tile_visits<B64>(tabA, kvb), use_b = tile_visits<B64>(tabB, kvb);
              const bool next_a = has_next && tile_visits<B64>(tabA, kvb_next);
              const bool next_b = has_next && tile_visits<B64>(tabB, kvb_next);
              if (!ring_ok) {
                wait_full(2 * e + 1);                 // V(e)
                if (has_next) wait_full(2 * e + 2);   // K(e+1)
              }
              tc_fence_after();
              bool pb_ok = false;
              if (use_a) issue_pv(tile_a, e, pa_ok);
              if (next_a) {
                issue_s(tile_a, e + 1, [&] { if (use_b) pb_ok = mbar_try_wait(bar_p + 8, n_p[1] & 1) != 0; });
              }
              if (use_b) issue_pv(tile_b, e, pb_ok);
              ring_ok = false;
              pa_ok = false;
              if (next_b) {
                issue_s(tile_b, e + 1, [&] {
                  bool ok = peek_full(2 * e + 3);                       // V(e+1)
                  if (e + 2 < n_sched) ok = peek_full(2 * e + 4) && ok; // K(e+2)
                  ring_ok = ok;
                  if (next_a) pa_ok = mbar_try_wait(bar_p, n_p[0] & 1) != 0;
                });
              }
              if (e + 2 == n_sched) tc_commit(bar_qfree);   // the last S of the unit has been issued
              release(2 * e + 1);
              if (has_next) release(2 * e + 2);
            }
          }
          if (!alive) break;
          fbase += 2 * n_sched;
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
            a = tile_visits<B64>(T.tab[0], kvb);
            b = tile_visits<B64>(T.tab[1], kvb);
          }
          const uint32_t any = __ballot_sync(0xFFFFFFFFu, a || b);
          ca += __popc(__ballot_sync(0xFFFFFFFFu, a));
          cb += __popc(__ballot_sync(0xFFFFFFFFu, b));
          if (a || b) T.sched[n + __popc(any & ((1u << lane) - 1u))] = static_cast<uint16_t>(kvb);
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
    if (2 * WsRegs<D>::kSoftmax + WsRegs<D>::kRole + WsRegs<D>::kOutput > 4 * fa.numRegs) {
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
