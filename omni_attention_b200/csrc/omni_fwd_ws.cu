// Warp-specialised, persistent sm_100a omni-attention forward kernel.
//
// One CTA per SM stays resident and works through a list of UNITS; a unit is a PAIR of adjacent Q
// blocks (tile A = block 2j, tile B = block 2j+1) of one (batch, head). For a unit the CTA walks the
// union of the two KV block lists once, so every K/V tile staged in shared memory feeds up to two Q
// tiles. Roles (384 threads = 3 warpgroups):
//   warps 0-3  softmax group of tile A   (thread = one query row, TMEM lane = row)
//   warps 4-7  softmax group of tile B
//   warp  8    TMA producer: Q tiles of a unit, then K,V tiles through a ring of shared-memory stages
//   warp  9    MMA issuer: tcgen05.mma for S = Q K^T (smem x smem) and O += P V (TMEM x smem)
//   warp  10   idle (completes the third warpgroup, which hands its registers to the softmax groups
//              with setmaxnreg: 208 registers per softmax thread, 88 elsewhere)
//   warp  11   unit scheduler: takes the next unit (atomic counter in caller-provided scratch, or a
//              fixed boustrophedon assignment without scratch), resolves its two block lists into
//              per-KV-block code tables and one ascending schedule, double buffered, one unit ahead
// TMEM (512 columns): S_A [0,128) S_B [128,256) O_A [256,256+D) O_B [256+D,256+2D). P (16-bit) is
// written over the first 64 columns of its S.
//
// Everything that is per-unit overhead in a one-unit-per-CTA kernel overlaps here with the
// previous unit: table building (scheduler warp), the Q/K/V loads of the next unit (the ring never
// drains; Q is reloaded as soon as the last S of the unit has been issued), and the first S MMAs of
// the next unit run while the softmax groups still normalise and store the previous output.
//
// Per tile the MMA order is PV(e), S(e+1), PV(e+1) ...; the two tiles' batches alternate in the
// tensor pipe, so while one tile's softmax runs on the CUDA cores the pipe works on the other tile.
// An S tile becomes visible to its softmax group through an mbarrier armed by tcgen05.commit, which
// also implies that every earlier MMA (in particular the previous P*V of the same tile) has
// finished; that is what lets the softmax group itself rescale O in TMEM when the running maximum
// moves, without a separate correction group.
//
// Block types: FULL tiles take a path with no mask arithmetic; CAUSAL (diagonal) and PARTIAL tiles
// build four 32-bit allow words per row (PARTIAL: one 16-byte load of the bit-packed row, or eight
// for the reference's byte-per-element format) before the scores arrive; blocks that are not listed
// are never loaded. The behaviour replaced is the reference's KV loop
// (omni-attn-mma/mma/omni_attn_shared_kv.cu:148-559) and epilogue (:560-646).
#include <type_traits>

#include "omni_common.cuh"
#include "omni_launch.h"

namespace omni {

// Per-unit block tables, built by the scheduler warp, read by every other role.
struct UnitTable {
  uint32_t tabA[kMaxKvBlocks];   // resolved entry code per KV block for tile A (0 = not visited)
  uint32_t tabB[kMaxKvBlocks];
  uint16_t sched[kMaxKvBlocks];  // KV blocks visited by either tile, ascending
  int n_sched;                   // entries in sched; -1 = no more units
  int cnt[2];                    // blocks visited by tile A / tile B
  int bh;                        // batch * H + head
  int pair;                      // Q block pair index: tile A = 2 * pair, tile B = 2 * pair + 1
  int pad[3];
};

template <int D>
struct WsCfg {
  static constexpr int kTileBytes = kBlock * D * 2;
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = kBlock * 128;
  static constexpr int kStages = (D == 128) ? 4 : 8;  // ring entries, each one K or one V tile
  static constexpr int kTmemCols = 512;
  // Softmax shape, chosen by measurement (C4 for D=128, C3 for D=64):
  //  * D=128: two passes over S in TMEM (row maximum over the whole row, then exponentials 64 columns at
  //    a time), so that the scores and the packed P are never live together and nothing spills; all exponentials on the MUFU unit (any share
  //    moved to the FMA pipe slows the MMA-issuing thread more than it saves).
  //  * D=64: one pass with the whole row in registers, a quarter of the exponentials evaluated by a
  //    polynomial on the FMA pipe (the MMAs are half as long, MUFU is the scarcer unit).
  static constexpr bool kTwoPass = (D == 128);
  static constexpr int kPolyNum = (D == 128) ? 0 : 1;   // element pairs per group of kPolyDen on the FMA pipe
  static constexpr int kPolyDen = (D == 128) ? 1 : 4;
  // q_full[2] q_free ring_full[S] ring_empty[S] s_full[2] p_ready[2] done[2] o_free[2] tab_full[2] tab_empty[2] near_end
  static constexpr int kNumBars = 3 + 2 * kStages + 13;
  static constexpr int kTableBytes = 2 * static_cast<int>(sizeof(UnitTable));
  static constexpr int kSmemBytes = (2 + kStages) * kTileBytes + kTableBytes + 8 * kNumBars + 64 + 1024;
};
static_assert(sizeof(UnitTable) % 16 == 0, "table slots stay aligned");

constexpr int kWsThreads = 384;
// Register split made with setmaxnreg. The kernel is compiled for 168 registers per thread (the most
// 384 threads can have); the increase of the two softmax warpgroups must be covered by the decrease
// of the third one, or setmaxnreg.inc waits forever.
constexpr int kLaunchRegs = 168;
constexpr int kSoftmaxRegs = 208;
constexpr int kOtherRegs = 88;
static_assert(2 * kSoftmaxRegs + kOtherRegs <= 3 * kLaunchRegs, "setmaxnreg split exceeds the launch allocation");
static_assert(kSoftmaxRegs % 8 == 0 && kOtherRegs % 8 == 0, "setmaxnreg counts are multiples of 8");

constexpr float kLazyRescaleLog2 = 8.f;
// The scheduler warp takes the next unit only when the producer is this many KV blocks from the end
// of the current one: early enough for the next unit's tables to be ready before the loads run dry,
// late enough that a CTA does not sit on a unit while other CTAs have already run out of work
// (measured: 4 against 12 is 5 % on the 4 K-token workload, 0.5 % on the 8 K one; 2 and 6 are the same).
constexpr int kNearEndBlocks = 4;
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

template <int D, bool BF16, bool SOFTCAP>
__global__ void __launch_bounds__(kWsThreads, 1)
omni_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using Cfg = WsCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);

  // ---- shared memory carve-up ----------------------------------------------------------------
  const uint32_t sQ0 = smem_u32(smem);                          // Q tile A, then Q tile B
  const uint32_t sRing = sQ0 + 2 * Cfg::kTileBytes;             // kStages K/V tiles
  uint8_t* after_tiles = smem + (2 + Cfg::kStages) * Cfg::kTileBytes;
  UnitTable* tables = reinterpret_cast<UnitTable*>(after_tiles);   // [2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(after_tiles + Cfg::kTableBytes);
  const uint32_t bar_q = smem_u32(bars + 0);                    // [2] Q tile landed
  const uint32_t bar_qfree = smem_u32(bars + 2);                // every S of the unit has been issued and is done
  const uint32_t bar_full = smem_u32(bars + 3);                 // [kStages] ring entry landed
  const uint32_t bar_empty = bar_full + 8 * Cfg::kStages;       // [kStages] ring entry consumed
  const uint32_t bar_s = bar_empty + 8 * Cfg::kStages;          // [2] S tile complete
  const uint32_t bar_p = bar_s + 16;                            // [2] P tile written (128 arrivals)
  const uint32_t bar_done = bar_p + 16;                         // [2] all MMAs of the unit complete
  const uint32_t bar_ofree = bar_done + 16;                     // [2] O of the unit read out of TMEM (128 arrivals)
  const uint32_t bar_tfull = bar_ofree + 16;                    // [2] unit table written
  const uint32_t bar_tempty = bar_tfull + 16;                   // [2] unit table no longer needed (10 arrivals)
  const uint32_t bar_near = bar_tempty + 16;                    // the producer is within a few blocks of the unit's end
  int* misc = reinterpret_cast<int*>(bars + Cfg::kNumBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 0);
  volatile int* abort_flag = misc + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int npairs = (p.nq + 1) >> 1;

  // ---- one-time set-up: barriers, TMEM -----------------------------------------------------------
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
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
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
  auto wait_table = [&](int k, int where) -> const UnitTable* {
    mbar_wait(bar_tfull + 8 * (k & 1), (k >> 1) & 1, abort_flag, p.status, where);
    return tables + (k & 1);
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

#ifdef OMNI_PROFILE_CTA
    auto gtime = [] { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return (long long)t; };
#define OMNI_USTAMP(i) if (tid == 0 && p.status != nullptr && k < 16) reinterpret_cast<long long*>(p.status + 4)[(blockIdx.x * 16 + k) * 8 + (i)] = gtime()
#else
#define OMNI_USTAMP(i)
#endif
    for (int k = 0;; ++k) {
      OMNI_USTAMP(0);
      const UnitTable* T = wait_table(k, 10 + g);
      const int n_sched = T->n_sched;
      if (n_sched < 0) break;
      OMNI_USTAMP(1);
#ifdef OMNI_PROFILE_CTA
      if (tid == 0 && p.status != nullptr && k < 16) reinterpret_cast<long long*>(p.status + 4)[(blockIdx.x * 16 + k) * 8 + 7] = T->cnt[0] + T->cnt[1];
#endif
      const uint32_t* tab = g == 0 ? T->tabA : T->tabB;
      const int my_cnt = T->cnt[g];
      const int qb = 2 * T->pair + g;
      const long long row0 = static_cast<long long>(T->bh) * p.N;

      RowState st{-INFINITY, 0.f};
      int cnt = 0;
      for (int e = 0; e < n_sched && cnt < my_cnt; ++e) {
        const int kvb = T->sched[e];
        const uint32_t code = tab[kvb];
        if (code == 0u) continue;
        const bool masked = (code & kCodeTypeMask) != kTypeFull || (code & kCodeClip);
        uint32_t allow[4];
        if (masked) build_allow(p, code, kvb, r, allow);

        mbar_wait(my_bar_s, n_tiles & 1, abort_flag, p.status, 12 + g);
        tc_fence_after();
        if (cnt == 0) { OMNI_USTAMP(2); }

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
              uint32_t r[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(s[32 * c + j]);
              tmem_st32(tS + 32 * c, r);
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
          sum += exp_and_pack64<BF16, Cfg::kPolyNum, Cfg::kPolyDen>(s, st.M, p.scale_log2, p.inv_scale_log2, pk);
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
        const float sum = exp_and_pack<BF16, Cfg::kPolyNum, Cfg::kPolyDen>(s, st.M, p.scale_log2, p.inv_scale_log2, pk);
        st.l = st.l * alpha + sum;
        store_p(tS, pk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(my_bar_p);
        ++cnt;
        ++n_tiles;
      }

      // ---- epilogue of the unit: O out of TMEM chunk by chunk, normalise, store; O is handed back
      // to the MMA issuer as soon as the last chunk has been read ----------------------------------
      OMNI_USTAMP(3);
      if (my_cnt > 0) {
        mbar_wait(bar_done + 8 * g, k & 1, abort_flag, p.status, 14 + g);
        tc_fence_after();
      }
      OMNI_USTAMP(4);
      const int q_abs = qb * kBlock + r;
      const bool have_row = qb < p.nq;
      const bool empty = my_cnt == 0 || q_abs >= p.seqlen_orig || st.M == -INFINITY || !(st.l > 0.f);
      const float inv = empty ? 0.f : 1.f / st.l;
      const long long row = row0 + q_abs;
      char* dst = static_cast<char*>(p.o) + row * (D * 2);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rr[32];
        if (my_cnt > 0) {   // uniform over the group
          tmem_ld32(tO + 32 * c, rr);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) rr[j] = 0u;
        }
        if (c == D / 32 - 1) {
          tc_fence_before();
          mbar_arrive(bar_ofree + 8 * g);   // the next unit may overwrite O now
        }
        if (have_row) {
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
      OMNI_USTAMP(5);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * (k & 1));
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
    if (warp == 8) {
      // =========================== TMA producer ===================================================
      if (lane == 0) {
        int fill = 0;              // ring entries filled so far, over all units
        for (int k = 0;; ++k) {
          const UnitTable* T = wait_table(k, 20);
          const int n_sched = T->n_sched;
          if (n_sched < 0) break;
          const long long row0 = static_cast<long long>(T->bh) * p.N;
          const int qbA = 2 * T->pair;
          // Q buffers are free once every S of the previous unit is done.
          if (k > 0) mbar_wait(bar_qfree, (k - 1) & 1, abort_flag, p.status, 21);
          for (int g = 0; g < 2; ++g) {
            if (T->cnt[g] > 0) {
              mbar_expect_tx(bar_q + 8 * g, Cfg::kTileBytes);
#pragma unroll
              for (int c = 0; c < Cfg::kChunks; ++c) {
                tma_load_2d(sQ0 + g * Cfg::kTileBytes + c * Cfg::kChunkBytes, &tmQ, bar_q + 8 * g, c * 64,
                            static_cast<int>(row0 + (qbA + g) * kBlock));
              }
            }
          }
          const int near_at = n_sched > kNearEndBlocks ? n_sched - kNearEndBlocks : 0;
          if (n_sched == 0) mbar_arrive(bar_near);
          for (int e = 0; e < n_sched; ++e) {
            if (e == near_at) mbar_arrive(bar_near);
            const int y = static_cast<int>(row0 + static_cast<int>(T->sched[e]) * kBlock);
#pragma unroll
            for (int kv = 0; kv < 2; ++kv, ++fill) {
              const int slot = fill % Cfg::kStages;
              if (fill >= Cfg::kStages) {
                mbar_wait(bar_empty + 8 * slot, ((fill / Cfg::kStages) - 1) & 1, abort_flag, p.status, 22);
              }
              const uint32_t dst = sRing + slot * Cfg::kTileBytes;
              const uint32_t full = bar_full + 8 * slot;
              mbar_expect_tx(full, Cfg::kTileBytes);
#pragma unroll
              for (int c = 0; c < Cfg::kChunks; ++c) {
                tma_load_2d(dst + c * Cfg::kChunkBytes, kv == 0 ? &tmK : &tmV, full, c * 64, y);
              }
            }
          }
          mbar_arrive(bar_tempty + 8 * (k & 1));
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
        int last_k = -1;

        for (int k = 0;; ++k) {
          const UnitTable* T = wait_table(k, 30);
          const int n_sched = T->n_sched;
          if (n_sched < 0) break;
          last_k = k;
          bool q_ready[2] = {false, false};
          int n_pv[2] = {0, 0};    // P*V batches issued in this unit

          auto slot_of = [&](int f) { return static_cast<uint32_t>((fbase + f) % Cfg::kStages); };
          auto wait_full = [&](int f) {
            mbar_wait(bar_full + 8 * ((fbase + f) % Cfg::kStages), ((fbase + f) / Cfg::kStages) & 1, abort_flag,
                      p.status, 31);
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
              mbar_wait(bar_q + 8 * g, n_q[g] & 1, abort_flag, p.status, 32);
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
            if (n_pv[g] == 0 && k > 0) {
              // first write to O_g in this unit: the softmax group must have read out the previous one
              mbar_wait(bar_ofree + 8 * g, (k - 1) & 1, abort_flag, p.status, 33);
            }
            if (!p_ready) mbar_wait(bar_p + 8 * g, n_p[g] & 1, abort_flag, p.status, 34 + g);
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < kBlock / 16; ++ks) {
              umma_ts(d_tmem, a_tmem + 8 * ks, vd + ks * 128, idesc_pv, ks > 0 ? 1u : first);
            }
            ++n_pv[g];
            ++n_p[g];
            // last P*V of this tile in the unit: its softmax group may start the epilogue as soon as
            // these MMAs retire, without waiting for the other tile
            if (n_pv[g] == T->cnt[g]) tc_commit(bar_done + 8 * g);
          };
          auto no_peek = [] {};
          constexpr std::integral_constant<int, 0> tile_a{};
          constexpr std::integral_constant<int, 1> tile_b{};

          if (n_sched > 0) {
            {  // prologue: scores of the first visited block
              const int kvb = T->sched[0];
              wait_full(0);
              tc_fence_after();
              if (T->tabA[kvb] != 0u) issue_s(tile_a, 0, no_peek);
              if (T->tabB[kvb] != 0u) issue_s(tile_b, 0, no_peek);
              release(0);
              if (n_sched == 1) tc_commit(bar_qfree);
            }
            bool ring_ok = false;   // V(e) and K(e+1) already seen complete
            bool pa_ok = false;     // P_A(e) already seen complete
            for (int e = 0; e < n_sched; ++e) {
              const int kvb = T->sched[e];
              const bool has_next = e + 1 < n_sched;
              const int kvb_next = has_next ? T->sched[e + 1] : 0;
              const bool use_a = T->tabA[kvb] != 0u, use_b = T->tabB[kvb] != 0u;
              const bool next_a = has_next && T->tabA[kvb_next] != 0u, next_b = has_next && T->tabB[kvb_next] != 0u;
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
          } else {
            tc_commit(bar_qfree);
          }
          // tiles that had nothing to do in this unit still complete their phase
          if (T->cnt[0] == 0) tc_commit(bar_done);
          if (T->cnt[1] == 0) tc_commit(bar_done + 8);
          fbase += 2 * n_sched;
          mbar_arrive(bar_tempty + 8 * (k & 1));
        }
        // Keep this thread (and with it the CTA's shared memory and TMEM) alive until every MMA
        // has retired, whatever the softmax groups do.
        if (last_k >= 0) {
          mbar_wait(bar_done, last_k & 1, abort_flag, p.status, 36);
          mbar_wait(bar_done + 8, last_k & 1, abort_flag, p.status, 37);
        }
      }
    } else if (warp == 11) {
      // =========================== unit scheduler =================================================
      const int grid = static_cast<int>(gridDim.x);
      for (int k = 0;; ++k) {
        UnitTable* T = tables + (k & 1);
        if (k >= 2) {
          if (lane == 0) mbar_wait(bar_tempty + 8 * (k & 1), ((k >> 1) - 1) & 1, abort_flag, p.status, 40);
          __syncwarp();
        }
        int unit = 0;
        if (lane == 0) {
          if (k >= 1) mbar_wait(bar_near, (k - 1) & 1, abort_flag, p.status, 41);
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
            T->n_sched = -1;
            mbar_arrive(bar_tfull + 8 * (k & 1));
          }
          break;
        }
        int bh, pair;
        decode_unit(p, unit, npairs, bh, pair);
        const int qbA = 2 * pair, qbB = 2 * pair + 1;
        for (int i = lane; i < p.nq; i += 32) {
          T->tabA[i] = 0u;
          T->tabB[i] = 0u;
        }
        __syncwarp();
        const long long headq = static_cast<long long>(bh) * p.nq;
        {
          int nA = __ldg(p.kv_num_blocks + headq + qbA);
          nA = max(0, min(nA, p.max_blocks));
          const long long baseA = (headq + qbA) * p.max_blocks;
          for (int i = lane; i < nA; i += 32) {
            int kvb;
            const uint32_t code = resolve_entry(p, baseA, i, qbA, kvb);
            if (code != 0u) T->tabA[kvb] = code;
          }
          if (qbB < p.nq) {
            int nB = __ldg(p.kv_num_blocks + headq + qbB);
            nB = max(0, min(nB, p.max_blocks));
            const long long baseB = (headq + qbB) * p.max_blocks;
            for (int i = lane; i < nB; i += 32) {
              int kvb;
              const uint32_t code = resolve_entry(p, baseB, i, qbB, kvb);
              if (code != 0u) T->tabB[kvb] = code;
            }
          }
        }
        __syncwarp();
        int n = 0, ca = 0, cb = 0;   // compact the visited KV blocks into an ascending list
        for (int base = 0; base < p.nq; base += 32) {
          const int kvb = base + lane;
          uint32_t a = 0u, b = 0u;
          if (kvb < p.nq) {
            a = T->tabA[kvb];
            b = T->tabB[kvb];
          }
          const uint32_t any = __ballot_sync(0xFFFFFFFFu, (a | b) != 0u);
          ca += __popc(__ballot_sync(0xFFFFFFFFu, a != 0u));
          cb += __popc(__ballot_sync(0xFFFFFFFFu, b != 0u));
          if ((a | b) != 0u) T->sched[n + __popc(any & ((1u << lane) - 1u))] = static_cast<uint16_t>(kvb);
          n += __popc(any);
        }
        if (lane == 0) {
          T->n_sched = n;
          T->cnt[0] = ca;
          T->cnt[1] = cb;
          T->bh = bh;
          T->pair = pair;
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

template <int D, bool BF16, bool SOFTCAP>
static cudaError_t launch_ws_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                               FwdParams p, cudaStream_t stream) {
  using Cfg = WsCfg<D>;
  auto kern = omni_fwd_ws_kernel<D, BF16, SOFTCAP>;
  static bool attr_done[64] = {};
  cudaError_t e = ensure_smem_attr(kern, Cfg::kSmemBytes, attr_done);
  if (e != cudaSuccess) return e;
  // The setmaxnreg split inside the kernel is only safe if the kernel was really compiled for
  // kLaunchRegs registers per thread; refuse to launch otherwise (an unsatisfiable increase would
  // wait forever).
  static int num_regs = -1;
  if (num_regs < 0) {
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess) return e;
    num_regs = fa.numRegs;
  }
  if (2 * kSoftmaxRegs + kOtherRegs > 3 * num_regs) return cudaErrorLaunchOutOfResources;
  static int num_sms[64] = {};
  int dev = 0;
  e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) dev = 63;
  if (num_sms[dev] == 0) {
    e = cudaDeviceGetAttribute(&num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const int npairs = (p.nq + 1) / 2;
  const long long units = static_cast<long long>(npairs) * p.BH;
  p.num_units = static_cast<int>(units);
  const int grid = static_cast<int>(units < num_sms[dev] ? units : num_sms[dev]);
  if (p.unit_counter != nullptr) {
    e = cudaMemsetAsync(p.unit_counter, 0, sizeof(int32_t), stream);
    if (e != cudaSuccess) return e;
  }
  kern<<<grid, kWsThreads, Cfg::kSmemBytes, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError();
}

cudaError_t launch_ws(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                      const CUtensorMap& tmV, const FwdParams& p, cudaStream_t stream) {
  const bool cap = p.cap_out != 0.f;
  if (head_dim == 64) {
    if (cap) {
      return bf16 ? launch_ws_t<64, true, true>(tmQ, tmK, tmV, p, stream)
                  : launch_ws_t<64, false, true>(tmQ, tmK, tmV, p, stream);
    }
    return bf16 ? launch_ws_t<64, true, false>(tmQ, tmK, tmV, p, stream)
                : launch_ws_t<64, false, false>(tmQ, tmK, tmV, p, stream);
  }
  if (cap) {
    return bf16 ? launch_ws_t<128, true, true>(tmQ, tmK, tmV, p, stream)
                : launch_ws_t<128, false, true>(tmQ, tmK, tmV, p, stream);
  }
  return bf16 ? launch_ws_t<128, true, false>(tmQ, tmK, tmV, p, stream)
              : launch_ws_t<128, false, false>(tmQ, tmK, tmV, p, stream);
}

}  // namespace omni
