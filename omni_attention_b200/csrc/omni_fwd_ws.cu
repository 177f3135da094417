// Warp-specialised sm_100a omni-attention forward kernel.
//
// One CTA owns a PAIR of adjacent Q blocks (tile A = block 2j, tile B = block 2j+1) of one
// (batch, head) and walks the union of their KV block lists once, so every K/V tile staged in
// shared memory feeds up to two Q tiles. Roles (384 threads = 3 warpgroups):
//   warps 0-3  softmax group of tile A   (thread = one query row, TMEM lane = row)
//   warps 4-7  softmax group of tile B
//   warp  8    TMA producer: Q tiles once, then K,V tiles through a ring of shared-memory stages
//   warp  9    MMA issuer: tcgen05.mma for S = Q K^T (smem x smem) and O += P V (TMEM x smem)
//   warps 10-11 idle; they exist so that the third warpgroup can hand its registers to the
//              softmax groups with setmaxnreg (208 registers per softmax thread, 88 elsewhere)
// TMEM (512 columns): S_A [0,128) S_B [128,256) O_A [256,256+D) O_B [256+D,256+2D). P (16-bit) is
// written over the first 64 columns of its S.
//
// The issue order per visited KV block e is   PV_A(e), S_A(e+1), PV_B(e), S_B(e+1):  while one
// tile's softmax runs on the CUDA cores the tensor pipe works on the other tile. An S tile becomes
// visible to its softmax group through an mbarrier armed by tcgen05.commit, which also implies that
// every earlier MMA (in particular the previous P*V of the same tile) has finished; that is what
// lets the softmax group itself rescale O in TMEM when the running maximum moves, without a
// separate correction group.
//
// Block types: FULL tiles take a path with no mask arithmetic; CAUSAL (diagonal) and PARTIAL tiles
// build four 32-bit allow words per row (PARTIAL: one 16-byte load of the bit-packed row, or eight
// for the reference's byte-per-element format) before the scores arrive; blocks that are not listed
// are never loaded. The behaviour replaced is the reference's KV loop
// (omni-attn-mma/mma/omni_attn_shared_kv.cu:148-559) and epilogue (:560-646).
#include "omni_common.cuh"
#include "omni_launch.h"

namespace omni {

template <int D>
struct WsCfg {
  static constexpr int kTileBytes = kBlock * D * 2;
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = kBlock * 128;
  static constexpr int kStages = (D == 128) ? 4 : 8;  // ring entries, each one K or one V tile
  static constexpr int kTmemCols = 512;
  static constexpr int kNumBars = 2 + 2 * kStages + 2 + 2 + 1;
  static constexpr int kTableBytes = kMaxKvBlocks * (4 + 4 + 2);
  static constexpr int kSmemBytes = (2 + kStages) * kTileBytes + kTableBytes + 512 + 1024;
};

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
// Share of the exponentials evaluated on the FMA pipe instead of the MUFU unit (pairs per group).
#ifndef OMNI_POLY_NUM
#define OMNI_POLY_NUM 0
#endif
#ifndef OMNI_POLY_DEN
#define OMNI_POLY_DEN 1
#endif
constexpr int kPolyNum = OMNI_POLY_NUM;
constexpr int kPolyDen = OMNI_POLY_DEN;

template <int D, bool BF16>
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
  uint32_t* tabA = reinterpret_cast<uint32_t*>(after_tiles);    // resolved entry code per KV block
  uint32_t* tabB = tabA + kMaxKvBlocks;
  uint16_t* sched = reinterpret_cast<uint16_t*>(tabB + kMaxKvBlocks);  // visited KV blocks, ascending
  uint64_t* bars = reinterpret_cast<uint64_t*>(after_tiles + Cfg::kTableBytes);
  const uint32_t bar_q = smem_u32(bars + 0);                    // [2] Q tile landed
  const uint32_t bar_full = smem_u32(bars + 2);                 // [kStages] ring entry landed
  const uint32_t bar_empty = bar_full + 8 * Cfg::kStages;       // [kStages] ring entry consumed
  const uint32_t bar_s = bar_empty + 8 * Cfg::kStages;          // [2] S tile complete
  const uint32_t bar_p = bar_s + 16;                            // [2] P tile written (128 arrivals)
  const uint32_t bar_done = bar_p + 16;                         // all MMAs complete
  int* misc = reinterpret_cast<int*>(bars + Cfg::kNumBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 0);
  volatile int* abort_flag = misc + 1;
  int* n_sched_slot = misc + 2;
  int* cnt_slot = misc + 3;  // [2] visited entries of tile A / tile B

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
#ifdef OMNI_PROFILE_CTA
  auto gtime = [] { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return (long long)t; };
  long long* crow = p.prof != nullptr ? p.prof + static_cast<long long>(blockIdx.x) * 8 : nullptr;
  if (tid == 0 && crow) { unsigned sm; asm("mov.u32 %0, %smid;" : "=r"(sm)); crow[0] = gtime(); crow[5] = sm; }
#endif

  // ---- which work unit ------------------------------------------------------------------------
  const int npairs = (p.nq + 1) >> 1;
  int unit = blockIdx.x;
  if (p.work_order != nullptr) unit = __ldg(p.work_order + unit);
  // Heads are taken in groups of `group_heads` (sized on the host so that the K and V of one group
  // fit in L2 together); inside a group the Q pairs run from last to first with the group's heads
  // adjacent. With causal-like masks the long lists of all heads of a group start first and the
  // short ones fill the tail, while co-resident CTAs keep re-reading the same few heads' K/V.
  const int G = p.group_heads;
  const int grp = unit / (G * npairs);
  const int heads_here = min(G, p.BH - grp * G);
  const int u = unit - grp * G * npairs;
  const int pair = npairs - 1 - u / heads_here;
  const int bh = grp * G + u % heads_here;
  const int qbA = 2 * pair;
  const int qbB = 2 * pair + 1;
  const bool haveB = qbB < p.nq;
  const long long row0 = static_cast<long long>(bh) * p.N;

  // ---- set-up: barriers, TMEM, block tables ----------------------------------------------------
  if (tid == 256) {
    mbar_init(bar_q, 1);
    mbar_init(bar_q + 8, 1);
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_p + 8, 128);
    mbar_init(bar_done, 1);
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
  for (int i = tid; i < p.nq; i += kWsThreads) {
    tabA[i] = 0u;
    tabB[i] = 0u;
  }
  __syncthreads();
  {
    const long long headq = static_cast<long long>(bh) * p.nq;
    int nA = __ldg(p.kv_num_blocks + headq + qbA);
    nA = max(0, min(nA, p.max_blocks));
    const long long baseA = (headq + qbA) * p.max_blocks;
    for (int i = tid; i < nA; i += kWsThreads) {
      int kvb;
      const uint32_t code = resolve_entry(p, baseA, i, qbA, kvb);
      if (code != 0u) tabA[kvb] = code;
    }
    if (haveB) {
      int nB = __ldg(p.kv_num_blocks + headq + qbB);
      nB = max(0, min(nB, p.max_blocks));
      const long long baseB = (headq + qbB) * p.max_blocks;
      for (int i = tid; i < nB; i += kWsThreads) {
        int kvb;
        const uint32_t code = resolve_entry(p, baseB, i, qbB, kvb);
        if (code != 0u) tabB[kvb] = code;
      }
    }
  }
  __syncthreads();
  if (warp == 0) {  // compact the visited KV blocks into an ascending list
    int n = 0, ca = 0, cb = 0;
    for (int base = 0; base < p.nq; base += 32) {
      const int kvb = base + lane;
      uint32_t a = 0u, b = 0u;
      if (kvb < p.nq) {
        a = tabA[kvb];
        b = tabB[kvb];
      }
      const uint32_t any = __ballot_sync(0xFFFFFFFFu, (a | b) != 0u);
      ca += __popc(__ballot_sync(0xFFFFFFFFu, a != 0u));
      cb += __popc(__ballot_sync(0xFFFFFFFFu, b != 0u));
      if ((a | b) != 0u) sched[n + __popc(any & ((1u << lane) - 1u))] = static_cast<uint16_t>(kvb);
      n += __popc(any);
    }
    if (lane == 0) {
      *n_sched_slot = n;
      cnt_slot[0] = ca;
      cnt_slot[1] = cb;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

#ifdef OMNI_PROFILE_CTA
  if (tid == 0 && crow) { crow[1] = gtime(); crow[6] = *n_sched_slot; crow[7] = cnt_slot[0] + cnt_slot[1]; }
#endif
  const uint32_t tmem_base = *tmem_slot;
  const int n_sched = *n_sched_slot;
  const int cntA = cnt_slot[0];
  const int cntB = cnt_slot[1];

  constexpr int fmt = BF16 ? 1 : 0;
  constexpr uint32_t idesc_qk = umma_idesc_f16(128, 128, fmt, 0);
  constexpr uint32_t idesc_pv = umma_idesc_f16(128, D, fmt, 1);

  if (warp < 8) {
    // =========================== softmax groups =================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int g = warp >> 2;                       // 0 = tile A, 1 = tile B
    const int r = tid & 127;                       // row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + 128 * g + lane_base;
    const uint32_t tO = tmem_base + 256 + D * g + lane_base;
    const uint32_t* tab = g == 0 ? tabA : tabB;
    const int my_cnt = g == 0 ? cntA : cntB;
    const int qb = g == 0 ? qbA : qbB;
    const uint32_t my_bar_s = bar_s + 8 * g;
    const uint32_t my_bar_p = bar_p + 8 * g;

    RowState st{-INFINITY, 0.f};
    int cnt = 0;
    for (int e = 0; e < n_sched && cnt < my_cnt; ++e) {
      const int kvb = sched[e];
      const uint32_t code = tab[kvb];
      if (code == 0u) continue;
      const bool masked = (code & kCodeTypeMask) != kTypeFull || (code & kCodeClip);
      uint32_t allow[4];
      if (masked) build_allow(p, code, kvb, r, allow);

      mbar_wait(my_bar_s, cnt & 1, abort_flag, p.status, 10 + g);
      tc_fence_after();

#if defined(OMNI_DEBUG_SKIP_SOFTMAX)
      // timing experiment only: no softmax work at all, P is whatever S holds
      tc_fence_before();
      mbar_arrive(my_bar_p);
      ++cnt;
      continue;
#endif
      float s[128];
      load_scores(tS, s);
      if (masked) apply_allow(allow, s);
      const float alpha = softmax_update(st, row_max(s), p.scale_log2, kLazyRescaleLog2);
      if (cnt > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.f)) rescale_o<D>(tO, alpha);
      uint32_t pk[64];
      const float sum = exp_and_pack<BF16, kPolyNum, kPolyDen>(s, st.M, p.scale_log2, p.inv_scale_log2, pk);
      st.l = st.l * alpha + sum;
      store_p(tS, pk);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(my_bar_p);
      ++cnt;
    }
    if (my_cnt > 0) {
      mbar_wait(bar_done, 0, abort_flag, p.status, 12 + g);
      tc_fence_after();
    }
#ifdef OMNI_PROFILE_CTA
    if (tid == 0 && crow) crow[2] = gtime();
#endif
    if (g == 0 || haveB) {
      const int q_abs = qb * kBlock + r;
      store_output_row<D, BF16>(tO, my_cnt > 0, st, p, row0 + q_abs, q_abs >= p.seqlen_orig);
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
    if (warp == 8) {
    // =========================== TMA producer ===================================================
    if (lane == 0) {
      if (cntA > 0) {
        mbar_expect_tx(bar_q, Cfg::kTileBytes);
#pragma unroll
        for (int c = 0; c < Cfg::kChunks; ++c) {
          tma_load_2d(sQ0 + c * Cfg::kChunkBytes, &tmQ, bar_q, c * 64, static_cast<int>(row0 + qbA * kBlock));
        }
      }
      if (cntB > 0) {
        mbar_expect_tx(bar_q + 8, Cfg::kTileBytes);
#pragma unroll
        for (int c = 0; c < Cfg::kChunks; ++c) {
          tma_load_2d(sQ0 + Cfg::kTileBytes + c * Cfg::kChunkBytes, &tmQ, bar_q + 8, c * 64,
                      static_cast<int>(row0 + qbB * kBlock));
        }
      }
      int fill = 0;
      for (int e = 0; e < n_sched; ++e) {
        const int y = static_cast<int>(row0 + static_cast<int>(sched[e]) * kBlock);
#pragma unroll
        for (int kv = 0; kv < 2; ++kv, ++fill) {
          const int slot = fill % Cfg::kStages;
          if (fill >= Cfg::kStages) {
            mbar_wait(bar_empty + 8 * slot, ((fill / Cfg::kStages) - 1) & 1, abort_flag, p.status, 20);
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
    }
    } else if (warp == 9) {
    // =========================== MMA issuer =====================================================
    if (lane == 0 && n_sched > 0) {
      const uint32_t tS[2] = {tmem_base, tmem_base + 128};
      const uint32_t tO[2] = {tmem_base + 256, tmem_base + 256 + D};
      int n_pv[2] = {0, 0};        // P*V products issued per tile (also the P barrier phase count)
      bool q_ready[2] = {false, false};

      // UMMA descriptors are built once; inside the loops a descriptor is "base + constant"
      // (start-address field, 16-byte units), so issuing one MMA costs a handful of instructions.
      const uint64_t q_desc[2] = {umma_smem_desc_sw128(sQ0, 16, 1024),
                                  umma_smem_desc_sw128(sQ0 + Cfg::kTileBytes, 16, 1024)};
      const uint64_t k_desc0 = umma_smem_desc_sw128(sRing, 16, 1024);                 // K-major view of a ring slot
      const uint64_t v_desc0 = umma_smem_desc_sw128(sRing, Cfg::kChunkBytes, 1024);   // MN-major view (V)
      constexpr uint32_t kSlotStep = Cfg::kTileBytes >> 4;
      constexpr uint32_t kChunkStep = Cfg::kChunkBytes >> 4;
      auto slot_of = [&](int fill) { return static_cast<uint32_t>(fill % Cfg::kStages); };
      auto wait_full = [&](int fill) {
        mbar_wait(bar_full + 8 * (fill % Cfg::kStages), (fill / Cfg::kStages) & 1, abort_flag, p.status, 30);
      };
      auto release = [&](int fill) { tc_commit(bar_empty + 8 * (fill % Cfg::kStages)); };
      // The tensor pipe accepts a tcgen05.mma only about as fast as it executes them, so the issuing
      // thread is busy for the whole execution time of a batch and every cycle it then spends
      // finding out whether the next batch may start (an mbarrier poll is a shared-memory round trip)
      // is a cycle the pipe idles. The polls for the NEXT batch are therefore started in the middle of
      // the current one (`peek`, non-blocking) and only fall back to a blocking wait when they failed.
      // Operand descriptors of a batch are computed before the batch starts, so that each MMA is a
      // single instruction for this thread: it shares its scheduler partition with two softmax warps
      // and every extra instruction per MMA waits for an issue slot behind their arithmetic.
      uint64_t qa[D / 16], qb_[D / 16];
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t off = (ks / 4) * kChunkStep + (ks % 4) * 2;
        qa[ks] = q_desc[0] + off;
        qb_[ks] = q_desc[1] + off;
      }
      auto issue_s = [&](int g, int e, auto&& peek) {   // S_g = Q_g * K(e)^T
        if (!q_ready[g]) {
          mbar_wait(bar_q + 8 * g, 0, abort_flag, p.status, 31);
          tc_fence_after();
          q_ready[g] = true;
        }
        const uint64_t kd0 = k_desc0 + slot_of(2 * e) * kSlotStep;
        uint64_t kd[D / 16];
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) kd[ks] = kd0 + ((ks / 4) * kChunkStep + (ks % 4) * 2);
        const uint32_t d_tmem = tS[g];
        if (g == 0) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            umma_ss(d_tmem, qa[ks], kd[ks], idesc_qk, ks > 0 ? 1u : 0u);
            if (ks == D / 16 - 4) peek();
          }
        } else {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            umma_ss(d_tmem, qb_[ks], kd[ks], idesc_qk, ks > 0 ? 1u : 0u);
            if (ks == D / 16 - 4) peek();
          }
        }
        tc_commit(bar_s + 8 * g);
      };
      auto issue_pv = [&](int g, int e, bool p_ready) {  // O_g += P_g * V(e)
        // 16 keys per step = 16 rows of 128 bytes = 2048 bytes; P advances 8 TMEM columns
        const uint64_t vd0 = v_desc0 + slot_of(2 * e + 1) * kSlotStep;
        uint64_t vd[kBlock / 16];
        uint32_t pa[kBlock / 16];
#pragma unroll
        for (int ks = 0; ks < kBlock / 16; ++ks) {
          vd[ks] = vd0 + ks * 128;
          pa[ks] = tS[g] + 8 * ks;
        }
        const uint32_t d_tmem = tO[g];
        const uint32_t first = n_pv[g] > 0 ? 1u : 0u;
        if (!p_ready) mbar_wait(bar_p + 8 * g, n_pv[g] & 1, abort_flag, p.status, 32 + g);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kBlock / 16; ++ks) {
          umma_ts(d_tmem, pa[ks], vd[ks], idesc_pv, ks > 0 ? 1u : first);
        }
        ++n_pv[g];
      };
      auto peek_full = [&](int fill) -> bool {
        return mbar_try_wait(bar_full + 8 * (fill % Cfg::kStages), (fill / Cfg::kStages) & 1) != 0;
      };
      auto no_peek = [] {};

      {  // prologue: scores of the first visited block
        const int kvb = sched[0];
        wait_full(0);
        tc_fence_after();
        if (tabA[kvb] != 0u) issue_s(0, 0, no_peek);
        if (tabB[kvb] != 0u) issue_s(1, 0, no_peek);
        release(0);
      }
      bool ring_ok = false;   // V(e) and K(e+1) already seen complete
      bool pa_ok = false;     // P_A(e) already seen complete
      for (int e = 0; e < n_sched; ++e) {
        const int kvb = sched[e];
        const bool has_next = e + 1 < n_sched;
        const int kvb_next = has_next ? sched[e + 1] : 0;
        const bool use_a = tabA[kvb] != 0u, use_b = tabB[kvb] != 0u;
        const bool next_a = has_next && tabA[kvb_next] != 0u, next_b = has_next && tabB[kvb_next] != 0u;
#ifdef OMNI_PROFILE
#define OMNI_STAMP(i) if (p.prof != nullptr && blockIdx.x == 0 && e < 64) p.prof[e * 8 + (i)] = clock64()
#else
#define OMNI_STAMP(i)
#endif
        OMNI_STAMP(0);
        if (!ring_ok) {
          wait_full(2 * e + 1);                 // V(e)
          if (has_next) wait_full(2 * e + 2);   // K(e+1)
        }
        tc_fence_after();
        bool pb_ok = false;
        OMNI_STAMP(1);
#ifdef OMNI_PROFILE
        if (p.prof != nullptr && blockIdx.x == 0 && e < 64) p.prof[512 + e] = (ring_ok ? 1 : 0) | (pa_ok ? 2 : 0);
#endif
        if (use_a) issue_pv(0, e, pa_ok);
        OMNI_STAMP(2);
        if (next_a) {
          issue_s(0, e + 1, [&] { if (use_b) pb_ok = mbar_try_wait(bar_p + 8, n_pv[1] & 1) != 0; });
        }
        OMNI_STAMP(3);
#ifdef OMNI_PROFILE
        if (p.prof != nullptr && blockIdx.x == 0 && e < 64) p.prof[512 + e] |= (pb_ok ? 4 : 0);
#endif
        if (use_b) issue_pv(1, e, pb_ok);
        OMNI_STAMP(4);
        ring_ok = false;
        pa_ok = false;
        if (next_b) {
          issue_s(1, e + 1, [&] {
            bool ok = peek_full(2 * e + 3);                       // V(e+1)
            if (e + 2 < n_sched) ok = peek_full(2 * e + 4) && ok; // K(e+2)
            ring_ok = ok;
            if (next_a) pa_ok = mbar_try_wait(bar_p, n_pv[0] & 1) != 0;
          });
        }
        OMNI_STAMP(5);
        release(2 * e + 1);
        if (has_next) release(2 * e + 2);
        OMNI_STAMP(6);
      }
      tc_commit(bar_done);
      // Keep this thread (and with it the CTA's shared memory and TMEM) alive until every MMA
      // has retired, whatever the softmax groups do.
      mbar_wait(bar_done, 0, abort_flag, p.status, 34);
    }
    }
  }

  tc_fence_before();
  __syncthreads();
#ifdef OMNI_PROFILE_CTA
  if (tid == 0 && crow) crow[3] = gtime();
#endif
  if (warp == 9) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int D, bool BF16>
static cudaError_t launch_ws_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                               const FwdParams& p, cudaStream_t stream) {
  using Cfg = WsCfg<D>;
  auto kern = omni_fwd_ws_kernel<D, BF16>;
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
  const int npairs = (p.nq + 1) / 2;
  const long long units = static_cast<long long>(npairs) * p.BH;
  kern<<<static_cast<unsigned>(units), kWsThreads, Cfg::kSmemBytes, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError();
}

cudaError_t launch_ws(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                      const CUtensorMap& tmV, const FwdParams& p, cudaStream_t stream) {
  if (head_dim == 64) {
    return bf16 ? launch_ws_t<64, true>(tmQ, tmK, tmV, p, stream)
                : launch_ws_t<64, false>(tmQ, tmK, tmV, p, stream);
  }
  return bf16 ? launch_ws_t<128, true>(tmQ, tmK, tmV, p, stream)
              : launch_ws_t<128, false>(tmQ, tmK, tmV, p, stream);
}

}  // namespace omni
