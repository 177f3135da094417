// sm_100a backward pass of block-mask ("omni") attention: dQ, dK, dV from dO with the block lists of
// the forward pass and its saved log-sum-exp. The reference is forward-only
// (omni-attn-mma/mma/omni_attn_shared_kv.cu has no gradient kernel); what is differentiated here is
// its forward definition, softmax((Q K^T) * scale + mask) V (omni-attn-mma/omni_attn_torch.py:348-387),
// with the same mask semantics as the forward kernels (omni_common.cuh).
//
//   P  = exp(S * scale - LSE)            S = Q K^T, masked entries give P = 0
//   dV = P^T dO
//   dP = dO V^T,  delta = rowsum(dO * O),  dS = P * (dP - delta)
//   dQ = scale * dS K,   dK = scale * dS^T Q
//
// Three launches on the caller's stream, all working memory in a caller-provided workspace:
//   1. omni_bwd_prep_kernel   resolves every (Q block, KV block) of the lists into a dense table of
//                             entry codes [BH, nq, nq] (so that the lists can be walked by column as
//                             well as by row) and computes delta.
//   2. omni_bwd_dkdv_kernel   one CTA per (KV block, batch*head): K, V stay in shared memory, the Q
//                             blocks that visit this KV block stream through a two-stage ring; S^T and
//                             dP^T are computed transposed (TMEM lane = key) so that P^T and dS^T can be
//                             fed to the tensor cores from TMEM for dV += P^T dO and dK += dS^T Q.
//   3. omni_bwd_dq_kernel     one CTA per (Q block, batch*head), the mirror image: Q, dO stay, the
//                             visited K, V stream; dQ += dS K with dS from TMEM.
// S and dP are recomputed in both kernels (7 tile contractions per visited tile instead of 5), which
// buys a deterministic result with no atomics and no fp32 dQ buffer.
// Both tile kernels are warp-specialised: 8 compute warps (a tile row = TMEM lane is shared by two
// threads, one per warpgroup, each taking 64 of its 128 columns), one warp whose first lane issues
// every tcgen05.mma and one whose first lane issues the TMA loads; everything is handed over through
// mbarriers (tcgen05.commit for "MMAs done", thread arrivals for "P / dS stored"). The per-element
// work of a visit is split in two (probabilities from S; dS from dP and the probabilities) and the
// MMAs of consecutive visits are interleaved so that the tensor pipe runs under both halves.
#include <type_traits>

#include "omni_common.cuh"
#include "omni_launch.h"

namespace omni {

template <int D>
struct BwdCfg {
  static constexpr int kTileBytes = kBlock * D * 2;
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = kBlock * 128;
  static constexpr int kTmemCols = 512;
  static constexpr int kVecBytes = 2 * 2 * kBlock * 4;   // LSE and delta of a Q block, two stages
  static constexpr int kBitsBytes = kBlock * 16;          // one bit-packed partial tile
  static constexpr int kListBytes = kMaxKvBlocks * 4 + kMaxKvBlocks * 2 + 16;   // codes, visit list, its length
  static constexpr int kSmemBytes = 6 * kTileBytes + kVecBytes + kBitsBytes + kListBytes + 256 + 1024;
};

constexpr int kBwdComputeThreads = 256;
constexpr int kBwdThreads = kBwdComputeThreads + 64;
constexpr int kBwdIssuer = kBwdComputeThreads;         // thread that issues the MMAs
constexpr int kBwdProducer = kBwdComputeThreads + 32;  // thread that issues the TMA loads


template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
  } else {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
  }
}

// ---------------------------------------------------------------------------------------------
// 1. Workspace: entry-code table and delta. Grid (nq, BH), 128 threads.
// ---------------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(128) omni_bwd_prep_kernel(const BwdParams p) {
  const int tid = threadIdx.x;
  const int qb = blockIdx.x;
  const int bh = blockIdx.y;
  const int nq = p.f.nq;

  uint32_t* codes = p.codes + (static_cast<long long>(bh) * nq + qb) * nq;
  for (int i = tid; i < nq; i += 128) codes[i] = 0u;
  __syncthreads();
  const long long list_base = (static_cast<long long>(bh) * nq + qb) * p.f.max_blocks;
  int n_list = __ldg(p.f.kv_num_blocks + static_cast<long long>(bh) * nq + qb);
  n_list = max(0, min(n_list, p.f.max_blocks));
  if (tid < 32) {   // one warp walks the list in order; a block listed twice resolves as in the forward
    for (int i0 = 0; i0 < n_list; i0 += 32) {
      const int i = i0 + tid;
      int kvb = -1;
      uint32_t code = 0u;
      if (i < n_list) code = resolve_entry(p.f, list_base, i, qb, kvb);
      table_put(codes, code != 0u ? kvb : -1, code);
    }
  }

  // delta: one warp per row at a time, D / 32 elements per lane
  const int warp = tid >> 5, lane = tid & 31;
  constexpr int kWords = D / 64;   // 32-bit words (2 elements) per lane
  for (int rr = 0; rr < 32; ++rr) {
    const long long row = static_cast<long long>(bh) * p.f.N + qb * kBlock + warp * 32 + rr;
    // rows are d_real elements long (head_dim 32 runs on the 64-wide instantiation: the upper lanes idle)
    const long long pitch = static_cast<long long>(p.f.d_real) * 2;
    const uint32_t* po = reinterpret_cast<const uint32_t*>(static_cast<const char*>(p.o) + row * pitch) + lane * kWords;
    const uint32_t* pd = reinterpret_cast<const uint32_t*>(static_cast<const char*>(p.d_o) + row * pitch) + lane * kWords;
    float acc = 0.f;
    if (lane * kWords * 2 < p.f.d_real) {
#pragma unroll
      for (int w = 0; w < kWords; ++w) {
        const float2 a = unpack2<BF16>(__ldg(po + w));
        const float2 b = unpack2<BF16>(__ldg(pd + w));
        acc = fmaf(a.x, b.x, acc);
        acc = fmaf(a.y, b.y, acc);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) p.delta[row] = acc;
  }
}

// ---------------------------------------------------------------------------------------------
// Pieces shared by the two tile kernels.
// ---------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void bwd_load_tile(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int y) {
#pragma unroll
  for (int c = 0; c < BwdCfg<D>::kChunks; ++c) tma_load_2d(dst + c * BwdCfg<D>::kChunkBytes, tm, bar, c * 64, y);
}

// Every tcgen05.mma occupies the issuing thread for about as long as the tensor pipe needs for it, so
// whatever else that thread executes per MMA is time with nothing queued: the descriptors are advanced
// as 32-bit low words (the high word is one constant) and the accumulate flags are compile-time
// constants wherever they can be.
constexpr uint32_t kBwdDescHi = umma_desc_hi_sw128(1024);

// acc[128 x 128] = A[128 x D] * B[128 x D]^T, both tiles row-major with D contiguous (K-major).
template <int D>
__device__ __forceinline__ void bwd_mma_ss(uint32_t d_tmem, uint32_t sA, uint32_t sB, uint32_t idesc) {
  const uint32_t a_lo = umma_desc_lo(sA, 16), b_lo = umma_desc_lo(sB, 16);
  umma_ss_lo<false>(d_tmem, a_lo, b_lo, kBwdDescHi, idesc);
#pragma unroll
  for (int k = 1; k < D / 16; ++k) {
    const uint32_t off = ((k / 4) * BwdCfg<D>::kChunkBytes + (k % 4) * 32) >> 4;
    umma_ss_lo<true>(d_tmem, a_lo + off, b_lo + off, kBwdDescHi, idesc);
  }
}

// acc[128 x D] (+)= A[128 x 128] * B[128 x D], A 16-bit in TMEM (lane = row of A), B a row-major
// tile whose rows are the contraction index (MN-major operand).
template <int D>
__device__ __forceinline__ void bwd_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t sB, uint32_t idesc,
                                           bool accumulate) {
  const uint32_t b_lo = umma_desc_lo(sB, BwdCfg<D>::kChunkBytes);
  umma_ts_lo(d_tmem, a_tmem, b_lo, kBwdDescHi, idesc, accumulate ? 1u : 0u);
#pragma unroll
  for (int k = 1; k < kBlock / 16; ++k) {
    umma_ts_lo_acc(d_tmem, a_tmem + 8 * k, b_lo + k * 128, kBwdDescHi, idesc);
  }
}

// The same with the 16-bit A operand stored as two runs of 32 TMEM columns, 64 columns apart
// (contraction indices [0,64) at a_region + a_off, [64,128) at a_region + 64 + a_off): the layout the
// tile kernels use so that each thread writes P / dS only over score columns it has read itself.
template <int D>
__device__ __forceinline__ void bwd_mma_ts_split(uint32_t d_tmem, uint32_t a_region, uint32_t a_off, uint32_t sB,
                                                 uint32_t idesc, bool accumulate) {
  const uint32_t b_lo = umma_desc_lo(sB, BwdCfg<D>::kChunkBytes);
  umma_ts_lo(d_tmem, a_region + a_off, b_lo, kBwdDescHi, idesc, accumulate ? 1u : 0u);
#pragma unroll
  for (int k = 1; k < kBlock / 16; ++k) {
    umma_ts_lo_acc(d_tmem, a_region + 64 * (k / 4) + a_off + 8 * (k % 4), b_lo + k * 128, kBwdDescHi, idesc);
  }
}

// One accumulator row (32-column chunks [kFirstChunk, kEndChunk) of it) out of TMEM, times `mul`, as
// 16-bit values to global memory (zeros when `have_acc` is false).
template <int D, bool BF16, int kFirstChunk = 0, int kEndChunk = D / 32>
__device__ __forceinline__ void bwd_store_row(uint32_t taddr_row, bool have_acc, float mul, void* base,
                                              long long row_index, int d_real) {
  // rows of the output are d_real elements long; accumulator columns beyond that (head_dim 32 on the
  // 64-wide instantiation) are zero and are not stored
  uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(base) + row_index * (static_cast<long long>(d_real) * 2));
#pragma unroll
  for (int c = kFirstChunk; c < kEndChunk; ++c) {
    if (32 * c >= d_real) break;
    uint32_t r[32];
    if (have_acc) {
      tmem_ld32(taddr_row + 32 * c, r);
      tc_wait_ld();
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = 0u;
    }
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      w[j] = pack2<BF16>(__uint_as_float(r[2 * j]) * mul, __uint_as_float(r[2 * j + 1]) * mul);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[4 * c + j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  }
}

// One row or column of the entry-code table -> shared memory, plus the ascending list of the blocks
// it visits (walking the table in global memory instead costs one dependent load per skipped
// block). Every thread of the CTA must call it.
__device__ __forceinline__ int bwd_build_visit_list(const uint32_t* src, long long stride, int n, uint32_t* code_s,
                                                    uint16_t* vis_s, int* n_vis_s) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) code_s[i] = __ldg(src + i * stride);
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int count = 0;
    for (int base = 0; base < n; base += 32) {
      const bool on = base + lane < n && code_s[base + lane] != 0u;
      const uint32_t any = __ballot_sync(0xFFFFFFFFu, on);
      if (on) vis_s[count + __popc(any & ((1u << lane) - 1u))] = static_cast<uint16_t>(base + lane);
      count += __popc(any);
    }
    if (lane == 0) *n_vis_s = count;
  }
  __syncthreads();
  return *n_vis_s;
}

// Tanh soft-cap in the backward pass (the forward's soft_cap_scores): the raw score s stands for the
// capped scaled score softcap * tanh(s * scale / softcap), whose derivative with respect to the
// scaled raw score is 1 - tanh^2. Replaces the pair of raw scores by their capped raw-equivalents
// (cap_out * tanh) and returns the two derivative factors.
__device__ __forceinline__ float2 bwd_soft_cap(float2& s, float cap_in, float cap_out) {
  const float2 y = __fmul2_rn(s, make_float2(cap_in, cap_in));
  float2 t;
  if (fmaxf(fabsf(y.x), fabsf(y.y)) <= kTanhPolyLimit) {
    t = tanh_small2(y);   // the forward's polynomial for small arguments: no MUFU work
  } else {
    t = make_float2(tanh_exact(y.x), tanh_exact(y.y));
  }
  s = __fmul2_rn(t, make_float2(cap_out, cap_out));
  return __ffma2_rn(make_float2(-t.x, -t.y), t, make_float2(1.f, 1.f));
}

// CTA index -> (block, batch*head) for the two tile kernels. Heads are taken in groups of
// `group_heads` (sized on the host so that a group's Q, K, V and dO stay in L2 together); inside a
// group the blocks run from the longest lists to the shortest for causal-like masks (`descending`:
// from the last block to the first) with the group's heads adjacent, so that the long CTAs of every
// head start early and the grid drains with short ones.
__device__ __forceinline__ void bwd_decode_cta(const FwdParams& f, int cta, bool descending, int& block, int& bh) {
  const int G = f.group_heads;
  const int grp = cta / (f.nq * G);
  const int rem = cta - grp * f.nq * G;
  const int heads_here = min(G, f.BH - grp * G);
  const int b = rem / heads_here;
  block = descending ? f.nq - 1 - b : b;
  bh = grp * G + rem % heads_here;
}

// log-sum-exp (natural log) -> subtrahend in the log2 domain; a row that attended nothing
// (-inf) gives +inf, which turns every probability of the row into exp2(-inf) = 0.
__device__ __forceinline__ float lse_to_log2(float lse) {
  return lse == -INFINITY ? INFINITY : lse * 1.4426950408889634f;
}

// ---------------------------------------------------------------------------------------------
// 2. dK, dV. One CTA per (KV block, batch*head), see bwd_decode_cta. 320 threads:
//   warps 0-7  per-element work; threads t and t + 128 own key row t of the block (query columns
//              [0,64) and [64,128) of the visited Q block)
//   warp  8    first lane issues every tcgen05.mma
//   warp  9    first lane issues the TMA loads
// TMEM: two score regions R0 = [0,128), R1 = [128,256), dV [256,256+D), dK [384,384+D). Visit i puts
// S^T in R(i&1) and dP^T in the other region; P^T and dS^T (16-bit) go over S^T, each thread writing
// only columns it has read itself, so dP^T's region is dead as soon as dS^T is stored.
//
// The per-element work is split in two so that the tensor pipe always has something to do:
//   E1(i): P^T  = exp2(S^T * c - LSE)        needs S^T(i)          -> feeds dV(i)
//   E2(i): dS^T = P^T * (dP^T - delta)       needs dP^T(i), E1(i)  -> feeds dK(i)
// and the MMAs of consecutive visits are interleaved in the order
//   S^T(i), dK(i-1), dP^T(i), dV(i)
// (S^T(i) overwrites dP^T(i-1), dead once E2(i-1) is done; dP^T(i) overwrites the region of visit
// i-1 right after dK(i-1) has read dS^T(i-1) from it; E1(i) runs under dK(i-1) and dP^T(i), E2(i)
// under dV(i)).
// ---------------------------------------------------------------------------------------------
template <int D, bool BF16, bool SOFTCAP>
__global__ void __launch_bounds__(kBwdThreads, 1)
omni_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const BwdParams p) {
  using Cfg = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);

  const uint32_t sK = smem_u32(smem);
  const uint32_t sV = sK + Cfg::kTileBytes;
  const uint32_t sQ = sV + Cfg::kTileBytes;            // two stages
  const uint32_t sdO = sQ + 2 * Cfg::kTileBytes;       // two stages
  // LSE (+inf for a dead row) and delta of the visited Q block as loaded, two stages
  float* lse_s = reinterpret_cast<float*>(smem + 6 * Cfg::kTileBytes);   // [2][128]
  float* delta_s = lse_s + 2 * kBlock;                                    // [2][128]
  uint32_t* bits_s = reinterpret_cast<uint32_t*>(delta_s + 2 * kBlock);   // [128][4]
  uint32_t* code_s = bits_s + kBlock * 4;                                   // [kMaxKvBlocks]
  uint16_t* vis_s = reinterpret_cast<uint16_t*>(code_s + kMaxKvBlocks);      // [kMaxKvBlocks]
  int* n_vis_s = reinterpret_cast<int*>(vis_s + kMaxKvBlocks);
  uint64_t* bars = reinterpret_cast<uint64_t*>(n_vis_s + 4);
  const uint32_t bar_kv = smem_u32(bars + 0);       // K, V landed
  const uint32_t bar_q = smem_u32(bars + 1);        // [2] Q stage landed
  const uint32_t bar_do = smem_u32(bars + 3);       // [2] dO stage landed
  const uint32_t bar_s = smem_u32(bars + 5);        // S^T of the visit complete
  const uint32_t bar_dp = smem_u32(bars + 6);       // dP^T of the visit complete
  const uint32_t bar_p = smem_u32(bars + 7);        // P^T stored (256 arrivals)
  const uint32_t bar_ds = smem_u32(bars + 8);       // dS^T stored (256 arrivals)
  const uint32_t bar_dvdone = smem_u32(bars + 9);   // [2] dV MMAs of the visit in this stage complete: dO stage free
  const uint32_t bar_dkdone = smem_u32(bars + 11);  // [2] dK MMAs complete: Q stage free
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const bool compute = tid < kBwdComputeThreads;
  const int half = (tid >> 7) & 1;  // which 64 query columns of the tile this thread works on
  const int t = tid & 127;          // key row of the tile = TMEM lane
  const int nq = p.f.nq;
  int kvb, bh;
  bwd_decode_cta(p.f, static_cast<int>(blockIdx.x), false, kvb, bh);

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_q + 8 * s, 1);
      mbar_init(bar_do + 8 * s, 1);
      mbar_init(bar_dvdone + 8 * s, 1);
      mbar_init(bar_dkdone + 8 * s, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_dp, 1);
    mbar_init(bar_p, kBwdComputeThreads);
    mbar_init(bar_ds, kBwdComputeThreads);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t tdV = tmem_base + 256;
  const uint32_t tdK = tmem_base + 384;
  constexpr int fmt = BF16 ? 1 : 0;
  constexpr uint32_t idesc_ss = umma_idesc_f16(128, 128, fmt, 0);
  constexpr uint32_t idesc_ts = umma_idesc_f16(128, D, fmt, 1);

  const long long row0 = static_cast<long long>(bh) * p.f.N;
  // column kvb of this head's code table: which Q blocks visit this KV block, and how
  const int n_vis = bwd_build_visit_list(p.codes + static_cast<long long>(bh) * nq * nq + kvb, nq, nq, code_s, vis_s,
                                         n_vis_s);
  auto stage_vectors = [&](int qb, int stage) {   // threads 0-127
    const int q_abs = qb * kBlock + tid;
    const long long row = row0 + q_abs;
    const bool live = q_abs < p.f.seqlen_orig;
    const float l = live ? __ldg(p.lse + row) : INFINITY;
    lse_s[stage * kBlock + tid] = l == -INFINITY ? INFINITY : l;   // a row that attended nothing is dead too
    delta_s[stage * kBlock + tid] = live ? __ldg(p.delta + row) : 0.f;
  };
  if (tid < kBlock) {
    if (n_vis > 0) stage_vectors(vis_s[0], 0);
    if (n_vis > 1) stage_vectors(vis_s[1], 1);
  }
  __syncthreads();   // the LSE / delta vectors are read by every compute thread

  if (tid == kBwdProducer) {
    // =========================== TMA producer ====================================================
    if (n_vis > 0) {
      mbar_expect_tx(bar_kv, 2 * Cfg::kTileBytes);
      const int y = static_cast<int>(row0 + kvb * kBlock);
      bwd_load_tile<D>(sK, &tmK, bar_kv, y);
      bwd_load_tile<D>(sV, &tmV, bar_kv, y);
    }
    for (int i = 0; i < n_vis; ++i) {
      const int stage = i & 1;
      const int y = static_cast<int>(row0 + static_cast<int>(vis_s[i]) * kBlock);
      const uint32_t prev = static_cast<uint32_t>(((i >> 1) - 1) & 1);   // parity of the stage's previous use
      // Q first: it is needed first (S^T opens the visit) although its stage is freed last (by dK)
      if (i >= 2) mbar_wait(bar_dkdone + 8 * stage, prev, abort_flag, p.f.status, 55);
      mbar_expect_tx(bar_q + 8 * stage, Cfg::kTileBytes);
      bwd_load_tile<D>(sQ + stage * Cfg::kTileBytes, &tmQ, bar_q + 8 * stage, y);
      if (i >= 2) mbar_wait(bar_dvdone + 8 * stage, prev, abort_flag, p.f.status, 56);
      mbar_expect_tx(bar_do + 8 * stage, Cfg::kTileBytes);
      bwd_load_tile<D>(sdO + stage * Cfg::kTileBytes, &tmdO, bar_do + 8 * stage, y);
    }
  } else if (tid == kBwdIssuer) {
    // =========================== MMA issuer ======================================================
    for (int i = 0; i < n_vis; ++i) {
      const int stage = i & 1;
      const uint32_t ph = static_cast<uint32_t>(i & 1);
      const uint32_t ld_ph = static_cast<uint32_t>((i >> 1) & 1);
      const uint32_t tS = tmem_base + 128 * (i & 1);
      const uint32_t tdP = tmem_base + 128 * ((i & 1) ^ 1);
      if (i == 0) {
        mbar_wait(bar_kv, 0, abort_flag, p.f.status, 50);
      } else {
        // E2 of the previous visit has read dP^T (its region takes this visit's S^T) and stored dS^T
        mbar_wait(bar_ds, ph ^ 1u, abort_flag, p.f.status, 57);
      }
      mbar_wait(bar_q + 8 * stage, ld_ph, abort_flag, p.f.status, 51);
      tc_fence_after();
      bwd_mma_ss<D>(tS, sK, sQ + stage * Cfg::kTileBytes, idesc_ss);                                  // S^T(i) = K Q^T
      tc_commit(bar_s);
      if (i > 0) {   // after S^T(i), not before: E1(i) is the long pole (dK first measured 7 % slower)
        bwd_mma_ts_split<D>(tdK, tdP, 32, sQ + (stage ^ 1) * Cfg::kTileBytes, idesc_ts, i > 1);      // dK += dS^T(i-1) Q(i-1)
        tc_commit(bar_dkdone + 8 * (stage ^ 1));
      }
      mbar_wait(bar_do + 8 * stage, ld_ph, abort_flag, p.f.status, 52);
      tc_fence_after();
      bwd_mma_ss<D>(tdP, sV, sdO + stage * Cfg::kTileBytes, idesc_ss);                                // dP^T(i) = V dO^T
      tc_commit(bar_dp);
      mbar_wait(bar_p, ph, abort_flag, p.f.status, 58);
      tc_fence_after();
      bwd_mma_ts_split<D>(tdV, tS, 0, sdO + stage * Cfg::kTileBytes, idesc_ts, i > 0);               // dV += P^T(i) dO(i)
      tc_commit(bar_dvdone + 8 * stage);
    }
    if (n_vis > 0) {
      const int last = n_vis - 1;
      mbar_wait(bar_ds, static_cast<uint32_t>(last & 1), abort_flag, p.f.status, 57);
      tc_fence_after();
      bwd_mma_ts_split<D>(tdK, tmem_base + 128 * (last & 1), 32, sQ + (last & 1) * Cfg::kTileBytes, idesc_ts, last > 0);
      tc_commit(bar_dkdone + 8 * (last & 1));
      // keep this thread alive until every MMA has retired
      mbar_wait(bar_dkdone + 8 * (last & 1), static_cast<uint32_t>((last >> 1) & 1), abort_flag, p.f.status, 59);
    }
  } else if (compute) {
    // =========================== per-element work ================================================
    const int k_abs = kvb * kBlock + t;
    const bool key_live = k_abs < p.f.seqlen_orig;
    const float2 c2 = make_float2(p.f.scale_log2, p.f.scale_log2);
    for (int i = 0; i < n_vis; ++i) {
      const int stage = i & 1;
      const uint32_t ph = static_cast<uint32_t>(i & 1);
      const int qb = vis_s[i];
      const uint32_t code = code_s[qb];
      const uint32_t my_s = tmem_base + 128 * (i & 1) + lane_base + 64 * half;
      const uint32_t my_dp = tmem_base + 128 * ((i & 1) ^ 1) + lane_base + 64 * half;
      // LSE / delta of the visit after next: the global loads are issued here and land in shared
      // memory at the end of this visit (stored as loaded), so their latency is off everybody's path
      float next_lse = INFINITY, next_delta = 0.f;
      if (tid < kBlock && i + 2 < n_vis) {
        const int q_abs = static_cast<int>(vis_s[i + 2]) * kBlock + tid;
        if (q_abs < p.f.seqlen_orig) {
          next_lse = __ldg(p.lse + row0 + q_abs);
          next_delta = __ldg(p.delta + row0 + q_abs);
        }
      }

      // Allow-bits of this thread's key over its 64 query rows of the block (bit r of word w = query
      // row 64 * half + 32 * w + r).
      const uint32_t type = code & kCodeTypeMask;
      uint32_t allow[2] = {0xFFFFFFFFu, 0xFFFFFFFFu};
      if (type == kTypePartial) {   // uniform over the compute threads
        if (tid < kBlock) {
          uint32_t rowbits[4];
          load_partial_row(p.f, code >> 3, tid, rowbits);   // row tid of the tile = query row tid
          *reinterpret_cast<uint4*>(bits_s + 4 * tid) = make_uint4(rowbits[0], rowbits[1], rowbits[2], rowbits[3]);
        }
        named_barrier_sync(1, kBwdComputeThreads);
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          uint32_t acc = 0u;
#pragma unroll
          for (int r = 0; r < 32; ++r) {
            acc |= ((bits_s[4 * (64 * half + 32 * w + r) + (t >> 5)] >> (t & 31)) & 1u) << r;
          }
          allow[w] = acc;
        }
      } else if (type == kTypeCausal) {
        // diagonal block: key t is seen by query rows r >= t
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          const int d = t - 64 * half - 32 * w;   // lowest allowed bit in this word
          allow[w] = d <= 0 ? 0xFFFFFFFFu : (d > 31 ? 0u : ~((1u << d) - 1u));
        }
      }
      if (!key_live) allow[0] = allow[1] = 0u;
      const bool masked = type != kTypeFull || (code & kCodeClip) || (qb + 1) * kBlock > p.f.seqlen_orig;
      const int q_live = p.f.seqlen_orig - qb * kBlock - 64 * half;   // query rows [0, q_live) of this half exist
      if (q_live < 64) {
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          const int d = q_live - 1 - 32 * w;
          allow[w] &= d >= 31 ? 0xFFFFFFFFu : (d < 0 ? 0u : ((2u << d) - 1u));
        }
      }

      // ---- E1: P^T -------------------------------------------------------------------------------
      const float* lse_c = lse_s + stage * kBlock + 64 * half;
      const float* del_c = delta_s + stage * kBlock + 64 * half;
      float pf[64];      // the unrounded probabilities (times the soft-cap slope, if any), kept for E2
      mbar_wait_warp(bar_s, ph, abort_flag, p.f.status, 52);
      tc_fence_after();
      auto e1 = [&](auto masked_c) {
        constexpr bool kMasked = decltype(masked_c)::value;
        uint32_t rs2[2][32];
        tmem_ld32(my_s, rs2[0]);
        tmem_ld32(my_s + 32, rs2[1]);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint32_t (&rs)[32] = rs2[c];
          uint32_t pp[16];
          const uint32_t aw = allow[c];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 nl = __fmul2_rn(*reinterpret_cast<const float2*>(lse_c + 32 * c + 2 * j),
                                         make_float2(-1.4426950408889634f, -1.4426950408889634f));   // +inf (dead row) -> -inf
            float2 sc = make_float2(__uint_as_float(rs[2 * j]), __uint_as_float(rs[2 * j + 1]));
            float2 slope = make_float2(1.f, 1.f);
            if constexpr (SOFTCAP) slope = bwd_soft_cap(sc, p.f.cap_in, p.f.cap_out);
            const float2 x = __ffma2_rn(sc, c2, nl);
            float2 pr = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            if constexpr (kMasked) {
              pr.x = ((aw >> (2 * j)) & 1u) ? pr.x : 0.f;
              pr.y = ((aw >> (2 * j + 1)) & 1u) ? pr.y : 0.f;
            }
            pp[j] = pack2<BF16>(pr.x, pr.y);
            if constexpr (SOFTCAP) pr = __fmul2_rn(pr, slope);
            pf[32 * c + 2 * j] = pr.x;
            pf[32 * c + 2 * j + 1] = pr.y;
          }
          // P^T over this thread's S^T columns [0,32) of its half: chunk 0 has been read completely
          tmem_st16(my_s + 16 * c, pp);
        }
      };
      if (masked) {   // uniform over the compute threads
        e1(std::true_type{});
      } else {
        e1(std::false_type{});
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p);

      // ---- E2: dS^T ------------------------------------------------------------------------------
      mbar_wait_warp(bar_dp, ph, abort_flag, p.f.status, 53);
      tc_fence_after();
      uint32_t rd2[2][32];
      tmem_ld32(my_dp, rd2[0]);
      tmem_ld32(my_dp + 32, rd2[1]);
      tc_wait_ld();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t (&rd)[32] = rd2[c];
        uint32_t dd[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 dl = *reinterpret_cast<const float2*>(del_c + 32 * c + 2 * j);
          const float2 ds = __fmul2_rn(make_float2(pf[32 * c + 2 * j], pf[32 * c + 2 * j + 1]),
                                       __fadd2_rn(make_float2(__uint_as_float(rd[2 * j]), __uint_as_float(rd[2 * j + 1])),
                                                  make_float2(-dl.x, -dl.y)));
          dd[j] = pack2<BF16>(ds.x, ds.y);
        }
        // dS^T over this thread's S^T columns [32,64) of its half (read in E1)
        tmem_st16(my_s + 32 + 16 * c, dd);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar_ds);

      // the vectors (and the partial-mask bits) of this visit are free once every compute thread is
      // through E2
      named_barrier_sync(2, kBwdComputeThreads);
      if (tid < kBlock && i + 2 < n_vis) {
        lse_s[stage * kBlock + tid] = next_lse == -INFINITY ? INFINITY : next_lse;
        delta_s[stage * kBlock + tid] = next_delta;
      }
    }
    if (n_vis > 0) {
      const int last = n_vis - 1;
      mbar_wait_warp(bar_dkdone + 8 * (last & 1), static_cast<uint32_t>((last >> 1) & 1), abort_flag, p.f.status, 54);
      tc_fence_after();
    }
    const long long out_row = row0 + k_abs;
    if (half == 0) {
      bwd_store_row<D, BF16>(tdV + lane_base, n_vis > 0, 1.f, p.dv, out_row, p.f.d_real);
    } else {
      bwd_store_row<D, BF16>(tdK + lane_base, n_vis > 0, p.f.scale, p.dk, out_row, p.f.d_real);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// 3. dQ. One CTA per (Q block, batch*head), see bwd_decode_cta. Same roles as the dK/dV kernel
// (threads t and t + 128 own query row t, key columns [0,64) and [64,128) of the visited KV block).
// TMEM: three score regions R0, R1, R2 = [0,128), [128,256), [256,384), dQ [384,384+D). Visit i puts
// S in R(i&1) and dP in R2; dS (16-bit) goes over S. The third region is what lets the scores run
// ahead: R2 is dead once E2(i) is done and takes dP(i+1) at once, R(i&1) is free once dQ(i) has read
// dS(i) and takes S(i+2), so the tensor pipe works in the order
//   dP(i+1), dQ(i), S(i+2)
// while the compute warps do E1(i+1) (probabilities, kept in registers) under dP(i+1) and E2(i+1)
// (dS) under dQ(i) / S(i+2). K is needed by S two visits ahead and by dQ, hence a ring of three K
// tiles (two for V); with Q and dO resident that is all of an SM's shared memory at D=128, so the
// buffer is declared 1024-byte aligned instead of being aligned by hand.
// ---------------------------------------------------------------------------------------------
template <int D>
struct DqCfg {
  static constexpr int kTileBytes = kBlock * D * 2;
  static constexpr int kListBytes = kMaxKvBlocks * 2 + 16;   // visit list, its length
  static constexpr int kSmemBytes = 7 * kTileBytes + kListBytes + 256;
};

template <int D, bool BF16, bool SOFTCAP>
__global__ void __launch_bounds__(kBwdThreads, 1)
omni_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const BwdParams p) {
  using Cfg = DqCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_dq[];
  uint8_t* smem = smem_dq;
  if ((smem_u32(smem) & 1023u) != 0u) {   // the swizzled tile layout needs it; uniform over the CTA
    if (threadIdx.x == 0 && p.f.status != nullptr) atomicExch(p.f.status, kStatusWaitTimeout | (69 << 8));
    return;
  }

  const uint32_t sQ = smem_u32(smem);
  const uint32_t sdO = sQ + Cfg::kTileBytes;
  const uint32_t sK = sdO + Cfg::kTileBytes;           // three stages
  const uint32_t sV = sK + 3 * Cfg::kTileBytes;        // two stages
  uint16_t* vis_s = reinterpret_cast<uint16_t*>(smem + 7 * Cfg::kTileBytes);   // [kMaxKvBlocks]
  int* n_vis_s = reinterpret_cast<int*>(vis_s + kMaxKvBlocks);
  uint64_t* bars = reinterpret_cast<uint64_t*>(n_vis_s + 4);
  const uint32_t bar_qdo = smem_u32(bars + 0);     // Q, dO landed
  const uint32_t bar_k = smem_u32(bars + 1);       // [3] K stage landed
  const uint32_t bar_v = smem_u32(bars + 4);       // [2] V stage landed
  const uint32_t bar_s = smem_u32(bars + 6);       // [2] S of a visit complete (by visit parity)
  const uint32_t bar_dp = smem_u32(bars + 8);      // dP of the visit complete
  const uint32_t bar_ds = smem_u32(bars + 9);      // dS stored (256 arrivals)
  const uint32_t bar_kfree = smem_u32(bars + 10);  // [3] dQ MMAs that read this K stage complete
  const uint32_t bar_vfree = smem_u32(bars + 13);  // [2] dP MMAs that read this V stage complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const bool compute = tid < kBwdComputeThreads;
  const int half = (tid >> 7) & 1;  // which 64 key columns of the tile this thread works on
  const int t = tid & 127;          // query row of the tile = TMEM lane
  const int nq = p.f.nq;
  int qb, bh;
  bwd_decode_cta(p.f, static_cast<int>(blockIdx.x), true, qb, bh);

  if (tid == 0) {
    mbar_init(bar_qdo, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(bar_k + 8 * s, 1);
      mbar_init(bar_kfree + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_v + 8 * s, 1);
      mbar_init(bar_vfree + 8 * s, 1);
      mbar_init(bar_s + 8 * s, 1);
    }
    mbar_init(bar_dp, 1);
    mbar_init(bar_ds, kBwdComputeThreads);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t tdQ = tmem_base + 384;
  auto region_s = [&](int i) { return tmem_base + 128u * static_cast<uint32_t>(i & 1); };
  auto region_dp = [&](int) { return tmem_base + 256u; };
  constexpr int fmt = BF16 ? 1 : 0;
  constexpr uint32_t idesc_ss = umma_idesc_f16(128, 128, fmt, 0);
  constexpr uint32_t idesc_ts = umma_idesc_f16(128, D, fmt, 1);

  const long long row0 = static_cast<long long>(bh) * p.f.N;
  // row qb of this head's code table: the KV blocks this Q block visits, and how
  const uint32_t* codes_row = p.codes + (static_cast<long long>(bh) * nq + qb) * nq;
  if (warp == 0) {
    const int lane = tid;
    int count = 0;
    for (int base = 0; base < nq; base += 32) {
      const bool on = base + lane < nq && __ldg(codes_row + base + lane) != 0u;
      const uint32_t any = __ballot_sync(0xFFFFFFFFu, on);
      if (on) vis_s[count + __popc(any & ((1u << lane) - 1u))] = static_cast<uint16_t>(base + lane);
      count += __popc(any);
    }
    if (lane == 0) *n_vis_s = count;
  }
  __syncthreads();
  const int n_vis = *n_vis_s;

  if (tid == kBwdProducer) {
    // =========================== TMA producer ====================================================
    if (n_vis > 0) {
      mbar_expect_tx(bar_qdo, 2 * Cfg::kTileBytes);
      const int y = static_cast<int>(row0 + qb * kBlock);
      bwd_load_tile<D>(sQ, &tmQ, bar_qdo, y);
      bwd_load_tile<D>(sdO, &tmdO, bar_qdo, y);
    }
    for (int j = 0; j < n_vis; ++j) {
      const int y = static_cast<int>(row0 + static_cast<int>(vis_s[j]) * kBlock);
      const int ks = j % 3, vs = j & 1;
      if (j >= 3) mbar_wait(bar_kfree + 8 * ks, static_cast<uint32_t>((j / 3 - 1) & 1), abort_flag, p.f.status, 65);
      mbar_expect_tx(bar_k + 8 * ks, Cfg::kTileBytes);
      bwd_load_tile<D>(sK + ks * Cfg::kTileBytes, &tmK, bar_k + 8 * ks, y);
      if (j >= 2) mbar_wait(bar_vfree + 8 * vs, static_cast<uint32_t>(((j >> 1) - 1) & 1), abort_flag, p.f.status, 66);
      mbar_expect_tx(bar_v + 8 * vs, Cfg::kTileBytes);
      bwd_load_tile<D>(sV + vs * Cfg::kTileBytes, &tmV, bar_v + 8 * vs, y);
    }
  } else if (tid == kBwdIssuer) {
    // =========================== MMA issuer ======================================================
    auto issue_s = [&](int j) {    // S(j) = Q K(j)^T
      mbar_wait(bar_k + 8 * (j % 3), static_cast<uint32_t>((j / 3) & 1), abort_flag, p.f.status, 61);
      tc_fence_after();
      bwd_mma_ss<D>(region_s(j), sQ, sK + (j % 3) * Cfg::kTileBytes, idesc_ss);
      tc_commit(bar_s + 8 * (j & 1));
    };
    auto issue_dp = [&](int j) {   // dP(j) = dO V(j)^T
      mbar_wait(bar_v + 8 * (j & 1), static_cast<uint32_t>((j >> 1) & 1), abort_flag, p.f.status, 62);
      tc_fence_after();
      bwd_mma_ss<D>(region_dp(j), sdO, sV + (j & 1) * Cfg::kTileBytes, idesc_ss);
      tc_commit(bar_dp);
      tc_commit(bar_vfree + 8 * (j & 1));
    };
    if (n_vis > 0) {
      mbar_wait(bar_qdo, 0, abort_flag, p.f.status, 60);
      issue_s(0);
      issue_dp(0);
      if (n_vis > 1) issue_s(1);
    }
    for (int i = 0; i < n_vis; ++i) {
      mbar_wait(bar_ds, static_cast<uint32_t>(i & 1), abort_flag, p.f.status, 63);
      tc_fence_after();
      if (i + 1 < n_vis) issue_dp(i + 1);   // first: E2(i+1) is waiting for it
      bwd_mma_ts_split<D>(tdQ, region_s(i), 0, sK + (i % 3) * Cfg::kTileBytes, idesc_ts, i > 0);   // dQ += dS(i) K(i)
      tc_commit(bar_kfree + 8 * (i % 3));
      if (i + 2 < n_vis) issue_s(i + 2);
    }
    if (n_vis > 0) {
      const int last = n_vis - 1;
      mbar_wait(bar_kfree + 8 * (last % 3), static_cast<uint32_t>((last / 3) & 1), abort_flag, p.f.status, 64);
    }
  } else if (compute) {
    // =========================== per-element work ================================================
    const int q_abs = qb * kBlock + t;
    const long long my_row = row0 + q_abs;
    const bool q_live = q_abs < p.f.seqlen_orig;
    // a row beyond the sequence (or one that attended nothing) gets -LSE = -inf: every probability 0
    const float neg_lse2 = q_live ? -lse_to_log2(__ldg(p.lse + my_row)) : -INFINITY;
    const float neg_delta = q_live ? -__ldg(p.delta + my_row) : 0.f;
    const float2 c2 = make_float2(p.f.scale_log2, p.f.scale_log2);
    const float2 nl2 = make_float2(neg_lse2, neg_lse2);
    const float2 nd2 = make_float2(neg_delta, neg_delta);

    for (int i = 0; i < n_vis; ++i) {
      const int kvb = vis_s[i];
      const uint32_t code = __ldg(codes_row + kvb);
      const uint32_t my_s = region_s(i) + lane_base + 64 * half;
      const uint32_t my_dp = region_dp(i) + lane_base + 64 * half;
      const bool masked = (code & kCodeTypeMask) != kTypeFull || (code & kCodeClip);
      uint32_t allow[4] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
      if (masked) build_allow(p.f, code, kvb, t, allow);

      // ---- E1: probabilities (times the soft-cap slope, if any), kept in registers ---------------
      float pf[64];
      mbar_wait_warp(bar_s + 8 * (i & 1), static_cast<uint32_t>((i >> 1) & 1), abort_flag, p.f.status, 67);
      tc_fence_after();
      auto e1 = [&](auto masked_c) {
        constexpr bool kMasked = decltype(masked_c)::value;
        uint32_t rs2[2][32];
        tmem_ld32(my_s, rs2[0]);
        tmem_ld32(my_s + 32, rs2[1]);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const uint32_t (&rs)[32] = rs2[c];
          const uint32_t aw = allow[2 * half + c];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float2 sc = make_float2(__uint_as_float(rs[2 * j]), __uint_as_float(rs[2 * j + 1]));
            float2 slope = make_float2(1.f, 1.f);
            if constexpr (SOFTCAP) slope = bwd_soft_cap(sc, p.f.cap_in, p.f.cap_out);
            const float2 x = __ffma2_rn(sc, c2, nl2);
            float2 pr = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            if constexpr (SOFTCAP) pr = __fmul2_rn(pr, slope);
            if constexpr (kMasked) {
              pr.x = ((aw >> (2 * j)) & 1u) ? pr.x : 0.f;
              pr.y = ((aw >> (2 * j + 1)) & 1u) ? pr.y : 0.f;
            }
            pf[32 * c + 2 * j] = pr.x;
            pf[32 * c + 2 * j + 1] = pr.y;
          }
        }
      };
      if (masked) {   // uniform over the compute threads
        e1(std::true_type{});
      } else {
        e1(std::false_type{});
      }

      // ---- E2: dS over this thread's S columns [0,32) of its half ---------------------------------
      mbar_wait_warp(bar_dp, static_cast<uint32_t>(i & 1), abort_flag, p.f.status, 68);
      tc_fence_after();
      uint32_t rd2[2][32];
      tmem_ld32(my_dp, rd2[0]);
      tmem_ld32(my_dp + 32, rd2[1]);
      tc_wait_ld();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t (&rd)[32] = rd2[c];
        uint32_t dd[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 ds = __fmul2_rn(make_float2(pf[32 * c + 2 * j], pf[32 * c + 2 * j + 1]),
                                       __fadd2_rn(make_float2(__uint_as_float(rd[2 * j]), __uint_as_float(rd[2 * j + 1])), nd2));
          dd[j] = pack2<BF16>(ds.x, ds.y);
        }
        tmem_st16(my_s + 16 * c, dd);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar_ds);
    }
    if (n_vis > 0) {
      const int last = n_vis - 1;
      mbar_wait_warp(bar_kfree + 8 * (last % 3), static_cast<uint32_t>((last / 3) & 1), abort_flag, p.f.status, 64);
      tc_fence_after();
    }
    if (half == 0) {
      bwd_store_row<D, BF16, 0, D / 64>(tdQ + lane_base, n_vis > 0, p.f.scale, p.dq, my_row, p.f.d_real);
    } else {
      bwd_store_row<D, BF16, D / 64, D / 32>(tdQ + lane_base, n_vis > 0, p.f.scale, p.dq, my_row, p.f.d_real);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

template <int D, bool BF16, bool SOFTCAP>
static cudaError_t launch_bwd_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                const CUtensorMap& tmdO, const BwdParams& p, cudaStream_t stream) {
  using Cfg = BwdCfg<D>;
  auto dkdv = omni_bwd_dkdv_kernel<D, BF16, SOFTCAP>;
  auto dq = omni_bwd_dq_kernel<D, BF16, SOFTCAP>;
  static SmemAttrOnce attr_dkdv[kMaxDevices];
  static SmemAttrOnce attr_dq[kMaxDevices];
  cudaError_t e = ensure_smem_attr(dkdv, Cfg::kSmemBytes, attr_dkdv);
  if (e != cudaSuccess) return e;
  e = ensure_smem_attr(dq, DqCfg<D>::kSmemBytes, attr_dq);
  if (e != cudaSuccess) return e;
  const dim3 grid(p.f.nq, p.f.BH);
  omni_bwd_prep_kernel<D, BF16><<<grid, 128, 0, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const unsigned ctas = static_cast<unsigned>(p.f.nq) * static_cast<unsigned>(p.f.BH);
  dkdv<<<ctas, kBwdThreads, Cfg::kSmemBytes, stream>>>(tmQ, tmK, tmV, tmdO, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dq<<<ctas, kBwdThreads, DqCfg<D>::kSmemBytes, stream>>>(tmQ, tmK, tmV, tmdO, p);
  return cudaGetLastError();
}

cudaError_t launch_bwd(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                       const CUtensorMap& tmV, const CUtensorMap& tmdO, const BwdParams& p, cudaStream_t stream) {
  const bool cap = p.f.cap_out != 0.f;
  if (head_dim == 64) {
    if (cap) {
      return bf16 ? launch_bwd_t<64, true, true>(tmQ, tmK, tmV, tmdO, p, stream)
                  : launch_bwd_t<64, false, true>(tmQ, tmK, tmV, tmdO, p, stream);
    }
    return bf16 ? launch_bwd_t<64, true, false>(tmQ, tmK, tmV, tmdO, p, stream)
                : launch_bwd_t<64, false, false>(tmQ, tmK, tmV, tmdO, p, stream);
  }
  if (cap) {
    return bf16 ? launch_bwd_t<128, true, true>(tmQ, tmK, tmV, tmdO, p, stream)
                : launch_bwd_t<128, false, true>(tmQ, tmK, tmV, tmdO, p, stream);
  }
  return bf16 ? launch_bwd_t<128, true, false>(tmQ, tmK, tmV, tmdO, p, stream)
              : launch_bwd_t<128, false, false>(tmQ, tmK, tmV, tmdO, p, stream);
}

}  // namespace omni
