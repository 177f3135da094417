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
// Both kernels are plain: one CTA of 8 compute warps plus one warp whose first lane issues TMA and
// tcgen05.mma (a lane that issues MMAs must not share its warp with lanes that spin on a barrier);
// a tile row (= TMEM lane) is shared by two compute threads, one per warpgroup, each taking 64 of
// its 128 columns. Loads are overlapped with compute; MMAs and the per-element work alternate.
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
constexpr int kBwdThreads = kBwdComputeThreads + 32;
constexpr int kBwdIssuer = kBwdComputeThreads;   // thread that issues TMA and MMAs

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
  for (int i = tid; i < n_list; i += 128) {
    int kvb;
    const uint32_t code = resolve_entry(p.f, list_base, i, qb, kvb);
    if (code != 0u) codes[kvb] = code;
  }

  // delta: one warp per row at a time, D / 32 elements per lane
  const int warp = tid >> 5, lane = tid & 31;
  constexpr int kWords = D / 64;   // 32-bit words (2 elements) per lane
  for (int rr = 0; rr < 32; ++rr) {
    const long long row = static_cast<long long>(bh) * p.f.N + qb * kBlock + warp * 32 + rr;
    const uint32_t* po = reinterpret_cast<const uint32_t*>(static_cast<const char*>(p.o) + row * (D * 2)) + lane * kWords;
    const uint32_t* pd = reinterpret_cast<const uint32_t*>(static_cast<const char*>(p.d_o) + row * (D * 2)) + lane * kWords;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < kWords; ++w) {
      const float2 a = unpack2<BF16>(__ldg(po + w));
      const float2 b = unpack2<BF16>(__ldg(pd + w));
      acc = fmaf(a.x, b.x, acc);
      acc = fmaf(a.y, b.y, acc);
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

// acc[128 x 128] = A[128 x D] * B[128 x D]^T, both tiles row-major with D contiguous (K-major).
template <int D>
__device__ __forceinline__ void bwd_mma_ss(uint32_t d_tmem, uint32_t sA, uint32_t sB, uint32_t idesc) {
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    const uint32_t off = (k / 4) * BwdCfg<D>::kChunkBytes + (k % 4) * 32;
    umma_ss(d_tmem, umma_smem_desc_sw128(sA + off, 16, 1024), umma_smem_desc_sw128(sB + off, 16, 1024), idesc,
            k > 0 ? 1u : 0u);
  }
}

// acc[128 x D] (+)= A[128 x 128] * B[128 x D], A 16-bit in TMEM (lane = row of A), B a row-major
// tile whose rows are the contraction index (MN-major operand).
template <int D>
__device__ __forceinline__ void bwd_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t sB, uint32_t idesc,
                                           bool accumulate) {
#pragma unroll
  for (int k = 0; k < kBlock / 16; ++k) {
    umma_ts(d_tmem, a_tmem + 8 * k, umma_smem_desc_sw128(sB + k * 2048, BwdCfg<D>::kChunkBytes, 1024), idesc,
            (accumulate || k > 0) ? 1u : 0u);
  }
}

// The same with the 16-bit A operand stored as two runs of 32 TMEM columns, 64 columns apart
// (contraction indices [0,64) at a_region + a_off, [64,128) at a_region + 64 + a_off): the layout the
// tile kernels use so that each thread writes P / dS only over score columns it has read itself.
template <int D>
__device__ __forceinline__ void bwd_mma_ts_split(uint32_t d_tmem, uint32_t a_region, uint32_t a_off, uint32_t sB,
                                                 uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int k = 0; k < kBlock / 16; ++k) {
    umma_ts(d_tmem, a_region + 64 * (k / 4) + a_off + 8 * (k % 4),
            umma_smem_desc_sw128(sB + k * 2048, BwdCfg<D>::kChunkBytes, 1024), idesc, (accumulate || k > 0) ? 1u : 0u);
  }
}

// One accumulator row (32-column chunks [kFirstChunk, kEndChunk) of it) out of TMEM, times `mul`, as
// 16-bit values to global memory (zeros when `have_acc` is false).
template <int D, bool BF16, int kFirstChunk = 0, int kEndChunk = D / 32>
__device__ __forceinline__ void bwd_store_row(uint32_t taddr_row, bool have_acc, float mul, void* base,
                                              long long row_index) {
  uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(base) + row_index * (D * 2));
#pragma unroll
  for (int c = kFirstChunk; c < kEndChunk; ++c) {
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
  const float k = cap_in * 2.8853900817779268f;   // 2 * log2(e)
  float r0, r1;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(ex2_approx(s.x * k) + 1.f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(ex2_approx(s.y * k) + 1.f));
  const float t0 = fmaf(-2.f, r0, 1.f), t1 = fmaf(-2.f, r1, 1.f);
  s = make_float2(cap_out * t0, cap_out * t1);
  return make_float2(fmaf(-t0, t0, 1.f), fmaf(-t1, t1, 1.f));
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
// 2. dK, dV. One CTA per (KV block, batch*head), see bwd_decode_cta. Threads t and t + 128 own key row t of the block
// (query columns [0,64) and [64,128)).
// TMEM: two score regions [0,128) and [128,256) that S^T and dP^T swap between visits, dV
// [256,256+D), dK [384,384+D). P^T and dS^T (16-bit) are written over S^T.
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
  float* lse_s = reinterpret_cast<float*>(smem + 6 * Cfg::kTileBytes);   // [2][128], -LSE in the log2 domain
  float* delta_s = lse_s + 2 * kBlock;                                    // [2][128], -delta
  uint32_t* bits_s = reinterpret_cast<uint32_t*>(delta_s + 2 * kBlock);   // [128][4]
  uint32_t* code_s = bits_s + kBlock * 4;                                   // [kMaxKvBlocks]
  uint16_t* vis_s = reinterpret_cast<uint16_t*>(code_s + kMaxKvBlocks);      // [kMaxKvBlocks]
  int* n_vis_s = reinterpret_cast<int*>(vis_s + kMaxKvBlocks);
  uint64_t* bars = reinterpret_cast<uint64_t*>(n_vis_s + 4);
  const uint32_t bar_kv = smem_u32(bars + 0);
  const uint32_t bar_ld = smem_u32(bars + 1);   // [2]
  const uint32_t bar_s = smem_u32(bars + 3);
  const uint32_t bar_acc = smem_u32(bars + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
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
    mbar_init(bar_ld, 1);
    mbar_init(bar_ld + 8, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_acc, 1);
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
  auto visited_at = [&](int i, uint32_t& code) -> int {
    if (i >= n_vis) {
      code = 0u;
      return nq;
    }
    const int qb = vis_s[i];
    code = code_s[qb];
    return qb;
  };
  // Staging of a Q block: the tiles (TMA, issuer thread) and the LSE / delta vectors (threads 0-127)
  // become possible at different times, hence two pieces.
  auto stage_tiles = [&](int qb, int stage) {
    const uint32_t bar = bar_ld + 8 * stage;
    mbar_expect_tx(bar, 2 * Cfg::kTileBytes);
    const int y = static_cast<int>(row0 + qb * kBlock);
    bwd_load_tile<D>(sQ + stage * Cfg::kTileBytes, &tmQ, bar, y);
    bwd_load_tile<D>(sdO + stage * Cfg::kTileBytes, &tmdO, bar, y);
  };
  auto stage_vectors = [&](int qb, int stage) {
    if (tid < kBlock) {
      const int q_abs = qb * kBlock + tid;
      const long long row = row0 + q_abs;
      const bool live = q_abs < p.f.seqlen_orig;
      lse_s[stage * kBlock + tid] = live ? -lse_to_log2(__ldg(p.lse + row)) : -INFINITY;   // negated
      delta_s[stage * kBlock + tid] = live ? -__ldg(p.delta + row) : 0.f;                   // negated
    }
  };
  // Visit i keeps S^T in TMEM region (i & 1) and dP^T in the other one (128 columns each). The
  // per-element pass writes P^T and dS^T over S^T only, so the dP^T region is free again as soon
  // as that pass ends and takes the S^T of visit i + 1 while dV / dK of visit i are still running.
  auto issue_scores = [&](int i) {   // issuer thread
    const int stage = i & 1;
    mbar_wait(bar_ld + 8 * stage, static_cast<uint32_t>((i >> 1) & 1), abort_flag, p.f.status, 51);
    tc_fence_after();
    bwd_mma_ss<D>(tmem_base + 128 * (i & 1), sK, sQ + stage * Cfg::kTileBytes, idesc_ss);            // S^T  = K Q^T
    bwd_mma_ss<D>(tmem_base + 128 * ((i & 1) ^ 1), sV, sdO + stage * Cfg::kTileBytes, idesc_ss);    // dP^T = V dO^T
    tc_commit(bar_s);
  };

  uint32_t code_cur = 0u, code_next = 0u;
  int qb_cur = visited_at(0, code_cur);
  if (n_vis > 0) {
    uint32_t unused;
    if (tid == kBwdIssuer) {
      mbar_expect_tx(bar_kv, 2 * Cfg::kTileBytes);
      const int y = static_cast<int>(row0 + kvb * kBlock);
      bwd_load_tile<D>(sK, &tmK, bar_kv, y);
      bwd_load_tile<D>(sV, &tmV, bar_kv, y);
      stage_tiles(qb_cur, 0);
      if (n_vis > 1) stage_tiles(visited_at(1, unused), 1);
      mbar_wait(bar_kv, 0, abort_flag, p.f.status, 50);
      issue_scores(0);
    }
    stage_vectors(qb_cur, 0);
    if (n_vis > 1) stage_vectors(visited_at(1, unused), 1);
  }
  __syncthreads();   // the LSE / delta vectors are read by every thread
  const int k_abs = kvb * kBlock + t;
  const bool key_live = k_abs < p.f.seqlen_orig;
  const float2 c2 = make_float2(p.f.scale_log2, p.f.scale_log2);

  for (int it = 0; it < n_vis; ++it) {
    const int stage = it & 1;
    const uint32_t tS = tmem_base + 128 * (it & 1);          // S^T, then P^T / dS^T
    const uint32_t tdP = tmem_base + 128 * ((it & 1) ^ 1);   // dP^T
    const int qb_next = visited_at(it + 1, code_next);

    // Allow-bits of this thread's key over its 64 query rows of the block (bit r of word w = query
    // row 64 * half + 32 * w + r).
    const uint32_t type = code_cur & kCodeTypeMask;
    uint32_t allow[2] = {0xFFFFFFFFu, 0xFFFFFFFFu};
    if (type == kTypePartial) {   // uniform over the CTA
      if (tid < kBlock) {
        uint32_t rowbits[4];
        load_partial_row(p.f, code_cur >> 3, tid, rowbits);   // row tid of the tile = query row tid
        *reinterpret_cast<uint4*>(bits_s + 4 * tid) = make_uint4(rowbits[0], rowbits[1], rowbits[2], rowbits[3]);
      }
      __syncthreads();
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
    const bool masked = type != kTypeFull || (code_cur & kCodeClip) || (qb_cur + 1) * kBlock > p.f.seqlen_orig;
    const int q_live = p.f.seqlen_orig - qb_cur * kBlock - 64 * half;   // query rows [0, q_live) of this half exist
    if (q_live < 64) {
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        const int d = q_live - 1 - 32 * w;
        allow[w] &= d >= 31 ? 0xFFFFFFFFu : (d < 0 ? 0u : ((2u << d) - 1u));
      }
    }

    if (compute) {
      mbar_wait_warp(bar_s, static_cast<uint32_t>(it & 1), abort_flag, p.f.status, 52);
      tc_fence_after();
      const float* lse_c = lse_s + stage * kBlock + 64 * half;
      const float* del_c = delta_s + stage * kBlock + 64 * half;
      const uint32_t my_s = tS + lane_base + 64 * half;
      const uint32_t my_dp = tdP + lane_base + 64 * half;
      uint32_t dd0[16];
      // two copies of the loop, so that tiles without any masking (the bulk) carry no select at all
      auto tile_math = [&](auto masked_c) {
        constexpr bool kMasked = decltype(masked_c)::value;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rs[32], rd[32];
          tmem_ld32(my_s + 32 * c, rs);
          tmem_ld32(my_dp + 32 * c, rd);
          tc_wait_ld();
          uint32_t pp[16], dd[16];
          const uint32_t aw = allow[c];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 nl = *reinterpret_cast<const float2*>(lse_c + 32 * c + 2 * j);
            const float2 nd = *reinterpret_cast<const float2*>(del_c + 32 * c + 2 * j);
            float2 sc = make_float2(__uint_as_float(rs[2 * j]), __uint_as_float(rs[2 * j + 1]));
            float2 slope;
            if constexpr (SOFTCAP) slope = bwd_soft_cap(sc, p.f.cap_in, p.f.cap_out);
            const float2 x = __ffma2_rn(sc, c2, nl);
            float2 pr = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            float2 ds = __fmul2_rn(pr, __fadd2_rn(make_float2(__uint_as_float(rd[2 * j]), __uint_as_float(rd[2 * j + 1])), nd));
            if constexpr (SOFTCAP) ds = __fmul2_rn(ds, slope);
            if constexpr (kMasked) {
              const bool ok0 = (aw >> (2 * j)) & 1u, ok1 = (aw >> (2 * j + 1)) & 1u;
              pr.x = ok0 ? pr.x : 0.f;
              pr.y = ok1 ? pr.y : 0.f;
              ds.x = ok0 ? ds.x : 0.f;
              ds.y = ok1 ? ds.y : 0.f;
            }
            pp[j] = pack2<BF16>(pr.x, pr.y);
            dd[j] = pack2<BF16>(ds.x, ds.y);
          }
          // P^T over this thread's S^T columns [0,32) of its half, dS^T over [32,64): chunk c has
          // been read completely (chunk 0 covers [0,32)), and nobody else touches these columns
          tmem_st16(my_s + 16 * c, pp);
          if (c == 1) {
            tmem_st16(my_s + 32, dd0);
            tmem_st16(my_s + 48, dd);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) dd0[j] = dd[j];
          }
        }
      };
      if (masked) {   // uniform over the CTA
        tile_math(std::true_type{});
      } else {
        tile_math(std::false_type{});
      }
      tc_wait_st();
    }
    tc_fence_before();
    __syncthreads();

    if (tid == kBwdIssuer) {
      tc_fence_after();
      bwd_mma_ts_split<D>(tdV, tS, 0, sdO + stage * Cfg::kTileBytes, idesc_ts, it > 0);   // dV += P^T dO
      bwd_mma_ts_split<D>(tdK, tS, 32, sQ + stage * Cfg::kTileBytes, idesc_ts, it > 0);   // dK += dS^T Q
      tc_commit(bar_acc);
      if (it + 1 < n_vis) issue_scores(it + 1);
      if (it + 2 < n_vis) {
        // the tiles of this visit are free once its dV / dK MMAs have completed
        mbar_wait(bar_acc, static_cast<uint32_t>(it & 1), abort_flag, p.f.status, 53);
        uint32_t unused;
        stage_tiles(visited_at(it + 2, unused), stage);
      }
    }
    if (it + 2 < n_vis) {
      uint32_t unused;
      stage_vectors(visited_at(it + 2, unused), stage);   // read two barriers from here
    }
    qb_cur = qb_next;
    code_cur = code_next;
  }
  const int it = n_vis;
  if (n_vis > 0) {
    if (compute) {
      mbar_wait_warp(bar_acc, static_cast<uint32_t>((n_vis - 1) & 1), abort_flag, p.f.status, 54);
    } else if (tid == kBwdIssuer) {
      mbar_wait(bar_acc, static_cast<uint32_t>((n_vis - 1) & 1), abort_flag, p.f.status, 54);
    }
    tc_fence_after();
  }

  const long long out_row = row0 + k_abs;
  if (compute && half == 0) {
    bwd_store_row<D, BF16>(tdV + lane_base, it > 0, 1.f, p.dv, out_row);
  } else if (compute) {
    bwd_store_row<D, BF16>(tdK + lane_base, it > 0, p.f.scale, p.dk, out_row);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// 3. dQ. One CTA per (Q block, batch*head), see bwd_decode_cta. Threads t and t + 128 own query row t of the block
// (key columns [0,64) and [64,128)).
// TMEM: two score regions [0,128) and [128,256) that S and dP swap between visits, dQ [256,256+D).
// dS (16-bit) is written over S.
// ---------------------------------------------------------------------------------------------
template <int D, bool BF16, bool SOFTCAP>
__global__ void __launch_bounds__(kBwdThreads, 1)
omni_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const BwdParams p) {
  using Cfg = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);

  const uint32_t sQ = smem_u32(smem);
  const uint32_t sdO = sQ + Cfg::kTileBytes;
  const uint32_t sK = sdO + Cfg::kTileBytes;           // two stages
  const uint32_t sV = sK + 2 * Cfg::kTileBytes;        // two stages
  uint32_t* code_s = reinterpret_cast<uint32_t*>(smem + 6 * Cfg::kTileBytes);   // [kMaxKvBlocks]
  uint16_t* vis_s = reinterpret_cast<uint16_t*>(code_s + kMaxKvBlocks);          // [kMaxKvBlocks]
  int* n_vis_s = reinterpret_cast<int*>(vis_s + kMaxKvBlocks);
  uint64_t* bars = reinterpret_cast<uint64_t*>(n_vis_s + 4);
  const uint32_t bar_q = smem_u32(bars + 0);
  const uint32_t bar_ld = smem_u32(bars + 1);   // [2]
  const uint32_t bar_s = smem_u32(bars + 3);
  const uint32_t bar_acc = smem_u32(bars + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
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
    mbar_init(bar_q, 1);
    mbar_init(bar_ld, 1);
    mbar_init(bar_ld + 8, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_acc, 1);
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
  const uint32_t tdQ = tmem_base + 256;
  constexpr int fmt = BF16 ? 1 : 0;
  constexpr uint32_t idesc_ss = umma_idesc_f16(128, 128, fmt, 0);
  constexpr uint32_t idesc_ts = umma_idesc_f16(128, D, fmt, 1);

  const long long row0 = static_cast<long long>(bh) * p.f.N;
  // row qb of this head's code table: the KV blocks this Q block visits, and how
  const int n_vis = bwd_build_visit_list(p.codes + (static_cast<long long>(bh) * nq + qb) * nq, 1, nq, code_s, vis_s,
                                         n_vis_s);
  auto visited_at = [&](int i, uint32_t& code) -> int {
    if (i >= n_vis) {
      code = 0u;
      return nq;
    }
    const int kvb = vis_s[i];
    code = code_s[kvb];
    return kvb;
  };
  auto stage_tiles = [&](int kvb, int stage) {   // issuer thread
    const uint32_t bar = bar_ld + 8 * stage;
    mbar_expect_tx(bar, 2 * Cfg::kTileBytes);
    const int y = static_cast<int>(row0 + kvb * kBlock);
    bwd_load_tile<D>(sK + stage * Cfg::kTileBytes, &tmK, bar, y);
    bwd_load_tile<D>(sV + stage * Cfg::kTileBytes, &tmV, bar, y);
  };
  // Visit i keeps S in TMEM region (i & 1) and dP in the other one; dS is written over S, so the dP
  // region takes the S of visit i + 1 while dQ of visit i is still running.
  auto issue_scores = [&](int i) {   // issuer thread
    const int stage = i & 1;
    mbar_wait(bar_ld + 8 * stage, static_cast<uint32_t>((i >> 1) & 1), abort_flag, p.f.status, 61);
    tc_fence_after();
    bwd_mma_ss<D>(tmem_base + 128 * (i & 1), sQ, sK + stage * Cfg::kTileBytes, idesc_ss);            // S  = Q K^T
    bwd_mma_ss<D>(tmem_base + 128 * ((i & 1) ^ 1), sdO, sV + stage * Cfg::kTileBytes, idesc_ss);    // dP = dO V^T
    tc_commit(bar_s);
  };

  const int q_abs = qb * kBlock + t;
  const long long my_row = row0 + q_abs;
  const bool q_live = q_abs < p.f.seqlen_orig;
  // a row beyond the sequence (or one that attended nothing) gets -LSE = -inf: every probability 0
  const float neg_lse2 = q_live ? -lse_to_log2(__ldg(p.lse + my_row)) : -INFINITY;
  const float neg_delta = q_live ? -__ldg(p.delta + my_row) : 0.f;
  const float2 c2 = make_float2(p.f.scale_log2, p.f.scale_log2);
  const float2 nl2 = make_float2(neg_lse2, neg_lse2);
  const float2 nd2 = make_float2(neg_delta, neg_delta);

  uint32_t code_cur = 0u, code_next = 0u;
  int kvb_cur = visited_at(0, code_cur);
  if (n_vis > 0 && tid == kBwdIssuer) {
    uint32_t unused;
    mbar_expect_tx(bar_q, 2 * Cfg::kTileBytes);
    const int y = static_cast<int>(row0 + qb * kBlock);
    bwd_load_tile<D>(sQ, &tmQ, bar_q, y);
    bwd_load_tile<D>(sdO, &tmdO, bar_q, y);
    stage_tiles(kvb_cur, 0);
    if (n_vis > 1) stage_tiles(visited_at(1, unused), 1);
    mbar_wait(bar_q, 0, abort_flag, p.f.status, 60);
    issue_scores(0);
  }

  for (int it = 0; it < n_vis; ++it) {
    const int stage = it & 1;
    const uint32_t tS = tmem_base + 128 * (it & 1);          // S, then dS
    const uint32_t tdP = tmem_base + 128 * ((it & 1) ^ 1);   // dP
    const int kvb_next = visited_at(it + 1, code_next);

    const bool masked = (code_cur & kCodeTypeMask) != kTypeFull || (code_cur & kCodeClip);
    uint32_t allow[4] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
    if (masked) build_allow(p.f, code_cur, kvb_cur, t, allow);

    if (compute) {
      mbar_wait_warp(bar_s, static_cast<uint32_t>(it & 1), abort_flag, p.f.status, 62);
      tc_fence_after();
      const uint32_t my_s = tS + lane_base + 64 * half;
      const uint32_t my_dp = tdP + lane_base + 64 * half;
      auto tile_math = [&](auto masked_c) {
        constexpr bool kMasked = decltype(masked_c)::value;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rs[32], rd[32];
          tmem_ld32(my_s + 32 * c, rs);
          tmem_ld32(my_dp + 32 * c, rd);
          tc_wait_ld();
          uint32_t dd[16];
          const uint32_t aw = allow[2 * half + c];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float2 sc = make_float2(__uint_as_float(rs[2 * j]), __uint_as_float(rs[2 * j + 1]));
            float2 slope;
            if constexpr (SOFTCAP) slope = bwd_soft_cap(sc, p.f.cap_in, p.f.cap_out);
            const float2 x = __ffma2_rn(sc, c2, nl2);
            const float2 pr = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            float2 ds = __fmul2_rn(pr, __fadd2_rn(make_float2(__uint_as_float(rd[2 * j]), __uint_as_float(rd[2 * j + 1])), nd2));
            if constexpr (SOFTCAP) ds = __fmul2_rn(ds, slope);
            if constexpr (kMasked) {
              ds.x = ((aw >> (2 * j)) & 1u) ? ds.x : 0.f;
              ds.y = ((aw >> (2 * j + 1)) & 1u) ? ds.y : 0.f;
            }
            dd[j] = pack2<BF16>(ds.x, ds.y);
          }
          // dS over this thread's S columns [0,32) of its half: columns it has read already
          tmem_st16(my_s + 16 * c, dd);
        }
      };
      if (masked) {   // uniform over the CTA
        tile_math(std::true_type{});
      } else {
        tile_math(std::false_type{});
      }
      tc_wait_st();
    }
    tc_fence_before();
    __syncthreads();

    if (tid == kBwdIssuer) {
      tc_fence_after();
      bwd_mma_ts_split<D>(tdQ, tS, 0, sK + stage * Cfg::kTileBytes, idesc_ts, it > 0);   // dQ += dS K
      tc_commit(bar_acc);
      if (it + 1 < n_vis) issue_scores(it + 1);
      if (it + 2 < n_vis) {
        mbar_wait(bar_acc, static_cast<uint32_t>(it & 1), abort_flag, p.f.status, 63);
        uint32_t unused;
        stage_tiles(visited_at(it + 2, unused), stage);
      }
    }
    kvb_cur = kvb_next;
    code_cur = code_next;
  }
  const int it = n_vis;
  if (n_vis > 0) {
    if (compute) {
      mbar_wait_warp(bar_acc, static_cast<uint32_t>((n_vis - 1) & 1), abort_flag, p.f.status, 64);
    } else if (tid == kBwdIssuer) {
      mbar_wait(bar_acc, static_cast<uint32_t>((n_vis - 1) & 1), abort_flag, p.f.status, 64);
    }
    tc_fence_after();
  }

  if (compute && half == 0) {
    bwd_store_row<D, BF16, 0, D / 64>(tdQ + lane_base, it > 0, p.f.scale, p.dq, my_row);
  } else if (compute) {
    bwd_store_row<D, BF16, D / 64, D / 32>(tdQ + lane_base, it > 0, p.f.scale, p.dq, my_row);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int D, bool BF16, bool SOFTCAP>
static cudaError_t launch_bwd_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                const CUtensorMap& tmdO, const BwdParams& p, cudaStream_t stream) {
  using Cfg = BwdCfg<D>;
  auto dkdv = omni_bwd_dkdv_kernel<D, BF16, SOFTCAP>;
  auto dq = omni_bwd_dq_kernel<D, BF16, SOFTCAP>;
  static bool attr_dkdv[64] = {};
  static bool attr_dq[64] = {};
  cudaError_t e = ensure_smem_attr(dkdv, Cfg::kSmemBytes, attr_dkdv);
  if (e != cudaSuccess) return e;
  e = ensure_smem_attr(dq, Cfg::kSmemBytes, attr_dq);
  if (e != cudaSuccess) return e;
  const dim3 grid(p.f.nq, p.f.BH);
  omni_bwd_prep_kernel<D, BF16><<<grid, 128, 0, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const unsigned ctas = static_cast<unsigned>(p.f.nq) * static_cast<unsigned>(p.f.BH);
  dkdv<<<ctas, kBwdThreads, Cfg::kSmemBytes, stream>>>(tmQ, tmK, tmV, tmdO, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dq<<<ctas, kBwdThreads, Cfg::kSmemBytes, stream>>>(tmQ, tmK, tmV, tmdO, p);
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
