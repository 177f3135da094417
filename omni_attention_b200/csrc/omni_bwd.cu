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
// Both kernels are plain (one 128-thread CTA, thread = TMEM lane = one row, thread 0 issues TMA and
// tcgen05.mma); loads are overlapped with compute, MMAs and the per-element work alternate.
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
  static constexpr int kSmemBytes = 6 * kTileBytes + kVecBytes + kBitsBytes + 256 + 1024;
};

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

// One accumulator row out of TMEM, times `mul`, as 16-bit values to global memory (zeros when
// `have_acc` is false).
template <int D, bool BF16>
__device__ __forceinline__ void bwd_store_row(uint32_t taddr_row, bool have_acc, float mul, void* base,
                                              long long row_index) {
  uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(base) + row_index * (D * 2));
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
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

// log-sum-exp (natural log) -> subtrahend in the log2 domain; a row that attended nothing
// (-inf) gives +inf, which turns every probability of the row into exp2(-inf) = 0.
__device__ __forceinline__ float lse_to_log2(float lse) {
  return lse == -INFINITY ? INFINITY : lse * 1.4426950408889634f;
}

// ---------------------------------------------------------------------------------------------
// 2. dK, dV. Grid (nq, BH): blockIdx.x = KV block. Thread t owns key row t of the block.
// TMEM: S^T [0,128)  dP^T [128,256)  dV [256,256+D)  dK [384,384+D). P^T (16-bit) is written over
// the first 64 columns of S^T, dS^T over the first 64 columns of dP^T.
// ---------------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(128, 1)
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
  float* lse_s = reinterpret_cast<float*>(smem + 6 * Cfg::kTileBytes);   // [2][128], log2 domain
  float* delta_s = lse_s + 2 * kBlock;                                    // [2][128]
  uint32_t* bits_s = reinterpret_cast<uint32_t*>(delta_s + 2 * kBlock);   // [128][4]
  uint64_t* bars = reinterpret_cast<uint64_t*>(bits_s + kBlock * 4);
  const uint32_t bar_kv = smem_u32(bars + 0);
  const uint32_t bar_ld = smem_u32(bars + 1);   // [2]
  const uint32_t bar_s = smem_u32(bars + 3);
  const uint32_t bar_acc = smem_u32(bars + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int kvb = blockIdx.x;
  const int bh = blockIdx.y;
  const int nq = p.f.nq;

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
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tSt = tmem_base;
  const uint32_t tdPt = tmem_base + 128;
  const uint32_t tdV = tmem_base + 256;
  const uint32_t tdK = tmem_base + 384;
  constexpr int fmt = BF16 ? 1 : 0;
  constexpr uint32_t idesc_ss = umma_idesc_f16(128, 128, fmt, 0);
  constexpr uint32_t idesc_ts = umma_idesc_f16(128, D, fmt, 1);

  const long long row0 = static_cast<long long>(bh) * p.f.N;
  // column kvb of this head's code table: which Q blocks visit this KV block, and how
  const uint32_t* col = p.codes + static_cast<long long>(bh) * nq * nq + kvb;
  auto next_visited = [&](int from, uint32_t& code) -> int {
    int qb = from;
    code = 0u;
    while (qb < nq) {
      code = __ldg(col + static_cast<long long>(qb) * nq);
      if (code != 0u) break;
      ++qb;
    }
    return qb;
  };
  // Stage a Q block: TMA for Q and dO (thread 0), LSE and delta by every thread for its own row.
  auto stage_q_block = [&](int qb, int stage) {
    if (tid == 0) {
      const uint32_t bar = bar_ld + 8 * stage;
      mbar_expect_tx(bar, 2 * Cfg::kTileBytes);
      const int y = static_cast<int>(row0 + qb * kBlock);
      bwd_load_tile<D>(sQ + stage * Cfg::kTileBytes, &tmQ, bar, y);
      bwd_load_tile<D>(sdO + stage * Cfg::kTileBytes, &tmdO, bar, y);
    }
    const int q_abs = qb * kBlock + tid;
    const long long row = row0 + q_abs;
    const bool live = q_abs < p.f.seqlen_orig;
    lse_s[stage * kBlock + tid] = live ? lse_to_log2(__ldg(p.lse + row)) : INFINITY;
    delta_s[stage * kBlock + tid] = live ? __ldg(p.delta + row) : 0.f;
  };

  uint32_t code_cur = 0u, code_next = 0u;
  int qb_cur = next_visited(0, code_cur);
  if (qb_cur < nq) {
    if (tid == 0) {
      mbar_expect_tx(bar_kv, 2 * Cfg::kTileBytes);
      const int y = static_cast<int>(row0 + kvb * kBlock);
      bwd_load_tile<D>(sK, &tmK, bar_kv, y);
      bwd_load_tile<D>(sV, &tmV, bar_kv, y);
    }
    stage_q_block(qb_cur, 0);
  }
  __syncthreads();   // the first block's LSE / delta vectors are read by every thread
  const int k_abs = kvb * kBlock + tid;
  const bool key_live = k_abs < p.f.seqlen_orig;

  int it = 0;
  while (qb_cur < nq) {
    const int stage = it & 1;
    const uint32_t ph = static_cast<uint32_t>(it & 1);
    // the other stage was last read by the MMAs of the previous iteration, which have completed
    const int qb_next = next_visited(qb_cur + 1, code_next);
    if (qb_next < nq) stage_q_block(qb_next, stage ^ 1);

    if (tid == 0) {
      if (it == 0) mbar_wait(bar_kv, 0, abort_flag, p.f.status, 50);
      mbar_wait(bar_ld + 8 * stage, static_cast<uint32_t>((it >> 1) & 1), abort_flag, p.f.status, 51);
      tc_fence_after();
      bwd_mma_ss<D>(tSt, sK, sQ + stage * Cfg::kTileBytes, idesc_ss);     // S^T  = K Q^T
      bwd_mma_ss<D>(tdPt, sV, sdO + stage * Cfg::kTileBytes, idesc_ss);   // dP^T = V dO^T
      tc_commit(bar_s);
    }

    // Allow-bits of this thread's key over the 128 query rows of the block (bit r = query row r).
    const uint32_t type = code_cur & kCodeTypeMask;
    uint32_t allow[4] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
    if (type == kTypePartial) {   // uniform over the CTA
      uint32_t rowbits[4];
      load_partial_row(p.f, code_cur >> 3, tid, rowbits);   // row tid of the tile = query row tid
      *reinterpret_cast<uint4*>(bits_s + 4 * tid) = make_uint4(rowbits[0], rowbits[1], rowbits[2], rowbits[3]);
      __syncthreads();
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t acc = 0u;
#pragma unroll
        for (int r = 0; r < 32; ++r) {
          acc |= ((bits_s[4 * (32 * w + r) + (tid >> 5)] >> (tid & 31)) & 1u) << r;
        }
        allow[w] = acc;
      }
    } else if (type == kTypeCausal) {
      // diagonal block: key t is seen by query rows r >= t
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const int d = tid - 32 * w;   // lowest allowed bit in this word
        allow[w] = d <= 0 ? 0xFFFFFFFFu : (d > 31 ? 0u : ~((1u << d) - 1u));
      }
    }
    if (!key_live) allow[0] = allow[1] = allow[2] = allow[3] = 0u;
    const int q_live = p.f.seqlen_orig - qb_cur * kBlock;   // query rows [0, q_live) exist
    if (q_live < kBlock) clip_row(q_live, allow);

    mbar_wait(bar_s, ph, abort_flag, p.f.status, 52);
    tc_fence_after();

    const float* lse_c = lse_s + stage * kBlock;
    const float* del_c = delta_s + stage * kBlock;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t rs[32], rd[32];
      tmem_ld32(tSt + lane_base + 32 * c, rs);
      tmem_ld32(tdPt + lane_base + 32 * c, rd);
      tc_wait_ld();
      uint32_t pp[16], dd[16];
      const uint32_t aw = allow[c];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float2 l2 = *reinterpret_cast<const float2*>(lse_c + 32 * c + 2 * j);
        const float2 dl = *reinterpret_cast<const float2*>(del_c + 32 * c + 2 * j);
        const bool ok0 = (aw >> (2 * j)) & 1u, ok1 = (aw >> (2 * j + 1)) & 1u;
        const float p0 = ok0 ? ex2_approx(fmaf(__uint_as_float(rs[2 * j]), p.f.scale_log2, -l2.x)) : 0.f;
        const float p1 = ok1 ? ex2_approx(fmaf(__uint_as_float(rs[2 * j + 1]), p.f.scale_log2, -l2.y)) : 0.f;
        const float d0 = ok0 ? p0 * (__uint_as_float(rd[2 * j]) - dl.x) : 0.f;
        const float d1 = ok1 ? p1 * (__uint_as_float(rd[2 * j + 1]) - dl.y) : 0.f;
        pp[j] = pack2<BF16>(p0, p1);
        dd[j] = pack2<BF16>(d0, d1);
      }
      tmem_st16(tSt + lane_base + 16 * c, pp);
      tmem_st16(tdPt + lane_base + 16 * c, dd);
    }
    tc_wait_st();
    tc_fence_before();
    __syncthreads();

    if (tid == 0) {
      tc_fence_after();
      bwd_mma_ts<D>(tdV, tSt, sdO + stage * Cfg::kTileBytes, idesc_ts, it > 0);   // dV += P^T dO
      bwd_mma_ts<D>(tdK, tdPt, sQ + stage * Cfg::kTileBytes, idesc_ts, it > 0);   // dK += dS^T Q
      tc_commit(bar_acc);
    }
    mbar_wait(bar_acc, ph, abort_flag, p.f.status, 53);
    tc_fence_after();
    qb_cur = qb_next;
    code_cur = code_next;
    ++it;
  }

  const long long out_row = row0 + k_abs;
  bwd_store_row<D, BF16>(tdV + lane_base, it > 0, 1.f, p.dv, out_row);
  bwd_store_row<D, BF16>(tdK + lane_base, it > 0, p.f.scale, p.dk, out_row);

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// 3. dQ. Grid (nq, BH): blockIdx.x = Q block. Thread t owns query row t of the block.
// TMEM: S [0,128)  dP [128,256)  dQ [256,256+D). dS (16-bit) is written over the first 64 columns
// of dP.
// ---------------------------------------------------------------------------------------------
template <int D, bool BF16>
__global__ void __launch_bounds__(128, 1)
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
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * Cfg::kTileBytes);
  const uint32_t bar_q = smem_u32(bars + 0);
  const uint32_t bar_ld = smem_u32(bars + 1);   // [2]
  const uint32_t bar_s = smem_u32(bars + 3);
  const uint32_t bar_acc = smem_u32(bars + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int qb = blockIdx.x;
  const int bh = blockIdx.y;
  const int nq = p.f.nq;

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
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tS = tmem_base;
  const uint32_t tdP = tmem_base + 128;
  const uint32_t tdQ = tmem_base + 256;
  constexpr int fmt = BF16 ? 1 : 0;
  constexpr uint32_t idesc_ss = umma_idesc_f16(128, 128, fmt, 0);
  constexpr uint32_t idesc_ts = umma_idesc_f16(128, D, fmt, 1);

  const long long row0 = static_cast<long long>(bh) * p.f.N;
  const uint32_t* codes = p.codes + (static_cast<long long>(bh) * nq + qb) * nq;   // row qb of the table
  auto next_visited = [&](int from, uint32_t& code) -> int {
    int kvb = from;
    code = 0u;
    while (kvb < nq) {
      code = __ldg(codes + kvb);
      if (code != 0u) break;
      ++kvb;
    }
    return kvb;
  };
  auto stage_kv_block = [&](int kvb, int stage) {
    if (tid == 0) {
      const uint32_t bar = bar_ld + 8 * stage;
      mbar_expect_tx(bar, 2 * Cfg::kTileBytes);
      const int y = static_cast<int>(row0 + kvb * kBlock);
      bwd_load_tile<D>(sK + stage * Cfg::kTileBytes, &tmK, bar, y);
      bwd_load_tile<D>(sV + stage * Cfg::kTileBytes, &tmV, bar, y);
    }
  };

  const int q_abs = qb * kBlock + tid;
  const long long my_row = row0 + q_abs;
  const bool q_live = q_abs < p.f.seqlen_orig;
  const float lse2 = q_live ? lse_to_log2(__ldg(p.lse + my_row)) : INFINITY;
  const float delta = q_live ? __ldg(p.delta + my_row) : 0.f;

  uint32_t code_cur = 0u, code_next = 0u;
  int kvb_cur = next_visited(0, code_cur);
  if (kvb_cur < nq) {
    if (tid == 0) {
      mbar_expect_tx(bar_q, 2 * Cfg::kTileBytes);
      const int y = static_cast<int>(row0 + qb * kBlock);
      bwd_load_tile<D>(sQ, &tmQ, bar_q, y);
      bwd_load_tile<D>(sdO, &tmdO, bar_q, y);
    }
    stage_kv_block(kvb_cur, 0);
  }

  int it = 0;
  while (kvb_cur < nq) {
    const int stage = it & 1;
    const uint32_t ph = static_cast<uint32_t>(it & 1);
    const int kvb_next = next_visited(kvb_cur + 1, code_next);
    if (kvb_next < nq) stage_kv_block(kvb_next, stage ^ 1);

    if (tid == 0) {
      if (it == 0) mbar_wait(bar_q, 0, abort_flag, p.f.status, 60);
      mbar_wait(bar_ld + 8 * stage, static_cast<uint32_t>((it >> 1) & 1), abort_flag, p.f.status, 61);
      tc_fence_after();
      bwd_mma_ss<D>(tS, sQ, sK + stage * Cfg::kTileBytes, idesc_ss);     // S  = Q K^T
      bwd_mma_ss<D>(tdP, sdO, sV + stage * Cfg::kTileBytes, idesc_ss);   // dP = dO V^T
      tc_commit(bar_s);
    }

    const bool masked = (code_cur & kCodeTypeMask) != kTypeFull || (code_cur & kCodeClip);
    uint32_t allow[4] = {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu};
    if (masked) build_allow(p.f, code_cur, kvb_cur, tid, allow);

    mbar_wait(bar_s, ph, abort_flag, p.f.status, 62);
    tc_fence_after();

#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t rs[32], rd[32];
      tmem_ld32(tS + lane_base + 32 * c, rs);
      tmem_ld32(tdP + lane_base + 32 * c, rd);
      tc_wait_ld();
      uint32_t dd[16];
      const uint32_t aw = allow[c];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const bool ok0 = (aw >> (2 * j)) & 1u, ok1 = (aw >> (2 * j + 1)) & 1u;
        const float p0 = ex2_approx(fmaf(__uint_as_float(rs[2 * j]), p.f.scale_log2, -lse2));
        const float p1 = ex2_approx(fmaf(__uint_as_float(rs[2 * j + 1]), p.f.scale_log2, -lse2));
        const float d0 = (ok0 && q_live) ? p0 * (__uint_as_float(rd[2 * j]) - delta) : 0.f;
        const float d1 = (ok1 && q_live) ? p1 * (__uint_as_float(rd[2 * j + 1]) - delta) : 0.f;
        dd[j] = pack2<BF16>(d0, d1);
      }
      tmem_st16(tdP + lane_base + 16 * c, dd);
    }
    tc_wait_st();
    tc_fence_before();
    __syncthreads();

    if (tid == 0) {
      tc_fence_after();
      bwd_mma_ts<D>(tdQ, tdP, sK + stage * Cfg::kTileBytes, idesc_ts, it > 0);   // dQ += dS K
      tc_commit(bar_acc);
    }
    mbar_wait(bar_acc, ph, abort_flag, p.f.status, 63);
    tc_fence_after();
    kvb_cur = kvb_next;
    code_cur = code_next;
    ++it;
  }

  bwd_store_row<D, BF16>(tdQ + lane_base, it > 0, p.f.scale, p.dq, my_row);

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int D, bool BF16>
static cudaError_t launch_bwd_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                const CUtensorMap& tmdO, const BwdParams& p, cudaStream_t stream) {
  using Cfg = BwdCfg<D>;
  auto dkdv = omni_bwd_dkdv_kernel<D, BF16>;
  auto dq = omni_bwd_dq_kernel<D, BF16>;
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
  dkdv<<<grid, 128, Cfg::kSmemBytes, stream>>>(tmQ, tmK, tmV, tmdO, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dq<<<grid, 128, Cfg::kSmemBytes, stream>>>(tmQ, tmK, tmV, tmdO, p);
  return cudaGetLastError();
}

cudaError_t launch_bwd(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                       const CUtensorMap& tmV, const CUtensorMap& tmdO, const BwdParams& p, cudaStream_t stream) {
  if (head_dim == 64) {
    return bf16 ? launch_bwd_t<64, true>(tmQ, tmK, tmV, tmdO, p, stream)
                : launch_bwd_t<64, false>(tmQ, tmK, tmV, tmdO, p, stream);
  }
  return bf16 ? launch_bwd_t<128, true>(tmQ, tmK, tmV, tmdO, p, stream)
              : launch_bwd_t<128, false>(tmQ, tmK, tmV, tmdO, p, stream);
}

}  // namespace omni
