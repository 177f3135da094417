// Plain sm_100a omni-attention forward kernel: one CTA of 128 threads per (Q block, batch*head),
// no warp specialisation. It exists for the same reason the reference keeps its scalar kernel
// (omni-attn-mma/mma/attn_naive.cu:21-302): a short, easy to audit statement of the block-list
// semantics that the fast kernel is cross-checked against. Unlike the reference's, it already
// runs on the Blackwell units: TMA tile loads, tcgen05 MMAs for Q*K^T and P*V, accumulators in TMEM.
//
// The tile's block list is first resolved into a code table in shared memory (one warp; a block that
// is listed twice is visited once, see table_put), then, per visited KV block in ascending order:
// TMA K,V -> smem;  S = Q K^T (TMEM);  each thread owns one query row: mask, online softmax, rescale
// O in TMEM, write P (16-bit) over S in TMEM;  O += P V. Lists in 64x64 blocks (B64) and head_dim 32
// (computed as 64, the missing columns read as zeros) are handled as in the warp-specialised kernel.
#include "omni_common.cuh"
#include "omni_launch.h"

namespace omni {

template <int D>
struct SimpleCfg {
  static constexpr int kTileBytes = kBlock * D * 2;
  static constexpr int kChunks = D / 64;              // 64-column (128-byte) swizzle chunks per row
  static constexpr int kChunkBytes = kBlock * 128;    // one chunk of a 128-row tile
  static constexpr int kTmemCols = 256;               // S/P: [0,128), O: [128,128+D)
  static constexpr int kFixedBytes = 3 * kTileBytes + 256 + 1024;  // Q,K,V + barriers + alignment
};

template <int D, bool BF16, bool B64>
__global__ void __launch_bounds__(128, 2)
omni_fwd_simple_kernel(const __grid_constant__ CUtensorMap tmQ,
                       const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  using Cfg = SimpleCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);

  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + Cfg::kTileBytes;
  const uint32_t sV = sK + Cfg::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * Cfg::kTileBytes);
  const uint32_t bar_q = smem_u32(bars + 0);
  const uint32_t bar_k = smem_u32(bars + 1);
  const uint32_t bar_v = smem_u32(bars + 2);
  const uint32_t bar_s = smem_u32(bars + 3);
  const uint32_t bar_o = smem_u32(bars + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* tab = reinterpret_cast<uint32_t*>(smem + 3 * Cfg::kTileBytes + 256);   // [nq * (B64 ? 4 : 1)]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int qb = blockIdx.x;
  const int bh = blockIdx.y;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const int tab_words = p.nq * (B64 ? 4 : 1);
  for (int i = tid; i < tab_words; i += 128) tab[i] = 0u;
  __syncthreads();
  if (warp == 1) build_tile_table<B64>(p, bh, qb, tab);
  __syncthreads();
  const uint32_t tab_addr = smem_u32(tab);

  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tS = tmem_base;          // scores, later overwritten by the packed P
  const uint32_t tO = tmem_base + 128;    // output accumulator

  constexpr int fmt = BF16 ? 1 : 0;
  constexpr uint32_t idesc_qk = umma_idesc_f16(128, 128, fmt, 0);
  constexpr uint32_t idesc_pv = umma_idesc_f16(128, D, fmt, 1);

  const long long row0 = static_cast<long long>(bh) * p.N;  // first row of this head in [BH*N, D]

  if (tid == 0) {
    mbar_expect_tx(bar_q, Cfg::kTileBytes);
#pragma unroll
    for (int c = 0; c < Cfg::kChunks; ++c) {
      tma_load_3d(sQ + c * Cfg::kChunkBytes, &tmQ, bar_q, c * 64, qb * kBlock, bh);
    }
  }

  RowState st{-INFINITY, 0.f};
  int visited = 0;
  uint32_t ph = 0;

  for (int kvb = 0; kvb < p.nq; ++kvb) {
    if (!tile_visits<B64>(tab_addr, kvb)) continue;   // identical in every thread

    if (tid == 0) {
      const int y = kvb * kBlock;
      mbar_expect_tx(bar_k, Cfg::kTileBytes);
#pragma unroll
      for (int c = 0; c < Cfg::kChunks; ++c) tma_load_3d(sK + c * Cfg::kChunkBytes, &tmK, bar_k, c * 64, y, bh);
      mbar_expect_tx(bar_v, Cfg::kTileBytes);
#pragma unroll
      for (int c = 0; c < Cfg::kChunks; ++c) tma_load_3d(sV + c * Cfg::kChunkBytes, &tmV, bar_v, c * 64, y, bh);

      if (visited == 0) mbar_wait(bar_q, 0, abort_flag, p.status, 1);
      mbar_wait(bar_k, ph, abort_flag, p.status, 2);
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        const uint32_t off = (k / 4) * Cfg::kChunkBytes + (k % 4) * 32;
        umma_ss(tS, umma_smem_desc_sw128(sQ + off, 16, 1024), umma_smem_desc_sw128(sK + off, 16, 1024),
                idesc_qk, k > 0 ? 1u : 0u);
      }
      tc_commit(bar_s);
    }

    // Fetch this row's allow-bits while the MMA runs.
    uint32_t allow[4];
    const bool masked = tile_row_allow<B64>(p, tab_addr, kvb, tid, allow) == 2;

    mbar_wait(bar_s, ph, abort_flag, p.status, 3);
    tc_fence_after();

    float s[128];
    load_scores(tS + lane_base, s);
    if (masked) apply_allow(allow, s);
    const float alpha = softmax_update(st, row_max(s), p.scale_log2, 0.f);
    if (visited > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.f)) rescale_o<D>(tO + lane_base, alpha);
    uint32_t pk[64];
    const float sum = exp_and_pack_n<BF16, 0, 1>(s, st.M, p.scale_log2, p.inv_scale_log2, pk);
    st.l = st.l * alpha + sum;
    store_p(tS + lane_base, pk);
    tc_wait_st();
    tc_fence_before();
    __syncthreads();

    if (tid == 0) {
      tc_fence_after();
      mbar_wait(bar_v, ph, abort_flag, p.status, 4);
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < kBlock / 16; ++k) {
        // V tile rows are keys: 16 keys per MMA = 2048 bytes; the two 64-wide d chunks are
        // kChunkBytes apart (leading byte offset), groups of 8 keys 1024 bytes apart.
        umma_ts(tO, tS + 8 * k, umma_smem_desc_sw128(sV + k * 2048, Cfg::kChunkBytes, 1024), idesc_pv,
                (visited > 0 || k > 0) ? 1u : 0u);
      }
      tc_commit(bar_o);
    }
    mbar_wait(bar_o, ph, abort_flag, p.status, 5);
    tc_fence_after();
    ph ^= 1u;
    ++visited;
  }

  if (visited == 0 && tid == 0) mbar_wait(bar_q, 0, abort_flag, p.status, 6);  // drain the Q copy

  const int q_abs = qb * kBlock + tid;
  if (q_abs < p.N) {   // with 64-blocks the last tile may have only 64 rows
    store_output_row<D, BF16>(tO + lane_base, visited > 0, st, p, row0 + q_abs, q_abs >= p.seqlen_orig);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int D, bool BF16, bool B64>
static cudaError_t launch_simple_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                   const FwdParams& p, cudaStream_t stream) {
  using Cfg = SimpleCfg<D>;
  // Ask for at least half an SM's shared memory so that no more than two CTAs (2 x 256 TMEM
  // columns) are ever resident per SM.
  const int need = Cfg::kFixedBytes + p.nq * (B64 ? 16 : 4);
  const int smem = need > 100 * 1024 ? need : 100 * 1024;
  constexpr int kMaxSmem = Cfg::kFixedBytes + kMaxKvBlocks * 4 > 100 * 1024 ? Cfg::kFixedBytes + kMaxKvBlocks * 4 : 100 * 1024;
  if (smem > kMaxSmem) return cudaErrorInvalidValue;   // the C-ABI layer refuses such lengths first
  auto kern = omni_fwd_simple_kernel<D, BF16, B64>;
  static SmemAttrOnce attr_once[kMaxDevices];
  cudaError_t e = ensure_smem_attr(kern, kMaxSmem, attr_once);
  if (e != cudaSuccess) return e;
  dim3 grid(p.nq, p.BH);
  kern<<<grid, 128, smem, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError();
}

template <int D, bool BF16>
static cudaError_t launch_simple_d(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                   const FwdParams& p, cudaStream_t stream) {
  return p.blk64 ? launch_simple_t<D, BF16, true>(tmQ, tmK, tmV, p, stream)
                 : launch_simple_t<D, BF16, false>(tmQ, tmK, tmV, p, stream);
}

// Longest sequence (in 128-row tiles) the plain kernel's code table has room for.
int simple_max_tiles(bool b64) { return b64 ? kMaxKvBlocks / 4 : kMaxKvBlocks; }

// head_dim is the width the kernel computes with: 64 (also for tensors of head_dim 32) or 128.
cudaError_t launch_simple(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                          const CUtensorMap& tmV, const FwdParams& p, cudaStream_t stream) {
  if (head_dim == 64) {
    return bf16 ? launch_simple_d<64, true>(tmQ, tmK, tmV, p, stream)
                : launch_simple_d<64, false>(tmQ, tmK, tmV, p, stream);
  }
  return bf16 ? launch_simple_d<128, true>(tmQ, tmK, tmV, p, stream)
              : launch_simple_d<128, false>(tmQ, tmK, tmV, p, stream);
}

}  // namespace omni
