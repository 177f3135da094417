// Shared device-side pieces of the omni-attention forward kernels: launch parameters, block-list
// entry resolution (what a listed KV block means for one Q block), per-row allow-bit masks for
// CAUSAL / PARTIAL / clipped tiles and the register-level online-softmax step.
//
// Semantics follow the reference's dense expansion of an OmniBlockMask
// (omni-attn-mma/omni_attn_torch.py:89-145) and its scalar kernel (omni-attn-mma/mma/attn_naive.cu:95-301):
//   * CAUSAL compares absolute positions (k_abs <= q_abs), so a CAUSAL entry below the diagonal is
//     a FULL tile and one above the diagonal contributes nothing;
//   * a PARTIAL entry without a usable per-element mask falls back to CAUSAL (omni_attn_torch.py:140-143);
//   * keys at positions >= seqlen_orig are never attended (attn_naive.cu:113);
//   * entries at index >= kv_num_blocks, MASKED entries and out-of-range block ids are ignored.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace omni {

constexpr int kBlock = 128;  // Q_BLOCK_SIZE == KV_BLOCK_SIZE == 128 is the only tile shape built.

// Block type codes of the reference (omni_attn_torch.py:30-41).
constexpr int kTypeMasked = 0;
constexpr int kTypeCausal = 1;
constexpr int kTypeFull = 2;
constexpr int kTypePartial = 3;

// Resolved entry code: bits [1:0] type (0 = not visited), bit 2 = clipped by seqlen_orig,
// bits [31:3] = index into the partial-mask pool.
constexpr uint32_t kCodeTypeMask = 3u;
constexpr uint32_t kCodeClip = 4u;

struct FwdParams {
  void* o;                        // [BH, N, D] 16-bit
  float* lse;                     // [BH, N] or null
  const int32_t* kv_num_blocks;   // [BH, nq]
  const int32_t* kv_indices;      // [BH, nq, max_blocks]
  const int32_t* types;           // [BH, nq, max_blocks]
  const int32_t* partial_idx;     // [BH, nq, max_blocks] or null
  const uint8_t* partial_bool;    // [P, 128, 128] bytes or null
  const uint32_t* partial_bits;   // [P, 128, 4] words (bit c of row r = attend) or null
  int32_t* status;                // device status word or null
  int32_t* unit_counter;          // zeroed int32 in caller scratch for dynamic unit hand-out, or null
  int BH;
  int N;            // padded sequence length (multiple of 128; of 64 with blk64)
  int seqlen_orig;  // unpadded length
  int nq;           // ceil(N / 128): 128-row tiles per (batch, head)
  int max_blocks;
  int num_partial;
  float scale;           // softmax scale
  float scale_log2;      // scale * log2(e)
  float inv_scale_log2;  // 1 / scale_log2
  float cap_in;          // soft-cap: scale / softcap (0 = no soft-cap)
  float cap_out;         // soft-cap: softcap / scale
  int group_heads;       // heads per scheduling group of the warp-specialised kernel (>= 1)
  int num_units;         // work units of the warp-specialised kernel: ceil(nq / 2) * BH
  int o_aligned32;       // output base address is 32-byte aligned (256-bit stores allowed)
  int d_real;            // head_dim of the tensors in memory: 32, 64 or 128 (32 is computed as 64 with the
                         // missing columns read as zeros by the TMA unit); row pitch of o is d_real * 2 bytes
  int blk64;             // 1: the lists, types and partial pool are in 64x64 blocks (N a multiple of 64)
  int nq_lists;          // Q blocks in the lists: N / 64 with blk64, else nq
  long long wait_cycles; // cycle budget of one bounded wait in the forward kernels
};

// Launch parameters of the backward kernels. `f` carries the block lists, the partial-mask pools,
// the sizes and the softmax scale exactly as the forward pass got them (its o / lse / unit_counter
// members are not used).
struct BwdParams {
  FwdParams f;
  const void* o;       // [BH, N, D] forward output
  const void* d_o;     // [BH, N, D] gradient of the output
  const float* lse;    // [BH, N] log-sum-exp saved by the forward pass (natural log)
  void* dq;            // [BH, N, D] results, same 16-bit type as the inputs
  void* dk;
  void* dv;
  uint32_t* codes;     // workspace: [BH, nq, nq] resolved entry code of every (Q block, KV block), 0 = not visited
  float* delta;        // workspace: [BH, N] rowsum(dO * O)
};

// One list entry as stored: KV block id, type code, index into the partial pool.
struct ListEntry {
  int kvb;
  int type;
  int pidx;
};

// The three loads of entry `i`, independent of one another (a caller that walks a list issues the
// loads of many entries before it looks at any of them).
__device__ __forceinline__ ListEntry load_entry(const FwdParams& p, long long list_base, int i) {
  ListEntry e;
  e.kvb = __ldg(p.kv_indices + list_base + i);
  e.type = __ldg(p.types + list_base + i);
  e.pidx = -1;
  if (p.partial_idx != nullptr && (p.partial_bool != nullptr || p.partial_bits != nullptr)) {
    e.pidx = __ldg(p.partial_idx + list_base + i);
  }
  return e;
}

// What entry `e` of the list of Q block `qb` means, for lists in BLK x BLK blocks: the code of the
// block, or 0 when the entry is not visited.
template <int BLK>
__device__ __forceinline__ uint32_t resolve_loaded(const FwdParams& p, const ListEntry& e, int qb) {
  const int kvb = e.kvb;
  int t = e.type;
  const int n_kv_blocks = BLK == kBlock ? p.nq : p.nq_lists;
  if (kvb < 0 || kvb >= n_kv_blocks) {
    if (p.status != nullptr) atomicCAS(p.status, 0, kStatusBadIndex);
    return 0;
  }
  if (t <= kTypeMasked || t > kTypePartial) return 0;
  const int kv_start = kvb * BLK;
  if (kv_start >= p.seqlen_orig) return 0;
  uint32_t pidx = 0;
  if (t == kTypePartial) {
    if (e.pidx >= 0 && e.pidx < p.num_partial) {
      pidx = static_cast<uint32_t>(e.pidx);
    } else {
      t = kTypeCausal;
    }
  }
  if (t == kTypeCausal) {
    if (kvb < qb) {
      t = kTypeFull;
    } else if (kvb > qb) {
      return 0;
    }
  }
  const uint32_t clip = (kv_start + BLK > p.seqlen_orig) ? kCodeClip : 0u;
  return static_cast<uint32_t>(t) | clip | (pidx << 3);
}

// Resolve entry `i` of the list of (bh, qb), lists in 128-blocks. Returns 0 when the entry is not visited.
__device__ __forceinline__ uint32_t resolve_entry(const FwdParams& p, long long list_base, int i,
                                                  int qb, int& kvb_out) {
  const ListEntry e = load_entry(p, list_base, i);
  kvb_out = e.kvb;
  return resolve_loaded<kBlock>(p, e, qb);
}

// Warp-collective write of one resolved entry per lane into a code table (`idx` < 0: this lane has
// nothing to write). A block that is listed more than once gets the meaning the reference's dense
// expansion gives it when it applies the entries in list order (omni-attn-mma/omni_attn_torch.py:
// 106-143): a FULL entry, a CAUSAL entry below the diagonal and a PARTIAL entry with its element mask
// replace whatever the block had (`strong`), a diagonal CAUSAL entry only adds to it, so it counts
// only for a block that has nothing yet. (The one combination this does not reproduce is a diagonal
// CAUSAL entry listed after a PARTIAL one for the same block: the reference takes the union, here the
// PARTIAL mask stands.) Callers feed the list 32 entries at a time, in order.
__device__ __forceinline__ void table_put(uint32_t* tab, int idx, uint32_t code) {
  const int lane = threadIdx.x & 31;
  const bool strong = idx >= 0 && (code & kCodeTypeMask) != kTypeCausal;
  const uint32_t peers = __match_any_sync(0xFFFFFFFFu, idx);
  const uint32_t strong_lanes = __ballot_sync(0xFFFFFFFFu, strong);
  if (idx >= 0) {
    const uint32_t sp = peers & strong_lanes;
    const int winner = 31 - __clz(sp != 0u ? sp : peers);
    if (lane == winner && (strong || tab[idx] == 0u)) tab[idx] = code;
  }
  __syncwarp();
}

// Code table of one 128-row Q tile (Q block `qb` in units of 128 rows) of (batch, head) `bh`, built by
// one warp. Lists in 128-blocks: tab[kvb] = code of KV block kvb. Lists in 64-blocks: four words per
// 128-wide KV block, tab[4 * kvb + 2 * qh + kh] = code of the 64x64 sub-block (rows 64 * qh ..,
// columns 64 * kh ..), resolved against the lists of Q blocks 2 * qb and 2 * qb + 1. The table must be
// zero on entry. A list is taken 128 entries at a time: all their loads first, then the writes in
// list order, so that a long list costs one memory latency per 128 entries and not one per 32.
template <int BLK>
__device__ __forceinline__ void put_list(const FwdParams& p, long long q_index, int q_block, uint32_t* tab,
                                         int sub_row) {
  const int lane = threadIdx.x & 31;
  int n = __ldg(p.kv_num_blocks + q_index);
  n = max(0, min(n, p.max_blocks));
  const long long base = q_index * p.max_blocks;
  constexpr int kBatch = 4;
  for (int i0 = 0; i0 < n; i0 += 32 * kBatch) {
    ListEntry ent[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + 32 * j + lane;
      ent[j].kvb = -1;
      ent[j].type = 0;
      ent[j].pidx = -1;
      if (i < n) ent[j] = load_entry(p, base, i);
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (i0 + 32 * j >= n) break;   // the same for every lane
      const int i = i0 + 32 * j + lane;
      const uint32_t code = i < n ? resolve_loaded<BLK>(p, ent[j], q_block) : 0u;
      int idx = -1;
      if (code != 0u) idx = BLK == kBlock ? ent[j].kvb : 4 * (ent[j].kvb >> 1) + 2 * sub_row + (ent[j].kvb & 1);
      table_put(tab, idx, code);
    }
  }
}

template <bool B64>
__device__ __forceinline__ void build_tile_table(const FwdParams& p, int bh, int qb, uint32_t* tab) {
  if constexpr (!B64) {
    if (qb >= p.nq) return;
    put_list<kBlock>(p, static_cast<long long>(bh) * p.nq + qb, qb, tab, 0);
  } else {
#pragma unroll 1
    for (int qh = 0; qh < 2; ++qh) {
      const int q64 = 2 * qb + qh;
      if (q64 >= p.nq_lists) break;
      put_list<64>(p, static_cast<long long>(bh) * p.nq_lists + q64, q64, tab, qh);
    }
  }
}

// Four 0/1 bytes -> 4 bits (byte i -> bit i). Any non-zero byte counts as true.
__device__ __forceinline__ uint32_t bytes_to_nibble(uint32_t w) {
  const uint32_t x = __vcmpne4(w, 0u) & 0x01010101u;
  return ((x * 0x01020408u) >> 24) & 0xFu;
}

// Load the 128 allow-bits of row `r` of partial tile `pidx` (bit c of word c/32 = attend).
__device__ __forceinline__ void load_partial_row(const FwdParams& p, uint32_t pidx, int r,
                                                 uint32_t (&allow)[4]) {
  if (p.partial_bits != nullptr) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.partial_bits) +
                          (static_cast<size_t>(pidx) * kBlock + r));
    allow[0] = v.x; allow[1] = v.y; allow[2] = v.z; allow[3] = v.w;
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(
        p.partial_bool + (static_cast<size_t>(pidx) * kBlock + r) * kBlock);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint4 a = __ldg(src + 2 * w);
      const uint4 b = __ldg(src + 2 * w + 1);
      allow[w] = bytes_to_nibble(a.x) | (bytes_to_nibble(a.y) << 4) | (bytes_to_nibble(a.z) << 8) |
                 (bytes_to_nibble(a.w) << 12) | (bytes_to_nibble(b.x) << 16) |
                 (bytes_to_nibble(b.y) << 20) | (bytes_to_nibble(b.z) << 24) |
                 (bytes_to_nibble(b.w) << 28);
    }
  }
}

// Allow-bits of row r for a diagonal CAUSAL tile: column c allowed iff c <= r.
__device__ __forceinline__ void causal_row(int r, uint32_t (&allow)[4]) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const int d = r - 32 * w;  // highest allowed bit in this word
      allow[w] = d >= 31 ? 0xFFFFFFFFu : (d < 0 ? 0u : ((2u << d) - 1u));
    }
}

// Keep only columns c < limit (1 <= limit <= 127).
__device__ __forceinline__ void clip_row(int limit, uint32_t (&allow)[4]) {
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const int d = limit - 1 - 32 * w;
    allow[w] &= d >= 31 ? 0xFFFFFFFFu : (d < 0 ? 0u : ((2u << d) - 1u));
  }
}

// Build the allow-bits of row r for a non-FULL or clipped tile.
__device__ __forceinline__ void build_allow(const FwdParams& p, uint32_t code, int kvb, int r,
                                            uint32_t (&allow)[4]) {
  const uint32_t t = code & kCodeTypeMask;
  if (t == kTypePartial) {
    load_partial_row(p, code >> 3, r, allow);
  } else if (t == kTypeCausal) {
    causal_row(r, allow);
  } else {
    allow[0] = allow[1] = allow[2] = allow[3] = 0xFFFFFFFFu;
  }
  if (code & kCodeClip) clip_row(p.seqlen_orig - kvb * kBlock, allow);
}

// ---- lists in 64x64 blocks: the allow-bits of one row over one 64-wide sub-block (two words) ----
// Pool layout with 64-blocks: bytes [P, 64, 64] (the reference's torch.bool tensor) or bits [P, 64, 2].
__device__ __forceinline__ void build_allow_sub64(const FwdParams& p, uint32_t code, int kv64, int r64,
                                                  uint32_t& a0, uint32_t& a1) {
  const uint32_t t = code & kCodeTypeMask;
  if (t == 0u) {
    a0 = a1 = 0u;
    return;
  }
  if (t == kTypePartial) {
    const size_t row = static_cast<size_t>(code >> 3) * 64 + r64;
    if (p.partial_bits != nullptr) {
      const uint2 v = __ldg(reinterpret_cast<const uint2*>(p.partial_bits) + row);
      a0 = v.x;
      a1 = v.y;
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(p.partial_bool + row * 64);
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint4 a = __ldg(src + 2 * h);
        const uint4 b = __ldg(src + 2 * h + 1);
        w[h] = bytes_to_nibble(a.x) | (bytes_to_nibble(a.y) << 4) | (bytes_to_nibble(a.z) << 8) |
               (bytes_to_nibble(a.w) << 12) | (bytes_to_nibble(b.x) << 16) | (bytes_to_nibble(b.y) << 20) |
               (bytes_to_nibble(b.z) << 24) | (bytes_to_nibble(b.w) << 28);
      }
      a0 = w[0];
      a1 = w[1];
    }
  } else if (t == kTypeCausal) {   // diagonal sub-block: column c allowed iff c <= r64
    a0 = r64 >= 31 ? 0xFFFFFFFFu : ((2u << r64) - 1u);
    a1 = r64 < 32 ? 0u : (r64 >= 63 ? 0xFFFFFFFFu : ((2u << (r64 - 32)) - 1u));
  } else {
    a0 = a1 = 0xFFFFFFFFu;
  }
  if (code & kCodeClip) {   // keep columns c < limit, 1 <= limit <= 63
    const int limit = p.seqlen_orig - kv64 * 64;
    a0 &= limit >= 32 ? 0xFFFFFFFFu : ((1u << limit) - 1u);
    a1 &= limit <= 32 ? 0u : ((1u << (limit - 32)) - 1u);
  }
}

// What a 128x128 tile means for row r, from the tile's code table (`tab` is the table's shared-memory
// address). Returns 0 when no row of the tile visits KV block kvb, 1 when row r attends all 128 keys,
// 2 when `allow` (bit c of word c / 32 = key c attended) has to be applied.
template <bool B64>
__device__ __forceinline__ int tile_row_allow(const FwdParams& p, uint32_t tab, int kvb, int r,
                                              uint32_t (&allow)[4]) {
  if constexpr (!B64) {
    const uint32_t code = lds_u32(tab + 4 * kvb);
    if (code == 0u) return 0;
    if ((code & kCodeTypeMask) == kTypeFull && !(code & kCodeClip)) return 1;
    build_allow(p, code, kvb, r, allow);
    return 2;
  } else {
    const uint4 c = lds_v4(tab + 16 * kvb);
    if ((c.x | c.y | c.z | c.w) == 0u) return 0;
    const uint32_t c0 = r < 64 ? c.x : c.z, c1 = r < 64 ? c.y : c.w;
    if (c0 == static_cast<uint32_t>(kTypeFull) && c1 == static_cast<uint32_t>(kTypeFull)) return 1;
    build_allow_sub64(p, c0, 2 * kvb, r & 63, allow[0], allow[1]);
    build_allow_sub64(p, c1, 2 * kvb + 1, r & 63, allow[2], allow[3]);
    return 2;
  }
}

// Does any row of the tile visit KV block kvb?
template <bool B64>
__device__ __forceinline__ bool tile_visits(uint32_t tab, int kvb) {
  if constexpr (!B64) {
    return lds_u32(tab + 4 * kvb) != 0u;
  } else {
    const uint4 c = lds_v4(tab + 16 * kvb);
    return (c.x | c.y | c.z | c.w) != 0u;
  }
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

// Running softmax state of one query row (one thread). The reference maximum is kept in the log2
// domain and is always an integer (the ceiling of scale*log2(e) times the largest raw score seen,
// moved lazily): exp2(s*c - M) then splits into an exact power of two and a fractional part, which
// is what lets part of the exponentials be evaluated on the FMA pipe. Any per-row constant factor
// in P cancels in O = (sum P V) / (sum P); the log-sum-exp is M*ln2 + ln(l).
struct RowState {
  float M;  // integer-valued reference maximum in log2 units, -inf before the first allowed key
  float l;  // running sum of exp2(s * scale_log2 - M)
};

// Read the 128 raw scores of this thread's row from TMEM.
__device__ __forceinline__ void load_scores(uint32_t taddr_row, float (&s)[128]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr_row + 32 * c, r);
#pragma unroll
    for (int j = 0; j < 32; ++j) s[32 * c + j] = __uint_as_float(r[j]);
  }
  tc_wait_ld();
}

__device__ __forceinline__ void apply_allow(const uint32_t (&allow)[4], float (&s)[128]) {
#pragma unroll
  for (int j = 0; j < 128; ++j) {
    s[j] = ((allow[j >> 5] >> (j & 31)) & 1u) ? s[j] : -INFINITY;
  }
}

// Tanh soft-cap of the Transfusion attention (transfusion_pytorch/transfusion.py:298-299, :358-364,
// :967): scaled score -> softcap * tanh(scaled score / softcap), applied before masking. The raw
// score s is replaced by the raw score that gives the capped value, (softcap / scale) * tanh(s *
// scale / softcap), so everything downstream is unchanged. tanh(y) = 1 - 2 / (exp(2y) + 1) with
// ex2.approx and rcp.approx (absolute error around 1e-7; tanh.approx would be 2^-11 relative, too
// coarse for a log-sum-exp tolerance of 1e-3 once multiplied by the cap).
// Small arguments, which is what a cap of 50 gives for ordinary scores, do not need the MUFU unit at
// all: for |y| <= 0.25 the odd Taylor polynomial of degree 7 is within 1e-7 of tanh. Rows whose largest
// |y| is beyond that take the exact form (a per-thread branch, rare).
constexpr float kTanhPolyLimit = 0.25f;
__device__ __forceinline__ float2 tanh_small2(float2 y) {
  const float2 y2 = __fmul2_rn(y, y);
  float2 p = __ffma2_rn(y2, make_float2(-17.f / 315.f, -17.f / 315.f), make_float2(2.f / 15.f, 2.f / 15.f));
  p = __ffma2_rn(p, y2, make_float2(-1.f / 3.f, -1.f / 3.f));
  p = __ffma2_rn(p, y2, make_float2(1.f, 1.f));
  return __fmul2_rn(y, p);
}
__device__ __forceinline__ float tanh_exact(float y) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(ex2_approx(y * 2.8853900817779268f) + 1.f));   // 2 * log2(e)
  return fmaf(-2.f, r, 1.f);
}

__device__ __forceinline__ float absmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(fabsf(b)), "f"(fabsf(c)));
  return d;
}

__device__ __forceinline__ void soft_cap_scores(float (&s)[128], float cap_in, float cap_out) {
  float a = 0.f, b = 0.f;
#pragma unroll
  for (int j = 0; j < 128; j += 4) {
    a = absmax3(a, s[j], s[j + 1]);
    b = absmax3(b, s[j + 2], s[j + 3]);
  }
  if (fmaxf(a, b) * cap_in <= kTanhPolyLimit) {
    // cap_out * tanh_small(s * cap_in) with the two factors folded into the coefficients
    // (cap_in * cap_out = 1): s + s * z * (b1 + z * (b2 + z * b3)), z = s * s
    const float c2 = cap_in * cap_in;
    const float b1 = (-1.f / 3.f) * c2, b2 = (2.f / 15.f) * c2 * c2, b3 = (-17.f / 315.f) * c2 * c2 * c2;
    const float2 b1v = make_float2(b1, b1), b2v = make_float2(b2, b2), b3v = make_float2(b3, b3);
#pragma unroll
    for (int j = 0; j < 128; j += 2) {
      const float2 x = make_float2(s[j], s[j + 1]);
      const float2 z = __fmul2_rn(x, x);
      float2 p = __ffma2_rn(z, b3v, b2v);
      p = __ffma2_rn(p, z, b1v);
      p = __fmul2_rn(p, z);
      const float2 t = __ffma2_rn(x, p, x);
      s[j] = t.x;
      s[j + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 128; ++j) s[j] = cap_out * tanh_exact(s[j] * cap_in);
  }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float row_max(const float (&s)[128]) {
  float a = s[0], b = s[1], c = s[2], d = s[3];
#pragma unroll
  for (int j = 4; j < 124; j += 8) {
    a = max3(a, s[j], s[j + 1]);
    b = max3(b, s[j + 2], s[j + 3]);
    c = max3(c, s[j + 4], s[j + 5]);
    d = max3(d, s[j + 6], s[j + 7]);
  }
  a = max3(a, s[124], s[125]);
  b = max3(b, s[126], s[127]);
  return fmaxf(max3(a, b, c), d);
}

// Online-softmax update for one tile. `lazy_log2` > 0 keeps the old reference maximum while the
// tile maximum exceeds it by at most that many powers of two (the exponentials then reach
// 2^lazy_log2, harmless in fp32 sums and in 16-bit P). Returns the factor the O accumulator and
// the running sum must be multiplied by before this tile is added (1 when the maximum did not move).
__device__ __forceinline__ float softmax_update(RowState& st, float tile_max, float scale_log2,
                                                float lazy_log2) {
  const float M_old = st.M;
  float M_new = fmaxf(M_old, ceilf(tile_max * scale_log2));
  if (lazy_log2 > 0.f && M_old != -INFINITY && M_new - M_old <= lazy_log2) M_new = M_old;
  float alpha = 1.f;
  if (M_new != M_old) {
    // M_old == -inf gives exp2(-inf) = 0: nothing accumulated so far survives, which is right.
    alpha = ex2_approx(M_old - M_new);
    st.M = M_new;
  }
  return alpha;
}

// 2^r on [-0.5, 0.5], degree-3 minimax polynomial (max relative error 7.5e-5; P is rounded to
// 8 or 11 mantissa bits afterwards).
constexpr float kExp2C0 = 0.9999280571937561f;
constexpr float kExp2C1 = 0.6932610273361206f;
constexpr float kExp2C2 = 0.24261116981506348f;
constexpr float kExp2C3 = 0.0551714189350605f;
constexpr float kRoundMagic = 12582912.f;  // 1.5 * 2^23: adding it rounds to the nearest integer

// P = exp2(s * scale_log2 - M) for NS scores of a row (the whole row, or half of it in the two-pass
// form), packed to 16-bit pairs; returns the sum of the unrounded exponentials. Packed two-wide fp32
// arithmetic throughout. Of every kPolyDen element pairs, kPolyNum are evaluated without the MUFU
// unit: n = round(x) comes out of one fused multiply-add against the rounding constant, 2^(x-n) from
// the polynomial, and 2^n is added into the exponent field; the other pairs use ex2.approx. That
// balances the 16/clk MUFU against the FMA pipe. A row with no allowed key so far has M = -inf and
// every s = -inf: P is then 0 (MUFU lanes) or below 2^-119 (polynomial lanes, wiped by the next rescale).
template <bool BF16, int kPolyNum, int kPolyDen, int NS>
__device__ __forceinline__ float exp_and_pack_n(const float (&s)[NS], float M, float scale_log2,
                                                float inv_scale_log2, uint32_t (&pk)[NS / 2]) {
  const float M_use = (M == -INFINITY) ? 0.f : M;
  const float2 c2 = make_float2(scale_log2, scale_log2);
  const float2 negM2 = make_float2(-M_use, -M_use);
  const float K = kRoundMagic - M_use;  // exact: both are integers below 2^24
  const float2 K2 = make_float2(K, K);
  const float2 minus1 = make_float2(-1.f, -1.f);
  const float s_min = (M_use - 120.f) * inv_scale_log2;  // keeps x >= -120 in the polynomial lanes
  float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < NS / 2; ++j) {
    float2 p2;
    if ((j % kPolyDen) < kPolyNum) {
      const float2 s2 = make_float2(fmaxf(s[2 * j], s_min), fmaxf(s[2 * j + 1], s_min));
      const float2 t2 = __ffma2_rn(s2, c2, K2);          // magic + round(x)
      const float2 a2 = __ffma2_rn(t2, minus1, K2);      // -(M + round(x))
      const float2 r2 = __ffma2_rn(s2, c2, a2);          // x - round(x)
      float2 q2 = __ffma2_rn(r2, make_float2(kExp2C3, kExp2C3), make_float2(kExp2C2, kExp2C2));
      q2 = __ffma2_rn(q2, r2, make_float2(kExp2C1, kExp2C1));
      q2 = __ffma2_rn(q2, r2, make_float2(kExp2C0, kExp2C0));
      p2.x = __int_as_float(__float_as_int(q2.x) + (__float_as_int(t2.x) << 23));
      p2.y = __int_as_float(__float_as_int(q2.y) + (__float_as_int(t2.y) << 23));
    } else {
      const float2 x2 = __ffma2_rn(make_float2(s[2 * j], s[2 * j + 1]), c2, negM2);
      p2.x = ex2_approx(x2.x);
      p2.y = ex2_approx(x2.y);
    }
    sum2 = __fadd2_rn(sum2, p2);
    pk[j] = pack2<BF16>(p2.x, p2.y);
  }
  return sum2.x + sum2.y;
}

// ---------------------------------------------------------------------------------------------
// Half-row (64 score) versions used by the warp-specialised kernel. It makes two passes over the
// scores in TMEM - first the row maximum, then exponentials - 64 columns at a time, so that only
// half a row is ever live in registers; re-reading S from TMEM costs a few tens of cycles, keeping
// all 128 scores plus the packed P in registers costs spills.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void load_scores64(uint32_t taddr_row, float (&s)[64]) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr_row + 32 * c, r);
#pragma unroll
    for (int j = 0; j < 32; ++j) s[32 * c + j] = __uint_as_float(r[j]);
  }
  tc_wait_ld();
}

// allow0/allow1: the two allow words of this half (columns [64h, 64h+64)).
__device__ __forceinline__ void apply_allow64(uint32_t allow0, uint32_t allow1, float (&s)[64]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) s[j] = ((allow0 >> j) & 1u) ? s[j] : -INFINITY;
#pragma unroll
  for (int j = 0; j < 32; ++j) s[32 + j] = ((allow1 >> j) & 1u) ? s[32 + j] : -INFINITY;
}

__device__ __forceinline__ float row_max64(const float (&s)[64]) {
  float a = s[0], b = s[1], c = s[2], d = s[3];
#pragma unroll
  for (int j = 4; j < 60; j += 8) {
    a = max3(a, s[j], s[j + 1]);
    b = max3(b, s[j + 2], s[j + 3]);
    c = max3(c, s[j + 4], s[j + 5]);
    d = max3(d, s[j + 6], s[j + 7]);
  }
  a = max3(a, s[60], s[61]);
  b = max3(b, s[62], s[63]);
  return fmaxf(max3(a, b, c), d);
}

// Write the packed P row (64 words) to TMEM columns [taddr_row, taddr_row + 64).
__device__ __forceinline__ void store_p(uint32_t taddr_row, const uint32_t (&pk)[64]) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = pk[32 * c + j];
    tmem_st32(taddr_row + 32 * c, r);
  }
}

// O[row, :] *= alpha in TMEM (D fp32 columns starting at taddr_row).
template <int D>
__device__ __forceinline__ void rescale_o(uint32_t taddr_row, float alpha) {
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr_row + 32 * c, r);
    tc_wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
    tmem_st32(taddr_row + 32 * c, r);
  }
}

// Final normalisation and store of one output row: O = acc / l (0 when the row attended nothing),
// LSE = M * ln2 + ln(l) (-inf when the row attended nothing). `zero_row` forces zeros (padding).
// Only the first p.d_real of the D accumulator columns exist in memory (head_dim 32 is computed as 64).
template <int D, bool BF16>
__device__ __forceinline__ void store_output_row(uint32_t taddr_row, bool have_acc,
                                                 const RowState& st, const FwdParams& p,
                                                 long long row_index, bool zero_row) {
  const bool empty = zero_row || !have_acc || st.M == -INFINITY || !(st.l > 0.f);
  const float inv = empty ? 0.f : 1.f / st.l;
  uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(p.o) + row_index * (p.d_real * 2));
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    if (32 * c >= p.d_real) break;
    uint32_t r[32];
    if (have_acc) {  // uniform across the CTA's softmax threads of this tile
      tmem_ld32(taddr_row + 32 * c, r);
      tc_wait_ld();
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = 0u;
    }
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float a = empty ? 0.f : __uint_as_float(r[2 * j]) * inv;
      const float b = empty ? 0.f : __uint_as_float(r[2 * j + 1]) * inv;
      w[j] = pack2<BF16>(a, b);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      dst[4 * c + j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    }
  }
  if (p.lse != nullptr) {
    p.lse[row_index] = empty ? -INFINITY : fmaf(st.M, 0.6931471805599453f, __logf(st.l));
  }
}

}  // namespace omni
