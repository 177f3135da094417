// Block-mask construction on the GPU from modality (image span) positions.
//
// Replaces the host-side builder create_omni_block_mask_from_modality_positions
// (omni-attn-mma/omni_attn_torch.py:1518-1736), which walks every (Q block, KV block) pair in Python,
// materialises the dense [B, N, N] mask of transfusion_pytorch/transfusion.py:496-515
// (causal | any_m(q >= offset_m & k < offset_m + length_m)) and cuts the PARTIAL tiles out of it
// (build_partial_block_data, omni_attn_torch.py:148-205).
//
// Here nothing N x N is ever built. Under that rule every query row q attends one contiguous key
// range [0, limit(q)], limit(q) = max(q, max over spans with offset <= q of offset + length - 1),
// clipped to the unpadded length. A (Q block, KV block) tile is therefore fully described by the
// smallest and largest limit of the block's 128 rows:
//     all keys allowed for all rows  -> FULL          no key allowed for any row -> not listed
//     diagonal tile of a block whose rows are all plain causal rows (no row inside a span) -> CAUSAL
//     anything else -> PARTIAL, element (r, c) allowed iff c <= limit(r) - 128 * kv_block
// which is the block-type derivation of omni-attn-mma/generate_attn_data.py:200-236 applied to the
// dense rule. PARTIAL tiles are written bit-packed ([P,128,4] words) and, optionally, in the
// reference's byte-per-element form; the pool is shared by all heads of a batch element.
//
// Three small kernels: (1) one CTA per (batch, Q block) classifies the row of tiles, compacts the
// listed KV blocks in ascending order for head 0 and counts its PARTIAL tiles; (2) one CTA turns the
// counts into pool offsets; (3) one CTA per (batch, Q block) writes the pool tiles and replicates
// the lists over the heads. All of it is HBM-write bound (the index tensors).
#include <cstdint>

#include "../../include/omni_attn_sm100.h"
#include "omni_common.cuh"

namespace omni {
namespace {

constexpr int kMaskThreads = 128;

struct MaskParams {
  const int32_t* modality_positions;  // [B, M, 3] (type, offset, length)
  int32_t* kv_num_blocks;             // [B, H, nq]
  int32_t* kv_indices;                // [B, H, nq, nq]
  int32_t* block_mask_types;          // [B, H, nq, nq]
  int32_t* partial_idx;               // [B, H, nq, nq]
  uint32_t* partial_bits;             // [capacity, 128, 4]
  uint8_t* partial_bool;              // [capacity, 128, 128] or null
  int32_t* num_partial_out;           // device int
  int32_t* counts;                    // scratch [B * nq]
  int32_t* bases;                     // scratch [B * nq]
  int B, M, H, seqlen, nq, capacity;
};

// limit of row q (-1 = the row attends nothing) and whether it is a plain causal row
__device__ __forceinline__ int row_limit(const MaskParams& p, int b, int q, bool& plain) {
  plain = true;
  if (q >= p.seqlen) {
    plain = false;
    return -1;
  }
  int lim = q;
  const int32_t* m = p.modality_positions + static_cast<long long>(b) * p.M * 3;
  for (int i = 0; i < p.M; ++i) {
    const int off = __ldg(m + 3 * i + 1);
    const int len = __ldg(m + 3 * i + 2);
    if (len > 0 && q >= off) {
      lim = max(lim, off + len - 1);
      if (q < off + len) plain = false;
    }
  }
  return min(lim, p.seqlen - 1);
}

__device__ __forceinline__ int tile_type(int lim_min, int lim_max, bool causal_block, int qb, int kb) {
  const int k0 = kb * kBlock;
  if (lim_max < k0) return kTypeMasked;
  if (lim_min >= k0 + kBlock - 1) return kTypeFull;
  if (kb == qb && causal_block) return kTypeCausal;
  return kTypePartial;
}

// block-wide min / max / and over 128 threads
__device__ __forceinline__ void block_limits(int lim, bool plain_and_causal, int* smem, int& lim_min, int& lim_max,
                                             bool& causal_block) {
  int mn = lim, mx = lim;
  int ok = plain_and_causal ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = min(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o));
    mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    ok &= __shfl_xor_sync(0xFFFFFFFFu, ok, o);
  }
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) {
    smem[w] = mn;
    smem[4 + w] = mx;
    smem[8 + w] = ok;
  }
  __syncthreads();
  lim_min = min(min(smem[0], smem[1]), min(smem[2], smem[3]));
  lim_max = max(max(smem[4], smem[5]), max(smem[6], smem[7]));
  causal_block = (smem[8] & smem[9] & smem[10] & smem[11]) != 0;
  __syncthreads();
}

__global__ void __launch_bounds__(kMaskThreads) mask_classify_kernel(const MaskParams p) {
  __shared__ int red[12];
  __shared__ int warp_tot[4], warp_part[4];
  const int qb = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
  bool plain;
  const int q = qb * kBlock + t;
  const int lim = row_limit(p, b, q, plain);
  int lim_min, lim_max;
  bool causal_block;
  block_limits(lim, plain && lim == q, red, lim_min, lim_max, causal_block);

  const long long row = (static_cast<long long>(b) * p.H * p.nq + qb) * p.nq;  // head 0
  int n_listed = 0, n_partial = 0;
  for (int base = 0; base < p.nq; base += kMaskThreads) {
    const int kb = base + t;
    const int type = kb < p.nq ? tile_type(lim_min, lim_max, causal_block, qb, kb) : kTypeMasked;
    const bool listed = type != kTypeMasked, part = type == kTypePartial;
    const uint32_t bl = __ballot_sync(0xFFFFFFFFu, listed), bp = __ballot_sync(0xFFFFFFFFu, part);
    const int w = t >> 5, lane = t & 31;
    if (lane == 0) {
      warp_tot[w] = __popc(bl);
      warp_part[w] = __popc(bp);
    }
    __syncthreads();
    int pos = n_listed, ppos = n_partial;
    for (int i = 0; i < w; ++i) {
      pos += warp_tot[i];
      ppos += warp_part[i];
    }
    pos += __popc(bl & ((1u << lane) - 1u));
    ppos += __popc(bp & ((1u << lane) - 1u));
    if (listed) {
      p.kv_indices[row + pos] = kb;
      p.block_mask_types[row + pos] = type;
      p.partial_idx[row + pos] = part ? ppos : -1;   // position among this row's PARTIAL tiles for now
    }
    n_listed += warp_tot[0] + warp_tot[1] + warp_tot[2] + warp_tot[3];
    n_partial += warp_part[0] + warp_part[1] + warp_part[2] + warp_part[3];
    __syncthreads();
  }
  for (int i = n_listed + t; i < p.nq; i += kMaskThreads) {   // unused tail of the list
    p.kv_indices[row + i] = 0;
    p.block_mask_types[row + i] = kTypeMasked;
    p.partial_idx[row + i] = -1;
  }
  if (t == 0) {
    p.kv_num_blocks[(static_cast<long long>(b) * p.H) * p.nq + qb] = n_listed;
    p.counts[b * p.nq + qb] = n_partial;
  }
}

// exclusive scan of counts[B * nq] by one CTA (a few thousand entries at most)
__global__ void __launch_bounds__(1024) mask_scan_kernel(const MaskParams p) {
  __shared__ int part[1024];
  const int n = p.B * p.nq;
  const int per = (n + 1023) / 1024;
  const int lo = min(n, static_cast<int>(threadIdx.x) * per), hi = min(n, lo + per);
  int s = 0;
  for (int i = lo; i < hi; ++i) s += p.counts[i];
  part[threadIdx.x] = s;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int v = threadIdx.x >= o ? part[threadIdx.x - o] : 0;
    __syncthreads();
    part[threadIdx.x] += v;
    __syncthreads();
  }
  int run = part[threadIdx.x] - s;
  for (int i = lo; i < hi; ++i) {
    p.bases[i] = run;
    run += p.counts[i];
  }
  if (threadIdx.x == 1023) *p.num_partial_out = part[1023];
}

__global__ void __launch_bounds__(kMaskThreads) mask_emit_kernel(const MaskParams p) {
  const int qb = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
  bool plain;
  const int lim = row_limit(p, b, qb * kBlock + t, plain);

  const long long row = (static_cast<long long>(b) * p.H * p.nq + qb) * p.nq;  // head 0
  const int n_listed = p.kv_num_blocks[(static_cast<long long>(b) * p.H) * p.nq + qb];
  const int base = p.bases[b * p.nq + qb];
  // pool tiles: thread t owns row t of every PARTIAL tile of this Q block
  for (int i = 0; i < n_listed; ++i) {
    const int local = p.partial_idx[row + i];
    if (local < 0) continue;
    const int pool = base + local;
    if (pool >= p.capacity) continue;   // reported through num_partial_out > capacity
    const int kb = p.kv_indices[row + i];
    const int cnt = min(max(lim + 1 - kb * kBlock, 0), kBlock);   // allowed columns of this row
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = cnt - 32 * j;
      w[j] = d >= 32 ? 0xFFFFFFFFu : (d <= 0 ? 0u : ((1u << d) - 1u));
    }
    reinterpret_cast<uint4*>(p.partial_bits)[static_cast<size_t>(pool) * kBlock + t] = make_uint4(w[0], w[1], w[2], w[3]);
    if (p.partial_bool != nullptr) {
      uint4* dst = reinterpret_cast<uint4*>(p.partial_bool + (static_cast<size_t>(pool) * kBlock + t) * kBlock);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t x[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c0 = 16 * j + 4 * k;
          x[k] = (c0 < cnt ? 1u : 0u) | (c0 + 1 < cnt ? 0x100u : 0u) | (c0 + 2 < cnt ? 0x10000u : 0u) |
                 (c0 + 3 < cnt ? 0x1000000u : 0u);
        }
        dst[j] = make_uint4(x[0], x[1], x[2], x[3]);
      }
    }
  }
  __syncthreads();
  // final pool indices for head 0, then the same list for every other head
  for (int i = t; i < p.nq; i += kMaskThreads) {
    const int kvb = p.kv_indices[row + i];
    const int typ = p.block_mask_types[row + i];
    int pi = p.partial_idx[row + i];
    if (pi >= 0) pi += base;
    p.partial_idx[row + i] = pi;
    for (int h = 1; h < p.H; ++h) {
      const long long r2 = row + static_cast<long long>(h) * p.nq * p.nq;
      p.kv_indices[r2 + i] = kvb;
      p.block_mask_types[r2 + i] = typ;
      p.partial_idx[r2 + i] = pi;
    }
  }
  if (t == 0) {
    for (int h = 1; h < p.H; ++h) {
      p.kv_num_blocks[(static_cast<long long>(b) * p.H + h) * p.nq + qb] = n_listed;
    }
  }
}

}  // namespace
}  // namespace omni

extern "C" int omni_attn_build_mask_sm100(const int32_t* modality_positions, int B, int M, int H, int seqlen,
                                          int seqlen_padded, int32_t* kv_num_blocks, int32_t* kv_indices,
                                          int32_t* block_mask_types, int32_t* partial_idx, uint32_t* partial_bits,
                                          uint8_t* partial_bool_or_null, int partial_capacity,
                                          int32_t* num_partial_out, void* scratch, long long scratch_bytes,
                                          void* cuda_stream) {
  using namespace omni;
  if (kv_num_blocks == nullptr || kv_indices == nullptr || block_mask_types == nullptr || partial_idx == nullptr ||
      num_partial_out == nullptr || scratch == nullptr || (M > 0 && modality_positions == nullptr) ||
      (partial_capacity > 0 && partial_bits == nullptr)) {
    return OMNI_ERR_NULL_POINTER;
  }
  if (B <= 0 || H <= 0 || M < 0 || B > 65535) return OMNI_ERR_SHAPE;
  if (seqlen_padded <= 0 || seqlen_padded % kBlock != 0 || seqlen <= 0 || seqlen > seqlen_padded) return OMNI_ERR_SEQLEN;
  const int nq = seqlen_padded / kBlock;
  if (nq > 1024) return OMNI_ERR_TOO_LONG;
  if (partial_capacity < 0) return OMNI_ERR_PARTIAL;
  if (scratch_bytes < 2LL * B * nq * static_cast<long long>(sizeof(int32_t))) return OMNI_ERR_SCRATCH;
  if ((reinterpret_cast<uintptr_t>(partial_bits) & 15u) || (reinterpret_cast<uintptr_t>(partial_bool_or_null) & 15u)) {
    return OMNI_ERR_ALIGNMENT;
  }
  MaskParams p;
  p.modality_positions = modality_positions;
  p.kv_num_blocks = kv_num_blocks;
  p.kv_indices = kv_indices;
  p.block_mask_types = block_mask_types;
  p.partial_idx = partial_idx;
  p.partial_bits = partial_bits;
  p.partial_bool = partial_bool_or_null;
  p.num_partial_out = num_partial_out;
  p.counts = static_cast<int32_t*>(scratch);
  p.bases = p.counts + static_cast<long long>(B) * nq;
  p.B = B; p.M = M; p.H = H; p.seqlen = seqlen; p.nq = nq; p.capacity = partial_capacity;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const dim3 grid(nq, B);
  mask_classify_kernel<<<grid, kMaskThreads, 0, st>>>(p);
  mask_scan_kernel<<<1, 1024, 0, st>>>(p);
  mask_emit_kernel<<<grid, kMaskThreads, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? OMNI_OK : OMNI_ERR_CUDA;
}
