// C-ABI layer of libomni_attn_sm100.so: argument validation (the checks of the reference's host
// launchers, omni-attn-mma/mma/omni_attn_shared_kv.cu:701-753, as error codes instead of
// exceptions), TMA tensor-map construction and kernel dispatch.
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "../../include/omni_attn_sm100.h"
#include "omni_launch.h"

namespace omni {
namespace {

thread_local int g_last_cuda_error = 0;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library has no link-time
// dependency on libcuda (it must load on a machine without a driver for symbol checks).
EncodeTiledFn get_encode_fn() {
  static const EncodeTiledFn fn = [] {   // initialised once, whichever host thread comes first
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) return reinterpret_cast<EncodeTiledFn>(ptr);
    (void)cudaGetLastError();
    return static_cast<EncodeTiledFn>(nullptr);
  }();
  return fn;
}

// [rows, head_dim] 16-bit row-major view of one of Q/K/V; box = 128 rows x 64 columns (128 bytes),
// 128-byte swizzle, which is the layout the UMMA shared-memory descriptors of the kernels expect.
int make_tile_map(CUtensorMap* tm, const void* base, long long rows, int head_dim, bool bf16) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return OMNI_ERR_NO_DRIVER_ENTRY;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(head_dim) * 2};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return OMNI_ERR_CUDA;
  }
  return OMNI_OK;
}

// [BH, N, head_dim] view of one of Q/K/V for the forward kernels; box = 128 rows x 64 columns of one
// (batch, head), 128-byte swizzle. Rows beyond N and columns beyond head_dim (head_dim 32) read as zeros.
int make_tile_map_3d(CUtensorMap* tm, const void* base, long long BH, int seqlen, int head_dim, bool bf16) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return OMNI_ERR_NO_DRIVER_ENTRY;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(seqlen),
                              static_cast<cuuint64_t>(BH)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2,
                                 static_cast<cuuint64_t>(head_dim) * 2 * static_cast<cuuint64_t>(seqlen)};
  const cuuint32_t box[3] = {64, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return OMNI_ERR_CUDA;
  }
  return OMNI_OK;
}

// Heads per scheduling group of the warp-specialised kernel: as many heads as keep the group's K and
// V (2 * N * D * 2 bytes per head) inside an L2 budget, 48 MB of the B200's 126 MB unless the
// environment variable OMNI_ATTN_L2_MB says otherwise.
int group_heads_for(long long BH, int seqlen, int head_dim) {
  static const long long budget = [] {
    const char* e = std::getenv("OMNI_ATTN_L2_MB");
    const long long mb = e != nullptr ? std::atoll(e) : 48;
    return (mb > 0 ? mb : 48) << 20;
  }();
  const long long per_head = 4LL * seqlen * head_dim;
  long long g = budget / per_head;
  if (g < 1) g = 1;
  if (g > BH) g = BH;
  return static_cast<int>(g);
}

// Cycle budget of the forward kernels' bounded waits (omni_attn_set_wait_cycles).
std::atomic<long long> g_wait_cycles{kWaitCycleLimit};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// cuTensorMapEncodeTiled is a driver call and wants a context current on the calling thread. A
// thread that has made no runtime call yet (a framework's worker thread that found its buffers in a
// cache, for instance) has none; setting the runtime's current device again binds the primary context.
int bind_context() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaSetDevice(dev);
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return OMNI_ERR_CUDA;
  }
  return OMNI_OK;
}

// The argument checks of the forward entry points: the list of the reference's launchers
// (omni-attn-mma/mma/omni_attn_shared_kv.cu:701-753) plus what plain pointers need. Nothing is
// launched and no CUDA call is made.
int validate_forward(bool simple, const void* q, const void* k, const void* v, void* o,
                     const int32_t* kv_num_blocks, const int32_t* kv_indices, const int32_t* types,
                     const uint8_t* partial_bool, const uint32_t* partial_bits, int B, int H, int seqlen_padded,
                     int seqlen_orig, int head_dim, int q_block, int kv_block, int max_blocks, int num_partial,
                     int dtype, const void* scratch, float softcap) {
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || kv_num_blocks == nullptr ||
      kv_indices == nullptr || types == nullptr) {
    return OMNI_ERR_NULL_POINTER;
  }
  if (dtype != OMNI_DTYPE_F16 && dtype != OMNI_DTYPE_BF16) return OMNI_ERR_DTYPE;
  if (head_dim != 32 && head_dim != 64 && head_dim != 128) return OMNI_ERR_HEAD_DIM;
  if (q_block != kv_block || (q_block != 64 && q_block != kBlock)) return OMNI_ERR_BLOCK_SIZE;
  if (seqlen_padded <= 0 || seqlen_padded % q_block != 0 || seqlen_orig <= 0 || seqlen_orig > seqlen_padded) {
    return OMNI_ERR_SEQLEN;
  }
  if (B <= 0 || H <= 0 || max_blocks <= 0) return OMNI_ERR_SHAPE;
  const long long BH = static_cast<long long>(B) * H;
  if (BH > 65535) return OMNI_ERR_SHAPE;
  if (softcap < 0.f || softcap != softcap) return OMNI_ERR_SOFTCAP;
  if (simple && softcap > 0.f) return OMNI_ERR_SOFTCAP;
  if (num_partial < 0) return OMNI_ERR_PARTIAL;
  if (num_partial > 0 && partial_bool == nullptr && partial_bits == nullptr) return OMNI_ERR_PARTIAL;
  const bool b64 = q_block == 64;
  const int nq = (seqlen_padded + kBlock - 1) / kBlock;
  const int max_tiles = simple ? simple_max_tiles(b64) : ws_max_tiles(head_dim == 128 ? 128 : 64, b64);
  if (nq > max_tiles) return OMNI_ERR_TOO_LONG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(partial_bool) ||
      !aligned16(partial_bits) || !aligned16(scratch)) {
    return OMNI_ERR_ALIGNMENT;
  }
  return OMNI_OK;
}

int forward(bool simple, const void* q, const void* k, const void* v, void* o, float* lse,
            const int32_t* kv_num_blocks, const int32_t* kv_indices, const int32_t* types,
            const int32_t* partial_idx, const uint8_t* partial_bool, const uint32_t* partial_bits, int B,
            int H, int seqlen_padded, int seqlen_orig, int head_dim, int q_block, int kv_block,
            int max_blocks, int num_partial, int dtype, float scale, void* stream, int32_t* status,
            void* scratch, float softcap = 0.f) {
  int rc = validate_forward(simple, q, k, v, o, kv_num_blocks, kv_indices, types, partial_bool, partial_bits, B, H,
                            seqlen_padded, seqlen_orig, head_dim, q_block, kv_block, max_blocks, num_partial, dtype,
                            scratch, softcap);
  if (rc != OMNI_OK) return rc;
  const long long BH = static_cast<long long>(B) * H;
  const bool bf16 = dtype == OMNI_DTYPE_BF16;
  // head_dim 32 is computed by the 64-wide kernels: the TMA unit reads the missing columns as zeros
  const int compute_dim = head_dim == 128 ? 128 : 64;
  CUtensorMap tmQ, tmK, tmV;
  rc = bind_context();
  if (rc != OMNI_OK) return rc;
  rc = make_tile_map_3d(&tmQ, q, BH, seqlen_padded, head_dim, bf16);
  if (rc != OMNI_OK) return rc;
  rc = make_tile_map_3d(&tmK, k, BH, seqlen_padded, head_dim, bf16);
  if (rc != OMNI_OK) return rc;
  rc = make_tile_map_3d(&tmV, v, BH, seqlen_padded, head_dim, bf16);
  if (rc != OMNI_OK) return rc;

  FwdParams p;
  p.o = o;
  p.lse = lse;
  p.kv_num_blocks = kv_num_blocks;
  p.kv_indices = kv_indices;
  p.types = types;
  p.partial_idx = num_partial > 0 ? partial_idx : nullptr;
  p.partial_bool = num_partial > 0 ? partial_bool : nullptr;
  p.partial_bits = num_partial > 0 ? partial_bits : nullptr;
  p.status = status;
  p.unit_counter = static_cast<int32_t*>(scratch);
  p.num_units = 0;
  p.o_aligned32 = (reinterpret_cast<uintptr_t>(o) & 31u) == 0 ? 1 : 0;
  p.BH = static_cast<int>(BH);
  p.N = seqlen_padded;
  p.seqlen_orig = seqlen_orig;
  p.nq = (seqlen_padded + kBlock - 1) / kBlock;
  p.max_blocks = max_blocks;
  p.num_partial = num_partial;
  p.scale = scale > 0.f ? scale : 1.f / std::sqrt(static_cast<float>(head_dim));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  p.inv_scale_log2 = 1.f / p.scale_log2;
  p.cap_in = softcap > 0.f ? p.scale / softcap : 0.f;
  p.cap_out = softcap > 0.f ? softcap / p.scale : 0.f;
  p.group_heads = group_heads_for(BH, seqlen_padded, head_dim);
  p.d_real = head_dim;
  p.blk64 = q_block == 64 ? 1 : 0;
  p.nq_lists = seqlen_padded / q_block;
  p.wait_cycles = g_wait_cycles.load(std::memory_order_relaxed);

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = simple ? launch_simple(compute_dim, bf16, tmQ, tmK, tmV, p, st)
                         : launch_ws(compute_dim, bf16, tmQ, tmK, tmV, p, st);
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return OMNI_ERR_CUDA;
  }
  return OMNI_OK;
}

long long bwd_workspace_bytes(long long BH, int seqlen_padded) {
  const long long nq = seqlen_padded / kBlock;
  const long long codes = ((BH * nq * nq * 4 + 255) / 256) * 256;
  return codes + BH * seqlen_padded * 4;
}

int backward(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
             void* dq, void* dk, void* dv, const int32_t* kv_num_blocks, const int32_t* kv_indices,
             const int32_t* types, const int32_t* partial_idx, const uint8_t* partial_bool,
             const uint32_t* partial_bits, int B, int H, int seqlen_padded, int seqlen_orig, int head_dim,
             int q_block, int kv_block, int max_blocks, int num_partial, int dtype, float scale, void* stream,
             int32_t* status, void* workspace, long long workspace_bytes, float softcap = 0.f) {
  if (softcap < 0.f || softcap != softcap) return OMNI_ERR_SOFTCAP;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || lse == nullptr || d_o == nullptr ||
      dq == nullptr || dk == nullptr || dv == nullptr || kv_num_blocks == nullptr || kv_indices == nullptr ||
      types == nullptr || workspace == nullptr) {
    return OMNI_ERR_NULL_POINTER;
  }
  if (dtype != OMNI_DTYPE_F16 && dtype != OMNI_DTYPE_BF16) return OMNI_ERR_DTYPE;
  if (head_dim != 32 && head_dim != 64 && head_dim != 128) return OMNI_ERR_HEAD_DIM;
  if (q_block != kBlock || kv_block != kBlock) return OMNI_ERR_BLOCK_SIZE;
  if (seqlen_padded <= 0 || seqlen_padded % kBlock != 0 || seqlen_orig <= 0 || seqlen_orig > seqlen_padded) {
    return OMNI_ERR_SEQLEN;
  }
  if (B <= 0 || H <= 0 || max_blocks <= 0) return OMNI_ERR_SHAPE;
  const long long BH = static_cast<long long>(B) * H;
  const long long rows = BH * seqlen_padded;
  if (rows >= (1LL << 31) || BH > 65535) return OMNI_ERR_SHAPE;
  if (num_partial < 0) return OMNI_ERR_PARTIAL;
  if (num_partial > 0 && partial_bool == nullptr && partial_bits == nullptr) return OMNI_ERR_PARTIAL;
  const int nq = seqlen_padded / kBlock;
  if (nq > kMaxKvBlocks) return OMNI_ERR_TOO_LONG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(d_o) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv) || !aligned16(partial_bool) || !aligned16(partial_bits) ||
      !aligned16(workspace)) {
    return OMNI_ERR_ALIGNMENT;
  }
  if (workspace_bytes < bwd_workspace_bytes(BH, seqlen_padded)) return OMNI_ERR_WORKSPACE;

  const bool bf16 = dtype == OMNI_DTYPE_BF16;
  CUtensorMap tmQ, tmK, tmV, tmdO;
  int rc = bind_context();
  if (rc != OMNI_OK) return rc;
  rc = make_tile_map(&tmQ, q, rows, head_dim, bf16);
  if (rc != OMNI_OK) return rc;
  rc = make_tile_map(&tmK, k, rows, head_dim, bf16);
  if (rc != OMNI_OK) return rc;
  rc = make_tile_map(&tmV, v, rows, head_dim, bf16);
  if (rc != OMNI_OK) return rc;
  rc = make_tile_map(&tmdO, d_o, rows, head_dim, bf16);
  if (rc != OMNI_OK) return rc;

  BwdParams p;
  p.f.o = nullptr;
  p.f.lse = nullptr;
  p.f.kv_num_blocks = kv_num_blocks;
  p.f.kv_indices = kv_indices;
  p.f.types = types;
  p.f.partial_idx = num_partial > 0 ? partial_idx : nullptr;
  p.f.partial_bool = num_partial > 0 ? partial_bool : nullptr;
  p.f.partial_bits = num_partial > 0 ? partial_bits : nullptr;
  p.f.status = status;
  p.f.unit_counter = nullptr;
  p.f.BH = static_cast<int>(BH);
  p.f.N = seqlen_padded;
  p.f.seqlen_orig = seqlen_orig;
  p.f.nq = nq;
  p.f.max_blocks = max_blocks;
  p.f.num_partial = num_partial;
  p.f.scale = scale > 0.f ? scale : 1.f / std::sqrt(static_cast<float>(head_dim));
  p.f.scale_log2 = p.f.scale * 1.4426950408889634f;
  p.f.inv_scale_log2 = 1.f / p.f.scale_log2;
  p.f.cap_in = softcap > 0.f ? p.f.scale / softcap : 0.f;
  p.f.cap_out = softcap > 0.f ? softcap / p.f.scale : 0.f;
  // Q, K, V and dO of a head group share L2: half as many heads per group as in the forward pass
  p.f.group_heads = group_heads_for(BH, seqlen_padded, head_dim) / 2 > 0 ? group_heads_for(BH, seqlen_padded, head_dim) / 2 : 1;
  p.f.num_units = 0;
  p.f.o_aligned32 = 0;
  p.f.d_real = head_dim;
  p.f.blk64 = 0;
  p.f.nq_lists = nq;
  p.f.wait_cycles = kWaitCycleLimit;
  p.o = o;
  p.d_o = d_o;
  p.lse = lse;
  p.dq = dq;
  p.dk = dk;
  p.dv = dv;
  p.codes = static_cast<uint32_t*>(workspace);
  p.delta = reinterpret_cast<float*>(static_cast<char*>(workspace) +
                                     ((BH * nq * nq * 4 + 255) / 256) * 256);
  // head_dim 32 runs on the 64-wide kernels: the tensor maps' innermost extent is 32, so the TMA unit
  // fills columns 32..63 of every tile with zeros, which changes none of the five contractions' first 32 columns
  cudaError_t e = launch_bwd(head_dim == 32 ? 64 : head_dim, bf16, tmQ, tmK, tmV, tmdO, p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return OMNI_ERR_CUDA;
  }
  return OMNI_OK;
}

// One thread per output word: 32 mask bytes -> 32 bits.
__global__ void pack_partial_kernel(const uint8_t* __restrict__ src, uint32_t* __restrict__ dst,
                                    long long n_words) {
  const long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  const uint4* s = reinterpret_cast<const uint4*>(src + w * 32);
  const uint4 a = __ldg(s);
  const uint4 b = __ldg(s + 1);
  dst[w] = bytes_to_nibble(a.x) | (bytes_to_nibble(a.y) << 4) | (bytes_to_nibble(a.z) << 8) |
           (bytes_to_nibble(a.w) << 12) | (bytes_to_nibble(b.x) << 16) | (bytes_to_nibble(b.y) << 20) |
           (bytes_to_nibble(b.z) << 24) | (bytes_to_nibble(b.w) << 28);
}

}  // namespace
}  // namespace omni

extern "C" {

int omni_attn_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* lse_or_null,
                        const int32_t* kv_num_blocks, const int32_t* kv_indices,
                        const int32_t* block_mask_types, const int32_t* partial_idx_or_null,
                        const uint8_t* partial_bool_or_null, const uint32_t* partial_bits_or_null,
                        int B, int H, int seqlen_padded, int seqlen_orig, int head_dim, int q_block,
                        int kv_block, int max_blocks, int num_partial, int dtype, float scale,
                        void* cuda_stream, int32_t* device_status_or_null) {
  return omni::forward(false, q, k, v, o, lse_or_null, kv_num_blocks, kv_indices, block_mask_types,
                       partial_idx_or_null, partial_bool_or_null, partial_bits_or_null, B, H,
                       seqlen_padded, seqlen_orig, head_dim, q_block, kv_block, max_blocks, num_partial,
                       dtype, scale, cuda_stream, device_status_or_null, nullptr);
}

int omni_attn_fwd_scratch_sm100(const void* q, const void* k, const void* v, void* o, float* lse_or_null,
                                const int32_t* kv_num_blocks, const int32_t* kv_indices,
                                const int32_t* block_mask_types, const int32_t* partial_idx_or_null,
                                const uint8_t* partial_bool_or_null, const uint32_t* partial_bits_or_null,
                                int B, int H, int seqlen_padded, int seqlen_orig, int head_dim, int q_block,
                                int kv_block, int max_blocks, int num_partial, int dtype, float scale,
                                void* cuda_stream, int32_t* device_status_or_null, void* scratch,
                                long long scratch_bytes) {
  if (scratch == nullptr) return OMNI_ERR_NULL_POINTER;
  if (scratch_bytes < OMNI_ATTN_SCRATCH_BYTES) return OMNI_ERR_SCRATCH;
  return omni::forward(false, q, k, v, o, lse_or_null, kv_num_blocks, kv_indices, block_mask_types,
                       partial_idx_or_null, partial_bool_or_null, partial_bits_or_null, B, H,
                       seqlen_padded, seqlen_orig, head_dim, q_block, kv_block, max_blocks, num_partial,
                       dtype, scale, cuda_stream, device_status_or_null, scratch);
}

int omni_attn_fwd_ex_sm100(const void* q, const void* k, const void* v, void* o, float* lse_or_null,
                           const int32_t* kv_num_blocks, const int32_t* kv_indices,
                           const int32_t* block_mask_types, const int32_t* partial_idx_or_null,
                           const uint8_t* partial_bool_or_null, const uint32_t* partial_bits_or_null, int B,
                           int H, int seqlen_padded, int seqlen_orig, int head_dim, int q_block, int kv_block,
                           int max_blocks, int num_partial, int dtype, float scale, void* cuda_stream,
                           int32_t* device_status_or_null, float softcap, void* scratch_or_null,
                           long long scratch_bytes) {
  if (softcap < 0.f || softcap != softcap) return OMNI_ERR_SOFTCAP;
  if (scratch_or_null != nullptr && scratch_bytes < OMNI_ATTN_SCRATCH_BYTES) return OMNI_ERR_SCRATCH;
  return omni::forward(false, q, k, v, o, lse_or_null, kv_num_blocks, kv_indices, block_mask_types,
                       partial_idx_or_null, partial_bool_or_null, partial_bits_or_null, B, H,
                       seqlen_padded, seqlen_orig, head_dim, q_block, kv_block, max_blocks, num_partial,
                       dtype, scale, cuda_stream, device_status_or_null, scratch_or_null, softcap);
}

int omni_attn_fwd_simple_sm100(const void* q, const void* k, const void* v, void* o,
                               float* lse_or_null, const int32_t* kv_num_blocks,
                               const int32_t* kv_indices, const int32_t* block_mask_types,
                               const int32_t* partial_idx_or_null,
                               const uint8_t* partial_bool_or_null,
                               const uint32_t* partial_bits_or_null, int B, int H,
                               int seqlen_padded, int seqlen_orig, int head_dim, int q_block,
                               int kv_block, int max_blocks, int num_partial, int dtype, float scale,
                               void* cuda_stream, int32_t* device_status_or_null) {
  return omni::forward(true, q, k, v, o, lse_or_null, kv_num_blocks, kv_indices, block_mask_types,
                       partial_idx_or_null, partial_bool_or_null, partial_bits_or_null, B, H,
                       seqlen_padded, seqlen_orig, head_dim, q_block, kv_block, max_blocks, num_partial,
                       dtype, scale, cuda_stream, device_status_or_null, nullptr);
}

int omni_attn_pack_partial_masks_blk_sm100(const uint8_t* partial_bool, uint32_t* partial_bits,
                                           int num_partial, int block, void* cuda_stream) {
  if (block != 64 && block != omni::kBlock) return OMNI_ERR_BLOCK_SIZE;
  if (num_partial < 0) return OMNI_ERR_PARTIAL;
  if (num_partial == 0) return OMNI_OK;
  if (partial_bool == nullptr || partial_bits == nullptr) return OMNI_ERR_NULL_POINTER;
  if (!omni::aligned16(partial_bool) || !omni::aligned16(partial_bits)) return OMNI_ERR_ALIGNMENT;
  const long long n_words = static_cast<long long>(num_partial) * block * (block / 32);
  const int threads = 256;
  const long long blocks = (n_words + threads - 1) / threads;
  omni::pack_partial_kernel<<<static_cast<unsigned>(blocks), threads, 0,
                              static_cast<cudaStream_t>(cuda_stream)>>>(partial_bool, partial_bits, n_words);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    omni::g_last_cuda_error = static_cast<int>(e);
    return OMNI_ERR_CUDA;
  }
  return OMNI_OK;
}

int omni_attn_pack_partial_masks_sm100(const uint8_t* partial_bool, uint32_t* partial_bits,
                                       int num_partial, void* cuda_stream) {
  return omni_attn_pack_partial_masks_blk_sm100(partial_bool, partial_bits, num_partial, omni::kBlock, cuda_stream);
}

// ---------------------------------------------------------------------------------------------
// Forward pass for callers that cannot give the library any device memory to work in.
//
// The scratch the persistent kernel wants (the unit counter, and room to bit-pack a byte-per-element
// partial mask pool) lives in this file-scope device array instead of a caller buffer. Every GPU
// that loads the library carries the array until the process exits; it is shared by all calls, so
// it still holds whatever the previous call left there: the counter is cleared at the start of every
// call and the packed pool is rewritten in full before it is read.
// ---------------------------------------------------------------------------------------------
namespace omni {
namespace {

constexpr long long kBuiltinPoolOffset = OMNI_ATTN_SCRATCH_BYTES;
constexpr long long kBuiltinScratchBytes =
    kBuiltinPoolOffset + static_cast<long long>(OMNI_ATTN_NOALLOC_MAX_PARTIAL) * kBlock * 16;

static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device address; the
// address has to be asked for, once per device, with that device current.
int builtin_scratch_address(unsigned char** out) {
  static std::mutex mu;
  static unsigned char* addr[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return OMNI_ERR_CUDA;
  }
  if (dev < 0 || dev >= 64) return OMNI_ERR_SHAPE;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_builtin_scratch);
    if (e != cudaSuccess || p == nullptr) {
      g_last_cuda_error = static_cast<int>(e);
      return OMNI_ERR_CUDA;
    }
    addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = addr[dev];
  return OMNI_OK;
}

}  // namespace
}  // namespace omni

int omni_attn_fwd_noalloc_sm100(const void* q, const void* k, const void* v, void* o, float* lse_or_null,
                                const int32_t* kv_num_blocks, const int32_t* kv_indices,
                                const int32_t* block_mask_types, const int32_t* partial_idx_or_null,
                                const uint8_t* partial_bool_or_null, const uint32_t* partial_bits_or_null,
                                int B, int H, int seqlen_padded, int seqlen_orig, int head_dim, int q_block,
                                int kv_block, int max_blocks, int num_partial, int dtype, float scale,
                                void* cuda_stream, int32_t* device_status_or_null) {
  // Every argument check comes first: a call that is going to be refused must not have touched the
  // shared array.
  int rc = omni::validate_forward(false, q, k, v, o, kv_num_blocks, kv_indices, block_mask_types, partial_bool_or_null,
                                  partial_bits_or_null, B, H, seqlen_padded, seqlen_orig, head_dim, q_block, kv_block,
                                  max_blocks, num_partial, dtype, nullptr, 0.f);
  if (rc != OMNI_OK) return rc;
  const bool pack_here = num_partial > 0 && partial_bits_or_null == nullptr && partial_bool_or_null != nullptr;
  // room for OMNI_ATTN_NOALLOC_MAX_PARTIAL bit-packed 128x128 tiles; a 64x64 tile takes a quarter of one
  const long long tile_bytes = static_cast<long long>(q_block) * q_block / 8;
  if (pack_here && num_partial * tile_bytes > static_cast<long long>(OMNI_ATTN_NOALLOC_MAX_PARTIAL) * omni::kBlock * 16) {
    return OMNI_ERR_NOALLOC_LIMIT;
  }
  unsigned char* scratch = nullptr;
  rc = omni::builtin_scratch_address(&scratch);
  if (rc != OMNI_OK) return rc;
  // The pack and the forward are two enqueues that belong together: without the lock two host
  // threads on one stream could interleave them (pack A, pack B, forward A, forward B) and A would
  // read B's masks although nothing overlaps on the GPU.
  static std::mutex enqueue_mu;
  std::lock_guard<std::mutex> lock(enqueue_mu);
  const uint32_t* bits = partial_bits_or_null;
  if (pack_here) {
    uint32_t* pool = reinterpret_cast<uint32_t*>(scratch + omni::kBuiltinPoolOffset);
    rc = omni_attn_pack_partial_masks_blk_sm100(partial_bool_or_null, pool, num_partial, q_block, cuda_stream);
    if (rc != OMNI_OK) return rc;
    bits = pool;
  }
  return omni::forward(false, q, k, v, o, lse_or_null, kv_num_blocks, kv_indices, block_mask_types,
                       partial_idx_or_null, partial_bool_or_null, bits, B, H, seqlen_padded, seqlen_orig,
                       head_dim, q_block, kv_block, max_blocks, num_partial, dtype, scale, cuda_stream,
                       device_status_or_null, scratch);
}

void omni_attn_set_wait_cycles(long long cycles) {
  omni::g_wait_cycles.store(cycles > 0 ? cycles : omni::kWaitCycleLimit, std::memory_order_relaxed);
}

int omni_attn_max_seqlen(int head_dim, int block, int simple_kernel) {
  if ((head_dim != 32 && head_dim != 64 && head_dim != 128) || (block != 64 && block != omni::kBlock)) return 0;
  const bool b64 = block == 64;
  const int tiles = simple_kernel ? omni::simple_max_tiles(b64) : omni::ws_max_tiles(head_dim == 128 ? 128 : 64, b64);
  return tiles * omni::kBlock;
}

long long omni_attn_bwd_workspace_bytes(int B, int H, int seqlen_padded) {
  if (B <= 0 || H <= 0 || seqlen_padded <= 0 || seqlen_padded % omni::kBlock != 0) return 0;
  return omni::bwd_workspace_bytes(static_cast<long long>(B) * H, seqlen_padded);
}

int omni_attn_bwd_sm100(const void* q, const void* k, const void* v, const void* o, const float* lse,
                        const void* d_o, void* dq, void* dk, void* dv, const int32_t* kv_num_blocks,
                        const int32_t* kv_indices, const int32_t* block_mask_types,
                        const int32_t* partial_idx_or_null, const uint8_t* partial_bool_or_null,
                        const uint32_t* partial_bits_or_null, int B, int H, int seqlen_padded, int seqlen_orig,
                        int head_dim, int q_block, int kv_block, int max_blocks, int num_partial, int dtype,
                        float scale, void* cuda_stream, int32_t* device_status_or_null, void* workspace,
                        long long workspace_bytes) {
  return omni::backward(q, k, v, o, lse, d_o, dq, dk, dv, kv_num_blocks, kv_indices, block_mask_types,
                        partial_idx_or_null, partial_bool_or_null, partial_bits_or_null, B, H, seqlen_padded,
                        seqlen_orig, head_dim, q_block, kv_block, max_blocks, num_partial, dtype, scale,
                        cuda_stream, device_status_or_null, workspace, workspace_bytes);
}

int omni_attn_bwd_ex_sm100(const void* q, const void* k, const void* v, const void* o, const float* lse,
                           const void* d_o, void* dq, void* dk, void* dv, const int32_t* kv_num_blocks,
                           const int32_t* kv_indices, const int32_t* block_mask_types,
                           const int32_t* partial_idx_or_null, const uint8_t* partial_bool_or_null,
                           const uint32_t* partial_bits_or_null, int B, int H, int seqlen_padded, int seqlen_orig,
                           int head_dim, int q_block, int kv_block, int max_blocks, int num_partial, int dtype,
                           float scale, void* cuda_stream, int32_t* device_status_or_null, void* workspace,
                           long long workspace_bytes, float softcap) {
  return omni::backward(q, k, v, o, lse, d_o, dq, dk, dv, kv_num_blocks, kv_indices, block_mask_types,
                        partial_idx_or_null, partial_bool_or_null, partial_bits_or_null, B, H, seqlen_padded,
                        seqlen_orig, head_dim, q_block, kv_block, max_blocks, num_partial, dtype, scale,
                        cuda_stream, device_status_or_null, workspace, workspace_bytes, softcap);
}

const char* omni_attn_error_string(int code) {
  switch (code) {
    case OMNI_OK: return "ok";
    case OMNI_ERR_NULL_POINTER: return "a required pointer is NULL";
    case OMNI_ERR_DTYPE: return "dtype must be fp16 (0) or bf16 (1)";
    case OMNI_ERR_HEAD_DIM: return "head_dim must be 32, 64 or 128 (backward pass: 64 or 128)";
    case OMNI_ERR_BLOCK_SIZE:
      return "Q_BLOCK_SIZE and KV_BLOCK_SIZE must be equal and 64 or 128 (backward pass and pack: see the header)";
    case OMNI_ERR_SEQLEN:
      return "seqlen_padded must be a positive multiple of the block size and 0 < seqlen_orig <= seqlen_padded";
    case OMNI_ERR_SHAPE:
      return "B, H, max_blocks must be positive and B*H <= 65535 (backward pass: also B*H*seqlen < 2^31)";
    case OMNI_ERR_PARTIAL: return "num_partial is negative, or positive without a partial mask pool";
    case OMNI_ERR_TOO_LONG:
      return "sequence longer than the kernel's block tables hold (131072 tokens with 128-blocks; see "
             "omni_attn_max_seqlen)";
    case OMNI_ERR_ALIGNMENT: return "q, k, v, o and the partial mask pools must be 16-byte aligned";
    case OMNI_ERR_CUDA: return "a CUDA call failed (see omni_attn_last_cuda_error)";
    case OMNI_ERR_NO_DRIVER_ENTRY: return "cuTensorMapEncodeTiled not available from the CUDA driver";
    case OMNI_ERR_SCRATCH: return "scratch buffer smaller than OMNI_ATTN_SCRATCH_BYTES";
    case OMNI_ERR_SOFTCAP: return "softcap must be >= 0 (0 = none); the plain kernel has no soft-cap";
    case OMNI_ERR_WORKSPACE: return "workspace smaller than omni_attn_bwd_workspace_bytes()";
    case OMNI_ERR_NOALLOC_LIMIT:
      return "byte-per-element partial pool has more than OMNI_ATTN_NOALLOC_MAX_PARTIAL (1024) tiles: too large for "
             "the built-in scratch; pass a bit-packed pool or use omni_attn_fwd_scratch_sm100";
    default: return "unknown error code";
  }
}

int omni_attn_last_cuda_error(void) { return omni::g_last_cuda_error; }

int omni_attn_abi_version(void) { return OMNI_ATTN_ABI_VERSION; }


}  // extern "C"
