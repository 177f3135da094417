// Internal launch interface between the C-ABI layer and the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "omni_common.cuh"

namespace omni {

// Longest sequence the warp-specialised kernel accepts: its per-CTA block tables hold this many
// KV blocks (128 tokens each).
constexpr int kMaxKvBlocks = 1024;

// Devices per process the per-device first-use state is kept for.
constexpr int kMaxDevices = 64;

// Longest sequence, in 128-row tiles, each forward kernel accepts for the given configuration
// (the unit / code tables live in shared memory beside the tiles).
int ws_max_tiles(int head_dim, bool b64);
int simple_max_tiles(bool b64);

cudaError_t launch_simple(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                          const CUtensorMap& tmV, const FwdParams& p, cudaStream_t stream);

cudaError_t launch_ws(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                      const CUtensorMap& tmV, const FwdParams& p, cudaStream_t stream);

// Backward pass: fills the workspace (entry codes, delta), then dK/dV (one CTA per KV block) and dQ
// (one CTA per Q block).
cudaError_t launch_bwd(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                       const CUtensorMap& tmV, const CUtensorMap& tmdO, const BwdParams& p, cudaStream_t stream);

// Sets a kernel's dynamic shared memory limit once per device (any host thread may be the first).
struct SmemAttrOnce {
  std::once_flag once;
  cudaError_t err = cudaSuccess;
};
template <typename K>
inline cudaError_t ensure_smem_attr(K kern, int bytes, SmemAttrOnce (&state)[kMaxDevices]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  SmemAttrOnce& s = state[dev];
  std::call_once(s.once, [&] { s.err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); });
  return s.err;
}

}  // namespace omni
