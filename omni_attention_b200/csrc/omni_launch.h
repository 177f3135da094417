// Internal launch interface between the C-ABI layer and the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "omni_common.cuh"

namespace omni {

// Longest sequence the warp-specialised kernel accepts: its per-CTA block tables hold this many
// KV blocks (128 tokens each).
constexpr int kMaxKvBlocks = 1024;

cudaError_t launch_simple(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                          const CUtensorMap& tmV, const FwdParams& p, cudaStream_t stream);

cudaError_t launch_ws(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                      const CUtensorMap& tmV, const FwdParams& p, cudaStream_t stream);

// Backward pass: fills the workspace (entry codes, delta), then dK/dV (one CTA per KV block) and dQ
// (one CTA per Q block).
cudaError_t launch_bwd(int head_dim, bool bf16, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                       const CUtensorMap& tmV, const CUtensorMap& tmdO, const BwdParams& p, cudaStream_t stream);

// Sets a kernel's dynamic shared memory limit once per device.
template <typename K>
inline cudaError_t ensure_smem_attr(K kern, int bytes, bool (&done)[64]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) dev = 63;
  if (dev == 63 || !done[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    done[dev] = true;
  }
  return cudaSuccess;
}

}  // namespace omni
