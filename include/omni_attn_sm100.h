/* C ABI of the B200 (sm_100a) omni-attention library, libomni_attn_sm100.so: the forward pass (the
 * reference's operator), and beside it the backward pass and the mask construction, which the
 * reference does not have as device code.
 *
 * Plain pointers and sizes only; no torch types. Every function returns 0 on success or a negative
 * OMNI_ERR_* code, never throws, allocates no device memory and keeps no reference to its
 * arguments after it returns. All work is enqueued on `cuda_stream` (a cudaStream_t; NULL = the
 * legacy default stream, which is what the reference's launchers use) and is asynchronous.
 *
 * The entry points replace the reference's host launchers
 *   omni-attn-mma/mma/omni_attn_shared_kv.cu:693-1009   omni_attn_mma_stages_split_q_shared_kv
 *   omni-attn-mma/mma/omni_attn_swizzle.cu:721-1036     ..._shared_kv_swizzle
 *   omni-attn-mma/mma/omni_attn_preftech.cu:636-930     omni_attn_preftech_kernel
 *   omni-attn-mma/mma/omni_attn_cp_async.cu:300-467     omni_attn_cp_async
 *   omni-attn-mma/mma/attn_naive.cu:305-408             omni_attn_simple_kernel
 * whose 13 tensor/int arguments (omni-attn-mma/pybind/omni_attn.cc:46-56) map one to one onto
 * the pointer/size arguments below.
 */
#ifndef OMNI_ATTN_SM100_H_
#define OMNI_ATTN_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OMNI_ATTN_ABI_VERSION 1

/* dtype argument */
#define OMNI_DTYPE_F16 0
#define OMNI_DTYPE_BF16 1

/* Block types, as stored in block_mask_types (omni-attn-mma/omni_attn_torch.py:30-41). */
#define OMNI_BLOCK_MASKED 0
#define OMNI_BLOCK_CAUSAL 1
#define OMNI_BLOCK_FULL 2
#define OMNI_BLOCK_PARTIAL 3

/* Error codes. The first group mirrors the reference launchers' std::runtime_error checks
 * (omni-attn-mma/mma/omni_attn_shared_kv.cu:701-753). */
#define OMNI_OK 0
#define OMNI_ERR_NULL_POINTER (-1)     /* a required pointer is NULL */
#define OMNI_ERR_DTYPE (-2)            /* dtype is neither fp16 nor bf16 */
#define OMNI_ERR_HEAD_DIM (-3)         /* head_dim not in {32, 64, 128} (omni-attn-mma/mma/omni_attn_shared_kv.cu:725-729) */
#define OMNI_ERR_BLOCK_SIZE (-4)       /* q_block/kv_block differ or are not 64 or 128 (omni_attn_shared_kv.cu:732-741); the backward pass takes 128 */
#define OMNI_ERR_SEQLEN (-5)           /* seqlen_padded not a positive multiple of the block, or seqlen_orig outside (0, seqlen_padded] */
#define OMNI_ERR_SHAPE (-6)            /* B, H or max_blocks not positive, or B*H > 65535 (backward pass: or B*H*seqlen >= 2^31) */
#define OMNI_ERR_PARTIAL (-7)          /* num_partial > 0 without any partial mask pool, or num_partial < 0 */
#define OMNI_ERR_TOO_LONG (-8)         /* longer than the kernel's block tables hold: see omni_attn_max_seqlen() */
#define OMNI_ERR_ALIGNMENT (-9)        /* q/k/v/o (or a partial mask pool) not 16-byte aligned */
#define OMNI_ERR_CUDA (-10)            /* a CUDA runtime/driver call failed; see omni_attn_last_cuda_error() */
#define OMNI_ERR_NO_DRIVER_ENTRY (-11) /* cuTensorMapEncodeTiled is not available from the driver */
#define OMNI_ERR_SCRATCH (-12)         /* scratch buffer smaller than OMNI_ATTN_SCRATCH_BYTES */
#define OMNI_ERR_SOFTCAP (-14)         /* softcap negative or NaN */
#define OMNI_ERR_WORKSPACE (-15)       /* omni_attn_bwd_sm100: workspace smaller than omni_attn_bwd_workspace_bytes() */
#define OMNI_ERR_NOALLOC_LIMIT (-13)   /* omni_attn_fwd_noalloc_sm100: byte mask pool larger than the built-in scratch holds */

/* Values a kernel can leave in *device_status (0 = clean run). Low byte = kind, upper bits = the
 * place in the kernel that gave up. */
#define OMNI_STATUS_WAIT_TIMEOUT 1 /* a bounded mbarrier wait ran out; the output is not valid */
#define OMNI_STATUS_BAD_INDEX 2    /* a kv_indices entry was outside [0, seqlen_padded/128); it was skipped */

/* Forward pass with the warp-specialised, persistent kernel (work units assigned to the resident
 * CTAs in a fixed pattern; see omni_attn_fwd_scratch_sm100 for dynamic assignment).
 *
 *  q, k, v           [B, H, seqlen_padded, head_dim], contiguous, 16-bit (dtype), device memory;
 *                    head_dim 32, 64 or 128; seqlen_padded a multiple of q_block
 *  o                 same shape and dtype, written in place (rows >= seqlen_orig are zeroed)
 *  lse_or_null       [B, H, seqlen_padded] fp32: natural-log sum of exp of the scaled, masked
 *                    scores of each row (-inf for a row that attends nothing), or NULL.
 *                    The reference has no such output.
 *  q_block, kv_block  both 128 or both 64, the two block shapes of the reference's launchers
 *                    (omni-attn-mma/mma/omni_attn_shared_kv.cu:780-888). The kernels always work on
 *                    128x128 tiles; lists in 64-blocks are read as they are, a tile being a 2x2 of
 *                    sub-blocks (no conversion pass, no extra memory).
 *  kv_num_blocks     [B, H, nq] int32, nq = seqlen_padded / q_block
 *  kv_indices        [B, H, nq, max_blocks] int32; the first kv_num_blocks entries are used
 *  block_mask_types  [B, H, nq, max_blocks] int32 (OMNI_BLOCK_*)
 *  partial_idx_or_null   [B, H, nq, max_blocks] int32 index into the partial pool (-1 = none), or NULL
 *  partial_bool_or_null  [num_partial, q_block, kv_block] one byte per element, non-zero = attend
 *                        (the reference's torch.bool tensor), or NULL
 *  partial_bits_or_null  [num_partial, q_block, kv_block / 32] uint32, bit (c % 32) of word c / 32 of
 *                        row r = attend; produced by omni_attn_pack_partial_masks_sm100 (128-blocks)
 *                        or omni_attn_pack_partial_masks_blk_sm100. Used in preference to the byte
 *                        form when both are given.
 *  scale             softmax scale; <= 0 selects 1/sqrt(head_dim), the reference's fixed choice
 *                    (omni-attn-mma/mma/omni_attn_shared_kv.cu:62)
 *  device_status_or_null  one int32 in device memory the kernel may set to an OMNI_STATUS_* value;
 *                    the caller zeroes it beforehand and reads it after synchronising.
 *
 * A PARTIAL entry whose index is negative or >= num_partial (or any PARTIAL entry when no pool is
 * given) is treated as CAUSAL, as the reference's dense expansion does
 * (omni-attn-mma/omni_attn_torch.py:140-143). CAUSAL compares absolute positions. A block that is
 * listed more than once is visited once, with the meaning the dense expansion gives it when it
 * applies the entries in list order (:106-143): a later FULL or PARTIAL entry replaces an earlier one, a
 * diagonal CAUSAL entry counts only for a block that has nothing else (the reference's union of a
 * PARTIAL mask with a later CAUSAL entry is the one combination not reproduced: the PARTIAL mask stands).
 * Longest sequence: omni_attn_max_seqlen(head_dim, q_block, 0).
 */
int omni_attn_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* lse_or_null,
                        const int32_t* kv_num_blocks, const int32_t* kv_indices,
                        const int32_t* block_mask_types, const int32_t* partial_idx_or_null,
                        const uint8_t* partial_bool_or_null, const uint32_t* partial_bits_or_null,
                        int B, int H, int seqlen_padded, int seqlen_orig, int head_dim, int q_block,
                        int kv_block, int max_blocks, int num_partial, int dtype, float scale,
                        void* cuda_stream, int32_t* device_status_or_null);

/* Same contract and same kernel, with a small scratch buffer in device memory owned by the caller
 * (at least OMNI_ATTN_SCRATCH_BYTES, 16-byte aligned; contents need not be initialised, the call
 * clears what it uses on `cuda_stream`). With scratch the resident CTAs take work units from a
 * shared counter as they become free instead of following a fixed assignment, which balances
 * masks whose block lists vary unpredictably in length. Two calls that may overlap on the GPU must
 * not share a scratch buffer. No counterpart in the reference (its grid is one CTA per Q block,
 * omni-attn-mma/mma/omni_attn_shared_kv.cu:789-790). */
#define OMNI_ATTN_SCRATCH_BYTES 256
int omni_attn_fwd_scratch_sm100(const void* q, const void* k, const void* v, void* o, float* lse_or_null,
                                const int32_t* kv_num_blocks, const int32_t* kv_indices,
                                const int32_t* block_mask_types, const int32_t* partial_idx_or_null,
                                const uint8_t* partial_bool_or_null,
                                const uint32_t* partial_bits_or_null, int B, int H, int seqlen_padded,
                                int seqlen_orig, int head_dim, int q_block, int kv_block, int max_blocks,
                                int num_partial, int dtype, float scale, void* cuda_stream,
                                int32_t* device_status_or_null, void* scratch, long long scratch_bytes);

/* Extended forward: everything omni_attn_fwd_sm100 does, plus
 *  softcap   > 0: the scaled scores go through softcap * tanh(x / softcap) before masking, the
 *            score_mod of the Transfusion attention (transfusion_pytorch/transfusion.py:358-364, applied
 *            at :953-961 and :967 with softcap_value = 50); 0 = none. The reference's kernels have no
 *            soft-cap.
 *  scratch_or_null / scratch_bytes   as in omni_attn_fwd_scratch_sm100, or NULL for the fixed unit
 *            assignment. */
int omni_attn_fwd_ex_sm100(const void* q, const void* k, const void* v, void* o, float* lse_or_null,
                           const int32_t* kv_num_blocks, const int32_t* kv_indices,
                           const int32_t* block_mask_types, const int32_t* partial_idx_or_null,
                           const uint8_t* partial_bool_or_null, const uint32_t* partial_bits_or_null, int B,
                           int H, int seqlen_padded, int seqlen_orig, int head_dim, int q_block, int kv_block,
                           int max_blocks, int num_partial, int dtype, float scale, void* cuda_stream,
                           int32_t* device_status_or_null, float softcap, void* scratch_or_null,
                           long long scratch_bytes);

/* Forward pass for callers that have no device memory to hand over and may not allocate any.
 * This entry point has no counterpart in the reference.
 *
 * Who needs it: a plug-in living inside a host program that owns every byte of device memory
 * through its own allocator and offers plug-ins no way to ask for some (the reference's own
 * 13-argument binding is such an interface: it has no workspace argument and its contract is that the
 * callee allocates nothing); a serving loop that must not call cudaMalloc/cudaFree on its hot path
 * because those calls synchronise the whole device and stall every other stream; a process that has
 * already given all of its memory budget away.
 *
 * Same arguments, results and error codes as omni_attn_fwd_sm100. The scratch that
 * omni_attn_fwd_scratch_sm100 takes from its caller (the counter from which the resident CTAs draw
 * work units) is kept in a fixed array inside the library instead, together with room to convert a
 * byte-per-element partial mask pool to the bit-packed form (one eighth of the mask traffic in
 * the kernel). The function calls no cudaMalloc, cudaFree or any other allocating routine.
 *
 * Limits and rules:
 *  - the array is OMNI_ATTN_SCRATCH_BYTES + OMNI_ATTN_NOALLOC_MAX_PARTIAL * 2048 bytes (about 2 MB) of
 *    device memory on every GPU that loads the library, held until the process exits;
 *  - a byte pool (partial_bool_or_null without partial_bits_or_null) of more than
 *    OMNI_ATTN_NOALLOC_MAX_PARTIAL 128x128 tiles (four times as many 64x64 tiles) is refused with
 *    OMNI_ERR_NOALLOC_LIMIT; a pool the caller has already bit-packed may have any size;
 *  - every argument check runs before anything is enqueued: a refused call leaves the array alone;
 *  - all calls on a device share the one array and it keeps the previous call's contents: each call
 *    clears the counter and rewrites the packed pool on `cuda_stream` before use. Two calls whose
 *    GPU work can overlap (different streams without an ordering between them) race on it and
 *    must be serialised by the caller. Host threads are serialised by the library itself for the
 *    time it takes to enqueue one call, so calls from several threads onto ONE stream are safe;
 *  - the first call on each device looks up the array's device address (with that device current);
 *    make that first call before starting any stream capture on the device.
 */
#define OMNI_ATTN_NOALLOC_MAX_PARTIAL 1024
int omni_attn_fwd_noalloc_sm100(const void* q, const void* k, const void* v, void* o, float* lse_or_null,
                                const int32_t* kv_num_blocks, const int32_t* kv_indices,
                                const int32_t* block_mask_types, const int32_t* partial_idx_or_null,
                                const uint8_t* partial_bool_or_null,
                                const uint32_t* partial_bits_or_null, int B, int H, int seqlen_padded,
                                int seqlen_orig, int head_dim, int q_block, int kv_block, int max_blocks,
                                int num_partial, int dtype, float scale, void* cuda_stream,
                                int32_t* device_status_or_null);

/* Same contract, computed by the plain one-tile-per-CTA kernel. It takes the place of the
 * reference's correctness-first kernel (omni-attn-mma/mma/attn_naive.cu:305-408). */
int omni_attn_fwd_simple_sm100(const void* q, const void* k, const void* v, void* o,
                               float* lse_or_null, const int32_t* kv_num_blocks,
                               const int32_t* kv_indices, const int32_t* block_mask_types,
                               const int32_t* partial_idx_or_null,
                               const uint8_t* partial_bool_or_null,
                               const uint32_t* partial_bits_or_null, int B, int H,
                               int seqlen_padded, int seqlen_orig, int head_dim, int q_block,
                               int kv_block, int max_blocks, int num_partial, int dtype, float scale,
                               void* cuda_stream, int32_t* device_status_or_null);

/* Packs the reference's byte-per-element partial masks ([num_partial,128,128], built by
 * build_partial_block_data, omni-attn-mma/omni_attn_torch.py:148-205) into one bit per element
 * ([num_partial,128,4] uint32). Both buffers are device memory owned by the caller. */
int omni_attn_pack_partial_masks_sm100(const uint8_t* partial_bool, uint32_t* partial_bits,
                                       int num_partial, void* cuda_stream);

/* The same for either block shape of build_partial_block_data: block = 128 or 64
 * ([num_partial, block, block] bytes -> [num_partial, block, block / 32] uint32). */
int omni_attn_pack_partial_masks_blk_sm100(const uint8_t* partial_bool, uint32_t* partial_bits,
                                           int num_partial, int block, void* cuda_stream);

/* Longest seqlen_padded the forward entry points accept for this head_dim (32, 64, 128) and block
 * shape (64, 128); simple_kernel != 0 asks for omni_attn_fwd_simple_sm100. 0 for unsupported
 * arguments. The block tables of a sequence live in shared memory beside the tiles, so lists in
 * 64-blocks, four codes per tile, reach less far (128-blocks: 131072 tokens). The reference's
 * launchers state no limit (omni-attn-mma/mma/omni_attn_shared_kv.cu:780-1003); its largest
 * published run is 2048 tokens (omni-attn-mma/logs/printed_mask.md:188-237). */
int omni_attn_max_seqlen(int head_dim, int block, int simple_kernel);

/* Every wait inside the forward kernels is bounded: a CTA that has waited `cycles` GPU clock cycles
 * for one hand-over sets *device_status to OMNI_STATUS_WAIT_TIMEOUT | (place << 8), waits for its
 * own copies and MMAs in flight and exits. The default is 2e9 cycles (about a second); cycles <= 0
 * restores it. Process-wide, read at every launch. The reference's kernels have no such bound (a
 * fault there surfaces as a hung or failed launch, omni-attn-mma/mma/omni_attn_shared_kv.cu:1005-1008). */
void omni_attn_set_wait_cycles(long long cycles);

/* Builds the block mask of an interleaved text / image sequence on the GPU, in the reference's
 * metadata format, from the image span positions. Replaces the host-side builder
 * create_omni_block_mask_from_modality_positions (omni-attn-mma/omni_attn_torch.py:1518-1736) together
 * with the dense mask (transfusion_pytorch/transfusion.py:496-515) and build_partial_block_data
 * (omni-attn-mma/omni_attn_torch.py:148-205) it relies on. Mask rule: key k is attended by query q iff
 * k <= q, or q >= offset_m and k < offset_m + length_m for some span m; nothing at or beyond `seqlen`.
 *
 *  modality_positions  [B, M, 3] int32 (type, offset, length), device; entries with length <= 0 are ignored
 *  seqlen              unpadded length; seqlen_padded = multiple of 128 >= seqlen (nq = seqlen_padded / 128)
 *  kv_num_blocks       out [B, H, nq];  kv_indices, block_mask_types, partial_idx  out [B, H, nq, nq]
 *                      (listed blocks first, ascending; the same lists for every head of a batch element)
 *  partial_bits        out [partial_capacity, 128, 4] bit-packed PARTIAL tiles (pool shared by the heads)
 *  partial_bool_or_null  out [partial_capacity, 128, 128] bytes, the reference's form, or NULL
 *  num_partial_out     out, one device int32: PARTIAL tiles the mask needs; when it exceeds
 *                      partial_capacity the tiles beyond the capacity were not written and the call must
 *                      be repeated with a larger pool
 *  scratch             device memory, at least 2 * B * nq * 4 bytes
 * Block types by content: all elements allowed -> FULL, none -> not listed, a diagonal block of plain
 * causal rows -> CAUSAL, anything else -> PARTIAL (the derivation of
 * omni-attn-mma/generate_attn_data.py:200-236; the reference builder's "dominant type" shortcut types
 * some fully allowed blocks PARTIAL with an all-true mask, which expands to the same dense mask). */
int omni_attn_build_mask_sm100(const int32_t* modality_positions, int B, int M, int H, int seqlen,
                               int seqlen_padded, int32_t* kv_num_blocks, int32_t* kv_indices,
                               int32_t* block_mask_types, int32_t* partial_idx, uint32_t* partial_bits,
                               uint8_t* partial_bool_or_null, int partial_capacity, int32_t* num_partial_out,
                               void* scratch, long long scratch_bytes, void* cuda_stream);

/* Backward pass: dQ, dK, dV from the gradient of the output, with the block lists of the forward
 * pass and the log-sum-exp it saved.
 *
 * No counterpart in the reference, which is forward-only (omni-attn-mma/pybind/omni_attn.cc:70-77
 * exports no gradient function, and omni-attn-mma/omni_attn_torch.py wraps the forward in no
 * autograd.Function). What is differentiated is the reference's forward definition
 * softmax((Q K^T) * scale + mask) V (omni-attn-mma/omni_attn_torch.py:348-387) with the mask semantics of
 * omni_attn_fwd_sm100; a row that attended nothing gets zero gradient.
 *
 *  q, k, v, o, d_o     in  [B, H, seqlen_padded, head_dim] 16-bit; o and lse are the results of the
 *                      forward call on the same q, k, v, lists and scale. Rows of q and d_o at positions
 *                      >= seqlen_orig take no part but must hold finite values.
 *  lse                 in  [B, H, seqlen_padded] fp32, natural log
 *  dq, dk, dv          out [B, H, seqlen_padded, head_dim], same 16-bit type; rows >= seqlen_orig are zero
 *  workspace           device memory, at least omni_attn_bwd_workspace_bytes(B, H, seqlen_padded) bytes,
 *                      16-byte aligned; holds no state between calls, and two calls that overlap in time
 *                      need two workspaces
 * The list, pool, size, dtype, scale, stream and status arguments are those of omni_attn_fwd_sm100.
 * head_dim 32, 64 or 128 as in the forward; the backward takes 128x128 blocks only (OMNI_ERR_BLOCK_SIZE for
 * 64x64: re-express such a mask on 128-tiles first, as the Python operator does).
 * Three kernels are enqueued on cuda_stream; the result is deterministic (no atomics). */
long long omni_attn_bwd_workspace_bytes(int B, int H, int seqlen_padded);
int omni_attn_bwd_sm100(const void* q, const void* k, const void* v, const void* o, const float* lse,
                        const void* d_o, void* dq, void* dk, void* dv, const int32_t* kv_num_blocks,
                        const int32_t* kv_indices, const int32_t* block_mask_types,
                        const int32_t* partial_idx_or_null, const uint8_t* partial_bool_or_null,
                        const uint32_t* partial_bits_or_null, int B, int H, int seqlen_padded, int seqlen_orig,
                        int head_dim, int q_block, int kv_block, int max_blocks, int num_partial, int dtype,
                        float scale, void* cuda_stream, int32_t* device_status_or_null, void* workspace,
                        long long workspace_bytes);

/* omni_attn_bwd_sm100 for a forward that was run with a tanh soft-cap (omni_attn_fwd_ex_sm100 with the
 * same softcap > 0; transfusion_pytorch/transfusion.py:298-299, :967): the chain rule adds the factor
 * 1 - tanh^2(score * scale / softcap) to dS. softcap == 0 is omni_attn_bwd_sm100. */
int omni_attn_bwd_ex_sm100(const void* q, const void* k, const void* v, const void* o, const float* lse,
                           const void* d_o, void* dq, void* dk, void* dv, const int32_t* kv_num_blocks,
                           const int32_t* kv_indices, const int32_t* block_mask_types,
                           const int32_t* partial_idx_or_null, const uint8_t* partial_bool_or_null,
                           const uint32_t* partial_bits_or_null, int B, int H, int seqlen_padded, int seqlen_orig,
                           int head_dim, int q_block, int kv_block, int max_blocks, int num_partial, int dtype,
                           float scale, void* cuda_stream, int32_t* device_status_or_null, void* workspace,
                           long long workspace_bytes, float softcap);

/* Text for an OMNI_ERR_* code; the pointer is static storage. */
const char* omni_attn_error_string(int code);

/* The cudaError_t (as int) of the most recent failing CUDA call on this thread, 0 if none. */
int omni_attn_last_cuda_error(void);

int omni_attn_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* OMNI_ATTN_SM100_H_ */
