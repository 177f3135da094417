"""Host-side operator: ``omni_attention(q, k, v, block_mask)``.

Same contract as the reference's wrappers ``omni_attention_shared_kv`` and siblings
(omni-attn-mma/omni_attn_torch.py:517-671): ``[B, H, N, D]`` inputs, an ``OmniBlockMask``, output
``[B, H, N, D]`` sliced back to the unpadded length. Differences, all deliberate:
  * the input dtype is kept (fp16 or bf16); the reference forces ``.half()`` (:609-611);
  * ``scale`` is honoured; the reference accepts and drops it (:517-523 vs :652-663);
  * the launch goes to torch's current stream and nothing synchronises the device (the reference
    calls ``torch.cuda.synchronize()`` after every launch, :666);
  * ``return_lse=True`` also returns the log-sum-exp rows;
  * mask tensors are converted / bit-packed once per mask object and cached on it.
The call goes through the C ABI of ``libomni_attn_sm100.so`` with raw device pointers. There is no
CPU or PyTorch fallback: a missing library or a non-CUDA tensor raises.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Tuple, Union

import torch
from torch import Tensor

from .block_mask import OmniBlockMask

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libomni_attn_sm100.so")
_lib = None

# symbols include/omni_attn_sm100.h declares
ABI_SYMBOLS = (
    "omni_attn_fwd_sm100",
    "omni_attn_fwd_scratch_sm100",
    "omni_attn_fwd_ex_sm100",
    "omni_attn_fwd_noalloc_sm100",
    "omni_attn_fwd_simple_sm100",
    "omni_attn_pack_partial_masks_sm100",
    "omni_attn_pack_partial_masks_blk_sm100",
    "omni_attn_max_seqlen",
    "omni_attn_set_wait_cycles",
    "omni_attn_build_mask_sm100",
    "omni_attn_bwd_workspace_bytes",
    "omni_attn_bwd_sm100",
    "omni_attn_bwd_ex_sm100",
    "omni_attn_error_string",
    "omni_attn_last_cuda_error",
    "omni_attn_abi_version",
)

SCRATCH_BYTES = 256  # OMNI_ATTN_SCRATCH_BYTES
STATUS_WAIT_TIMEOUT = 1
STATUS_BAD_INDEX = 2


class OmniAttnError(RuntimeError):
    """A C-ABI call returned an error code, or a kernel reported a bad status."""


def load_library() -> ctypes.CDLL:
    """Load libomni_attn_sm100.so from the package directory (built by ``omni_attention_b200.build``);
    the environment variable OMNI_ATTN_LIBRARY names another build of the same library."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("OMNI_ATTN_LIBRARY", _LIB_PATH)
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build it with `python -m omni_attention_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(path)
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fwd_args = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp] + [i32] * 10 + [f32, vp, vp]
    for name in ("omni_attn_fwd_sm100", "omni_attn_fwd_simple_sm100", "omni_attn_fwd_noalloc_sm100"):
        fn = getattr(lib, name)
        fn.argtypes = fwd_args
        fn.restype = i32
    lib.omni_attn_fwd_scratch_sm100.argtypes = fwd_args + [vp, ctypes.c_longlong]
    lib.omni_attn_fwd_scratch_sm100.restype = i32
    lib.omni_attn_fwd_ex_sm100.argtypes = fwd_args + [f32, vp, ctypes.c_longlong]
    lib.omni_attn_fwd_ex_sm100.restype = i32
    lib.omni_attn_pack_partial_masks_sm100.argtypes = [vp, vp, i32, vp]
    lib.omni_attn_pack_partial_masks_sm100.restype = i32
    lib.omni_attn_pack_partial_masks_blk_sm100.argtypes = [vp, vp, i32, i32, vp]
    lib.omni_attn_pack_partial_masks_blk_sm100.restype = i32
    lib.omni_attn_max_seqlen.argtypes = [i32, i32, i32]
    lib.omni_attn_max_seqlen.restype = i32
    lib.omni_attn_set_wait_cycles.argtypes = [ctypes.c_longlong]
    lib.omni_attn_set_wait_cycles.restype = None
    lib.omni_attn_build_mask_sm100.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, i32, vp, vp,
                                               ctypes.c_longlong, vp]
    lib.omni_attn_build_mask_sm100.restype = i32
    lib.omni_attn_bwd_workspace_bytes.argtypes = [i32, i32, i32]
    lib.omni_attn_bwd_workspace_bytes.restype = ctypes.c_longlong
    lib.omni_attn_bwd_sm100.argtypes = [vp] * 15 + [i32] * 10 + [f32, vp, vp, vp, ctypes.c_longlong]
    lib.omni_attn_bwd_sm100.restype = i32
    lib.omni_attn_bwd_ex_sm100.argtypes = lib.omni_attn_bwd_sm100.argtypes + [f32]
    lib.omni_attn_bwd_ex_sm100.restype = i32
    lib.omni_attn_error_string.argtypes = [i32]
    lib.omni_attn_error_string.restype = ctypes.c_char_p
    lib.omni_attn_last_cuda_error.argtypes = []
    lib.omni_attn_last_cuda_error.restype = i32
    lib.omni_attn_abi_version.argtypes = []
    lib.omni_attn_abi_version.restype = i32
    _lib = lib
    return lib


def _check(rc: int) -> None:
    if rc != 0:
        lib = load_library()
        msg = lib.omni_attn_error_string(rc).decode()
        extra = f", CUDA error {lib.omni_attn_last_cuda_error()}" if rc == -10 else ""
        raise OmniAttnError(f"omni_attn: {msg} (code {rc}{extra})")


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def pack_partial_masks(partial_block_masks: Tensor) -> Tensor:
    """[P, blk, blk] bool (CUDA; blk = 128 or 64) -> [P, blk, blk / 32] int32 bit masks, on the current stream."""
    assert partial_block_masks.is_cuda and partial_block_masks.dtype == torch.bool
    P, blk = partial_block_masks.shape[0], int(partial_block_masks.shape[1])
    if blk not in (64, 128) or partial_block_masks.shape[2] != blk:
        raise OmniAttnError(f"partial_block_masks must be [P, 64, 64] or [P, 128, 128], got {tuple(partial_block_masks.shape)}")
    src = partial_block_masks.contiguous()
    bits = torch.empty(P, blk, blk // 32, dtype=torch.int32, device=src.device)
    if P > 0:
        with torch.cuda.device(src.device):
            stream = torch.cuda.current_stream().cuda_stream
            _check(load_library().omni_attn_pack_partial_masks_blk_sm100(src.data_ptr(), bits.data_ptr(), P, blk, stream))
    return bits


def build_block_mask_cuda(modality_positions: Tensor, batch: int, nheads: int, seq_len: int, padded: int,
                          device: torch.device) -> OmniBlockMask:
    """Runs omni_attn_build_mask_sm100 on ``device`` and wraps its outputs in an OmniBlockMask whose
    tensors stay on the device. Nothing here waits for the GPU when ``modality_positions`` is a host
    tensor: the number of PARTIAL tiles, which sizes the pool, is counted on the host from the span
    table (O(B*N*M) integer arithmetic). The kernels write the pool bit-packed, which is what the
    attention kernels read; the container's byte-per-element ``partial_block_masks`` is expanded from it
    only if somebody reads that field."""
    from .block_mask import _limits_from_modality_tensor, count_partial_tiles

    lib = load_library()
    limits, plain = _limits_from_modality_tensor(modality_positions, int(seq_len), int(padded))
    need = count_partial_tiles(limits, plain)
    mp = modality_positions.to(device=device, dtype=torch.int32).contiguous()
    M = int(mp.shape[1])
    nq = padded // 128
    nb = torch.empty(batch, nheads, nq, dtype=torch.int32, device=device)
    idx = torch.empty(batch, nheads, nq, nq, dtype=torch.int32, device=device)
    typ = torch.empty_like(idx)
    pidx = torch.empty_like(idx)
    count = torch.zeros(1, dtype=torch.int32, device=device)
    scratch = torch.empty(2 * batch * nq, dtype=torch.int32, device=device)
    bits = torch.empty(max(need, 1), 128, 4, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream().cuda_stream
        _check(lib.omni_attn_build_mask_sm100(_ptr(mp), batch, M, nheads, int(seq_len), int(padded), nb.data_ptr(),
                                              idx.data_ptr(), typ.data_ptr(), pidx.data_ptr(), bits.data_ptr(), None,
                                              need, count.data_ptr(), scratch.data_ptr(), scratch.numel() * 4,
                                              stream))
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(device))
        built_on = torch.cuda.current_stream(device).cuda_stream
    bits = bits[:need]
    bm = OmniBlockMask(nb, idx, typ, padded, padded, 128, 128, pidx, None)

    def expand_pool() -> Tensor:
        # first read of the reference-shaped pool: also the place where the host count is checked
        # against the one the kernels made (reading it waits for the GPU, which this read does anyway)
        cur = torch.cuda.current_stream(device)
        if cur.cuda_stream != built_on:
            cur.wait_event(ready)
        if int(count.item()) != need:
            raise RuntimeError(f"mask builder: the kernels counted {int(count.item())} PARTIAL tiles, the host {need}")
        shifts = torch.arange(32, dtype=torch.int32, device=device)
        return ((bits.unsqueeze(-1) >> shifts) & 1).bool().view(need, 128, 128)

    bm.set_lazy_partial_pool(expand_pool)
    # what the attention calls use; a caller that asks for the byte-per-element pool (pack_bits=False)
    # gets it through the container's field, expanded then
    bm._cache[(str(device), True)] = {"nb": nb, "idx": idx, "typ": typ, "pidx": pidx, "pbool": None,
                                      "pbits": bits if need > 0 else None, "num_partial": need,
                                      "ready": ready, "stream": built_on}
    return bm


def _device_mask(bm: OmniBlockMask, device: torch.device, pack_bits: bool) -> dict:
    """int32 contiguous copies of the mask tensors on ``device`` (+ bit-packed pool), cached on the mask."""
    key = (str(device), pack_bits)
    hit = bm._cache.get(key)
    if hit is not None:
        # The copies and the pack kernel were enqueued on the stream that was current when the entry
        # was built; a call on another stream must not run ahead of them.
        cur = torch.cuda.current_stream(device)
        if hit.get("ready") is not None and cur.cuda_stream != hit.get("stream"):
            cur.wait_event(hit["ready"])
        return hit
    cv = lambda t: t.to(device=device, dtype=torch.int32).contiguous()
    d = {"nb": cv(bm.kv_num_blocks), "idx": cv(bm.kv_indices), "typ": cv(bm.block_mask_types),
         "pidx": None, "pbool": None, "pbits": None, "num_partial": 0}
    if bm.partial_block_mask_indices is not None and bm.partial_block_masks is not None:
        d["pidx"] = cv(bm.partial_block_mask_indices)
        pool = bm.partial_block_masks.to(device=device, dtype=torch.bool).contiguous()
        d["num_partial"] = int(pool.shape[0])
        if pool.shape[0] > 0:
            if pack_bits:
                d["pbits"] = pack_partial_masks(pool)
            else:
                d["pbool"] = pool
    with torch.cuda.device(device):
        d["ready"] = torch.cuda.Event()
        d["ready"].record(torch.cuda.current_stream(device))
        d["stream"] = torch.cuda.current_stream(device).cuda_stream
    bm._cache[key] = d
    return d


def omni_attention_forward_out(q: Tensor, k: Tensor, v: Tensor, out: Tensor, block_mask: OmniBlockMask,
                               seqlen_orig: int, scale: Optional[float] = None, lse: Optional[Tensor] = None,
                               status: Optional[Tensor] = None, kernel: str = "ws", pack_bits: bool = True,
                               softcap: Optional[float] = None) -> None:
    """Launch the forward on padded, contiguous CUDA tensors; writes ``out`` (and ``lse``) in place."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda and out.is_cuda):
        raise OmniAttnError("omni_attention needs CUDA tensors (there is no CPU path)")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise OmniAttnError(f"unsupported dtype {q.dtype}: fp16 or bf16")
    for t in (k, v, out):
        if t.dtype != q.dtype or t.shape != q.shape:
            raise OmniAttnError("q, k, v, out must share dtype and shape (Q_len == KV_len)")
    for t in (q, k, v, out):
        if not t.is_contiguous():
            raise OmniAttnError("q, k, v, out must be contiguous")
    B, H, N, D = q.shape
    m = _device_mask(block_mask, q.device, pack_bits)
    nq = N // block_mask.Q_BLOCK_SIZE if block_mask.Q_BLOCK_SIZE else 0
    if tuple(m["nb"].shape) != (B, H, nq):
        raise OmniAttnError(f"kv_num_blocks shape {tuple(m['nb'].shape)} != {(B, H, nq)}")
    if tuple(m["idx"].shape[:3]) != (B, H, nq) or m["typ"].shape != m["idx"].shape:
        raise OmniAttnError("kv_indices / block_mask_types shape mismatch")
    if m["pidx"] is not None and m["pidx"].shape != m["idx"].shape:
        raise OmniAttnError("partial_block_mask_indices shape mismatch")
    if lse is not None and (lse.dtype != torch.float32 or lse.numel() != B * H * N or not lse.is_contiguous()):
        raise OmniAttnError("lse must be contiguous float32 [B, H, N]")
    lib = load_library()
    if kernel not in ("ws", "ws_static", "simple"):
        raise OmniAttnError(f"unknown kernel {kernel!r}")
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _ptr(lse), m["nb"].data_ptr(),
                m["idx"].data_ptr(), m["typ"].data_ptr(), _ptr(m["pidx"]), _ptr(m["pbool"]), _ptr(m["pbits"]),
                B, H, N, int(seqlen_orig), D, block_mask.Q_BLOCK_SIZE, block_mask.KV_BLOCK_SIZE,
                int(m["idx"].shape[3]), m["num_partial"], 1 if q.dtype == torch.bfloat16 else 0,
                float(scale) if scale is not None else 0.0, stream, _ptr(status))
        if softcap is not None and softcap > 0:
            if kernel == "simple":
                raise OmniAttnError("the plain kernel has no soft-cap")
            sc = _scratch_for(q.device, stream) if kernel == "ws" else None
            rc = lib.omni_attn_fwd_ex_sm100(*args, float(softcap), _ptr(sc), SCRATCH_BYTES if sc is not None else 0)
        elif kernel == "ws":
            # dynamic unit hand-out: one small scratch buffer per (device, stream), reused by every
            # call on that stream (calls on one stream never overlap)
            rc = lib.omni_attn_fwd_scratch_sm100(*args, _scratch_for(q.device, stream).data_ptr(), SCRATCH_BYTES)
        elif kernel == "ws_static":
            rc = lib.omni_attn_fwd_sm100(*args)
        else:
            rc = lib.omni_attn_fwd_simple_sm100(*args)
    _check(rc)


_scratch = {}


def _scratch_for(device: torch.device, stream: int) -> Tensor:
    key = (str(device), int(stream))
    t = _scratch.get(key)
    if t is None:
        t = torch.zeros(SCRATCH_BYTES // 4, dtype=torch.int32, device=device)
        _scratch[key] = t
    return t


def _pad_to_block(x: Tensor, block: int) -> Tuple[Tensor, int]:
    n = x.shape[2]
    rem = (-n) % block
    if rem == 0:
        return x, n
    return torch.nn.functional.pad(x, (0, 0, 0, rem)), n


def _prepare(query: Tensor, key: Tensor, value: Tensor, block_mask: OmniBlockMask, scale: Optional[float],
             for_backward: bool = False):
    """Shape checks and padding. The forward kernels take everything the reference's launchers accept
    (omni-attn-mma/mma/omni_attn_shared_kv.cu:725-741: head_dim 32/64/128, blocks 64 or 128) as it is,
    so all that happens here is the reference wrapper's zero-padding of the sequence to a multiple of
    the mask's block size (omni_attn_torch.py:1261-1284).

    The backward kernels take 128x128 blocks only; with ``for_backward`` a 64x64-block mask is
    re-expressed on 128-tiles once (quadrant by quadrant, cached on the mask object).
    Returns padded contiguous q, k, v, the mask to use, the scale, and the original length / head_dim."""
    B, H, Q, D = query.shape
    if key.shape != (B, H, Q, D) or value.shape != (B, H, Q, D):
        raise OmniAttnError(f"key/value shape must equal query shape {(B, H, Q, D)} (Q_len == KV_len)")
    if D not in (32, 64, 128):
        raise ValueError(f"Unsupported head_dim={D}. Supported: 32, 64, 128.")
    sizes = (block_mask.Q_BLOCK_SIZE, block_mask.KV_BLOCK_SIZE)
    if sizes not in ((64, 64), (128, 128)):
        raise ValueError("Unsupported block size: Q_BLOCK_SIZE and KV_BLOCK_SIZE must both be 64 or both be 128.")
    if for_backward:
        if sizes == (64, 64):
            hit = block_mask._cache.get("retiled128")
            if hit is None:
                from .block_mask import retile_block_mask

                hit = retile_block_mask(block_mask, 128)
                block_mask._cache["retiled128"] = hit
            block_mask = hit
    blk = block_mask.Q_BLOCK_SIZE
    qp, n_orig = _pad_to_block(query, blk)
    kp, _ = _pad_to_block(key, blk)
    vp, _ = _pad_to_block(value, blk)
    if qp.shape[2] != block_mask.q_len or kp.shape[2] != block_mask.kv_len:
        raise OmniAttnError(
            f"padded length {qp.shape[2]} does not match the mask's q_len/kv_len ({block_mask.q_len}/{block_mask.kv_len})")
    return qp.contiguous(), kp.contiguous(), vp.contiguous(), block_mask, scale, n_orig, D


def omni_attention(query: Tensor, key: Tensor, value: Tensor, block_mask: OmniBlockMask,
                   scale: Optional[float] = None, return_lse: bool = False, kernel: str = "ws",
                   check_status: bool = False, softcap: Optional[float] = None) -> Union[Tensor, Tuple[Tensor, Tensor]]:
    """Block-mask attention forward on a B200.

    query/key/value: [B, H, N, D] fp16 or bf16 CUDA tensors with Q_len == KV_len, D in {32, 64, 128};
    ``block_mask`` with 128x128 or 64x64 blocks, built for the length padded to its block size. Returns ``out[:, :, :N]`` (and
    ``lse[:, :, :N]``, natural log, when ``return_lse``). ``softcap`` > 0 applies the Transfusion attention's
    tanh soft-cap to the scaled scores before masking (transfusion_pytorch/transfusion.py:358-364). ``check_status=True`` synchronises and
    raises if the kernel reported a bounded-wait timeout or an out-of-range block index.
    """
    B, H = query.shape[:2]
    qp, kp, vp, block_mask, scale, n_orig, d_orig = _prepare(query, key, value, block_mask, scale)
    out = torch.empty_like(qp)
    lse = torch.empty(B, H, qp.shape[2], dtype=torch.float32, device=qp.device) if return_lse else None
    status = torch.zeros(1, dtype=torch.int32, device=qp.device) if check_status else None
    omni_attention_forward_out(qp, kp, vp, out, block_mask, n_orig, scale, lse, status, kernel, softcap=softcap)
    if check_status:
        code = int(status.item())
        if code & 0xFF == STATUS_WAIT_TIMEOUT:
            raise OmniAttnError(f"kernel gave up waiting (status {code:#x}); output is not valid")
        if code & 0xFF == STATUS_BAD_INDEX:
            raise OmniAttnError("kv_indices holds a block id outside [0, num_kv_blocks); the entry was skipped")
    out = out[:, :, :n_orig, :d_orig]
    if return_lse:
        return out, lse[:, :, :n_orig]
    return out


def omni_attention_backward_out(q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor, d_out: Tensor,
                                dq: Tensor, dk: Tensor, dv: Tensor, block_mask: OmniBlockMask, seqlen_orig: int,
                                scale: Optional[float] = None, status: Optional[Tensor] = None,
                                workspace: Optional[Tensor] = None, softcap: Optional[float] = None) -> None:
    """Launch the backward on padded, contiguous CUDA tensors; writes ``dq``, ``dk``, ``dv`` in place.
    ``out`` and ``lse`` are what the forward returned for the same inputs, mask and scale. The
    reference has no backward; this is the gradient of its forward definition. ``softcap`` must be
    the value the forward was run with."""
    tensors = (q, k, v, out, d_out, dq, dk, dv)
    if not all(t.is_cuda for t in tensors) or not lse.is_cuda:
        raise OmniAttnError("omni_attention backward needs CUDA tensors (there is no CPU path)")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise OmniAttnError(f"unsupported dtype {q.dtype}: fp16 or bf16")
    for t in tensors:
        if t.dtype != q.dtype or t.shape != q.shape or not t.is_contiguous():
            raise OmniAttnError("q, k, v, out, d_out, dq, dk, dv must be contiguous and share dtype and shape")
    B, H, N, D = q.shape
    if lse.dtype != torch.float32 or lse.numel() != B * H * N or not lse.is_contiguous():
        raise OmniAttnError("lse must be contiguous float32 [B, H, N]")
    m = _device_mask(block_mask, q.device, True)
    lib = load_library()
    need = int(lib.omni_attn_bwd_workspace_bytes(B, H, N))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), d_out.data_ptr(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), m["nb"].data_ptr(), m["idx"].data_ptr(),
                m["typ"].data_ptr(), _ptr(m["pidx"]), _ptr(m["pbool"]), _ptr(m["pbits"]), B, H, N, int(seqlen_orig), D,
                block_mask.Q_BLOCK_SIZE, block_mask.KV_BLOCK_SIZE, int(m["idx"].shape[3]), m["num_partial"],
                1 if q.dtype == torch.bfloat16 else 0, float(scale) if scale is not None else 0.0, stream,
                _ptr(status), workspace.data_ptr(), workspace.numel() * workspace.element_size())
        if softcap is not None and softcap > 0:
            rc = lib.omni_attn_bwd_ex_sm100(*args, float(softcap))
        else:
            rc = lib.omni_attn_bwd_sm100(*args)
    _check(rc)


class _OmniAttentionFn(torch.autograd.Function):
    """Forward and backward kernels as one differentiable op on padded tensors."""

    @staticmethod
    def forward(ctx, q, k, v, block_mask, seqlen_orig, scale, softcap):
        out = torch.empty_like(q)
        lse = torch.empty(q.shape[0], q.shape[1], q.shape[2], dtype=torch.float32, device=q.device)
        omni_attention_forward_out(q, k, v, out, block_mask, seqlen_orig, scale, lse, softcap=softcap)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.block_mask, ctx.seqlen_orig, ctx.scale, ctx.softcap = block_mask, seqlen_orig, scale, softcap
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse = ctx.saved_tensors
        d_out = d_out.contiguous()
        if ctx.seqlen_orig < q.shape[2]:
            d_out = d_out.clone()
            d_out[:, :, ctx.seqlen_orig:] = 0   # padded rows take no part but must be finite
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        omni_attention_backward_out(q, k, v, out, lse, d_out, dq, dk, dv, ctx.block_mask, ctx.seqlen_orig, ctx.scale,
                                    softcap=ctx.softcap)
        return dq, dk, dv, None, None, None, None


def omni_attention_autograd(query: Tensor, key: Tensor, value: Tensor, block_mask: OmniBlockMask,
                            scale: Optional[float] = None, softcap: Optional[float] = None) -> Tensor:
    """``omni_attention`` for training: same inputs and output, differentiable with respect to
    query, key and value (the gradients come from omni_attn_bwd_sm100 / omni_attn_bwd_ex_sm100)."""
    qp, kp, vp, block_mask, scale, n_orig, d_orig = _prepare(query, key, value, block_mask, scale, for_backward=True)
    out = _OmniAttentionFn.apply(qp, kp, vp, block_mask, n_orig, scale, softcap if softcap else None)
    return out[:, :, :n_orig, :d_orig]


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
