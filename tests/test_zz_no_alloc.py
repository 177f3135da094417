"""omni_attn_fwd_noalloc_sm100: the forward entry point for callers that cannot allocate device memory
and have no workspace to hand over (for instance a plug-in behind the reference's 13-argument binding,
which has no workspace argument, or a serving loop that must keep cudaMalloc off its hot path).
It keeps its scratch in an array built into the library, so nothing is allocated by the call.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test. The GPU test calls the entry point through the C ABI and compares it with the existing
omni_attn_fwd_sm100 on two calls in a row, the second with another mask and pool, because the
built-in scratch keeps what the first call left in it.
"""
import ctypes
import os
import re

import pytest
import torch

from conftest import OUT_ATOL, OUT_RTOL, LSE_ATOL, ROOT, load_golden
from omni_attention_b200 import ops


def _header_constant(name):
    src = open(os.path.join(ROOT, "include", "omni_attn_sm100.h")).read()
    return int(re.search(r"#define\s+" + name + r"\s+\(?(-?\d+)\)?", src).group(1))


def test_refuses_byte_pool_beyond_builtin_scratch_without_touching_the_gpu():
    lib = ops.load_library()
    limit = _header_constant("OMNI_ATTN_NOALLOC_MAX_PARTIAL")
    buf = (ctypes.c_char * 4096)()
    a = (ctypes.addressof(buf) + 15) & ~15
    rc = lib.omni_attn_fwd_noalloc_sm100(a, a, a, a, None, a, a, a, a, a, None, 1, 1, 128, 128, 64, 128, 128, 1,
                                         limit + 1, 0, 0.0, None, None)
    assert rc == _header_constant("OMNI_ERR_NOALLOC_LIMIT")
    assert b"OMNI_ATTN_NOALLOC_MAX_PARTIAL" in lib.omni_attn_error_string(rc)


def _call(fn, q, k, v, bm, dev):
    """One forward through the C ABI with the reference's byte-per-element pool; returns (out, lse, status)."""
    B, H, N, D = q.shape
    i32 = lambda t: t.to(device=dev, dtype=torch.int32).contiguous()
    nb, idx, typ = i32(bm.kv_num_blocks), i32(bm.kv_indices), i32(bm.block_mask_types)
    pidx = i32(bm.partial_block_mask_indices)
    pool = bm.partial_block_masks.to(dev).contiguous()
    out = torch.empty_like(q)
    lse = torch.empty(B, H, N, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), nb.data_ptr(), idx.data_ptr(),
            typ.data_ptr(), pidx.data_ptr(), pool.data_ptr(), None, B, H, N, N, D, 128, 128, int(idx.shape[3]),
            int(pool.shape[0]), 1 if q.dtype == torch.bfloat16 else 0, 0.0, torch.cuda.current_stream().cuda_stream,
            status.data_ptr())
    assert rc == 0, ops.load_library().omni_attn_error_string(rc)
    torch.cuda.synchronize()
    return out, lse, int(status.item())


def test_argument_checks_come_before_anything_else():
    """A call that is going to be refused is refused before the built-in array is touched: every code of
    the ordinary entry point comes back from this one too, without a GPU."""
    lib = ops.load_library()
    buf = (ctypes.c_char * 4096)()
    a = (ctypes.addressof(buf) + 15) & ~15
    call = lambda **kw: lib.omni_attn_fwd_noalloc_sm100(
        kw.get("q", a), a, a, a, None, a, a, a, a, a, None, 1, 1, kw.get("N", 128), 128, kw.get("D", 64), 128, 128, 1,
        kw.get("npart", 1), kw.get("dtype", 0), 0.0, None, None)
    assert call(q=None) == _header_constant("OMNI_ERR_NULL_POINTER")
    assert call(D=96) == _header_constant("OMNI_ERR_HEAD_DIM")
    assert call(dtype=5) == _header_constant("OMNI_ERR_DTYPE")
    assert call(N=100) == _header_constant("OMNI_ERR_SEQLEN")
    assert call(npart=-2) == _header_constant("OMNI_ERR_PARTIAL")


def _device_memory_in_use(dev):
    free, total = torch.cuda.mem_get_info(dev)
    return total - free, torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)


@pytest.mark.gpu
def test_noalloc_entry_matches_existing_entry_on_two_calls_in_a_row(cuda_device):
    lib = ops.load_library()
    for name in ("ref_interleaved_n512_d64", "ref_fcp_n512_d64"):   # second call: other mask, smaller pool
        g = load_golden(name)
        q, k, v = (g[x].to(cuda_device).contiguous() for x in "qkv")
        ref_out, ref_lse, ref_status = _call(lib.omni_attn_fwd_sm100, q, k, v, g["bm"], cuda_device)
        out, lse, status = _call(lib.omni_attn_fwd_noalloc_sm100, q, k, v, g["bm"], cuda_device)
        # once its first call on the device is behind it, the entry point takes no device memory: neither
        # the driver's count of bytes in use nor torch's allocator moves across a call
        # (everything the call needs is allocated by _call's caller side before `before` is read)
        B, H, N, D = q.shape
        i32 = lambda t: t.to(device=cuda_device, dtype=torch.int32).contiguous()
        bm = g["bm"]
        nb, idx, typ, pidx = i32(bm.kv_num_blocks), i32(bm.kv_indices), i32(bm.block_mask_types), i32(bm.partial_block_mask_indices)
        pool = bm.partial_block_masks.to(cuda_device).contiguous()
        o2 = torch.empty_like(q)
        stream = torch.cuda.current_stream().cuda_stream
        torch.cuda.synchronize()
        before = _device_memory_in_use(cuda_device)
        rc = lib.omni_attn_fwd_noalloc_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), o2.data_ptr(), None, nb.data_ptr(),
                                             idx.data_ptr(), typ.data_ptr(), pidx.data_ptr(), pool.data_ptr(), None, B, H, N, N,
                                             D, 128, 128, int(idx.shape[3]), int(pool.shape[0]), 0, 0.0, stream, None)
        torch.cuda.synchronize()
        assert rc == 0 and _device_memory_in_use(cuda_device) == before
        assert torch.equal(o2, out)
        assert status == 0 and ref_status == 0
        err = (out.float() - ref_out.float()).abs()
        assert bool((err <= OUT_ATOL + OUT_RTOL * ref_out.float().abs()).all()), f"{name}: max abs err {float(err.max())}"
        assert float((lse - ref_lse).abs().max()) <= LSE_ATOL
        # and both agree with the reference's own output for the case
        gerr = (out.float().cpu() - g["out"]).abs()
        assert bool((gerr <= OUT_ATOL + OUT_RTOL * g["out"].abs()).all())
    # a pool the caller has already bit-packed goes through unchanged
    g = load_golden("ref_fcp_n384_d128")
    q, k, v = (g[x].to(cuda_device).contiguous() for x in "qkv")
    bits = ops.pack_partial_masks(g["bm"].partial_block_masks.to(cuda_device))
    B, H, N, D = q.shape
    i32 = lambda t: t.to(device=cuda_device, dtype=torch.int32).contiguous()
    nb, idx, typ, pidx = (i32(getattr(g["bm"], n)) for n in ("kv_num_blocks", "kv_indices", "block_mask_types",
                                                               "partial_block_mask_indices"))
    out = torch.empty_like(q)
    rc = lib.omni_attn_fwd_noalloc_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), None, nb.data_ptr(),
                                         idx.data_ptr(), typ.data_ptr(), pidx.data_ptr(), None, bits.data_ptr(), B, H, N, N,
                                         D, 128, 128, int(idx.shape[3]), int(bits.shape[0]), 0, 0.0,
                                         torch.cuda.current_stream().cuda_stream, None)
    assert rc == 0
    torch.cuda.synchronize()
    gerr = (out.float().cpu() - g["out"]).abs()
    assert bool((gerr <= OUT_ATOL + OUT_RTOL * g["out"].abs()).all())


@pytest.mark.gpu
def test_noalloc_entry_at_its_pool_limit(cuda_device):
    """A byte pool of exactly OMNI_ATTN_NOALLOC_MAX_PARTIAL tiles is the largest the built-in array can
    bit-pack; the last tile is used. Same result as the ordinary entry point on the byte pool."""
    from omni_attention_b200.block_mask import BlockMaskType, OmniBlockMask

    lib = ops.load_library()
    limit = _header_constant("OMNI_ATTN_NOALLOC_MAX_PARTIAL")
    torch.manual_seed(4)
    B, H, N, D = 1, 8, 2048, 64
    nq = N // 128
    q, k, v = (torch.randn(B, H, N, D).half().to(cuda_device) for _ in range(3))
    pool = torch.rand(limit, 128, 128) < 0.5
    pool[:, torch.arange(128), torch.arange(128)] = True          # every row keeps a key in every tile
    qb = torch.arange(nq).view(nq, 1)
    pos = torch.arange(nq).view(1, nq)
    listed = pos <= qb
    idx = torch.where(listed, pos, 0).to(torch.int32).expand(B, H, nq, nq).contiguous()
    typ = torch.where(listed, int(BlockMaskType.PARTIAL), 0).to(torch.int32).expand(B, H, nq, nq).contiguous()
    nb = listed.sum(-1).to(torch.int32).expand(B, H, nq).contiguous()
    n_entries = B * H * nq * nq
    pidx = (limit - 1 - torch.arange(n_entries) % limit).to(torch.int32).view(B, H, nq, nq)   # entry 0 -> the last tile
    pidx = torch.where(typ == int(BlockMaskType.PARTIAL), pidx, torch.full_like(pidx, -1))
    bm = OmniBlockMask(nb, idx, typ, N, N, 128, 128, pidx, pool)
    ref_out, ref_lse, ref_status = _call(lib.omni_attn_fwd_sm100, q, k, v, bm, cuda_device)
    out, lse, status = _call(lib.omni_attn_fwd_noalloc_sm100, q, k, v, bm, cuda_device)
    assert status == 0 and ref_status == 0
    err = (out.float() - ref_out.float()).abs()
    assert bool((err <= OUT_ATOL + OUT_RTOL * ref_out.float().abs()).all()), float(err.max())
    assert float((lse - ref_lse).abs().max()) <= LSE_ATOL
