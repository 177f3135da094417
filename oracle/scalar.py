"""ctypes binding of the scalar C oracle (oracle/omni_oracle_scalar.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from typing import Optional, Tuple

import numpy as np
import torch

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, "libomni_oracle_scalar.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_DIR, "omni_oracle_scalar.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", src, "-o", _SO, "-lm"], check=True)
    return _SO


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        _lib.omni_oracle_rows.argtypes = [vp] * 8 + [i32] * 7 + [ctypes.c_float, vp, vp, i32, vp, vp, i32]
        _lib.omni_oracle_rows.restype = i32
    return _lib


def oracle_rows(q, k, v, bm, rows_bh, rows_q, scale: Optional[float] = None, seqlen_orig: Optional[int] = None,
                partial_fallback_causal: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Output rows [n, D] and lse [n] for the listed (batch*head, query) rows. q/k/v: [B, H, N, D]
    (any float dtype; upcast to fp32), ``bm`` any object with the OmniBlockMask fields."""
    B, H, N, D = q.shape
    f32 = lambda t: np.ascontiguousarray(t.detach().cpu().float().reshape(B * H, N, D).numpy())
    i32 = lambda t: np.ascontiguousarray(t.detach().cpu().to(torch.int32).numpy())
    qn, kn, vn = f32(q), f32(k), f32(v)
    nb, idx, typ = i32(bm.kv_num_blocks), i32(bm.kv_indices), i32(bm.block_mask_types)
    pidx = pool = None
    num_partial = 0
    if bm.partial_block_mask_indices is not None and bm.partial_block_masks is not None:
        pidx = i32(bm.partial_block_mask_indices)
        pool = np.ascontiguousarray(bm.partial_block_masks.detach().cpu().to(torch.uint8).numpy())
        num_partial = int(pool.shape[0])
    rb = np.ascontiguousarray(np.asarray(rows_bh, dtype=np.int32))
    rq = np.ascontiguousarray(np.asarray(rows_q, dtype=np.int32))
    n = int(rb.shape[0])
    out = np.zeros((n, D), dtype=np.float32)
    lse = np.zeros((n,), dtype=np.float32)
    p = lambda a: None if a is None or a.size == 0 else a.ctypes.data
    rc = _load().omni_oracle_rows(
        p(qn), p(kn), p(vn), p(nb), p(idx), p(typ), p(pidx), p(pool), num_partial, B * H, N,
        int(seqlen_orig if seqlen_orig is not None else N), D, int(bm.Q_BLOCK_SIZE), int(idx.shape[-1]),
        float(scale if scale is not None else 1.0 / math.sqrt(D)), p(rb), p(rq), n, p(out), p(lse),
        1 if partial_fallback_causal else 0)
    if rc != 0:
        raise ValueError("row index out of range")
    return torch.from_numpy(out), torch.from_numpy(lse)
