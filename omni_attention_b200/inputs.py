"""Seeded synthetic workloads: the five benchmark configurations (Q/K/V and block masks).

The reference's own inputs are synthetic too (``torch.randn`` Q/K/V and generated masks,
omni-attn-mma/generate_debug_data.py:20-25, :270-344; omni-attn-mma/generate_attn_data.py:155-281);
these generators follow the same recipes at the benchmark shapes, on a CPU generator so that a
seed gives the same data everywhere. Masks are built block by block, never as an N x N tensor.

  C1  causal,              B1  H8  N512   D64  fp16
  C2  random F/C/P/skip,   B1  H8  N2048  D64  fp16
  C3  interleaved,         B2  H16 N4096  D64  bf16   image spans 256, text U[64,512]
  C4  large interleaved,   B1  H32 N8192  D128 bf16   4-6 image spans of 1024, text U[128,1024]
  C5  long multi-image,    B4  H32 N32768 D128 bf16   8-16 images from {256,1024,4096}, text U[256,2048]
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor

from .block_mask import (BlockMaskType, OmniBlockMask, block_mask_from_row_limits,
                         create_causal_omni_block_mask, row_limits_from_modality_positions, _pack_lists)


@dataclass(frozen=True)
class Config:
    name: str
    B: int
    H: int
    N: int
    D: int
    dtype: torch.dtype
    pattern: str
    qkv_scale: float = 1.0


CONFIGS: Dict[str, Config] = {
    "C1": Config("C1", 1, 8, 512, 64, torch.float16, "causal"),
    "C2": Config("C2", 1, 8, 2048, 64, torch.float16, "random_fcp"),
    "C3": Config("C3", 2, 16, 4096, 64, torch.bfloat16, "interleaved_256"),
    "C4": Config("C4", 1, 32, 8192, 128, torch.bfloat16, "interleaved_1024", 0.5),
    "C5": Config("C5", 4, 32, 32768, 128, torch.bfloat16, "multi_image", 0.5),
}


def make_qkv(B: int, H: int, N: int, D: int, dtype: torch.dtype, seed: int, qkv_scale: float = 1.0,
             bh_range: Optional[Tuple[int, int]] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """i.i.d. N(0,1)*qkv_scale, drawn in fp32 per (batch*head) slice and rounded to ``dtype``.

    Each slice has its own generator seeded by (seed, slice index), so a rank holding only
    ``bh_range`` of the flattened batch*head axis gets exactly the values the full tensor has.
    Returned shape: [1, n, N, D] for a range, else [B, H, N, D]. CPU tensors.
    """
    lo, hi = (0, B * H) if bh_range is None else bh_range
    outs = [torch.empty(hi - lo, N, D, dtype=dtype) for _ in range(3)]
    g = torch.Generator(device="cpu")
    for i in range(lo, hi):
        g.manual_seed(seed * 1000003 + i)
        for t in outs:
            x = torch.randn(N, D, generator=g, dtype=torch.float32)
            if qkv_scale != 1.0:
                x = x * qkv_scale
            t[i - lo] = x.to(dtype)
    if bh_range is None:
        return tuple(t.view(B, H, N, D) for t in outs)
    return tuple(t.unsqueeze(0) for t in outs)


def random_fcp_block_mask(B: int, H: int, N: int, seed: int, p_skip: float = 0.2, p_full: float = 0.4,
                          block: int = 128) -> OmniBlockMask:
    """Random block types: diagonal CAUSAL; each block below it independently not listed
    (p_skip), FULL (p_full) or PARTIAL with a Bernoulli(0.5) element mask (the rest). One draw shared
    by all heads and batch elements, as omni-attn-mma/generate_debug_data.py:285-305 does. Every
    query row keeps at least its own position (the diagonal block is always listed)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    nq = N // block
    u = torch.rand(nq, nq, generator=g)
    grid = torch.full((nq, nq), int(BlockMaskType.PARTIAL), dtype=torch.int32)
    grid[u < p_skip + p_full] = int(BlockMaskType.FULL)
    grid[u < p_skip] = int(BlockMaskType.MASKED)
    qb = torch.arange(nq).view(nq, 1)
    kb = torch.arange(nq).view(1, nq)
    grid[kb > qb] = int(BlockMaskType.MASKED)
    grid[kb == qb] = int(BlockMaskType.CAUSAL)
    nb, idx, typ = _pack_lists(grid)
    is_p = typ == BlockMaskType.PARTIAL
    m = int(is_p.sum())
    pidx = torch.full((nq, nq), -1, dtype=torch.int32)
    pidx[is_p] = torch.arange(m, dtype=torch.int32)
    pool = torch.rand(m, block, block, generator=g) < 0.5
    ex = lambda t: t.view(1, 1, *t.shape).expand(B, H, *t.shape).contiguous()
    return OmniBlockMask(ex(nb), ex(idx), ex(typ), N, N, block, block, ex(pidx), pool)


def _draw_spans(N: int, g: torch.Generator, text_range: Tuple[int, int], image_sizes: List[int],
                n_images: Optional[Tuple[int, int]]) -> List[Tuple[int, int]]:
    """Alternate causal text spans and bidirectional image spans until N tokens; returns the image
    spans as (offset, length). With ``n_images`` = (lo, hi) the number of images is drawn first and
    the sequence is text afterwards; otherwise images repeat until the sequence is full."""
    ri = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    budget = ri(*n_images) if n_images is not None else 1 << 30
    spans, pos = [], 0
    while pos < N:
        pos += ri(*text_range)
        if pos >= N or budget == 0:
            break
        size = image_sizes[ri(0, len(image_sizes) - 1)]
        if pos + size > N:
            break
        spans.append((pos, size))
        pos += size
        budget -= 1
    return spans


def interleaved_block_mask(cfg: Config, seed: int, share_partial_across_heads: bool = True) -> Tuple[OmniBlockMask, list]:
    g = torch.Generator(device="cpu").manual_seed(seed + 7919)
    if cfg.pattern == "interleaved_256":
        kw = dict(text_range=(64, 512), image_sizes=[256], n_images=None)
    elif cfg.pattern == "interleaved_1024":
        kw = dict(text_range=(128, 1024), image_sizes=[1024], n_images=(4, 6))
    elif cfg.pattern == "multi_image":
        kw = dict(text_range=(256, 2048), image_sizes=[256, 1024, 4096], n_images=(8, 16))
    else:
        raise ValueError(cfg.pattern)
    spans = [_draw_spans(cfg.N, g, **kw) for _ in range(cfg.B)]
    limits, causal_rows = row_limits_from_modality_positions(cfg.N, spans)
    bm = block_mask_from_row_limits(limits, cfg.H, causal_rows, 128, share_partial_across_heads)
    return bm, spans


def make_block_mask(cfg: Config, seed: int = 0, B: Optional[int] = None) -> Tuple[OmniBlockMask, dict]:
    """Block mask of a configuration (``B`` overrides the batch size, e.g. one element per GPU)."""
    if B is not None and B != cfg.B:
        cfg = Config(cfg.name, B, cfg.H, cfg.N, cfg.D, cfg.dtype, cfg.pattern, cfg.qkv_scale)
    meta: dict = {"config": cfg.name, "seed": seed}
    if cfg.pattern == "causal":
        bm = create_causal_omni_block_mask(cfg.B, cfg.H, cfg.N, cfg.N, 128, 128, "cpu")
    elif cfg.pattern == "random_fcp":
        bm = random_fcp_block_mask(cfg.B, cfg.H, cfg.N, seed)
    else:
        bm, spans = interleaved_block_mask(cfg, seed)
        meta["image_spans"] = spans
    return bm, meta


def make_inputs(name: str, seed: int = 0, bh_range: Optional[Tuple[int, int]] = None,
                B: Optional[int] = None) -> Tuple[Tensor, Tensor, Tensor, OmniBlockMask, dict]:
    """(q, k, v, block_mask, meta) of configuration ``name`` on the CPU.

    ``bh_range`` restricts everything to a range of the flattened batch*head axis (the shard one
    GPU owns); the mask is then the matching ``slice_heads`` view.
    """
    cfg = CONFIGS[name]
    if B is not None and B != cfg.B:
        cfg = Config(cfg.name, B, cfg.H, cfg.N, cfg.D, cfg.dtype, cfg.pattern, cfg.qkv_scale)
    bm, meta = make_block_mask(cfg, seed)
    q, k, v = make_qkv(cfg.B, cfg.H, cfg.N, cfg.D, cfg.dtype, seed, cfg.qkv_scale, bh_range)
    if bh_range is not None:
        bm = bm.slice_heads(*bh_range)
    meta.update(B=cfg.B, H=cfg.H, N=cfg.N, D=cfg.D, dtype=str(cfg.dtype).replace("torch.", ""))
    return q, k, v, bm, meta


def effective_flops(bm: OmniBlockMask, head_dim: int) -> int:
    """4 * 128 * 128 * D per visited block: Q K^T and P V of every listed FULL/CAUSAL/PARTIAL block
    counted as full tiles, nothing for softmax, masks or blocks that are not listed."""
    return 4 * bm.Q_BLOCK_SIZE * bm.KV_BLOCK_SIZE * head_dim * bm.visited_blocks()
