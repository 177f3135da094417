"""Block-mask metadata of omni-attention: the same container and type codes as the reference's
operator surface, with vectorised builders.

Mirrors (same names, fields and meaning):
  * ``BlockMaskType``  - omni-attn-mma/omni_attn_torch.py:30-41
  * ``OmniBlockMask``  - omni-attn-mma/omni_attn_torch.py:48-145 (fields, ``num_q_blocks``, ``shape``,
    ``to_dense_mask``)
  * ``build_partial_block_data`` - omni-attn-mma/omni_attn_torch.py:148-205
  * ``create_causal_omni_block_mask`` - omni-attn-mma/omni_attn_torch.py:1950-2015

The reference builds these with Python loops over every block (and every element for CAUSAL
blocks); here everything is tensor arithmetic so that 32K-token masks are built in milliseconds,
and masks that follow the "every query row attends keys 0..limit" pattern of interleaved
text/image sequences (transfusion_pytorch/transfusion.py:496-515) are classified block by block
without ever materialising an N x N tensor.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import IntEnum
from typing import Optional, Sequence, Tuple

import torch
from torch import Tensor


class BlockMaskType(IntEnum):
    MASKED = 0   # block not visited
    CAUSAL = 1   # key position <= query position (absolute positions)
    FULL = 2     # every element attends
    PARTIAL = 3  # per-element mask from the partial pool


@dataclass
class OmniBlockMask:
    """Block-sparse attention mask.

    kv_num_blocks     [B, H, nq]              number of listed KV blocks per Q block
    kv_indices        [B, H, nq, max_blocks]  listed KV block ids (first kv_num_blocks valid)
    block_mask_types  [B, H, nq, max_blocks]  BlockMaskType per listed block
    q_len, kv_len     padded lengths (multiples of the block sizes)
    partial_block_mask_indices  [B, H, nq, max_blocks] index into the pool, -1 = none
    partial_block_masks         [P, Q_BLOCK_SIZE, KV_BLOCK_SIZE] bool, True = attend
    """

    kv_num_blocks: Tensor
    kv_indices: Tensor
    block_mask_types: Tensor
    q_len: int
    kv_len: int
    Q_BLOCK_SIZE: int = 128
    KV_BLOCK_SIZE: int = 128
    partial_block_mask_indices: Optional[Tensor] = None
    partial_block_masks: Optional[Tensor] = None   # a property, see below: may be expanded on first read
    # Device-side copies and the bit-packed partial pool, filled lazily by the operator.
    _cache: dict = field(default_factory=dict, repr=False, compare=False)

    def set_lazy_partial_pool(self, make) -> None:
        """``make()`` returns the bool pool; it is called the first time ``partial_block_masks`` is read.
        Used by builders that hold the pool in another form (bit-packed on the GPU) and whose consumers
        never need the byte-per-element copy."""
        self.__dict__["_pool"] = None
        self.__dict__["_pool_make"] = make

    @property
    def num_q_blocks(self) -> int:
        return (self.q_len + self.Q_BLOCK_SIZE - 1) // self.Q_BLOCK_SIZE

    @property
    def num_kv_blocks(self) -> int:
        return (self.kv_len + self.KV_BLOCK_SIZE - 1) // self.KV_BLOCK_SIZE

    @property
    def device(self) -> torch.device:
        return self.kv_num_blocks.device

    @property
    def shape(self) -> Tuple[int, int, int, int]:
        B, H, _ = self.kv_num_blocks.shape
        return (B, H, self.q_len, self.kv_len)

    def to(self, device) -> "OmniBlockMask":
        mv = lambda t: None if t is None else t.to(device)
        return OmniBlockMask(
            mv(self.kv_num_blocks), mv(self.kv_indices), mv(self.block_mask_types), self.q_len,
            self.kv_len, self.Q_BLOCK_SIZE, self.KV_BLOCK_SIZE, mv(self.partial_block_mask_indices),
            mv(self.partial_block_masks))

    def slice_heads(self, start: int, stop: int) -> "OmniBlockMask":
        """Mask of the flattened (batch*head) range [start, stop), as a [1, stop-start] batch.

        This is the unit multi-GPU sharding works in: every (batch, head) pair is independent.
        The partial pool is shared, not re-indexed.
        """
        B, H, nq = self.kv_num_blocks.shape
        fl = lambda t: None if t is None else t.reshape(B * H, *t.shape[2:])[start:stop].unsqueeze(0)
        out = OmniBlockMask(
            fl(self.kv_num_blocks), fl(self.kv_indices), fl(self.block_mask_types), self.q_len,
            self.kv_len, self.Q_BLOCK_SIZE, self.KV_BLOCK_SIZE, fl(self.partial_block_mask_indices), None)
        # the pool is shared as it is: expanded, or still to be expanded on first read
        out.__dict__["_pool"] = self.__dict__.get("_pool")
        out.__dict__["_pool_make"] = (lambda: self.partial_block_masks) if self.__dict__.get("_pool_make") else None
        return out

    def visited_blocks(self) -> int:
        """Listed entries that are actually computed (type FULL, CAUSAL or PARTIAL)."""
        nb = self.kv_num_blocks.long().clamp(0, self.kv_indices.shape[-1])
        pos = torch.arange(self.kv_indices.shape[-1], device=self.device)
        listed = pos < nb.unsqueeze(-1)
        t = self.block_mask_types
        return int((listed & (t >= BlockMaskType.CAUSAL) & (t <= BlockMaskType.PARTIAL)).sum().item())

    def sparsity(self) -> float:
        """Percentage of (Q block, KV block) pairs that are not listed."""
        B, H, nq = self.kv_num_blocks.shape
        total = B * H * nq * self.num_kv_blocks
        return 100.0 * (1.0 - float(self.kv_num_blocks.sum().item()) / total)

    def to_dense_mask(self) -> Tensor:
        """Boolean [B, H, q_len, kv_len], True = attend."""
        return dense_mask_from_blocks(self)


def _get_partial_pool(self):
    pool = self.__dict__.get("_pool")
    make = self.__dict__.get("_pool_make")
    if pool is None and make is not None:
        pool = make()
        self.__dict__["_pool"] = pool
        self.__dict__["_pool_make"] = None
    return pool


def _set_partial_pool(self, value):
    self.__dict__["_pool"] = value
    self.__dict__["_pool_make"] = None


# The dataclass keeps the reference's field name and position; reads and writes go through a
# property so that a builder may leave the byte-per-element pool unexpanded until someone asks.
OmniBlockMask.partial_block_masks = property(_get_partial_pool, _set_partial_pool)


def dense_mask_from_blocks(bm: OmniBlockMask, bh_range: Optional[Tuple[int, int]] = None) -> Tensor:
    """Expand listed blocks to a dense boolean mask (optionally only a flattened batch*head range,
    returned as [n, q_len, kv_len]).

    Semantics of omni-attn-mma/omni_attn_torch.py:89-145: FULL sets the block; CAUSAL sets key <=
    query by absolute position; PARTIAL copies its pool entry, or falls back to CAUSAL when there is
    no usable pool entry; MASKED and unlisted blocks stay False.
    """
    B, H, nq, mb = bm.kv_indices.shape
    Bq, Bk = bm.Q_BLOCK_SIZE, bm.KV_BLOCK_SIZE
    nk = bm.num_kv_blocks
    dev = bm.device
    lo, hi = (0, B * H) if bh_range is None else bh_range
    n = hi - lo
    flat = lambda t: t.reshape(B * H, *t.shape[2:])[lo:hi]
    nb = flat(bm.kv_num_blocks).long().clamp(0, mb)
    idx = flat(bm.kv_indices).long()
    typ = flat(bm.block_mask_types).long()
    listed = torch.arange(mb, device=dev) < nb.unsqueeze(-1)
    listed &= (idx >= 0) & (idx < nk)
    pidx = None
    if bm.partial_block_mask_indices is not None and bm.partial_block_masks is not None:
        pidx = flat(bm.partial_block_mask_indices).long()
        P = bm.partial_block_masks.shape[0]
        usable = (pidx >= 0) & (pidx < P)
    else:
        usable = torch.zeros_like(listed)
    is_partial = listed & (typ == BlockMaskType.PARTIAL) & usable
    is_causal = listed & ((typ == BlockMaskType.CAUSAL) | ((typ == BlockMaskType.PARTIAL) & ~usable))
    is_full = listed & (typ == BlockMaskType.FULL)

    # block-level grids [n, nq, nk]; a later list entry for the same block overrides nothing
    # here because FULL/CAUSAL only ever add and PARTIAL entries are written last.
    blocks = torch.zeros(n, nq, Bq, nk, Bk, dtype=torch.bool, device=dev)
    qpos = (torch.arange(nq, device=dev) * Bq).view(nq, 1, 1, 1) + torch.arange(Bq, device=dev).view(1, Bq, 1, 1)
    kpos = (torch.arange(nk, device=dev) * Bk).view(1, 1, nk, 1) + torch.arange(Bk, device=dev).view(1, 1, 1, Bk)
    causal_pat = kpos <= qpos  # [nq, Bq, nk, Bk]

    def block_grid(sel: Tensor) -> Tensor:
        g = torch.zeros(n, nq, nk, dtype=torch.bool, device=dev)
        i0, i1, i2 = sel.nonzero(as_tuple=True)
        g[i0, i1, idx[i0, i1, i2]] = True
        return g

    blocks |= block_grid(is_full).view(n, nq, 1, nk, 1)
    blocks |= block_grid(is_causal).view(n, nq, 1, nk, 1) & causal_pat.unsqueeze(0)
    if pidx is not None and bool(is_partial.any()):
        i0, i1, i2 = is_partial.nonzero(as_tuple=True)
        tiles = bm.partial_block_masks[pidx[i0, i1, i2]].to(torch.bool)  # [m, Bq, Bk]
        blocks[i0, i1, :, idx[i0, i1, i2], :] = tiles
    dense = blocks.view(n, nq * Bq, nk * Bk)[:, : bm.q_len, : bm.kv_len]
    if bh_range is None:
        return dense.reshape(B, H, bm.q_len, bm.kv_len)
    return dense


def build_partial_block_data(block_mask: OmniBlockMask, dense_mask: Tensor) -> Tuple[Tensor, Tensor]:
    """Per-element masks of the PARTIAL blocks, cut out of ``dense_mask`` [B, H, q, kv].

    Returns ``(partial_block_mask_indices, partial_block_masks)`` in the reference's format and
    order (pool entries numbered in (b, h, q_block, list position) order, one entry per listed
    PARTIAL block, no sharing), omni-attn-mma/omni_attn_torch.py:148-205.
    """
    B, H, nq, mb = block_mask.block_mask_types.shape
    Bq, Bk = block_mask.Q_BLOCK_SIZE, block_mask.KV_BLOCK_SIZE
    dev = dense_mask.device
    ql, kl = block_mask.q_len, block_mask.kv_len
    if dense_mask.shape[2] != ql or dense_mask.shape[3] != kl:
        padded = torch.zeros(B, H, ql, kl, dtype=dense_mask.dtype, device=dev)
        a, b = min(dense_mask.shape[2], ql), min(dense_mask.shape[3], kl)
        padded[:, :, :a, :b] = dense_mask[:, :, :a, :b]
        dense_mask = padded
    nqp, nkp = nq * Bq, block_mask.num_kv_blocks * Bk
    if (ql, kl) != (nqp, nkp):
        padded = torch.zeros(B, H, nqp, nkp, dtype=dense_mask.dtype, device=dev)
        padded[:, :, :ql, :kl] = dense_mask
        dense_mask = padded
    nb = block_mask.kv_num_blocks.long().clamp(0, mb)
    listed = torch.arange(mb, device=dev) < nb.unsqueeze(-1)
    sel = listed & (block_mask.block_mask_types == BlockMaskType.PARTIAL)
    indices = torch.full((B, H, nq, mb), -1, dtype=torch.int32, device=dev)
    b_, h_, q_, i_ = sel.nonzero(as_tuple=True)  # row-major order = the reference's loop order
    m = b_.numel()
    if m == 0:
        return indices, torch.empty(0, Bq, Bk, dtype=torch.bool, device=dev)
    indices[b_, h_, q_, i_] = torch.arange(m, dtype=torch.int32, device=dev)
    kvb = block_mask.kv_indices[b_, h_, q_, i_].long()
    tiles = dense_mask.view(B, H, nq, Bq, block_mask.num_kv_blocks, Bk)[b_, h_, q_, :, kvb, :]
    return indices, tiles.to(torch.bool).contiguous()


def create_causal_omni_block_mask(batch: int, nheads: int, q_len: int, kv_len: int,
                                  Q_BLOCK_SIZE: int = 128, KV_BLOCK_SIZE: int = 128,
                                  device="cpu") -> OmniBlockMask:
    """Causal mask: diagonal blocks CAUSAL, blocks below FULL, blocks above not listed
    (omni-attn-mma/omni_attn_torch.py:1950-2015)."""
    qp = -(-q_len // Q_BLOCK_SIZE) * Q_BLOCK_SIZE
    kp = -(-kv_len // KV_BLOCK_SIZE) * KV_BLOCK_SIZE
    nq, nk = qp // Q_BLOCK_SIZE, kp // KV_BLOCK_SIZE
    qb = torch.arange(nq, device=device).view(nq, 1)
    pos = torch.arange(nk, device=device).view(1, nk)
    listed = pos <= qb
    idx = torch.where(listed, pos, 0).to(torch.int32)
    typ = torch.where(listed, torch.where(pos == qb, int(BlockMaskType.CAUSAL), int(BlockMaskType.FULL)),
                      int(BlockMaskType.MASKED)).to(torch.int32)
    nb = listed.sum(-1).to(torch.int32)
    ex = lambda t: t.unsqueeze(0).unsqueeze(0).expand(batch, nheads, *t.shape).contiguous()
    return OmniBlockMask(ex(nb), ex(idx), ex(typ), qp, kp, Q_BLOCK_SIZE, KV_BLOCK_SIZE)


def _pack_lists(grid_type: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """[..., nq, nk] type grid (0 = not listed) -> (kv_num_blocks, kv_indices, block_mask_types) with
    listed blocks first, ascending, max_blocks = nk."""
    nk = grid_type.shape[-1]
    listed = grid_type != 0
    # stable sort: listed blocks first, ascending block id
    key = (~listed).to(torch.int32) * nk + torch.arange(nk, device=grid_type.device, dtype=torch.int32)
    order = key.argsort(dim=-1, stable=True)
    nb = listed.sum(-1).to(torch.int32)
    typ = torch.gather(grid_type, -1, order).to(torch.int32)
    idx = torch.where(typ != 0, order.to(torch.int32), torch.zeros((), dtype=torch.int32, device=grid_type.device))
    return nb, idx.contiguous(), typ.contiguous()


def block_mask_from_row_limits(limits: Tensor, nheads: int, causal_rows: Optional[Tensor] = None,
                               block: int = 128, share_partial_across_heads: bool = True) -> OmniBlockMask:
    """Mask where query row q of batch element b attends keys ``0 .. limits[b, q]`` inclusive.

    That is the shape of every interleaved text/image mask: ``limits[q] = q`` on text tokens and the
    last token of the enclosing span on image tokens (causal | modality rule,
    transfusion_pytorch/transfusion.py:496-515). Block types follow the reference's derivation from
    a dense mask (omni-attn-mma/generate_attn_data.py:200-236): all elements set -> FULL; none ->
    not listed; a diagonal block whose rows are all plain-causal rows -> CAUSAL; anything else ->
    PARTIAL with its element mask in the pool. ``causal_rows`` [B, N] marks rows that may form a
    CAUSAL block (default: rows with ``limits == q``).

    Partial pool entries are shared by all heads of a batch element unless
    ``share_partial_across_heads`` is False, in which case each head gets its own copy exactly as
    the reference's ``build_partial_block_data`` lays them out. Never builds an N x N tensor.
    """
    B, N = limits.shape
    assert N % block == 0, "sequence length must be a multiple of the block size"
    dev = limits.device
    nq = N // block
    lim = limits.long().view(B, nq, block)
    if causal_rows is None:
        causal_rows = limits.long() == torch.arange(N, device=dev)
    pure = causal_rows.view(B, nq, block).all(-1)  # [B, nq]
    kstart = torch.arange(nq, device=dev) * block
    # allowed columns of row (b, qb, r) inside KV block kb: clamp(lim + 1 - kb*block, 0, block)
    cnt = (lim.unsqueeze(-1) + 1 - kstart.view(1, 1, 1, nq)).clamp(0, block)  # [B, nq, block, nk]
    all_full = (cnt == block).all(2)
    all_empty = (cnt == 0).all(2)
    diag = torch.eye(nq, dtype=torch.bool, device=dev).unsqueeze(0)
    r = torch.arange(block, device=dev)
    looks_causal = (cnt == (r + 1).view(1, 1, block, 1)).all(2)  # only ever true on the diagonal
    grid = torch.full((B, nq, nq), int(BlockMaskType.PARTIAL), dtype=torch.int32, device=dev)
    grid[diag.expand(B, -1, -1) & looks_causal & pure.unsqueeze(-1)] = int(BlockMaskType.CAUSAL)
    grid[all_full] = int(BlockMaskType.FULL)
    grid[all_empty] = int(BlockMaskType.MASKED)
    nb, idx, typ = _pack_lists(grid)

    is_p = typ == BlockMaskType.PARTIAL  # [B, nq, mb]
    b_, q_, i_ = is_p.nonzero(as_tuple=True)
    m = b_.numel()
    pidx = torch.full((B, nq, nq), -1, dtype=torch.int32, device=dev)
    pool = torch.empty(0, block, block, dtype=torch.bool, device=dev)
    if m > 0:
        pidx[b_, q_, i_] = torch.arange(m, dtype=torch.int32, device=dev)
        c = cnt[b_, q_, :, idx[b_, q_, i_].long()]  # [m, block] allowed-column counts per row
        pool = torch.arange(block, device=dev).view(1, 1, block) < c.unsqueeze(-1)
    exh = lambda t: t.unsqueeze(1).expand(B, nheads, *t.shape[1:]).contiguous()
    nb, idx, typ, pidx = exh(nb), exh(idx), exh(typ), exh(pidx)
    if m > 0 and not share_partial_across_heads:
        # reference layout: entries numbered in (b, h, q_block, position) order, one copy per head
        per_b = torch.bincount(b_, minlength=B)                      # partial blocks per batch element
        first = torch.cumsum(per_b, 0) - per_b                       # first shared index of element b
        local = pidx.long() - first.view(B, 1, 1, 1)                 # index within the batch element
        base = (first * nheads).view(B, 1, 1, 1) + torch.arange(nheads, device=dev).view(1, nheads, 1, 1) * per_b.view(B, 1, 1, 1)
        new = torch.where(pidx >= 0, (base + local).to(torch.int32), pidx)
        order = torch.empty(m * nheads, dtype=torch.long, device=dev)
        src = pidx[pidx >= 0].long()           # shared index of every (b,h,q,i) entry, row-major
        order[new[new >= 0].long()] = src
        pool = pool[order]
        pidx = new
    return OmniBlockMask(nb, idx, typ, N, N, block, block, pidx, pool.contiguous())


def block_mask_from_dense(dense: Tensor, block: int = 128, causal_ok: Optional[Tensor] = None) -> OmniBlockMask:
    """Derive an OmniBlockMask from a dense boolean mask [B, H, N, N] (N a multiple of ``block``).

    FULL / not listed / CAUSAL (block equals the absolute-position causal pattern, and, when
    ``causal_ok`` [nq] is given, only where it allows) / PARTIAL, as in
    omni-attn-mma/generate_attn_data.py:200-236. For small sizes and tests.
    """
    B, H, N, _ = dense.shape
    nq = N // block
    dev = dense.device
    t = dense.view(B, H, nq, block, nq, block).permute(0, 1, 2, 4, 3, 5)  # [B,H,nq,nk,Bq,Bk]
    all_ = t.all(-1).all(-1)
    any_ = t.any(-1).any(-1)
    pos = torch.arange(N, device=dev)
    causal = (pos.view(1, N) <= pos.view(N, 1)).view(nq, block, nq, block).permute(0, 2, 1, 3)
    is_c = (t == causal.view(1, 1, nq, nq, block, block)).all(-1).all(-1)
    if causal_ok is not None:
        is_c &= causal_ok.view(1, 1, nq, 1).to(dev)
    grid = torch.full((B, H, nq, nq), int(BlockMaskType.PARTIAL), dtype=torch.int32, device=dev)
    grid[is_c] = int(BlockMaskType.CAUSAL)
    grid[all_] = int(BlockMaskType.FULL)
    grid[~any_] = int(BlockMaskType.MASKED)
    nb, idx, typ = _pack_lists(grid)
    bm = OmniBlockMask(nb, idx, typ, N, N, block, block)
    if bool((typ == BlockMaskType.PARTIAL).any()):
        bm.partial_block_mask_indices, bm.partial_block_masks = build_partial_block_data(bm, dense)
    return bm


def row_limits_from_modality_positions(seq_len: int, modality_positions: Sequence[Sequence[Tuple[int, int]]],
                                       device="cpu") -> Tuple[Tensor, Tensor]:
    """Per-row attention limits for the causal | modality rule.

    ``modality_positions[b]`` lists ``(offset, length)`` of the bidirectional (image) spans of batch
    element b. Returns ``(limits [B, N], causal_rows [B, N])``: a token inside a span attends
    through the span's last token, any other token attends causally.
    """
    B = len(modality_positions)
    limits = torch.arange(seq_len, device=device).repeat(B, 1)
    causal_rows = torch.ones(B, seq_len, dtype=torch.bool, device=device)
    for b, spans in enumerate(modality_positions):
        for off, length in spans:
            lo, hi = max(0, int(off)), min(seq_len, int(off) + int(length))
            if hi > lo:
                limits[b, lo:hi] = torch.maximum(limits[b, lo:hi], torch.tensor(hi - 1, device=device))
                causal_rows[b, lo:hi] = False
    return limits, causal_rows


def _limits_from_modality_tensor(modality_positions: Tensor, seq_len: int, padded: int) -> Tuple[Tensor, Tensor]:
    """Row limits (-1 on padding rows) and plain-causal-row flags for a [B, M, 3] (type, offset, length) tensor."""
    mp = modality_positions.detach().cpu().long()
    B = mp.shape[0]
    q = torch.arange(padded).view(1, padded)
    limits = q.repeat(B, 1)
    plain = torch.ones(B, padded, dtype=torch.bool)
    for m in range(mp.shape[1]):
        off, ln = mp[:, m, 1].view(B, 1), mp[:, m, 2].view(B, 1)
        started = (ln > 0) & (q >= off)
        limits = torch.where(started, torch.maximum(limits, off + ln - 1), limits)
        plain &= ~(started & (q < off + ln))
    limits = limits.clamp(max=seq_len - 1)
    pad = q >= seq_len
    limits = torch.where(pad, torch.full_like(limits, -1), limits)
    plain &= ~pad
    return limits, plain


def count_partial_tiles(limits: Tensor, plain: Tensor, block: int = 128) -> int:
    """Number of PARTIAL tiles of the row-limit mask ``limits`` [B, N] (the same typing rule as
    ``block_mask_from_row_limits`` and the GPU builder, evaluated from the smallest and largest limit
    of every block of rows; the pool is shared by the heads)."""
    B, N = limits.shape
    nq = N // block
    lim = limits.long().view(B, nq, block)
    lim_min, lim_max = lim.min(-1).values, lim.max(-1).values
    q = torch.arange(N, device=limits.device).view(1, nq, block)
    causal_block = (plain.view(B, nq, block) & (lim == q)).all(-1)
    lo = torch.div(lim_min + 1, block, rounding_mode="floor")   # first KV block that is not FULL
    hi = torch.div(lim_max, block, rounding_mode="floor")       # last KV block that is listed
    cnt = (hi - lo + 1).clamp(min=0)
    qb = torch.arange(nq, device=limits.device).view(1, nq)
    cnt = cnt - ((lo <= qb) & (qb <= hi) & causal_block).long()  # a CAUSAL diagonal tile is not PARTIAL
    return int(cnt.sum().item())


def create_omni_block_mask_from_modality_positions(modality_positions: Tensor, batch: int, nheads: int, q_len: int,
                                                   kv_len: int, Q_BLOCK_SIZE: int = 128, KV_BLOCK_SIZE: int = 128,
                                                   device="cpu") -> OmniBlockMask:
    """Block mask of an interleaved text / image sequence from ``modality_positions`` [B, M, 3] =
    (type, offset, length); same name, arguments and padding behaviour as the reference's builder
    (omni-attn-mma/omni_attn_torch.py:1518-1736).

    The dense mask it stands for is the reference's: key <= query, or query >= offset and key <
    offset + length for some span (transfusion_pytorch/transfusion.py:496-515); nothing at or beyond the
    unpadded length. Blocks are typed by content (all allowed -> FULL, none -> not listed, a diagonal
    block of plain causal rows -> CAUSAL, else PARTIAL); the reference types some fully allowed blocks
    PARTIAL with an all-true tile, which expands to the same dense mask. The PARTIAL pool is shared by
    the heads of a batch element. On a CUDA device the mask is built by the library's kernels and stays
    on the device; on the CPU it is built with tensor arithmetic. Neither builds an N x N tensor.
    """
    if q_len != kv_len:
        raise ValueError("Q_len must equal KV_len")
    if Q_BLOCK_SIZE != 128 or KV_BLOCK_SIZE != 128:
        raise ValueError("Unsupported block size: Q_BLOCK_SIZE and KV_BLOCK_SIZE must be 128.")
    if modality_positions.dim() != 3 or modality_positions.shape[0] != batch or modality_positions.shape[2] != 3:
        raise ValueError("modality_positions must be [batch, M, 3]")
    padded = -(-q_len // 128) * 128
    dev = torch.device(device)
    if dev.type == "cuda":
        from .ops import build_block_mask_cuda

        return build_block_mask_cuda(modality_positions, batch, nheads, q_len, padded, dev)
    limits, plain = _limits_from_modality_tensor(modality_positions, q_len, padded)
    return block_mask_from_row_limits(limits, nheads, plain, 128, True).to(dev)


def _stack_block_masks(parts, B: int, H: int) -> OmniBlockMask:
    """Join per-(batch, head) single-slice masks (row-major over B*H, equal geometry) into one mask;
    partial pools are concatenated and the indices shifted."""
    first = parts[0]
    nb = torch.cat([p.kv_num_blocks for p in parts], 0).view(B, H, -1)
    idx = torch.cat([p.kv_indices for p in parts], 0).view(B, H, *first.kv_indices.shape[2:])
    typ = torch.cat([p.block_mask_types for p in parts], 0).view(B, H, *first.block_mask_types.shape[2:])
    pools, pidx, base = [], [], 0
    cache = {}
    for p in parts:
        if p.partial_block_masks is None or p.partial_block_masks.shape[0] == 0:
            pidx.append(torch.full_like(p.kv_indices, -1))
            continue
        key = id(p)
        if key not in cache:            # a slice object shared by several heads brings its tiles once
            cache[key] = base
            pools.append(p.partial_block_masks)
            base += p.partial_block_masks.shape[0]
        off = cache[key]
        pi = p.partial_block_mask_indices
        pidx.append(torch.where(pi >= 0, pi + off, pi))
    bm = OmniBlockMask(nb.contiguous(), idx.contiguous(), typ.contiguous(), first.q_len, first.kv_len,
                       first.Q_BLOCK_SIZE, first.KV_BLOCK_SIZE)
    if pools:
        bm.partial_block_mask_indices = torch.cat(pidx, 0).view(idx.shape).to(torch.int32).contiguous()
        bm.partial_block_masks = torch.cat(pools, 0).contiguous()
    return bm


def _retile_by_quadrants(bm: OmniBlockMask, block: int) -> OmniBlockMask:
    """``retile_block_mask`` for a source block size that divides ``block``: every target tile is r x r
    source blocks (r = block / source size), so its type and, where it is PARTIAL, its element mask
    follow from those r*r list entries alone. Nothing of size N x N is built; the work is one small
    grid per (batch, head) plus one [block, block] tile per PARTIAL target tile. Same expansion rules
    as ``dense_mask_from_blocks``; heads of a batch element whose lists equal head 0's share its
    pool entries."""
    src = bm.Q_BLOCK_SIZE
    r = block // src
    B, H, nqs, mb = bm.kv_indices.shape
    nks = bm.num_kv_blocks
    dev = bm.device
    BH = B * H
    n_pad = -(-max(bm.q_len, bm.kv_len) // block) * block
    nq = n_pad // block
    G = nq * r                                   # source blocks per side after padding
    flat = lambda t: t.reshape(BH, *t.shape[2:])
    nb = flat(bm.kv_num_blocks).long().clamp(0, mb)
    idx = flat(bm.kv_indices).long()
    typ = flat(bm.block_mask_types).long()
    listed = (torch.arange(mb, device=dev) < nb.unsqueeze(-1)) & (idx >= 0) & (idx < nks)
    have_pool = bm.partial_block_mask_indices is not None and bm.partial_block_masks is not None
    if have_pool:
        pidx = flat(bm.partial_block_mask_indices).long()
        usable = (pidx >= 0) & (pidx < bm.partial_block_masks.shape[0])
    else:
        pidx = torch.full_like(idx, -1)
        usable = torch.zeros_like(listed)
    is_partial = listed & (typ == BlockMaskType.PARTIAL) & usable
    is_causal = listed & ((typ == BlockMaskType.CAUSAL) | ((typ == BlockMaskType.PARTIAL) & ~usable))
    is_full = listed & (typ == BlockMaskType.FULL)

    # state of every source block: bit 0 = FULL listed, bit 1 = CAUSAL listed, pool index of a PARTIAL entry
    def scatter(sel: Tensor, value: Tensor, into: Tensor) -> None:
        i0, i1, i2 = sel.nonzero(as_tuple=True)
        into[i0, i1, idx[i0, i1, i2]] = value[i0, i1, i2] if value.dim() else value

    one = torch.ones((), dtype=torch.bool, device=dev)
    g_full = torch.zeros(BH, G, G, dtype=torch.bool, device=dev)
    g_causal = torch.zeros_like(g_full)
    g_pool = torch.full((BH, G, G), -1, dtype=torch.long, device=dev)
    scatter(is_full, one, g_full)
    scatter(is_causal, one, g_causal)
    scatter(is_partial, pidx, g_pool)
    rr = torch.arange(G, device=dev)
    below, on_diag = rr.view(G, 1) > rr.view(1, G), rr.view(G, 1) == rr.view(1, G)
    # a CAUSAL entry off the diagonal is all-true below it and empty above it (absolute positions)
    full_s = (g_full | (g_causal & below)) & (g_pool < 0)
    tril_s = g_causal & on_diag & ~g_full & (g_pool < 0)
    part_s = g_pool >= 0
    quad = lambda t: t.view(BH, nq, r, nq, r).permute(0, 1, 3, 2, 4).reshape(BH, nq, nq, r * r)
    qf, qt, qp = quad(full_s), quad(tril_s), quad(part_s)
    empty_q = ~(qf | qt | qp)
    all_full, all_empty = qf.all(-1), empty_q.all(-1)
    # the causal pattern of a diagonal target tile: tril on its diagonal quadrants, full below, empty above
    a_ = torch.arange(r, device=dev)
    want_t = (a_.view(r, 1) == a_.view(1, r)).reshape(-1)
    want_f = (a_.view(r, 1) > a_.view(1, r)).reshape(-1)
    tile_diag = torch.eye(nq, dtype=torch.bool, device=dev).unsqueeze(0)
    is_c = tile_diag & (qt == want_t).all(-1) & (qf == want_f).all(-1) & ~qp.any(-1)
    grid = torch.full((BH, nq, nq), int(BlockMaskType.PARTIAL), dtype=torch.int32, device=dev)
    grid[is_c] = int(BlockMaskType.CAUSAL)
    grid[all_full] = int(BlockMaskType.FULL)
    grid[all_empty] = int(BlockMaskType.MASKED)
    nb2, idx2, typ2 = _pack_lists(grid)

    # heads whose source lists are those of their batch element's head 0 reuse its tiles
    key = (g_full.to(torch.int64) | (g_causal.to(torch.int64) << 1) | ((g_pool + 1) << 2)).view(B, H, -1)
    same_as_first = (key == key[:, :1]).all(-1)                       # [B, H]
    owner = torch.where(same_as_first, torch.arange(B, device=dev).view(B, 1) * H,
                        torch.arange(BH, device=dev).view(B, H)).reshape(BH)

    is_p = (typ2 == BlockMaskType.PARTIAL) & (torch.arange(nq, device=dev) < nb2.unsqueeze(-1))
    pidx2 = torch.full((BH, nq, nq), -1, dtype=torch.int32, device=dev)
    pool2 = torch.empty(0, block, block, dtype=torch.bool, device=dev)
    own = owner.view(BH, 1, 1).expand_as(is_p)
    mine = is_p & (own == torch.arange(BH, device=dev).view(BH, 1, 1))
    s0, s1, s2 = mine.nonzero(as_tuple=True)
    m = s0.numel()
    if m > 0:
        tile_grid = torch.full((BH, nq, nq), -1, dtype=torch.long, device=dev)
        kv = idx2[s0, s1, s2].long()
        tile_grid[s0, s1, kv] = torch.arange(m, device=dev)
        o0, o1, o2 = is_p.nonzero(as_tuple=True)
        pidx2[o0, o1, o2] = tile_grid[owner[o0], o1, idx2[o0, o1, o2].long()].to(torch.int32)
        # element masks, quadrant by quadrant
        tril = torch.ones(src, src, dtype=torch.bool, device=dev).tril()
        pool2 = torch.zeros(m, r, src, r, src, dtype=torch.bool, device=dev)
        for qa in range(r):
            for qb in range(r):
                gi, gj = s1 * r + qa, kv * r + qb
                f, t_, pi = full_s[s0, gi, gj], tril_s[s0, gi, gj], g_pool[s0, gi, gj]
                tile = f.view(m, 1, 1) | (t_.view(m, 1, 1) & tril)
                if have_pool and bool((pi >= 0).any()):
                    from_pool = bm.partial_block_masks[pi.clamp(min=0)].to(torch.bool)
                    tile = torch.where((pi >= 0).view(m, 1, 1), from_pool, tile)
                pool2[:, qa, :, qb, :] = tile
        pool2 = pool2.view(m, block, block)
    sh = lambda t: t.view(B, H, *t.shape[1:]).contiguous()
    out = OmniBlockMask(sh(nb2), sh(idx2), sh(typ2), n_pad, n_pad, block, block)
    if m > 0:
        out.partial_block_mask_indices = sh(pidx2)
        out.partial_block_masks = pool2
    return out


def retile_block_mask(bm: OmniBlockMask, block: int = 128) -> OmniBlockMask:
    """The same attention pattern on another square block size.

    The reference's launchers accept 64x64 as well as 128x128 blocks
    (omni-attn-mma/mma/omni_attn_shared_kv.cu:780-888). The forward kernels take both; the backward
    kernels and FlexAttention conversions work on 128x128, so other masks are re-expressed here. When
    the source block size divides ``block`` (64 -> 128, the case that matters) the target tiles are
    composed from their quadrants and nothing N x N is built. Otherwise each slice is expanded with
    ``dense_mask_from_blocks`` and re-derived with ``block_mask_from_dense``, one [N, N] boolean
    slice at a time (heads that share one pattern are converted once); for small sizes and tests.
    """
    if bm.Q_BLOCK_SIZE == bm.KV_BLOCK_SIZE and block % bm.Q_BLOCK_SIZE == 0 and bm.q_len == bm.kv_len:
        return _retile_by_quadrants(bm, block)
    B, H = bm.kv_num_blocks.shape[:2]
    n_pad = -(-max(bm.q_len, bm.kv_len) // block) * block
    parts, seen = [], {}
    have_pool = bm.partial_block_mask_indices is not None and bm.partial_block_masks is not None
    for b in range(B):
        for h in range(H):
            fields = [bm.kv_num_blocks[b, h], bm.kv_indices[b, h], bm.block_mask_types[b, h]]
            if have_pool:
                fields.append(bm.partial_block_mask_indices[b, h])
            hit = None
            for (ob, oh), part in seen.items():
                if ob == b and all(torch.equal(x, y) for x, y in zip(fields, part[1])):
                    hit = part[0]
                    break
            if hit is None:
                dense = dense_mask_from_blocks(bm, (b * H + h, b * H + h + 1))[0]
                full = torch.zeros(n_pad, n_pad, dtype=torch.bool, device=dense.device)
                full[: dense.shape[0], : dense.shape[1]] = dense
                hit = block_mask_from_dense(full[None, None], block)
                seen[(b, h)] = (hit, fields)
            parts.append(hit)
    return _stack_block_masks(parts, B, H)


def omni_block_mask_from_flex_block_mask(flex_block_mask, materialize_partial: bool = True) -> OmniBlockMask:
    """OmniBlockMask from a ``torch.nn.attention.flex_attention.BlockMask``
    (omni-attn-mma/omni_attn_torch.py:226-290).

    ``materialize_partial=False`` is the reference's conversion to the letter: the blocks flex lists
    as needing ``mask_mod`` (``kv_indices``) become PARTIAL entries without element masks - which the
    expansion and the kernels read as CAUSAL - and flex's full blocks are dropped, as there.
    The default also carries over ``full_kv_indices`` as FULL entries and evaluates ``mask_mod`` on
    every partial block into the element-mask pool, so that the result attends exactly where flex
    does. Flex masks on another block size come back re-tiled to 128 (``retile_block_mask``).
    """
    q_len, kv_len = (int(x) for x in flex_block_mask.seq_lengths)
    bs = getattr(flex_block_mask, "BLOCK_SIZE", None)
    Bq = int(getattr(flex_block_mask, "Q_BLOCK_SIZE", bs[0] if bs is not None else 128))
    Bk = int(getattr(flex_block_mask, "KV_BLOCK_SIZE", bs[1] if bs is not None else 128))

    def lift(t):
        while t.dim() < 3:
            t = t.unsqueeze(0)
        return t

    p_nb = lift(flex_block_mask.kv_num_blocks.clone()).to(torch.int32)
    p_idx = flex_block_mask.kv_indices.clone()
    while p_idx.dim() < 4:
        p_idx = p_idx.unsqueeze(0)
    p_idx = p_idx.to(torch.int32)
    B, H, nq = p_nb.shape
    mb = p_idx.shape[3]
    dev = p_nb.device
    slot = torch.arange(mb, device=dev).view(1, 1, 1, mb)
    if not materialize_partial:
        typ = torch.where(slot < p_nb.unsqueeze(-1), int(BlockMaskType.PARTIAL), int(BlockMaskType.MASKED)).to(torch.int32)
        return OmniBlockMask(p_nb, p_idx.contiguous(), typ.contiguous(), q_len, kv_len, Bq, Bk)

    nk = -(-kv_len // Bk)
    grid = torch.zeros(B, H, nq, nk, dtype=torch.int32, device=dev)
    b_, h_, q_, i_ = (slot < p_nb.unsqueeze(-1)).nonzero(as_tuple=True)
    grid[b_, h_, q_, p_idx[b_, h_, q_, i_].long()] = int(BlockMaskType.PARTIAL)
    f_nb = getattr(flex_block_mask, "full_kv_num_blocks", None)
    if f_nb is not None:
        f_nb = lift(f_nb).to(torch.int32)
        f_idx = flex_block_mask.full_kv_indices
        while f_idx.dim() < 4:
            f_idx = f_idx.unsqueeze(0)
        fslot = torch.arange(f_idx.shape[3], device=dev).view(1, 1, 1, -1)
        fb, fh, fq, fi = (fslot < f_nb.unsqueeze(-1)).nonzero(as_tuple=True)
        grid[fb, fh, fq, f_idx[fb, fh, fq, fi].long()] = int(BlockMaskType.FULL)
    # element masks of the partial blocks, straight from mask_mod
    pb, ph, pq, pk = (grid == int(BlockMaskType.PARTIAL)).nonzero(as_tuple=True)
    m = pb.numel()
    tiles = torch.zeros(m, Bq, Bk, dtype=torch.bool, device=dev)
    mask_mod = flex_block_mask.mask_mod
    r = torch.arange(Bq, device=dev).view(Bq, 1)
    c = torch.arange(Bk, device=dev).view(1, Bk)
    for j in range(m):
        qi = pq[j] * Bq + r
        ki = pk[j] * Bk + c
        t = mask_mod(pb[j], ph[j], qi, ki)
        tiles[j] = torch.as_tensor(t, dtype=torch.bool, device=dev).expand(Bq, Bk) & (qi < q_len) & (ki < kv_len)
    # a partial block that turns out to allow everything is typed FULL, one that allows nothing is dropped
    allf = tiles.flatten(1).all(1)
    none = ~tiles.flatten(1).any(1)
    grid[pb[allf], ph[allf], pq[allf], pk[allf]] = int(BlockMaskType.FULL)
    grid[pb[none], ph[none], pq[none], pk[none]] = int(BlockMaskType.MASKED)
    keep = ~(allf | none)
    nb, idx, typ = _pack_lists(grid)
    bm = OmniBlockMask(nb, idx, typ, -(-q_len // Bq) * Bq, nk * Bk, Bq, Bk)
    if bool(keep.any()):
        number = torch.full((B, H, nq, nk), -1, dtype=torch.int32, device=dev)
        number[pb[keep], ph[keep], pq[keep], pk[keep]] = torch.arange(int(keep.sum()), dtype=torch.int32, device=dev)
        pidx = torch.gather(number, -1, idx.long())
        pidx = torch.where(typ == int(BlockMaskType.PARTIAL), pidx, torch.full_like(pidx, -1))
        bm.partial_block_mask_indices = pidx.contiguous()
        bm.partial_block_masks = tiles[keep].contiguous()
    if Bq != 128 or Bk != 128:
        bm = retile_block_mask(bm, 128)
    return bm
