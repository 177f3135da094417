"""Host-side mask builders of the package against the oracle's restatements of the reference."""
import os
import sys

import pytest
import torch

from conftest import GOLDEN_CASES, load_golden
from omni_attention_b200 import inputs
from omni_attention_b200.block_mask import (BlockMaskType, OmniBlockMask, block_mask_from_dense,
                                            block_mask_from_row_limits, build_partial_block_data,
                                            create_causal_omni_block_mask, dense_mask_from_blocks,
                                            row_limits_from_modality_positions)
from oracle import omni_oracle as orc

# the reference checkout, when there is one: next to this repository unless OMNI_REFERENCE_DIR says otherwise
REF_DIR = os.environ.get("OMNI_REFERENCE_DIR") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference", "omni-attn-mma"))


def test_type_codes_match_reference_enum():
    assert (int(BlockMaskType.MASKED), int(BlockMaskType.CAUSAL), int(BlockMaskType.FULL), int(BlockMaskType.PARTIAL)) == (0, 1, 2, 3)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_vectorised_expansion_matches_golden_dense_mask(name):
    g = load_golden(name)
    assert torch.equal(dense_mask_from_blocks(g["bm"]), g["dense"])
    assert torch.equal(g["bm"].to_dense_mask(), g["dense"])
    B, H = g["dense"].shape[:2]
    part = dense_mask_from_blocks(g["bm"], (B * H - 1, B * H))
    assert torch.equal(part[0], g["dense"][B - 1, H - 1])


@pytest.mark.parametrize("name", ["ref_fcp_n512_d64", "ref_interleaved_n512_d64"])
def test_build_partial_block_data_matches_reference_layout(name):
    g = load_golden(name)
    bm = g["bm"]
    idx, pool = build_partial_block_data(bm, g["dense"])
    assert torch.equal(idx, bm.partial_block_mask_indices)
    assert torch.equal(pool, bm.partial_block_masks)


def test_partial_without_pool_falls_back_to_causal():
    g = load_golden("ref_fcp_n512_d64")
    bm = g["bm"]
    stripped = OmniBlockMask(bm.kv_num_blocks, bm.kv_indices, bm.block_mask_types, bm.q_len, bm.kv_len)
    assert torch.equal(dense_mask_from_blocks(stripped), orc.to_dense_mask_loops(stripped))


def test_causal_builder():
    bm = create_causal_omni_block_mask(2, 3, 500, 500)
    assert bm.q_len == 512 and bm.kv_num_blocks.shape == (2, 3, 4)
    dense = bm.to_dense_mask()
    want = torch.tril(torch.ones(512, 512, dtype=torch.bool))
    assert torch.equal(dense[1, 2], want)
    assert bm.kv_num_blocks[0, 0].tolist() == [1, 2, 3, 4]
    assert bm.visited_blocks() == 2 * 3 * 10


@pytest.mark.parametrize("share", [True, False])
def test_row_limit_builder_matches_dense_derivation(share):
    N, H = 1024, 2
    spans = [[(100, 256), (600, 130)], [(0, 128), (128, 128), (700, 300)]]
    limits, causal_rows = row_limits_from_modality_positions(N, spans)
    bm = block_mask_from_row_limits(limits, H, causal_rows, 128, share_partial_across_heads=share)
    mods = [torch.tensor([[1, o, l] for o, l in s] + [[1, 0, 0]] * (3 - len(s))) for s in spans]
    dense = orc.naive_attn_mask(N, torch.stack(mods))  # [B, N, N]
    got = bm.to_dense_mask()
    for b in range(2):
        for h in range(H):
            assert torch.equal(got[b, h], dense[b])
        bounds = [x for o, l in spans[b] for x in (o, o + l)]
        want_types = orc.block_types_from_dense(dense[b], 128, bounds)
        grid = torch.zeros(8, 8, dtype=torch.int32)
        for qb in range(8):
            n = int(bm.kv_num_blocks[b, 0, qb])
            ids = bm.kv_indices[b, 0, qb, :n].long()
            assert ids.tolist() == sorted(ids.tolist())
            grid[qb, ids] = bm.block_mask_types[b, 0, qb, :n]
        assert torch.equal(grid, want_types)
    if not share:
        idx, pool = build_partial_block_data(bm, got)
        assert torch.equal(idx, bm.partial_block_mask_indices)
        assert torch.equal(pool, bm.partial_block_masks)


def test_block_mask_from_dense_round_trip():
    torch.manual_seed(0)
    dense = torch.rand(1, 2, 384, 384) < 0.5
    dense[:, :, :128, 128:] = False
    dense[:, :, 128:256, :128] = True
    dense[0, 0, :128, :128] = torch.tril(torch.ones(128, 128, dtype=torch.bool))
    bm = block_mask_from_dense(dense)
    assert torch.equal(bm.to_dense_mask(), dense)
    assert int(bm.block_mask_types[0, 0, 0, 0]) == BlockMaskType.CAUSAL
    assert int(bm.kv_num_blocks[0, 0, 0]) == 1


@pytest.mark.parametrize("name", ["C1", "C2", "C3"])
def test_config_generators(name):
    cfg = inputs.CONFIGS[name]
    bm, meta = inputs.make_block_mask(cfg, seed=0)
    bm2, _ = inputs.make_block_mask(cfg, seed=0)
    assert torch.equal(bm.kv_indices, bm2.kv_indices) and torch.equal(bm.block_mask_types, bm2.block_mask_types)
    assert bm.kv_num_blocks.shape == (cfg.B, cfg.H, cfg.N // 128)
    dense = dense_mask_from_blocks(bm, (0, 1))[0]
    assert bool(dense.any(-1).all()), "every query row must keep at least one key"
    assert torch.equal(dense, orc.to_dense_mask_slice(bm, 0, 0))
    assert not bool(torch.triu(dense, 1).any()) or name == "C3"
    if name == "C3":
        spans = meta["image_spans"][0]
        mods = torch.tensor([[[1, o, l] for o, l in spans]])
        assert torch.equal(dense, orc.naive_attn_mask(cfg.N, mods)[0])
    assert inputs.effective_flops(bm, cfg.D) == 4 * 128 * 128 * cfg.D * bm.visited_blocks()


def test_qkv_sharding_is_consistent():
    q, k, v = inputs.make_qkv(1, 4, 256, 64, torch.bfloat16, seed=3, qkv_scale=0.5)
    qs, ks, vs = inputs.make_qkv(1, 4, 256, 64, torch.bfloat16, seed=3, qkv_scale=0.5, bh_range=(2, 4))
    assert torch.equal(qs[0], q[0, 2:4]) and torch.equal(vs[0], v[0, 2:4])
    bm = create_causal_omni_block_mask(2, 2, 256, 256)
    sl = bm.slice_heads(1, 3)
    assert sl.kv_num_blocks.shape == (1, 2, 2)
    assert torch.equal(sl.kv_indices[0, 0], bm.kv_indices[0, 1])
    assert torch.equal(sl.kv_indices[0, 1], bm.kv_indices[1, 0])


@pytest.mark.skipif(not os.path.isdir(REF_DIR), reason="reference checkout not present")
def test_builders_against_reference_in_process():
    sys.path.insert(0, REF_DIR)
    import omni_attn_torch as ref  # reference module

    r = ref.create_causal_omni_block_mask(1, 2, 300, 300, 128, 128, device="cpu")
    m = create_causal_omni_block_mask(1, 2, 300, 300)
    for f in ("kv_num_blocks", "kv_indices", "block_mask_types"):
        assert torch.equal(getattr(r, f), getattr(m, f))
    assert (r.q_len, r.kv_len) == (m.q_len, m.kv_len)
    g = load_golden("ref_interleaved_n512_d64")
    idx, pool = ref.build_partial_block_data(g["bm"], g["dense"])
    mi, mp = build_partial_block_data(g["bm"], g["dense"])
    assert torch.equal(idx, mi) and torch.equal(pool, mp)


@pytest.mark.parametrize("seq_len", [1000, 1024])
def test_mask_from_modality_positions_matches_dense_rule(seq_len):
    """CPU builder with the reference's name and arguments against the oracle's restatement of the
    dense rule (transfusion_pytorch/transfusion.py:496-515), with and without padding."""
    from omni_attention_b200 import create_omni_block_mask_from_modality_positions

    mp = torch.tensor([[[1, 100, 256], [1, 600, 130], [0, 0, 0]], [[1, 0, 128], [1, 128, 128], [1, 700, 300]]])
    bm = create_omni_block_mask_from_modality_positions(mp, 2, 3, seq_len, seq_len)
    pad = -(-seq_len // 128) * 128
    assert (bm.q_len, bm.kv_len) == (pad, pad) and bm.kv_num_blocks.shape == (2, 3, pad // 128)
    want = torch.zeros(2, pad, pad, dtype=torch.bool)
    want[:, :seq_len, :seq_len] = orc.naive_attn_mask(seq_len, mp)
    got = bm.to_dense_mask()
    for h in range(3):
        assert torch.equal(got[:, h], want)
    with pytest.raises(ValueError):
        create_omni_block_mask_from_modality_positions(mp, 2, 3, 512, 256)


def _flex_mask_mod(b, h, q, k):
    # causal | one bidirectional span | a head-dependent extra span
    return (k <= q) | ((q >= 100) & (q < 300) & (k < 300)) | ((h == 1) & (q >= 400) & (k < 450))


def _flex_dense(n, heads):
    pos = torch.arange(n)
    return torch.stack([_flex_mask_mod(torch.tensor(0), torch.tensor(h), pos.view(n, 1), pos.view(1, n))
                        for h in range(heads)])[None]


@pytest.mark.parametrize("flex_block", [128, 64])
def test_flex_block_mask_converter_attends_where_flex_does(flex_block):
    """omni_block_mask_from_flex_block_mask (omni-attn-mma/omni_attn_torch.py:226-290): with the element
    masks materialised the converted mask expands to mask_mod itself, on 128- and 64-wide flex blocks."""
    from torch.nn.attention.flex_attention import create_block_mask

    from omni_attention_b200.block_mask import omni_block_mask_from_flex_block_mask

    n = 512
    flex = create_block_mask(_flex_mask_mod, 1, 2, n, n, device="cpu", BLOCK_SIZE=flex_block)
    bm = omni_block_mask_from_flex_block_mask(flex)
    assert (bm.Q_BLOCK_SIZE, bm.KV_BLOCK_SIZE) == (128, 128)
    assert torch.equal(dense_mask_from_blocks(bm), _flex_dense(n, 2))
    assert torch.equal(dense_mask_from_blocks(bm), orc.to_dense_mask_loops(bm))
    # the reference's conversion to the letter: flex's partial lists typed PARTIAL without element masks
    ref_style = omni_block_mask_from_flex_block_mask(flex, materialize_partial=False)
    assert ref_style.partial_block_masks is None
    assert torch.equal(ref_style.kv_num_blocks, flex.kv_num_blocks.to(torch.int32))
    listed = torch.arange(ref_style.kv_indices.shape[3]).view(1, 1, 1, -1) < ref_style.kv_num_blocks.unsqueeze(-1)
    assert torch.all(ref_style.block_mask_types[listed] == int(BlockMaskType.PARTIAL))
    assert torch.all(ref_style.block_mask_types[~listed] == int(BlockMaskType.MASKED))


def test_retile_64_blocks_to_128_keeps_the_pattern():
    from omni_attention_b200.block_mask import retile_block_mask

    dense = _flex_dense(512, 2)
    bm64 = block_mask_from_dense(dense, 64)
    assert bm64.Q_BLOCK_SIZE == 64 and bm64.kv_indices.shape[2] == 8
    bm128 = retile_block_mask(bm64, 128)
    assert bm128.Q_BLOCK_SIZE == 128 and bm128.kv_indices.shape[2:] == (4, 4)
    assert torch.equal(dense_mask_from_blocks(bm128), dense)
    # ragged: 300 tokens on 64-blocks (padded to 320) re-tiled for a length padded to 384
    d300 = torch.zeros(1, 1, 320, 320, dtype=torch.bool)
    d300[:, :, :300, :300] = torch.tril(torch.ones(300, 300, dtype=torch.bool))
    r = retile_block_mask(block_mask_from_dense(d300, 64), 128)
    assert r.q_len == 384
    assert torch.equal(dense_mask_from_blocks(r)[:, :, :320, :320], d300)
    assert not bool(dense_mask_from_blocks(r)[:, :, 320:].any())


def test_partial_tile_count_from_row_limits_is_the_pool_size():
    """The host-side count that sizes the GPU builder's pool is the number of pool entries the CPU
    builder makes, for span tables with unaligned, overlapping, empty and out-of-range spans and
    lengths with and without padding."""
    from omni_attention_b200.block_mask import _limits_from_modality_tensor, count_partial_tiles

    g = torch.Generator().manual_seed(5)
    for trial in range(40):
        B = int(torch.randint(1, 4, (1,), generator=g))
        M = int(torch.randint(0, 6, (1,), generator=g))
        seq_len = int(torch.randint(1, 1500, (1,), generator=g))
        pad = -(-seq_len // 128) * 128
        mp = torch.zeros(B, M, 3, dtype=torch.long)
        if M:
            mp[:, :, 1] = torch.randint(0, seq_len + 200, (B, M), generator=g)
            mp[:, :, 2] = torch.randint(0, 700, (B, M), generator=g)
        limits, plain = _limits_from_modality_tensor(mp, seq_len, pad)
        bm = block_mask_from_row_limits(limits, 2, plain, 128, True)
        assert count_partial_tiles(limits, plain) == bm.partial_block_masks.shape[0], (trial, seq_len, mp.tolist())


def test_partial_pool_can_be_left_unexpanded_until_it_is_read():
    bm = create_causal_omni_block_mask(1, 2, 256, 256)
    calls = []

    def make():
        calls.append(1)
        return torch.ones(3, 128, 128, dtype=torch.bool)

    bm.set_lazy_partial_pool(make)
    part = bm.slice_heads(0, 1)            # shares the pool without expanding it
    assert calls == []
    assert part.partial_block_masks.shape == (3, 128, 128) and calls == [1]
    assert bm.partial_block_masks is part.partial_block_masks and calls == [1]
    bm.partial_block_masks = None          # plain assignment still works
    assert bm.partial_block_masks is None
    fresh = OmniBlockMask(bm.kv_num_blocks, bm.kv_indices, bm.block_mask_types, 256, 256, 128, 128, None,
                          torch.zeros(1, 128, 128, dtype=torch.bool))
    assert fresh.partial_block_masks.shape == (1, 128, 128)


@pytest.mark.parametrize("src,nblk", [(64, 6), (64, 5), (32, 8)])
def test_retile_by_quadrants_expands_to_the_same_dense_mask(src, nblk):
    """Random lists on small blocks (every type, CAUSAL entries off the diagonal, PARTIAL entries with
    and without a pool tile, listed MASKED entries, an odd block count, heads that do and do not share
    head 0's lists): the 128-tile mask composed from quadrants expands to the same dense mask."""
    from omni_attention_b200.block_mask import retile_block_mask

    g = torch.Generator().manual_seed(100 + nblk + src)
    B, H = 2, 3
    n = src * nblk
    grid = torch.randint(0, 4, (B, H, nblk, nblk), generator=g).to(torch.int32)
    grid[:, 1] = grid[:, 0]                      # head 1 shares head 0's lists
    grid[0, :, 2] = 0                            # an empty row of blocks
    order = torch.argsort(torch.rand(B, H, nblk, nblk, generator=g), dim=-1)   # lists in random order
    listed = torch.gather(grid, -1, order) != 0
    keep = torch.argsort((~listed).to(torch.int32), dim=-1, stable=True)
    idx = torch.gather(order, -1, keep).to(torch.int32)
    typ = torch.gather(grid, -1, idx.long())
    nb = (typ != 0).sum(-1).to(torch.int32)
    nb[1, 2, 0] = min(nblk, int(nb[1, 2, 0]) + 1)            # one listed MASKED entry
    is_p = typ == int(BlockMaskType.PARTIAL)
    pidx = torch.full_like(idx, -1)
    count = int(is_p.sum())
    pidx[is_p] = torch.arange(count, dtype=torch.int32)
    drop = is_p & (torch.rand(B, H, nblk, nblk, generator=g) < 0.2)
    pidx[drop] = -1                                          # PARTIAL without a tile: read as CAUSAL
    for t in (nb, idx, typ, pidx):                           # head 1 is head 0 once more
        t[:, 1] = t[:, 0]
    pool = torch.rand(max(count, 1), src, src, generator=g) < 0.5
    bm = OmniBlockMask(nb, idx, typ, n, n, src, src, pidx, pool)
    want = dense_mask_from_blocks(bm)
    out = retile_block_mask(bm, 128)
    n_pad = -(-n // 128) * 128
    assert (out.Q_BLOCK_SIZE, out.q_len, out.kv_len) == (128, n_pad, n_pad)
    got = dense_mask_from_blocks(out)
    assert torch.equal(got[:, :, :n, :n], want)
    assert not bool(got[:, :, n:].any()) and not bool(got[:, :, :, n:].any())
    if out.partial_block_masks is not None:
        # heads 0 and 1 share their tiles
        assert torch.equal(out.partial_block_mask_indices[:, 0], out.partial_block_mask_indices[:, 1])
