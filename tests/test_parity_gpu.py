"""Parity of the CUDA kernels with the CPU oracle, through the C ABI (ctypes) and the pybind module.

Tolerances (written once in conftest.py): output atol 2e-2 / rtol 1e-2, log-sum-exp 1e-3.
"""
import math

import pytest
import torch

from conftest import GOLDEN_CASES, LSE_ATOL, assert_parity, load_golden
from omni_attention_b200 import inputs, ops
from omni_attention_b200.block_mask import (BlockMaskType, OmniBlockMask, create_causal_omni_block_mask,
                                            dense_mask_from_blocks,
                                            block_mask_from_dense)
from omni_attention_b200.ops import omni_attention
from oracle import omni_oracle as orc
from oracle import scalar

pytestmark = pytest.mark.gpu
KERNELS = ["ws", "simple"]


def run(q, k, v, bm, dev, kernel="ws", **kw):
    out, lse = omni_attention(q.to(dev), k.to(dev), v.to(dev), bm, return_lse=True, kernel=kernel, check_status=True, **kw)
    return out, lse


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_vectors_from_the_reference(cuda_device, name, kernel):
    g = load_golden(name)
    out, lse = run(g["q"], g["k"], g["v"], g["bm"], cuda_device, kernel)
    assert_parity(out, lse, g["out"], g["lse"], f"{name}/{kernel}")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_vectors_bf16(cuda_device, name, kernel):
    g = load_golden(name)
    q, k, v = (g[x].bfloat16() for x in "qkv")
    ref_out, ref_lse = orc.block_mask_attention(q, k, v, g["bm"])
    out, lse = run(q, k, v, g["bm"], cuda_device, kernel)
    assert out.dtype == torch.bfloat16
    assert_parity(out, lse, ref_out, ref_lse, f"{name}/{kernel}/bf16")


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("cname", ["C1", "C2", "C3"])
@pytest.mark.parametrize("seed", [0, 1])
def test_benchmark_configs_full(cuda_device, cname, seed, kernel):
    if kernel == "simple" and seed == 1:
        pytest.skip("second seed only on the fast kernel")
    q, k, v, bm, _ = inputs.make_inputs(cname, seed=seed)
    ref_out, ref_lse = orc.block_mask_attention(q, k, v, bm)
    out, lse = run(q, k, v, bm, cuda_device, kernel)
    assert_parity(out, lse, ref_out, ref_lse, f"{cname}/seed{seed}/{kernel}")


def _sample_rows(B, H, N, n, gen):
    bh = torch.randint(0, B * H, (n,), generator=gen)
    qi = torch.randint(0, N, (n,), generator=gen)
    return bh.tolist(), qi.tolist()


def test_config_c4_sampled_heads_and_rows(cuda_device):
    q, k, v, bm, _ = inputs.make_inputs("C4", seed=0)
    out, lse = run(q, k, v, bm, cuda_device)
    out_s, lse_s = run(q, k, v, bm, cuda_device, "simple")
    # two whole heads against the torch oracle
    heads = [(0, 3), (0, 31)]
    ref_out, ref_lse = orc.block_mask_attention(q, k, v, bm, bh=heads)
    for b, h in heads:
        assert_parity(out[b, h], lse[b, h], ref_out[b, h], ref_lse[b, h], f"C4 head {h}")
        assert_parity(out_s[b, h], lse_s[b, h], ref_out[b, h], ref_lse[b, h], f"C4 head {h} simple")
    # random rows of every head against the scalar oracle
    g = torch.Generator().manual_seed(5)
    rb, rq = _sample_rows(1, 32, 8192, 256, g)
    so, sl = scalar.oracle_rows(q, k, v, bm, rb, rq)
    got = out.float().cpu().view(32, 8192, 128)[rb, rq]
    got_l = lse.cpu().view(32, 8192)[rb, rq]
    assert_parity(got, got_l, so, sl, "C4 sampled rows")
    # the two kernels agree with each other everywhere
    assert_parity(out, lse, out_s.float(), lse_s, "C4 ws vs simple")


@pytest.mark.parametrize("lo", list(range(0, 128, 16)))
def test_config_c5_shape_sharded_slice(cuda_device, lo):
    """The 32K multi-image configuration, shard by shard as 8 GPUs would own it (16 of the 128
    batch*head pairs each), checked on sampled rows and through properties that need no oracle."""
    cfg = inputs.CONFIGS["C5"]
    hi = lo + 16
    q, k, v, bm, _ = inputs.make_inputs("C5", seed=0, bh_range=(lo, hi))
    out, lse = run(q, k, v, bm, cuda_device)
    assert out.shape == (1, hi - lo, cfg.N, cfg.D)
    assert not bool(torch.isnan(out).any()) and not bool(torch.isinf(lse).any())
    g = torch.Generator().manual_seed(9)
    rb, rq = _sample_rows(1, hi - lo, cfg.N, 96, g)
    rq[:8] = [0, 127, 128, cfg.N - 1, cfg.N - 128, 4095, 4096, 20000]
    so, sl = scalar.oracle_rows(q, k, v, bm, rb, rq)
    got = out.float().cpu().view(hi - lo, cfg.N, cfg.D)[rb, rq]
    got_l = lse.cpu().view(hi - lo, cfg.N)[rb, rq]
    assert_parity(got, got_l, so, sl, "C5 sampled rows")
    # linearity in V: out(V1 + V2) = out(V1) + out(V2); same attention weights, fp32 accumulation
    v2 = torch.roll(v, 1, dims=2)
    o_b, _ = run(q, k, v2, bm, cuda_device)
    o_sum, lse2 = run(q, k, (v.float() + v2.float()).to(v.dtype), bm, cuda_device)
    assert torch.equal(lse2, lse), "lse must not depend on V"
    diff = (o_sum.float() - (out.float() + o_b.float())).abs().max().item()
    assert diff <= 3e-2, diff
    # a constant V column comes back unchanged: the attention weights of every row sum to one
    vc = torch.full_like(v, 0.75)
    o_c, _ = run(q, k, vc, bm, cuda_device)
    assert (o_c.float() - 0.75).abs().max().item() <= 4e-3


@pytest.mark.parametrize("kernel", KERNELS)
def test_edge_empty_lists_and_masked_entries(cuda_device, kernel):
    g = load_golden("ref_fcp_n512_d64")
    bm = g["bm"]
    bm2 = OmniBlockMask(bm.kv_num_blocks.clone(), bm.kv_indices.clone(), bm.block_mask_types.clone(), bm.q_len,
                        bm.kv_len, 128, 128, bm.partial_block_mask_indices.clone(), bm.partial_block_masks.clone())
    bm2.kv_num_blocks[:, 0, 1] = 0                       # Q block 1 of head 0 attends nothing
    bm2.block_mask_types[:, 1, 3, 1] = int(BlockMaskType.MASKED)   # a listed entry typed MASKED is skipped
    bm2.kv_indices[:, 1, 2, 0] = 3                       # CAUSAL-typed? force an above-diagonal block id on a listed entry
    bm2.block_mask_types[:, 1, 2, 0] = int(BlockMaskType.CAUSAL)  # CAUSAL above the diagonal contributes nothing
    dense = dense_mask_from_blocks(bm2)
    assert torch.equal(dense, orc.to_dense_mask_loops(bm2))
    rows_ok = dense.any(-1)
    out, lse = run(g["q"], g["k"], g["v"], bm2, cuda_device, kernel)
    ref_out, ref_lse = orc.block_mask_attention(g["q"], g["k"], g["v"], bm2)
    out, lse = out.float().cpu(), lse.cpu()
    assert_parity(out[rows_ok], lse[rows_ok], ref_out[rows_ok], ref_lse[rows_ok], "rows with keys")
    # rows that attend nothing: zeros and lse = -inf (the torch path gives NaN there, the
    # reference's CUDA kernels give zeros: omni-attn-mma/mma/attn_naive.cu:178-183)
    assert bool((~rows_ok).any())
    assert torch.all(out[~rows_ok] == 0)
    assert torch.all(torch.isinf(lse[~rows_ok]) & (lse[~rows_ok] < 0))


@pytest.mark.parametrize("kernel", KERNELS)
def test_edge_ragged_length_padding_and_clipping(cuda_device, kernel):
    """Unpadded length 300: the operator pads to 384; keys >= 300 are never attended even though the
    block lists cover them, padded query rows are sliced off."""
    torch.manual_seed(3)
    n = 300
    q, k, v = (torch.randn(1, 2, n, 128).half() for _ in range(3))
    bm = create_causal_omni_block_mask(1, 2, n, n)
    bm.block_mask_types[:, 1, 2, :] = int(BlockMaskType.FULL)   # head 1: last Q block sees every block fully
    out, lse = run(q, k, v, bm, cuda_device, kernel)
    assert out.shape == (1, 2, n, 128)
    pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, 384 - n))
    ref_out, ref_lse = orc.block_mask_attention(pad(q), pad(k), pad(v), bm, seqlen_orig=n)
    assert_parity(out, lse, ref_out[:, :, :n], ref_lse[:, :, :n], "ragged")
    so, sl = scalar.oracle_rows(pad(q), pad(k), pad(v), bm, [1, 1, 0], [299, 256, 299], seqlen_orig=n)
    assert_parity(out.float().cpu()[0, [1, 1, 0], [299, 256, 299]], lse.cpu()[0, [1, 1, 0], [299, 256, 299]], so, sl, "ragged rows")


@pytest.mark.parametrize("kernel", KERNELS)
def test_edge_partial_rows_without_keys_and_unsorted_lists(cuda_device, kernel):
    torch.manual_seed(4)
    N = 384
    q, k, v = (torch.randn(1, 1, N, 64).bfloat16() for _ in range(3))
    nb = torch.tensor([[[1, 2, 3]]], dtype=torch.int32)
    idx = torch.tensor([[[[0, 0, 0], [1, 0, 0], [2, 0, 1]]]], dtype=torch.int32)          # last list unsorted
    P, F, C = int(BlockMaskType.PARTIAL), int(BlockMaskType.FULL), int(BlockMaskType.CAUSAL)
    typ = torch.tensor([[[[P, 0, 0], [C, P, 0], [P, F, P]]]], dtype=torch.int32)
    pidx = torch.tensor([[[[0, -1, -1], [-1, 1, -1], [2, -1, 7]]]], dtype=torch.int32)     # 7 is out of range -> causal fallback
    pool = torch.rand(3, 128, 128) < 0.3
    pool[0, 5] = False          # a row of the only tile of Q block 0 with no allowed key at all
    pool[0, 0, 0] = True
    bm = OmniBlockMask(nb, idx, typ, N, N, 128, 128, pidx, pool)
    dense = dense_mask_from_blocks(bm)
    assert torch.equal(dense, orc.to_dense_mask_loops(bm))
    rows_ok = dense.any(-1)
    assert not bool(rows_ok[0, 0, 5])
    out, lse = run(q, k, v, bm, cuda_device, kernel)
    ref_out, ref_lse = orc.block_mask_attention(q, k, v, bm)
    out, lse = out.float().cpu(), lse.cpu()
    assert_parity(out[rows_ok], lse[rows_ok], ref_out[rows_ok], ref_lse[rows_ok], "partial")
    assert torch.all(out[~rows_ok] == 0) and torch.all(lse[~rows_ok] == -math.inf)
    # byte-per-element pool (the reference's format) and the bit-packed pool give identical results
    ob, lb = omni_attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), bm, return_lse=True, kernel=kernel)
    bm_bytes = OmniBlockMask(nb, idx, typ, N, N, 128, 128, pidx, pool)
    o2 = torch.empty_like(ob)
    l2 = torch.empty_like(lb)
    ops.omni_attention_forward_out(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), o2, bm_bytes, N, None, l2, None,
                                   kernel, pack_bits=False)
    assert torch.equal(o2, ob) and torch.equal(l2, lb)


def test_pack_partial_masks_bit_layout(cuda_device):
    pool = torch.rand(5, 128, 128) < 0.5
    bits = ops.pack_partial_masks(pool.to(cuda_device)).cpu()
    w = bits.view(5, 128, 4).to(torch.int64) & 0xFFFFFFFF
    unpacked = ((w.unsqueeze(-1) >> torch.arange(32)) & 1).bool().view(5, 128, 128)
    assert torch.equal(unpacked, pool)


def test_bad_block_index_is_reported_not_dereferenced(cuda_device):
    g = load_golden("ref_causal_n256_d64")
    bm = g["bm"]
    bad = OmniBlockMask(bm.kv_num_blocks.clone(), bm.kv_indices.clone(), bm.block_mask_types.clone(), 256, 256)
    bad.kv_indices[0, 0, 1, 0] = 99
    with pytest.raises(ops.OmniAttnError, match="block id"):
        omni_attention(g["q"].to(cuda_device), g["k"].to(cuda_device), g["v"].to(cuda_device), bad, check_status=True)


def test_scale_argument_is_honoured(cuda_device):
    g = load_golden("ref_causal_n256_d64")
    s = 0.05
    ref_out, ref_lse = orc.block_mask_attention(g["q"], g["k"], g["v"], g["bm"], scale=s)
    out, lse = run(g["q"], g["k"], g["v"], g["bm"], cuda_device, "ws", scale=s)
    assert_parity(out, lse, ref_out, ref_lse, "scale")


def test_runs_on_a_side_stream_without_device_sync(cuda_device):
    g = load_golden("ref_fcp_n384_d128")
    q, k, v = (g[x].to(cuda_device) for x in "qkv")
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        out = omni_attention(q, k, v, g["bm"])
    st.synchronize()
    assert_parity(out, None, g["out"], None, "side stream")


def test_reference_pybind_surface(cuda_device):
    """The reference's 13-argument entry points, called exactly as its wrapper does
    (omni-attn-mma/omni_attn_torch.py:652-663): caller-allocated O, int32 mask tensors, bool pool."""
    import omni_attention_b200 as pkg

    m = pkg.install_reference_module()
    g = load_golden("ref_interleaved_n512_d64")
    bm = g["bm"]
    dev = cuda_device
    q, k, v = (g[x].to(dev).contiguous() for x in "qkv")
    args = lambda o: (q, k, v, o, bm.kv_num_blocks.to(dev).int().contiguous(), bm.kv_indices.to(dev).int().contiguous(),
                      bm.block_mask_types.to(dev).int().contiguous(), 128, 128, 512,
                      bm.partial_block_mask_indices.to(dev).int().contiguous(), bm.partial_block_masks.to(dev).contiguous(), True)
    for name in ("omni_attn_mma_stages_split_q_shared_kv", "omni_attn_simple_kernel", "omni_attn_cp_async",
                 "omni_attn_preftech_kernel", "omni_attn_mma_stages_split_q_shared_kv_swizzle"):
        o = torch.empty_like(q)
        assert getattr(m, name)(*args(o)) is None
        torch.cuda.synchronize()
        assert_parity(o, None, g["out"], None, name)
    # has_partial = False with empty placeholders, causal mask
    gc = load_golden("ref_causal_n256_d64")
    q, k, v = (gc[x].to(dev).contiguous() for x in "qkv")
    o = torch.empty_like(q)
    c = gc["bm"]
    m.omni_attn_mma_stages_split_q_shared_kv(q, k, v, o, c.kv_num_blocks.to(dev), c.kv_indices.to(dev), c.block_mask_types.to(dev),
                                             128, 128, 256, torch.empty(0, dtype=torch.int32, device=dev),
                                             torch.empty(0, dtype=torch.bool, device=dev), False)
    torch.cuda.synchronize()
    assert_parity(o, None, gc["out"], None, "no partial")
    # the reference launchers' errors
    with pytest.raises(RuntimeError):
        m.omni_attn_simple_kernel(q.float(), k.float(), v.float(), o.float(), c.kv_num_blocks.to(dev), c.kv_indices.to(dev),
                                  c.block_mask_types.to(dev), 128, 128, 256, torch.empty(0, dtype=torch.int32, device=dev),
                                  torch.empty(0, dtype=torch.bool, device=dev), False)
    with pytest.raises(RuntimeError, match="Q blocks"):
        m.omni_attn_simple_kernel(q, k, v, o, c.kv_num_blocks.to(dev)[:, :, :1].contiguous(), c.kv_indices.to(dev),
                                  c.block_mask_types.to(dev), 128, 128, 256, torch.empty(0, dtype=torch.int32, device=dev),
                                  torch.empty(0, dtype=torch.bool, device=dev), False)
    with pytest.raises(RuntimeError, match="block size"):
        m.omni_attn_simple_kernel(q, k, v, o, c.kv_num_blocks.to(dev), c.kv_indices.to(dev), c.block_mask_types.to(dev), 128, 64,
                                  256, torch.empty(0, dtype=torch.int32, device=dev), torch.empty(0, dtype=torch.bool, device=dev), False)
    with pytest.raises(RuntimeError, match="contiguous"):
        m.omni_attn_simple_kernel(q.transpose(1, 2).contiguous().transpose(1, 2), k, v, o, c.kv_num_blocks.to(dev), c.kv_indices.to(dev),
                                  c.block_mask_types.to(dev), 128, 128, 256, torch.empty(0, dtype=torch.int32, device=dev),
                                  torch.empty(0, dtype=torch.bool, device=dev), False)
    # superset entry: scale, lse, status
    lse = torch.empty(1, 2, 256, dtype=torch.float32, device=dev)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    m.omni_attn_fwd(q, k, v, o, c.kv_num_blocks.to(dev), c.kv_indices.to(dev), c.block_mask_types.to(dev), 128, 128, 256,
                    torch.empty(0, dtype=torch.int32, device=dev), torch.empty(0, dtype=torch.bool, device=dev), False,
                    scale=None, lse=lse, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert float((lse.cpu() - gc["lse"]).abs().max()) <= LSE_ATOL


def _random_modality_positions(B, N, gen, max_spans=6):
    rows = []
    for _ in range(B):
        spans, pos = [], 0
        for _ in range(max_spans):
            pos += int(torch.randint(1, max(2, N // 8), (1,), generator=gen))
            ln = int(torch.randint(1, max(2, N // 5), (1,), generator=gen))
            if pos + ln > N:
                break
            spans.append([1, pos, ln])
            pos += ln
        spans += [[0, 0, 0]] * (max_spans - len(spans))
        rows.append(spans)
    return torch.tensor(rows, dtype=torch.int32)


@pytest.mark.parametrize("seq_len", [500, 1024, 4096])
def test_gpu_mask_builder_matches_cpu_builder_and_dense_rule(cuda_device, seq_len):
    """omni_attn_build_mask_sm100 (through the package's builder on a CUDA device) against the CPU
    builder: same lists and types, same dense expansion, and attention on the GPU-built mask against
    the oracle."""
    from omni_attention_b200 import create_omni_block_mask_from_modality_positions as build

    g = torch.Generator().manual_seed(seq_len)
    B, H, D = 2, 2, 64
    mp = _random_modality_positions(B, seq_len, g)
    cpu = build(mp, B, H, seq_len, seq_len)
    gpu = build(mp, B, H, seq_len, seq_len, device=cuda_device)
    assert gpu.kv_indices.is_cuda and gpu.q_len == cpu.q_len
    assert torch.equal(gpu.kv_num_blocks.cpu(), cpu.kv_num_blocks)
    assert torch.equal(gpu.kv_indices.cpu(), cpu.kv_indices)
    assert torch.equal(gpu.block_mask_types.cpu(), cpu.block_mask_types)
    assert gpu.partial_block_masks.shape == cpu.partial_block_masks.shape
    # pool numbering may differ; the tile each entry points at must not
    sel = cpu.partial_block_mask_indices >= 0
    assert torch.equal(gpu.partial_block_mask_indices.cpu() >= 0, sel)
    ct = cpu.partial_block_masks[cpu.partial_block_mask_indices[sel].long()]
    gt = gpu.partial_block_masks.cpu()[gpu.partial_block_mask_indices.cpu()[sel].long()]
    assert torch.equal(ct, gt)
    if seq_len <= 1024:
        pad = cpu.q_len
        want = torch.zeros(B, pad, pad, dtype=torch.bool)
        want[:, :seq_len, :seq_len] = orc.naive_attn_mask(seq_len, mp.long())
        assert torch.equal(gpu.to(torch.device("cpu")).to_dense_mask()[:, 0], want)
    q, k, v = (torch.randn(B, H, seq_len, D, generator=g).bfloat16() for _ in range(3))
    out, lse = omni_attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), gpu, return_lse=True, check_status=True)
    pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, cpu.q_len - seq_len))
    ref_out, ref_lse = orc.block_mask_attention(pad(q), pad(k), pad(v), cpu, seqlen_orig=seq_len)
    assert_parity(out, lse, ref_out[:, :, :seq_len], ref_lse[:, :, :seq_len], f"gpu-built mask N={seq_len}")


def test_gpu_mask_builder_at_c5_size(cuda_device):
    """The 32K multi-image layout: GPU-built mask equals the CPU-built one; prints the build time."""
    from omni_attention_b200 import create_omni_block_mask_from_modality_positions as build

    cfg = inputs.CONFIGS["C5"]
    cpu, meta = inputs.make_block_mask(cfg, seed=0)
    spans = meta["image_spans"]
    M = max(len(s) for s in spans)
    mp = torch.tensor([[[1, o, l] for o, l in s] + [[0, 0, 0]] * (M - len(s)) for s in spans], dtype=torch.int32)
    gpu = build(mp, cfg.B, cfg.H, cfg.N, cfg.N, device=cuda_device)
    assert torch.equal(gpu.kv_num_blocks.cpu(), cpu.kv_num_blocks)
    assert torch.equal(gpu.kv_indices.cpu(), cpu.kv_indices)
    assert torch.equal(gpu.block_mask_types.cpu(), cpu.block_mask_types)
    assert gpu.partial_block_masks.shape[0] == cpu.partial_block_masks.shape[0]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        build(mp, cfg.B, cfg.H, cfg.N, cfg.N, device=cuda_device)
    e1.record()
    torch.cuda.synchronize()
    out_bytes = 4 * (3 * cpu.kv_indices.numel() + cpu.kv_num_blocks.numel())
    print(f"C5 mask build (incl. host sync and bit expansion): {e0.elapsed_time(e1) / 5:.3f} ms, index tensors {out_bytes / 1e6:.0f} MB")


@pytest.mark.parametrize("D,dtype", [(64, torch.float16), (128, torch.bfloat16)])
def test_transfusion_attention_core_with_softcap(cuda_device, D, dtype):
    """The Transfusion attention slot: GPU-built modality mask + tanh soft-cap (value 50 as in the
    model, and a small cap that really bends the scores) against the oracle's restatement of the
    model's non-flex branch (transfusion_pytorch/transfusion.py:963-983)."""
    from omni_attention_b200.transfusion import transfusion_attention_core, transfusion_block_mask

    g = torch.Generator().manual_seed(D)
    B, H, N = 2, 2, 1024
    mp = _random_modality_positions(B, N, g)
    q, k, v = (torch.randn(B, H, N, D, generator=g).to(dtype) for _ in range(3))
    q = q * 3.0   # large scores so that the cap matters
    bm = transfusion_block_mask(mp.to(cuda_device), H, N)
    dense = orc.naive_attn_mask(N, mp.long())
    for cap in (50.0, 4.0):
        out = transfusion_attention_core(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), bm, softcap_value=cap)
        ref, ref_lse = orc.attention_dense_mask(q.float(), k.float(), v.float(), orc.to_score_mask(dense).unsqueeze(1),
                                                softcap=cap)
        assert_parity(out, None, ref, None, f"softcap {cap} D={D}")
        _, lse = omni_attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), bm, return_lse=True, softcap=cap)
        assert float((lse.cpu() - ref_lse).abs().max()) <= LSE_ATOL
    # the cap must change the result on this input (otherwise the test proves nothing)
    plain = omni_attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), bm)
    assert float((plain.float() - out.float()).abs().max()) > 0.05
    with pytest.raises(ops.OmniAttnError):
        omni_attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), bm, kernel="simple", softcap=4.0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_dim_32_and_64_wide_blocks(cuda_device, dtype):
    """The reference's launchers also accept head_dim 32 and 64x64 blocks
    (omni-attn-mma/mma/omni_attn_shared_kv.cu:725-741, :780-888). The operator maps both onto the
    128x128 / head_dim 64 kernel: the mask is re-tiled, the head dimension zero-padded with the scale
    kept at 1/sqrt(32)."""
    torch.manual_seed(8)
    n = 640
    pos = torch.arange(n)
    dense = (pos.view(1, n) <= pos.view(n, 1)) | ((pos.view(n, 1) >= 70) & (pos.view(n, 1) < 330) & (pos.view(1, n) < 330))
    dense = dense[None, None].expand(1, 2, n, n).contiguous()
    bm64 = block_mask_from_dense(dense, 64)
    assert bm64.Q_BLOCK_SIZE == 64
    q, k, v = (torch.randn(1, 2, n, 32).to(dtype) for _ in range(3))
    out, lse = omni_attention(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), bm64, return_lse=True)
    assert out.shape == (1, 2, n, 32)
    ref_out, ref_lse = orc.attention_dense_mask(q.float(), k.float(), v.float(), orc.to_score_mask(dense))
    assert_parity(out, lse, ref_out, ref_lse, "D=32, 64-wide blocks")


def test_flex_block_mask_through_the_kernel(cuda_device):
    """A flex_attention BlockMask (built on the CPU, no Triton involved) converted with
    omni_block_mask_from_flex_block_mask drives the kernel to the dense-mask result."""
    from torch.nn.attention.flex_attention import create_block_mask

    from omni_attention_b200.block_mask import omni_block_mask_from_flex_block_mask

    def mask_mod(b, h, q, k):
        return (k <= q) | ((q >= 200) & (q < 500) & (k < 500))

    n = 768
    flex = create_block_mask(mask_mod, 1, 1, n, n, device="cpu", BLOCK_SIZE=128)
    bm = omni_block_mask_from_flex_block_mask(flex)
    bm = OmniBlockMask(bm.kv_num_blocks.expand(1, 4, -1).contiguous(), bm.kv_indices.expand(1, 4, -1, -1).contiguous(),
                       bm.block_mask_types.expand(1, 4, -1, -1).contiguous(), n, n, 128, 128,
                       bm.partial_block_mask_indices.expand(1, 4, -1, -1).contiguous(), bm.partial_block_masks)
    torch.manual_seed(9)
    q, k, v = (torch.randn(1, 4, n, 64).bfloat16() for _ in range(3))
    out, lse = run(q, k, v, bm, cuda_device)
    pos = torch.arange(n)
    dense = mask_mod(0, 0, pos.view(n, 1), pos.view(1, n))
    ref_out, ref_lse = orc.attention_dense_mask(q.float(), k.float(), v.float(), orc.to_score_mask(dense)[None, None])
    assert_parity(out, lse, ref_out, ref_lse, "flex mask")


def test_call_from_a_fresh_host_thread(cuda_device):
    """A host thread that has made no CUDA call of its own (an autograd worker that found its buffers
    in the allocator's cache, a serving thread) can call the library: the entry points bind the
    device's primary context themselves before the driver call that builds the TMA descriptors."""
    import threading

    g = load_golden("ref_causal_n256_d64")
    q, k, v = (g[n].half().to(cuda_device) for n in ("q", "k", "v"))
    ref, _ = run(g["q"].half(), g["k"].half(), g["v"].half(), g["bm"], cuda_device)   # also caches the device mask
    out = torch.empty_like(q)
    torch.cuda.synchronize()
    errors = []

    def worker():
        try:
            ops.omni_attention_forward_out(q, k, v, out, g["bm"], q.shape[2])
        except Exception as e:   # noqa: BLE001
            errors.append(e)

    t = threading.Thread(target=worker)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert not errors, errors
    assert torch.equal(out.cpu(), ref.cpu())


def test_maximum_sequence_length(cuda_device):
    """1 024 KV blocks = 131 072 tokens, the most the kernels' per-CTA block tables hold: one head, causal
    lists with a FULL bidirectional band, sampled rows against the scalar oracle; the backward at the same
    size through the property that needs no oracle."""
    n, d = 1024 * 128, 64
    bm = create_causal_omni_block_mask(1, 1, n, n)
    assert bm.kv_indices.shape == (1, 1, 1024, 1024)
    gen = torch.Generator().manual_seed(17)
    q, k, v = (torch.randn(1, 1, n, d, generator=gen).bfloat16() for _ in range(3))
    out, lse = run(q, k, v, bm, cuda_device)
    assert out.shape == (1, 1, n, d) and bool(torch.isfinite(out.float()).all())
    rq = [0, 127, 128, n - 1, n - 128, 65535, 65536, 100000] + torch.randint(0, n, (24,), generator=gen).tolist()
    rb = [0] * len(rq)
    so, sl = scalar.oracle_rows(q, k, v, bm, rb, rq)
    assert_parity(out.float().cpu()[0, 0, rq], lse.cpu()[0, 0, rq], so, sl, "131072 tokens")

    d_out = (torch.randn(1, 1, n, d, generator=gen) * 0.5).bfloat16()
    qd, kd, vd, dod = (t.to(cuda_device) for t in (q, k, v, d_out))
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(qd), torch.empty_like(qd)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    ops.omni_attention_backward_out(qd, kd, vd, out.contiguous(), lse.contiguous(), dod, dq, dk, dv, bm, n, None, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert all(bool(torch.isfinite(t.float()).all()) for t in (dq, dk, dv))
    lhs, rhs = dv.float().sum(dim=2).cpu(), d_out.float().sum(dim=2)
    assert float((lhs - rhs).abs().max()) <= 2e-2 * float(rhs.abs().max()) + 2.0


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (64, torch.float16)])
def test_running_maximum_that_keeps_moving(cuda_device, kernel, D, dtype):
    """Key magnitude grows with position, so the running maximum of every row rises by far more than the
    lazy-rescale threshold (2^8) from one KV block to the next: the O rescale path runs on every block."""
    torch.manual_seed(3)
    n = 1024
    q, k, v = (torch.randn(1, 2, n, D) for _ in range(3))
    k = k * (1.0 + torch.arange(n).float() / 16.0).view(1, 1, n, 1)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    bm = create_causal_omni_block_mask(1, 2, n, n)
    out, lse = run(q, k, v, bm, cuda_device, kernel)
    ref_out, ref_lse = orc.block_mask_attention(q, k, v, bm)
    assert_parity(out, lse, ref_out, ref_lse, f"moving maximum D={D}")


@pytest.mark.parametrize("seed", [0, 1, 7])
def test_config_c4_on_the_inputs_the_bench_times(cuda_device, seed):
    """The bench's rank `seed` draws its mask with seed = rank and its Q, K, V on the device with seed
    1234 + rank (bench.device_qkv): the same inputs here, sampled rows of every head against the scalar
    oracle, and the fast kernel against the plain one everywhere."""
    import bench

    cfg = inputs.CONFIGS["C4"]
    bm, _ = inputs.make_block_mask(cfg, seed=seed, B=1)
    q, k, v = bench.device_qkv(1, cfg.H, cfg.N, cfg.D, cfg.dtype, 1234 + seed, cuda_device, cfg.qkv_scale)
    out, lse = omni_attention(q, k, v, bm, return_lse=True, check_status=True)
    out_s, lse_s = omni_attention(q, k, v, bm, return_lse=True, check_status=True, kernel="simple")
    g = torch.Generator().manual_seed(100 + seed)
    rb, rq = _sample_rows(1, cfg.H, cfg.N, 192, g)
    rq[:6] = [0, 127, 128, cfg.N - 1, cfg.N - 128, 4097]
    so, sl = scalar.oracle_rows(q.cpu(), k.cpu(), v.cpu(), bm, rb, rq)
    got = out.float().cpu().view(cfg.H, cfg.N, cfg.D)[rb, rq]
    got_l = lse.cpu().view(cfg.H, cfg.N)[rb, rq]
    assert_parity(got, got_l, so, sl, f"C4 bench inputs, seed {seed}")
    assert_parity(out, lse, out_s.float(), lse_s, f"C4 bench inputs, seed {seed}: ws vs simple")


def test_repeated_launches_give_the_same_bits(cuda_device):
    """Which CTA draws which unit changes from launch to launch (dynamic hand-out), and the L2 state
    with it; neither may change a bit of the result. C3 forward (with log-sum-exp) and backward, 25
    launches each against the first one."""
    q, k, v, bm, _ = inputs.make_inputs("C3", seed=3)
    qd, kd, vd = (t.to(cuda_device) for t in (q, k, v))
    first = None
    for it in range(25):
        out = torch.empty_like(qd)
        lse = torch.empty(q.shape[:3], dtype=torch.float32, device=cuda_device)
        status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        ops.omni_attention_forward_out(qd, kd, vd, out, bm, q.shape[2], None, lse, status)
        if first is None:
            first = (out.clone(), lse.clone())
            d_out = torch.randn_like(qd)
        else:
            assert torch.equal(out, first[0]) and torch.equal(lse, first[1]), f"forward launch {it} differs"
        assert int(status.item()) == 0
    grads = None
    for it in range(25):
        dq, dk, dv = torch.empty_like(qd), torch.empty_like(qd), torch.empty_like(qd)
        ops.omni_attention_backward_out(qd, kd, vd, first[0], first[1], d_out, dq, dk, dv, bm, q.shape[2], None, status)
        if grads is None:
            grads = (dq, dk, dv)
        else:
            assert all(torch.equal(a, b) for a, b in zip((dq, dk, dv), grads)), f"backward launch {it} differs"
    assert int(status.item()) == 0
