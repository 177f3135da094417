"""Backward kernels (omni_attn_bwd_sm100) against the oracle's gradient, through the C ABI.

The reference has no backward pass; the oracle's gradient is torch autograd through its pinned
forward (oracle/omni_oracle.py: block_mask_attention_backward). Tolerance, stated here: every
gradient element within ``GRAD_RTOL[dtype] * max|reference gradient of that tensor and head|`` -
P and dS are rounded to the 16-bit input type before the tensor-core contractions and the results are
stored in that type, so the error scales with the largest entries (8 mantissa bits for bf16, 11 for
fp16)."""
import math

import pytest
import torch

from conftest import GOLDEN_CASES, GOLDEN_CASES_64_32, load_golden
from omni_attention_b200 import (BlockMaskType, OmniBlockMask, create_causal_omni_block_mask, inputs, omni_attention,
                                 omni_attention_autograd, ops)
from omni_attention_b200.block_mask import dense_mask_from_blocks
from oracle import omni_oracle as orc

pytestmark = pytest.mark.gpu

GRAD_RTOL = {torch.float16: 4e-3, torch.bfloat16: 2e-2}


def backward(q, k, v, d_out, bm, dev, seqlen_orig=None, scale=None):
    """Forward (for out, lse) then backward on padded tensors; returns (dq, dk, dv) on the CPU as fp32."""
    B, H, N, D = q.shape
    so = N if seqlen_orig is None else seqlen_orig
    qd, kd, vd, dod = (t.to(dev).contiguous() for t in (q, k, v, d_out))
    out = torch.empty_like(qd)
    lse = torch.empty(B, H, N, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.omni_attention_forward_out(qd, kd, vd, out, bm, so, scale, lse, status)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(qd), torch.empty_like(qd)
    ops.omni_attention_backward_out(qd, kd, vd, out, lse, dod, dq, dk, dv, bm, so, scale, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return dq.float().cpu(), dk.float().cpu(), dv.float().cpu()


def assert_grads(got, ref, dtype, heads, what=""):
    for name, a, r in zip(("dq", "dk", "dv"), got, ref):
        for b, h in heads:
            x, y = a[b, h], r[b, h]
            assert bool(torch.isfinite(x).all()), f"{what} {name}[{b},{h}] has non-finite entries"
            tol = GRAD_RTOL[dtype] * float(y.abs().max())
            err = float((x - y).abs().max())
            assert err <= tol, f"{what} {name}[{b},{h}]: max abs err {err:.4g} > {tol:.4g}"


def all_heads(B, H):
    return [(b, h) for b in range(B) for h in range(H)]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_backward_on_the_golden_cases(cuda_device, name, dtype):
    g = load_golden(name)
    q, k, v = (g[n].to(dtype) for n in ("q", "k", "v"))
    torch.manual_seed(11)
    d_out = torch.randn(q.shape).to(dtype)
    heads = all_heads(q.shape[0], q.shape[1])
    ref = orc.block_mask_attention_backward(q, k, v, g["bm"], d_out)
    assert_grads(backward(q, k, v, d_out, g["bm"], cuda_device), ref, dtype, heads, name)


@pytest.mark.parametrize("name", GOLDEN_CASES_64_32)
def test_autograd_op_on_64_blocks_and_head_dim_32(cuda_device, name):
    """The differentiable operator on the reference's other block shape and head_dim: the forward takes
    them as they are, the backward gets the mask re-tiled to 128 (quadrant by quadrant) and head_dim 32
    zero-padded; gradients against autograd through the oracle on the original mask."""
    g = load_golden(name)
    dtype = torch.float16
    q, k, v = (g[n].to(dtype) for n in ("q", "k", "v"))
    torch.manual_seed(13)
    d_out = torch.randn(q.shape).to(dtype)
    heads = all_heads(q.shape[0], q.shape[1])
    n = q.shape[2]
    assert g["bm"].q_len == n   # the goldens are stored at the padded length
    ref = orc.block_mask_attention_backward(q, k, v, g["bm"], d_out)
    qd, kd, vd = (t.to(cuda_device).requires_grad_(True) for t in (q, k, v))
    out = omni_attention_autograd(qd, kd, vd, g["bm"])
    assert torch.equal(out.detach(), omni_attention(qd.detach(), kd.detach(), vd.detach(), g["bm"]))
    out.backward(d_out.to(cuda_device))
    got = tuple(t.grad.float().cpu() for t in (qd, kd, vd))
    assert_grads(got, ref, dtype, heads, name)


@pytest.mark.parametrize("cname,heads", [("C1", None), ("C2", None), ("C3", [(0, 0), (1, 7), (1, 15)])])
def test_backward_benchmark_configs(cuda_device, cname, heads):
    q, k, v, bm, _ = inputs.make_inputs(cname, 1)
    torch.manual_seed(12)
    d_out = (torch.randn(q.shape) * 0.5).to(q.dtype)
    heads = heads or all_heads(q.shape[0], q.shape[1])
    ref = orc.block_mask_attention_backward(q, k, v, bm, d_out, bh=heads)
    assert_grads(backward(q, k, v, d_out, bm, cuda_device), ref, q.dtype, heads, cname)


def test_backward_c4_one_head_and_full_size_properties(cuda_device):
    q, k, v, bm, _ = inputs.make_inputs("C4", 0)
    torch.manual_seed(13)
    d_out = (torch.randn(q.shape) * 0.5).to(q.dtype)
    heads = [(0, 17)]
    ref = orc.block_mask_attention_backward(q, k, v, bm, d_out, bh=heads)
    got = backward(q, k, v, d_out, bm, cuda_device)
    assert_grads(got, ref, q.dtype, heads, "C4")
    dq, dk, dv = got
    # every head, no oracle needed:
    # the rows of P sum to one, so the dV of a head summed over its keys is the dO summed over its rows
    lhs = dv.sum(dim=2)
    rhs = d_out.float().sum(dim=2)
    assert float((lhs - rhs).abs().max()) <= 2e-2 * float(rhs.abs().max()) + 0.5
    # the same inputs give the same bits (no atomics anywhere)
    again = backward(q, k, v, d_out, bm, cuda_device)
    assert all(torch.equal(a, b) for a, b in zip(got, again))
    # with every key row equal, dS K = (sum_k dS) k0 = 0: each row of dS sums to zero
    k_const = k[:, :, :1].expand_as(k).contiguous()
    dq0, _, _ = backward(q, k_const, v, d_out, bm, cuda_device)
    assert float(dq0.abs().max()) <= 2e-2 * float(dq.abs().max())


def test_backward_edge_cases_empty_rows_masked_entries_unsorted_lists(cuda_device):
    torch.manual_seed(4)
    N = 384
    q, k, v, d_out = (torch.randn(1, 1, N, 64).bfloat16() for _ in range(4))
    nb = torch.tensor([[[1, 2, 3]]], dtype=torch.int32)
    idx = torch.tensor([[[[0, 0, 0], [1, 0, 0], [2, 0, 1]]]], dtype=torch.int32)          # last list unsorted
    P, F, C = int(BlockMaskType.PARTIAL), int(BlockMaskType.FULL), int(BlockMaskType.CAUSAL)
    typ = torch.tensor([[[[P, 0, 0], [C, P, 0], [P, F, P]]]], dtype=torch.int32)
    pidx = torch.tensor([[[[0, -1, -1], [-1, 1, -1], [2, -1, 7]]]], dtype=torch.int32)     # 7: out of range -> causal fallback
    pool = torch.rand(3, 128, 128) < 0.3
    pool[0, 5] = False          # query row 5 attends nothing at all
    pool[0, 0, 0] = True
    bm = OmniBlockMask(nb, idx, typ, N, N, 128, 128, pidx, pool)
    dense = dense_mask_from_blocks(bm)
    assert not bool(dense[0, 0, 5].any())
    ref = orc.block_mask_attention_backward(q, k, v, bm, d_out)
    got = backward(q, k, v, d_out, bm, cuda_device)
    assert_grads(got, ref, torch.bfloat16, [(0, 0)], "partial")
    assert torch.all(got[0][0, 0, 5] == 0)

    # a Q block with an empty list, a listed entry typed MASKED, CAUSAL above the diagonal
    g = load_golden("ref_fcp_n512_d64")
    bm = g["bm"]
    bm2 = OmniBlockMask(bm.kv_num_blocks.clone(), bm.kv_indices.clone(), bm.block_mask_types.clone(), bm.q_len,
                        bm.kv_len, 128, 128, bm.partial_block_mask_indices.clone(), bm.partial_block_masks.clone())
    bm2.kv_num_blocks[:, 0, 1] = 0
    bm2.block_mask_types[:, 1, 3, 1] = int(BlockMaskType.MASKED)
    bm2.kv_indices[:, 1, 2, 0] = 3
    bm2.block_mask_types[:, 1, 2, 0] = int(BlockMaskType.CAUSAL)
    q, k, v = g["q"], g["k"], g["v"]
    d_out = torch.randn(q.shape).half()
    ref = orc.block_mask_attention_backward(q, k, v, bm2, d_out)
    got = backward(q, k, v, d_out, bm2, cuda_device)
    heads = all_heads(q.shape[0], q.shape[1])
    assert_grads(got, ref, torch.float16, heads, "empty lists")
    assert torch.all(got[0][:, 0, 128:256] == 0)   # the Q block that attends nothing


@pytest.mark.parametrize("D,dtype", [(128, torch.float16), (64, torch.bfloat16)])
def test_autograd_op_with_ragged_length(cuda_device, D, dtype):
    """Unpadded length 300 through the differentiable operator: padding, clipping of keys >= 300 and
    the slicing of the padded rows all sit inside the autograd graph."""
    torch.manual_seed(5)
    n = 300
    q, k, v, d_out = (torch.randn(1, 2, n, D).to(dtype) for _ in range(4))
    bm = create_causal_omni_block_mask(1, 2, n, n)
    bm.block_mask_types[:, 1, 2, :] = int(BlockMaskType.FULL)   # head 1: last Q block sees every block fully
    qd, kd, vd = (t.to(cuda_device).requires_grad_(True) for t in (q, k, v))
    out = omni_attention_autograd(qd, kd, vd, bm)
    assert out.shape == (1, 2, n, D)
    assert torch.equal(out.detach(), omni_attention(qd.detach(), kd.detach(), vd.detach(), bm))
    out.backward(d_out.to(cuda_device))
    pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, 384 - n))
    ref = orc.block_mask_attention_backward(pad(q), pad(k), pad(v), bm, pad(d_out), seqlen_orig=n)
    got = tuple(t.grad.float().cpu() for t in (qd, kd, vd))
    assert_grads(got, tuple(r[:, :, :n] for r in ref), dtype, [(0, 0), (0, 1)], "ragged")


def test_backward_rejects_a_small_workspace(cuda_device):
    lib = ops.load_library()
    assert lib.omni_attn_bwd_workspace_bytes(1, 2, 256) >= 2 * 2 * 2 * 4 + 2 * 256 * 4
    assert lib.omni_attn_bwd_workspace_bytes(1, 2, 100) == 0
    q = torch.zeros(1, 2, 256, 64, dtype=torch.float16, device=cuda_device)
    lse = torch.zeros(1, 2, 256, device=cuda_device)
    bm = create_causal_omni_block_mask(1, 2, 256, 256)
    ws = torch.empty(64, dtype=torch.uint8, device=cuda_device)
    with pytest.raises(ops.OmniAttnError, match="workspace"):
        ops.omni_attention_backward_out(q, q, q, q, lse, q, q.clone(), q.clone(), q.clone(), bm, 256, workspace=ws)


@pytest.mark.parametrize("D,dtype", [(64, torch.float16), (128, torch.bfloat16)])
def test_backward_with_softcap_through_the_transfusion_core(cuda_device, D, dtype):
    """Training path of the Transfusion attention slot: soft-capped scores
    (transfusion_pytorch/transfusion.py:298-299, :967) forward and backward. Scores are made large
    enough for the cap to bend them."""
    from omni_attention_b200.transfusion import transfusion_attention_core

    torch.manual_seed(21)
    n, cap = 512, 3.0
    q, k, v, d_out = (torch.randn(1, 2, n, D).to(dtype) for _ in range(4))
    q = (q.float() * 2.0).to(dtype)
    bm = create_causal_omni_block_mask(1, 2, n, n)
    bm.block_mask_types[:, :, 3, 1] = int(BlockMaskType.FULL)
    qd, kd, vd = (t.to(cuda_device).requires_grad_(True) for t in (q, k, v))
    out = transfusion_attention_core(qd, kd, vd, bm, softcap_value=cap)
    assert out.requires_grad
    out.backward(d_out.to(cuda_device))
    ref_out, _ = orc.block_mask_attention(q, k, v, bm, softcap=cap)
    assert float((out.detach().float().cpu() - ref_out).abs().max()) <= 2e-2 + 1e-2 * float(ref_out.abs().max())
    ref = orc.block_mask_attention_backward(q, k, v, bm, d_out, softcap=cap)
    got = tuple(t.grad.float().cpu() for t in (qd, kd, vd))
    assert_grads(got, ref, dtype, [(0, 0), (0, 1)], "softcap")
    # and the cap really matters for these inputs
    plain = orc.block_mask_attention_backward(q, k, v, bm, d_out)
    assert float((plain[0] - ref[0]).abs().max()) > 10 * GRAD_RTOL[dtype] * float(ref[0].abs().max())


def test_backward_c5_shape_sampled_rows_and_columns(cuda_device):
    """The 32K multi-image configuration: two of the 128 (batch, head) pairs on the GPU, one of them
    checked at sampled query rows (dq) and key rows (dk, dv) against the block-at-a-time oracle, both
    through properties that need no oracle."""
    cfg = inputs.CONFIGS["C5"]
    lo, hi = 48, 50
    q, k, v, bm, _ = inputs.make_inputs("C5", seed=0, bh_range=(lo, hi))
    torch.manual_seed(31)
    d_out = (torch.randn(q.shape) * 0.5).to(q.dtype)
    dq, dk, dv = backward(q, k, v, d_out, bm, cuda_device)
    assert all(bool(torch.isfinite(t).all()) for t in (dq, dk, dv))
    lhs, rhs = dv.sum(dim=2), d_out.float().sum(dim=2)
    assert float((lhs - rhs).abs().max()) <= 2e-2 * float(rhs.abs().max()) + 1.0
    g = torch.Generator().manual_seed(5)
    rows = torch.randint(0, cfg.N, (48,), generator=g).tolist() + [0, 127, 128, cfg.N - 1, 4095, 4096]
    cols = torch.randint(0, cfg.N, (48,), generator=g).tolist() + [0, 127, 128, cfg.N - 1, 20000, 20001]
    rq, rk, rv = orc.blockwise_gradients(q, k, v, bm, d_out, 0, 1, rows, cols)
    tol = GRAD_RTOL[q.dtype]
    for name, got, ref in (("dq", dq[0, 1, rows], rq), ("dk", dk[0, 1, cols], rk), ("dv", dv[0, 1, cols], rv)):
        err = float((got - ref).abs().max())
        assert err <= tol * float(ref.abs().max()), f"C5 {name}: {err:.4g} vs max {float(ref.abs().max()):.4g}"


def test_backward_through_the_pybind_module(cuda_device):
    """`omni_attn.omni_attn_bwd` (torch tensors) gives the bits of the ctypes path."""
    import omni_attention_b200 as pkg

    m = pkg.install_reference_module()
    g = load_golden("ref_fcp_n512_d64")
    q, k, v = (g[n].half().to(cuda_device) for n in ("q", "k", "v"))
    bm = g["bm"]
    B, H, N, D = q.shape
    torch.manual_seed(3)
    d_out = torch.randn(q.shape).half().to(cuda_device)
    dev = lambda t: t.to(cuda_device, torch.int32).contiguous()
    nb, idx, typ, pidx = dev(bm.kv_num_blocks), dev(bm.kv_indices), dev(bm.block_mask_types), dev(bm.partial_block_mask_indices)
    pool = bm.partial_block_masks.to(cuda_device).contiguous()
    out = torch.empty_like(q)
    lse = torch.empty(B, H, N, dtype=torch.float32, device=cuda_device)
    m.omni_attn_fwd(q, k, v, out, nb, idx, typ, 128, 128, N, pidx, pool, True, lse=lse)
    ws = torch.empty(m.omni_attn_bwd_workspace_bytes(B, H, N), dtype=torch.uint8, device=cuda_device)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    m.omni_attn_bwd(q, k, v, out, lse, d_out, dq, dk, dv, nb, idx, typ, 128, 128, N, pidx, pool, True, ws)
    ref = backward(g["q"].half(), g["k"].half(), g["v"].half(), d_out.cpu(), bm, cuda_device)
    for a, b in zip((dq, dk, dv), ref):
        assert torch.equal(a.float().cpu(), b)
    with pytest.raises(RuntimeError, match="workspace"):
        m.omni_attn_bwd(q, k, v, out, lse, d_out, dq, dk, dv, nb, idx, typ, 128, 128, N, pidx, pool, True, ws[:16])


@pytest.mark.parametrize("n,D", [(128, 64), (128, 128), (200, 128), (640, 64)])
def test_small_and_odd_shapes_forward_and_backward(cuda_device, n, D):
    """One Q block, an odd number of Q blocks, a batch*head count that no grouping divides, a length
    that needs padding: forward and backward against the oracle."""
    torch.manual_seed(n + D)
    B, H = 3, 5
    q, k, v, d_out = (torch.randn(B, H, n, D).half() for _ in range(4))
    bm = create_causal_omni_block_mask(B, H, n, n)
    qd, kd, vd = (t.to(cuda_device).requires_grad_(True) for t in (q, k, v))
    out = omni_attention_autograd(qd, kd, vd, bm)
    out.backward(d_out.to(cuda_device))
    n_pad = bm.q_len
    pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, n_pad - n))
    ref_out, _ = orc.block_mask_attention(pad(q), pad(k), pad(v), bm, seqlen_orig=n)
    err = (out.detach().float().cpu() - ref_out[:, :, :n]).abs()
    assert float(err.max()) <= 2e-2 + 1e-2 * float(ref_out[:, :, :n].abs().max())
    ref = orc.block_mask_attention_backward(pad(q), pad(k), pad(v), bm, pad(d_out), seqlen_orig=n)
    got = tuple(t.grad.float().cpu() for t in (qd, kd, vd))
    assert_grads(got, tuple(r[:, :, :n] for r in ref), torch.float16, all_heads(B, H), f"n={n} D={D}")
