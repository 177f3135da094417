"""Pins the CPU oracle: against the golden vectors produced by running the reference
(tests/golden/make_golden.py) and, where the reference checkout is present, against the reference's
own functions called in-process on fresh seeded inputs."""
import math
import os
import sys

import pytest
import torch

from conftest import GOLDEN_CASES, GOLDEN_CASES_64_32, load_golden

ALL_GOLDEN = GOLDEN_CASES + GOLDEN_CASES_64_32
from oracle import omni_oracle as orc
from oracle import scalar

# the reference checkout, when there is one: next to this repository unless OMNI_REFERENCE_DIR says otherwise
REF_DIR = os.environ.get("OMNI_REFERENCE_DIR") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference", "omni-attn-mma"))


@pytest.mark.parametrize("name", ALL_GOLDEN)
def test_dense_mask_matches_reference_expansion(name):
    g = load_golden(name)
    bm = g["bm"]
    assert torch.equal(orc.to_dense_mask_loops(bm), g["dense"])
    B, H = g["dense"].shape[:2]
    for b in range(B):
        for h in range(H):
            assert torch.equal(orc.to_dense_mask_slice(bm, b, h), g["dense"][b, h])


@pytest.mark.parametrize("name", ALL_GOLDEN)
def test_attention_matches_reference_output(name):
    g = load_golden(name)
    out, lse = orc.block_mask_attention(g["q"], g["k"], g["v"], g["bm"])
    # same torch ops on the same values: bit-exact on the same build, allow rounding noise across builds
    assert torch.allclose(out, g["out"], atol=2e-6, rtol=1e-6)
    assert torch.allclose(lse, g["lse"], atol=2e-6, rtol=1e-6)


@pytest.mark.parametrize("name", ALL_GOLDEN)
def test_scalar_oracle_matches_reference_output(name):
    g = load_golden(name)
    B, H, N, D = g["q"].shape
    rows_bh = [bh for bh in range(B * H) for _ in range(N)]
    rows_q = list(range(N)) * (B * H)
    out, lse = scalar.oracle_rows(g["q"], g["k"], g["v"], g["bm"], rows_bh, rows_q)
    assert torch.allclose(out.view(B, H, N, D), g["out"], atol=5e-6, rtol=1e-5)
    assert torch.allclose(lse.view(B, H, N), g["lse"], atol=5e-6, rtol=1e-5)


def test_scalar_oracle_clips_keys_and_zeroes_empty_rows():
    g = load_golden("ref_causal_n256_d64")
    B, H, N, D = g["q"].shape
    bm = g["bm"]
    seqlen_orig = 200
    out, lse = scalar.oracle_rows(g["q"], g["k"], g["v"], bm, [0] * N, list(range(N)), seqlen_orig=seqlen_orig)
    ro, rl = orc.block_mask_attention(g["q"], g["k"], g["v"], bm, bh=[(0, 0)], seqlen_orig=seqlen_orig)
    assert torch.allclose(out[:seqlen_orig], ro[0, 0, :seqlen_orig], atol=5e-6)
    assert torch.all(out[seqlen_orig:] == 0) and torch.all(torch.isinf(lse[seqlen_orig:]))
    # a Q block with an empty list attends nothing: zeros, lse = -inf
    bm2 = load_golden("ref_causal_n256_d64")["bm"]
    bm2.kv_num_blocks[:, :, 1] = 0
    out, lse = scalar.oracle_rows(g["q"], g["k"], g["v"], bm2, [0, 0], [5, 130])
    assert torch.all(out[1] == 0) and math.isinf(float(lse[1])) and float(lse[1]) < 0
    assert torch.any(out[0] != 0)


def test_naive_attn_mask_rule():
    mods = torch.tensor([[[1, 3, 4], [1, 10, 2]]])
    m = orc.naive_attn_mask(16, mods)[0]
    for i in range(16):
        for j in range(16):
            want = j <= i or (i >= 3 and j < 7) or (i >= 10 and j < 12)
            assert bool(m[i, j]) == want


@pytest.mark.skipif(not os.path.isdir(REF_DIR), reason="reference checkout not present")
def test_oracle_against_reference_in_process():
    sys.path.insert(0, REF_DIR)
    import naive_attn as ref_naive  # reference module
    import omni_attn_torch as ref  # reference module

    torch.manual_seed(123)
    B, H, N, D = 1, 2, 384, 64
    q, k, v = (torch.randn(B, H, N, D).half().float() for _ in range(3))
    # random F/C/P/skip lists, PARTIAL blocks with Bernoulli masks, built with the reference's types
    nq = N // 128
    nb = torch.zeros(B, H, nq, dtype=torch.int32)
    idx = torch.zeros(B, H, nq, nq, dtype=torch.int32)
    typ = torch.zeros(B, H, nq, nq, dtype=torch.int32)
    for h in range(H):
        for qb in range(nq):
            n = 0
            for kb in range(qb + 1):
                t = int(ref.BlockMaskType.CAUSAL) if kb == qb else int(torch.randint(0, 4, (1,)))
                if t == 0:
                    continue
                idx[0, h, qb, n], typ[0, h, qb, n] = kb, t
                n += 1
            nb[0, h, qb] = n
    rbm = ref.OmniBlockMask(nb, idx, typ, N, N, 128, 128)
    dense_src = torch.rand(B, H, N, N) < 0.5
    rbm.partial_block_mask_indices, rbm.partial_block_masks = ref.build_partial_block_data(rbm, dense_src)
    dense = rbm.to_dense_mask()
    assert torch.equal(orc.to_dense_mask_loops(rbm), dense)
    ref_out = ref.naive_attention_with_dense_mask(q, k, v, mask=ref.to_score_mask(rbm))
    ref_out2 = ref_naive.naive_attention(q, k, v, dense)
    out, _ = orc.block_mask_attention(q, k, v, rbm)
    assert torch.allclose(out, ref_out, atol=1e-6, rtol=1e-6)
    assert torch.allclose(out, ref_out2, atol=1e-6, rtol=1e-6)
    # dtype behaviour of the torch path with 16-bit inputs (softmax in fp32, cast back)
    o16, _ = orc.attention_dense_mask(q.bfloat16(), k.bfloat16(), v.bfloat16(), ref.to_score_mask(rbm))
    r16 = ref.naive_attention_with_dense_mask(q.bfloat16(), k.bfloat16(), v.bfloat16(), mask=ref.to_score_mask(rbm))
    assert torch.equal(o16, r16)


def test_oracle_gradient_matches_torch_sdpa_autograd():
    """The oracle's backward is autograd through its own forward; cross-check it on a causal mask
    with the gradient of torch's scaled_dot_product_attention."""
    import torch.nn.functional as F
    from omni_attention_b200 import create_causal_omni_block_mask
    from oracle import omni_oracle as orc

    torch.manual_seed(0)
    q, k, v, d_out = (torch.randn(1, 2, 256, 64) for _ in range(4))
    bm = create_causal_omni_block_mask(1, 2, 256, 256)
    dq, dk, dv = orc.block_mask_attention_backward(q, k, v, bm, d_out)
    qs, ks, vs = (t.clone().requires_grad_(True) for t in (q, k, v))
    F.scaled_dot_product_attention(qs, ks, vs, is_causal=True).backward(d_out)
    for a, b in ((dq, qs.grad), (dk, ks.grad), (dv, vs.grad)):
        assert float((a - b).abs().max()) < 2e-5


def test_blockwise_gradient_oracle_matches_the_autograd_oracle():
    """The sampled, block-at-a-time gradient used at 32 K tokens equals the autograd oracle where both run."""
    from conftest import load_golden
    from oracle import omni_oracle as orc

    g = load_golden("ref_fcp_n512_d64")
    q, k, v, bm = g["q"], g["k"], g["v"], g["bm"]
    torch.manual_seed(2)
    d_out = torch.randn(q.shape)
    ref = orc.block_mask_attention_backward(q, k, v, bm, d_out)
    rows = [0, 5, 127, 128, 300, 511]
    cols = [0, 64, 129, 255, 256, 510]
    for h in (0, q.shape[1] - 1):
        dq, dk, dv = orc.blockwise_gradients(q, k, v, bm, d_out, 0, h, rows, cols)
        assert float((dq - ref[0][0, h, rows]).abs().max()) < 1e-4
        assert float((dk - ref[1][0, h, cols]).abs().max()) < 1e-4
        assert float((dv - ref[2][0, h, cols]).abs().max()) < 1e-4
        dense = orc.to_dense_mask_slice(bm, 0, h)
        for qb in range(4):
            assert torch.equal(orc.mask_block_rows(bm, 0, h, qb), dense[qb * 128:(qb + 1) * 128])


# ---- the Transfusion attention core with its tanh soft-cap ---------------------------------------------------
TRANSFUSION_SRC = os.path.normpath(os.path.join(REF_DIR, "..", "transfusion_pytorch", "transfusion.py"))


def _softcap_golden():
    import numpy as np
    from conftest import GOLDEN_DIR

    z = np.load(os.path.join(GOLDEN_DIR, "ref_softcap_interleaved_n512_d64.npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def test_softclamp_is_the_references_function():
    """oracle.softclamp against the reference's own two-line function (transfusion_pytorch/transfusion.py:
    298-299), taken out of its source file (the package itself cannot be imported: einx is missing)."""
    if not os.path.exists(TRANSFUSION_SRC):
        pytest.skip("reference checkout not present")
    import ast

    ns = {"torch": torch}
    for node in ast.parse(open(TRANSFUSION_SRC).read()).body:
        if isinstance(node, ast.FunctionDef) and node.name == "softclamp":
            exec(compile(ast.Module([node], []), TRANSFUSION_SRC, "exec"), ns)
    t = torch.randn(4, 97, generator=torch.Generator().manual_seed(2)) * 30
    for cap in (50.0, 4.0, 15.0):
        assert torch.equal(orc.softclamp(t, cap), ns["softclamp"](t, cap))
    assert torch.equal(orc.softclamp(t), ns["softclamp"](t))


@pytest.mark.parametrize("cap", [50, 4])
def test_softcap_branch_of_the_oracle_matches_the_reference_core(cap):
    """attention_dense_mask(softcap=) against the golden written from the reference's own softclamp /
    max_neg_value and the operators of its attention core (tests/golden/make_golden.py, case 9)."""
    g = load_golden("ref_interleaved_n512_d64")
    s = _softcap_golden()
    out, lse = orc.attention_dense_mask(g["q"].float(), g["k"].float(), g["v"].float(), orc.to_score_mask(g["dense"]),
                                        softcap=float(cap))
    assert torch.allclose(out, s[f"out_cap{cap}"], atol=3e-6, rtol=1e-5)
    assert torch.allclose(lse, s[f"lse_cap{cap}"], atol=3e-6, rtol=1e-5)


def test_attention_forward_restatement_reproduces_the_core_golden():
    """transfusion_attention_forward with pass-through projections is the bare core: it must give the
    cap-50 golden."""
    g = load_golden("ref_interleaved_n512_d64")
    s = _softcap_golden()

    class Bare:
        scale, softcap_value, laser, laser_softclamp_value, to_gates = 64 ** -0.5, 50.0, False, 15.0, None
        to_qk = staticmethod(lambda x: (g["q"].float(), g["k"].float()))
        to_v = staticmethod(lambda x: g["v"].float())
        to_out = staticmethod(lambda o: o)
        dropout = staticmethod(lambda a: a)

    out = orc.transfusion_attention_forward(Bare, None, attn_mask=g["dense"][:, 0])
    assert torch.allclose(out, s["out_cap50"], atol=3e-6, rtol=1e-5)


def test_modality_position_builder_matches_the_references_builder():
    """create_omni_block_mask_from_modality_positions (this package, CPU path) against the reference's
    builder of the same name (omni-attn-mma/omni_attn_torch.py:1518-1736) on spans aligned to the block
    size, where the reference needs nothing from the transfusion package: equal dense expansions."""
    if not os.path.exists(os.path.join(REF_DIR, "omni_attn_torch.py")):
        pytest.skip("reference checkout not present")
    sys.path.insert(0, REF_DIR)
    try:
        import omni_attn_torch as ref
    finally:
        sys.path.remove(REF_DIR)
    from omni_attention_b200.block_mask import create_omni_block_mask_from_modality_positions

    gen = torch.Generator().manual_seed(12)
    for N in (512, 1024):
        nb = N // 128
        rows = []
        for _ in range(2):                      # two batch elements, up to three aligned image spans each
            spans, pos = [], 0
            while pos < nb and len(spans) < 3:
                pos += int(torch.randint(0, 3, (1,), generator=gen))
                ln = int(torch.randint(1, 3, (1,), generator=gen))
                if pos + ln > nb:
                    break
                spans.append([1, pos * 128, ln * 128])
                pos += ln
            rows.append(spans + [[0, 0, 0]] * (3 - len(spans)))
        mp = torch.tensor(rows, dtype=torch.int32)
        theirs = ref.create_omni_block_mask_from_modality_positions(mp, 2, 2, N, N, 128, 128, device="cpu")
        assert theirs.partial_block_masks is None          # aligned spans: the reference built no PARTIAL block
        mine = create_omni_block_mask_from_modality_positions(mp, 2, 2, N, N, 128, 128, device="cpu")
        assert torch.equal(mine.to_dense_mask(), theirs.to_dense_mask())
        assert torch.equal(orc.to_dense_mask_loops(mine), orc.naive_attn_mask(N, mp)[:, None].expand(-1, 2, -1, -1))
