"""Everything the reference's launchers accept (omni-attn-mma/mma/omni_attn_shared_kv.cu:725-741, :780-888:
blocks of 64 or 128, head_dim 32 / 64 / 128) goes through the C ABI and the drop-in `omni_attn` module as it
is: golden vectors written by the reference's own generators with Q_BLOCK_SIZE = KV_BLOCK_SIZE = 64 and
head_dim 32, the reference wrappers' recorded argument forms replayed on the real module, and the list
edge cases that only show with these shapes (units without any work, blocks listed twice).

Tolerances (conftest.py): output atol 2e-2 / rtol 1e-2, log-sum-exp 1e-3.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

from conftest import GOLDEN_CASES_64_32, GOLDEN_DIR, LSE_ATOL, ROOT, assert_parity, load_golden
from omni_attention_b200 import ops
from omni_attention_b200.block_mask import BlockMaskType, OmniBlockMask, dense_mask_from_blocks, retile_block_mask
from omni_attention_b200.ops import omni_attention
from oracle import omni_oracle as orc

pytestmark = pytest.mark.gpu
KERNELS = ["ws", "ws_static", "simple"]


def run(q, k, v, bm, dev, kernel="ws", **kw):
    return omni_attention(q.to(dev), k.to(dev), v.to(dev), bm, return_lse=True, kernel=kernel, check_status=True, **kw)


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", GOLDEN_CASES_64_32)
def test_golden_vectors_64_blocks_and_head_dim_32(cuda_device, name, kernel):
    g = load_golden(name)
    out, lse = run(g["q"], g["k"], g["v"], g["bm"], cuda_device, kernel)
    assert out.shape == g["out"].shape
    assert_parity(out, lse, g["out"], g["lse"], f"{name}/{kernel}")
    # bf16 inputs against the oracle on the rounded values
    q, k, v = (g[x].bfloat16() for x in "qkv")
    ref_out, ref_lse = orc.block_mask_attention(q, k, v, g["bm"])
    out, lse = run(q, k, v, g["bm"], cuda_device, kernel)
    assert_parity(out, lse, ref_out, ref_lse, f"{name}/{kernel}/bf16")


@pytest.mark.parametrize("name", ["ref_fcp_n448_d64_blk64", "ref_interleaved_n512_d32_blk64"])
def test_byte_pool_equals_bit_pool_with_64_blocks(cuda_device, name):
    g = load_golden(name)
    dev = cuda_device
    q, k, v = (g[x].to(dev).contiguous() for x in "qkv")
    outs = []
    for pack in (True, False):
        o = torch.empty_like(q)
        ops.omni_attention_forward_out(q, k, v, o, g["bm"], q.shape[2], pack_bits=pack)
        outs.append(o)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])


def test_64_block_lists_equal_the_same_mask_in_128_blocks(cuda_device):
    """A 64-block mask and its 128-block re-expression (built on the host from the dense expansion) put
    the same allow bits on the same tiles in the same order: the results are bit-identical."""
    g = load_golden("ref_interleaved_n512_d32_blk64")
    bm128 = retile_block_mask(g["bm"], 128)
    assert bm128.Q_BLOCK_SIZE == 128
    a, la = run(g["q"], g["k"], g["v"], g["bm"], cuda_device)
    b, lb = run(g["q"], g["k"], g["v"], bm128, cuda_device)
    assert torch.equal(a, b) and torch.equal(la, lb)


def test_ragged_length_with_64_blocks(cuda_device):
    """Unpadded length 490 under a mask built for 512 = 8 blocks of 64: keys at and beyond 490 are never
    attended, rows beyond it come back sliced off (omni-attn-mma/mma/attn_naive.cu:113)."""
    g = load_golden("ref_interleaved_n512_d32_blk64")
    n = 490
    q, k, v = (g[x][:, :, :n] for x in "qkv")
    ref_out, ref_lse = orc.block_mask_attention(g["q"], g["k"], g["v"], g["bm"], seqlen_orig=n)
    for kernel in KERNELS:
        out, lse = run(q, k, v, g["bm"], cuda_device, kernel)
        assert out.shape[2] == n
        assert_parity(out, lse, ref_out[:, :, :n], ref_lse[:, :, :n], f"ragged 64 / {kernel}")


def _forms():
    return json.load(open(os.path.join(GOLDEN_DIR, "ref_wrapper_calls.json")))


@pytest.mark.parametrize("form", _forms(), ids=lambda f: f"{f['wrapper']}-{f['case']}")
def test_recorded_reference_wrapper_calls_replayed_on_the_module(cuda_device, form):
    """The 13 arguments the reference's unmodified wrappers were recorded to pass
    (tests/golden/ref_wrapper_calls.json), rebuilt with the recorded dtypes, shapes and placeholders
    from the golden case they were recorded on, and handed to the real module function."""
    import omni_attention_b200 as pkg

    mod = pkg.install_reference_module()
    g = load_golden(form["case"])
    bm, n_orig, dev = g["bm"], form["n_orig"], cuda_device
    a = form["args"]
    dt = lambda e: getattr(torch, e["tensor"]["dtype"])
    N = a[0]["tensor"]["shape"][2]

    def padded(x, e):   # what the wrapper does: slice to the caller's length, pad with zeros, cast
        t = torch.zeros(e["tensor"]["shape"], dtype=dt(e), device=dev)
        t[:, :, :n_orig] = x[:, :, :n_orig].to(dev)
        return t

    q, k, v = (padded(g[x], e) for x, e in zip("qkv", a[:3]))
    o = torch.empty(a[3]["tensor"]["shape"], dtype=dt(a[3]), device=dev)
    nb, idx, typ = (getattr(bm, n).to(device=dev, dtype=dt(e)).contiguous()
                    for n, e in zip(("kv_num_blocks", "kv_indices", "block_mask_types"), a[4:7]))
    assert list(nb.shape) == a[4]["tensor"]["shape"] and list(idx.shape) == a[5]["tensor"]["shape"]
    has_partial = a[12]["bool"]
    if has_partial:
        pidx = bm.partial_block_mask_indices.to(device=dev, dtype=dt(a[10])).contiguous()
        pool = bm.partial_block_masks.to(device=dev, dtype=dt(a[11])).contiguous()
        assert list(pool.shape) == a[11]["tensor"]["shape"]
    else:
        pidx = torch.full(a[10]["tensor"]["shape"], -1, dtype=dt(a[10]), device=dev)
        pool = torch.empty(a[11]["tensor"]["shape"], dtype=dt(a[11]), device=dev)
    res = getattr(mod, form["function"])(q, k, v, o, nb, idx, typ, a[7]["int"], a[8]["int"], a[9]["int"], pidx, pool,
                                         has_partial)
    assert res is None
    torch.cuda.synchronize()
    ref_out, _ = orc.block_mask_attention(q.cpu(), k.cpu(), v.cpu(), bm, seqlen_orig=n_orig)
    assert_parity(o[:, :, :n_orig], None, ref_out[:, :, :n_orig], None, f"{form['wrapper']} on {form['case']}")
    assert N == bm.q_len


def _clone(bm):
    c = lambda t: None if t is None else t.clone()
    return OmniBlockMask(c(bm.kv_num_blocks), c(bm.kv_indices), c(bm.block_mask_types), bm.q_len, bm.kv_len,
                         bm.Q_BLOCK_SIZE, bm.KV_BLOCK_SIZE, c(bm.partial_block_mask_indices), c(bm.partial_block_masks))


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("blocks", [128, 64])
def test_units_without_any_work(cuda_device, kernel, blocks):
    """Whole Q-block pairs with empty lists, many in a row and on every head (a resident CTA then gets
    several units in succession that load no Q and issue no MMA): zeros, lse = -inf, status 0, and the
    rows that do have work still match the oracle."""
    torch.manual_seed(3)
    B, H, N, D = 1, 24, 8192, 64
    q, k, v = (torch.randn(B, H, N, D).half() for _ in range(3))
    nq = N // blocks
    from omni_attention_b200.block_mask import create_causal_omni_block_mask

    bm = create_causal_omni_block_mask(B, H, N, N, blocks, blocks)
    per256 = 256 // blocks
    keep = torch.zeros(nq, dtype=torch.bool)
    for pair in (0, 5):                       # only two 256-row pairs of every head keep their lists
        keep[pair * per256:(pair + 1) * per256] = True
    keep[7 * per256] = True                   # and one pair keeps only its first block
    bm.kv_num_blocks[:, :, ~keep] = 0
    out, lse = run(q, k, v, bm, cuda_device, kernel)
    rows = keep.repeat_interleave(blocks)
    assert bool((out[:, :, ~rows] == 0).all()) and bool(torch.isinf(lse[:, :, ~rows]).all())
    ref_out, ref_lse = orc.block_mask_attention(q, k, v, bm, bh=[(0, 0), (0, 23)])
    for h in (0, 23):
        assert_parity(out[0, h][rows], lse[0, h][rows], ref_out[0, h][rows], ref_lse[0, h][rows], f"head {h}")
    # every head saw the same lists and gets an answer of the same quality
    o2, l2 = run(q[:, :1].expand(B, H, N, D).contiguous(), k[:, :1].expand(B, H, N, D).contiguous(),
                 v[:, :1].expand(B, H, N, D).contiguous(), bm, cuda_device, kernel)
    assert bool((o2 == o2[:, :1]).all()) and bool((l2 == l2[:, :1]).all())


@pytest.mark.parametrize("kernel", KERNELS)
def test_block_listed_twice(cuda_device, kernel):
    """A KV block that appears twice in a list is visited once, with the meaning the reference's dense
    expansion gives the pair when it applies the entries in list order
    (omni-attn-mma/omni_attn_torch.py:106-143): same type twice = once; FULL after PARTIAL = FULL;
    PARTIAL after FULL = the PARTIAL mask; CAUSAL next to FULL = FULL."""
    g = load_golden("ref_fcp_n512_d64")
    base = g["bm"]
    F, C, P = int(BlockMaskType.FULL), int(BlockMaskType.CAUSAL), int(BlockMaskType.PARTIAL)
    pool_idx = int(base.partial_block_mask_indices.max())
    assert pool_idx >= 0
    cases = {
        "same type twice": [(0, F, -1), (1, F, -1), (1, F, -1), (3, C, -1)],
        "full after partial": [(0, P, pool_idx), (0, F, -1), (3, C, -1)],
        "partial after full": [(0, F, -1), (0, P, pool_idx), (1, F, -1), (3, C, -1)],
        "causal beside full": [(1, C, -1), (1, F, -1), (2, F, -1), (2, C, -1), (3, C, -1)],
        "diagonal causal twice": [(0, F, -1), (3, C, -1), (3, C, -1)],
    }
    for what, entries in cases.items():
        bm = _clone(base)
        mb = max(bm.kv_indices.shape[3], 8)
        B, H, nq, _ = bm.kv_indices.shape
        bm.kv_indices = torch.zeros(B, H, nq, mb, dtype=torch.int32)
        bm.block_mask_types = torch.zeros(B, H, nq, mb, dtype=torch.int32)
        bm.partial_block_mask_indices = torch.full((B, H, nq, mb), -1, dtype=torch.int32)
        bm.kv_num_blocks = torch.zeros(B, H, nq, dtype=torch.int32)
        # Q block 3 carries the list under test, the others a plain diagonal entry
        for qb in range(nq):
            lst = entries if qb == 3 else [(qb, C, -1)]
            bm.kv_num_blocks[:, :, qb] = len(lst)
            for i, (kb, t, pi) in enumerate(lst):
                bm.kv_indices[:, :, qb, i] = kb
                bm.block_mask_types[:, :, qb, i] = t
                bm.partial_block_mask_indices[:, :, qb, i] = pi
        dense = orc.to_dense_mask_loops(bm)   # the reference's expansion, entry by entry in list order
        ref_out, ref_lse = orc.attention_dense_mask(g["q"].float(), g["k"].float(), g["v"].float(), orc.to_score_mask(dense))
        out, lse = run(g["q"], g["k"], g["v"], bm, cuda_device, kernel)
        assert_parity(out, lse, ref_out, ref_lse, f"{what}/{kernel}")


def test_block_listed_twice_backward(cuda_device):
    from omni_attention_b200.ops import omni_attention_autograd

    g = load_golden("ref_fcp_n512_d64")
    bm = _clone(g["bm"])
    F = int(BlockMaskType.FULL)
    # Q block 2: FULL entry for KV block 0 listed twice, then its diagonal
    bm.kv_num_blocks[:, :, 2] = 3
    bm.kv_indices[:, :, 2, :3] = torch.tensor([0, 0, 2], dtype=torch.int32)
    bm.block_mask_types[:, :, 2, :3] = torch.tensor([F, F, int(BlockMaskType.CAUSAL)], dtype=torch.int32)
    bm.partial_block_mask_indices[:, :, 2, :3] = -1
    torch.manual_seed(1)
    d_out = torch.randn(g["q"].shape).half()
    dense = orc.to_dense_mask_loops(bm)
    leaves = [g[x].float().clone().requires_grad_(True) for x in "qkv"]
    o, _ = orc.attention_dense_mask(*leaves, orc.to_score_mask(dense))
    o.backward(d_out.float())
    dev = cuda_device
    mine = [g[x].to(dev).requires_grad_(True) for x in "qkv"]
    omni_attention_autograd(*mine, bm).backward(d_out.to(dev))
    for name, t, r in zip(("dq", "dk", "dv"), mine, leaves):
        err = float((t.grad.float().cpu() - r.grad).abs().max())
        assert err <= 4e-3 * float(r.grad.abs().max()), f"{name}: {err}"


def test_length_limits_are_reported(cuda_device):
    lib = ops.load_library()
    assert lib.omni_attn_max_seqlen(128, 128, 0) == 131072 and lib.omni_attn_max_seqlen(64, 128, 0) == 131072
    lim = lib.omni_attn_max_seqlen(128, 64, 0)
    assert 32768 <= lim < 131072 and lim % 128 == 0
    assert lib.omni_attn_max_seqlen(96, 128, 0) == 0


def test_first_calls_from_four_host_threads_at_once():
    """A fresh process whose first four calls into the library come from four threads at the same
    moment (the per-device first-use state is set up under std::call_once): all four results are
    right."""
    code = r"""
import sys, threading, torch
sys.path.insert(0, %r); sys.path.insert(0, %r)
from conftest import load_golden, assert_parity
from omni_attention_b200.ops import omni_attention
g = load_golden("ref_fcp_n512_d64")
dev = torch.device("cuda:0")
q, k, v = (g[x].to(dev) for x in "qkv")
torch.cuda.synchronize()
res, go = [None] * 4, threading.Barrier(4)
def work(i):
    go.wait()
    s = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(s):
        res[i] = omni_attention(q, k, v, g["bm"].to("cpu"), return_lse=True, kernel=("ws", "simple", "ws_static", "ws")[i])
    s.synchronize()
ts = [threading.Thread(target=work, args=(i,)) for i in range(4)]
[t.start() for t in ts]; [t.join() for t in ts]
for i, (o, l) in enumerate(res):
    assert_parity(o, l, g["out"], g["lse"], "thread %%d" %% i)
print("threads ok")
""" % (ROOT, os.path.join(ROOT, "tests"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "threads ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_right(cuda_device):
    """Bounded waits: with a budget of one cycle (omni_attn_set_wait_cycles) every hand-over that is not
    already there when a role asks for it counts as run out; the CTAs give up cleanly - status
    OMNI_STATUS_WAIT_TIMEOUT with the place in the upper bits, the call returns, nothing is left in flight -
    and an ordinary call right afterwards, on the same context, is correct."""
    lib = ops.load_library()
    g = load_golden("ref_fcp_n384_d128")
    dev = cuda_device
    q, k, v = (g[x].to(dev).contiguous() for x in "qkv")
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    lib.omni_attn_set_wait_cycles(1)
    try:
        ops.omni_attention_forward_out(q, k, v, out, g["bm"], q.shape[2], status=status, kernel="ws")
        torch.cuda.synchronize()
    finally:
        lib.omni_attn_set_wait_cycles(0)       # back to the default budget
    code = int(status.item())
    assert code & 0xFF == ops.STATUS_WAIT_TIMEOUT and (code >> 8) > 0, hex(code)
    with pytest.raises(ops.OmniAttnError, match="gave up waiting"):
        lib.omni_attn_set_wait_cycles(1)
        try:
            omni_attention(q, k, v, g["bm"], check_status=True)
        finally:
            lib.omni_attn_set_wait_cycles(0)
    good, lse = run(g["q"], g["k"], g["v"], g["bm"], dev)
    assert_parity(good, lse, g["out"], g["lse"], "call after a timed-out one")


def _random_case(seed):
    """A small random mask and inputs: either block size, any head_dim and dtype, lists in random order
    with every type (MASKED entries, PARTIAL entries with and without a pool tile), garbage behind the
    list ends, sometimes a ragged length."""
    import random

    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    blk = rnd.choice([64, 128])
    nblk = rnd.randint(1, 9 if blk == 64 else 5)
    D = rnd.choice([32, 64, 128])
    dtype = rnd.choice([torch.float16, torch.bfloat16])
    B, H = rnd.choice([1, 2]), rnd.choice([1, 3])
    N = blk * nblk
    n_orig = rnd.choice([N, N, rnd.randint(N - blk + 1, N)])
    mb = nblk + rnd.choice([0, 0, 2])
    nb = torch.zeros(B, H, nblk, dtype=torch.int32)
    idx = torch.zeros(B, H, nblk, mb, dtype=torch.int32)
    typ = torch.zeros_like(idx)
    pidx = torch.full_like(idx, -1)
    pools = []
    for b in range(B):
        for h in range(H):
            for qb in range(nblk):
                ks = [kb for kb in range(nblk) if rnd.random() < 0.6]
                rnd.shuffle(ks)
                nb[b, h, qb] = len(ks)
                for i, kb in enumerate(ks):
                    t = rnd.choice([0, 1, 2, 2, 3, 3])
                    idx[b, h, qb, i], typ[b, h, qb, i] = kb, t
                    if t == 3 and rnd.random() < 0.85:
                        pidx[b, h, qb, i] = len(pools)
                        pools.append(torch.rand(blk, blk, generator=g) < rnd.choice([0.05, 0.5, 0.95]))
                for i in range(len(ks), mb):
                    idx[b, h, qb, i], typ[b, h, qb, i] = rnd.randint(0, nblk - 1), rnd.choice([0, 1, 2, 3])
    pool = torch.stack(pools) if pools else None
    bm = OmniBlockMask(nb, idx, typ, N, N, blk, blk, pidx if pool is not None else None, pool)
    q, k, v, d_out = (torch.randn(B, H, n_orig, D, generator=g).to(dtype) for _ in range(4))
    return bm, q, k, v, d_out, N, n_orig, dtype


@pytest.mark.parametrize("chunk", range(4))
def test_random_small_masks_forward_and_dv(cuda_device, chunk):
    """15 random cases per chunk: both kernels against the oracle on every row that may attend a key
    (exact zeros and -inf on the others), and dV of the differentiable operator (dV does not depend on
    the rounded output the way dQ and dK do through delta; those two are checked to be finite and within
    4x the tolerance of tests/test_backward_gpu.py)."""
    from omni_attention_b200 import omni_attention_autograd

    for case in range(15):
        seed = 7000 + 100 * chunk + case
        bm, q, k, v, d_out, N, n_orig, dtype = _random_case(seed)
        pad = lambda t: torch.nn.functional.pad(t, (0, 0, 0, N - n_orig))
        ref_o, ref_l = orc.block_mask_attention(pad(q), pad(k), pad(v), bm, seqlen_orig=n_orig)
        dense = dense_mask_from_blocks(bm).clone()
        dense[..., n_orig:] = False
        live = dense.any(-1)[:, :, :n_orig]
        for kernel in KERNELS:
            out, lse = run(q, k, v, bm, cuda_device, kernel)
            out, lse = out.float().cpu(), lse.cpu()
            assert bool((out[~live] == 0).all()) and bool(torch.isinf(lse[~live]).all()), f"seed {seed} {kernel}: dead rows"
            if bool(live.any()):
                assert_parity(out[live], lse[live], ref_o[:, :, :n_orig][live], ref_l[:, :, :n_orig][live], f"seed {seed} {kernel}")
        qd, kd, vd = (t.to(cuda_device).requires_grad_(True) for t in (q, k, v))
        omni_attention_autograd(qd, kd, vd, bm).backward(d_out.to(cuda_device))
        ref = orc.block_mask_attention_backward(pad(q), pad(k), pad(v), bm, pad(d_out), seqlen_orig=n_orig)
        rt = 4e-3 if dtype == torch.float16 else 2e-2
        for name, got, r, slack in (("dq", qd.grad, ref[0], 4.0), ("dk", kd.grad, ref[1], 4.0), ("dv", vd.grad, ref[2], 1.0)):
            got, r = got.float().cpu(), r[:, :, :n_orig]
            assert bool(torch.isfinite(got).all()), f"seed {seed} {name}"
            for b in range(q.shape[0]):
                for h in range(q.shape[1]):
                    scale_ = float(r[b, h].abs().max())
                    if scale_ > 0.05:   # heads whose true gradient is (almost) zero have no relative tolerance
                        err = float((got[b, h] - r[b, h]).abs().max())
                        assert err <= slack * rt * scale_, f"seed {seed} {name}[{b},{h}]: {err:.3g} > {slack * rt * scale_:.3g}"


def test_c3_pattern_listed_in_64_blocks_gives_the_same_bits(cuda_device):
    """The interleaved 4K-token workload listed in 64x64 blocks (four times as many entries, PARTIAL
    tiles of 64x64) against the same pattern in 128x128 blocks: same kernel, same allow bits, same bits
    out, on both kernels."""
    from omni_attention_b200 import inputs
    from omni_attention_b200.block_mask import block_mask_from_row_limits, row_limits_from_modality_positions

    cfg = inputs.CONFIGS["C3"]
    q, k, v, bm128, meta = inputs.make_inputs("C3", seed=2)
    limits, causal_rows = row_limits_from_modality_positions(cfg.N, meta["image_spans"])
    bm64 = block_mask_from_row_limits(limits, cfg.H, causal_rows, 64, True)
    assert bm64.Q_BLOCK_SIZE == 64 and bm64.visited_blocks() > 3 * bm128.visited_blocks()
    for kernel in ("ws", "simple"):
        o128, l128 = run(q, k, v, bm128, cuda_device, kernel)
        o64, l64 = run(q, k, v, bm64, cuda_device, kernel)
        assert torch.equal(o128, o64) and torch.equal(l128, l64), kernel
