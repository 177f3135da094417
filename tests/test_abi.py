"""The C-ABI library loads without a GPU, exports every function include/omni_attn_sm100.h declares,
and rejects bad arguments with the documented codes before touching the device."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT
from omni_attention_b200 import ops

HEADER = os.path.join(ROOT, "include", "omni_attn_sm100.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(omni_attn_\w+)\s*\(", src)))


def error_codes():
    src = open(HEADER).read()
    return {m.group(1): int(m.group(2)) for m in re.finditer(r"#define\s+(OMNI_\w+)\s+\(?(-?\d+)\)?", src)}


def test_library_exports_every_declared_symbol():
    lib = ops.load_library()
    names = declared_functions()
    assert sorted(names) == sorted(ops.ABI_SYMBOLS)
    for n in names:
        assert getattr(lib, n) is not None
    assert lib.omni_attn_abi_version() == error_codes()["OMNI_ATTN_ABI_VERSION"]


def test_pybind_module_exports_reference_names():
    import omni_attention_b200 as pkg

    m = pkg.install_reference_module()
    for n in ("omni_attn_mma_stages_split_q_shared_kv", "omni_attn_simple_kernel", "omni_attn_cp_async",
              "omni_attn_preftech_kernel", "omni_attn_mma_stages_split_q_shared_kv_swizzle", "omni_attn_fwd",
              "omni_attn_bwd", "omni_attn_bwd_workspace_bytes"):
        assert callable(getattr(m, n))
    # the reference's wrappers pass 13 positional arguments; anything else is a TypeError
    with pytest.raises(TypeError):
        m.omni_attn_simple_kernel(1, 2, 3)


def _call(lib, fn="omni_attn_fwd_sm100", **kw):
    buf = (ctypes.c_char * 4096)()
    a = ctypes.addressof(buf)
    a = (a + 15) & ~15
    d = dict(q=a, k=a, v=a, o=a, lse=None, nb=a, idx=a, typ=a, pidx=None, pbool=None, pbits=None, B=1, H=1, N=128,
             orig=128, D=64, qb=128, kb=128, mb=1, npart=0, dtype=0, scale=0.0, stream=None, status=None)
    d.update(kw)
    return getattr(lib, fn)(d["q"], d["k"], d["v"], d["o"], d["lse"], d["nb"], d["idx"], d["typ"], d["pidx"], d["pbool"],
                            d["pbits"], d["B"], d["H"], d["N"], d["orig"], d["D"], d["qb"], d["kb"], d["mb"], d["npart"],
                            d["dtype"], d["scale"], d["stream"], d["status"])


@pytest.mark.parametrize("fn", ["omni_attn_fwd_sm100", "omni_attn_fwd_simple_sm100"])
def test_argument_validation_codes(fn):
    lib = ops.load_library()
    E = error_codes()
    assert _call(lib, fn, q=None) == E["OMNI_ERR_NULL_POINTER"]
    assert _call(lib, fn, typ=None) == E["OMNI_ERR_NULL_POINTER"]
    assert _call(lib, fn, dtype=2) == E["OMNI_ERR_DTYPE"]
    assert _call(lib, fn, D=48) == E["OMNI_ERR_HEAD_DIM"]
    assert _call(lib, fn, D=96) == E["OMNI_ERR_HEAD_DIM"]
    assert _call(lib, fn, D=256) == E["OMNI_ERR_HEAD_DIM"]
    assert _call(lib, fn, qb=32, kb=32) == E["OMNI_ERR_BLOCK_SIZE"]
    assert _call(lib, fn, qb=128, kb=64) == E["OMNI_ERR_BLOCK_SIZE"]
    assert _call(lib, fn, qb=64, kb=128) == E["OMNI_ERR_BLOCK_SIZE"]
    assert _call(lib, fn, N=100) == E["OMNI_ERR_SEQLEN"]
    assert _call(lib, fn, N=192) == E["OMNI_ERR_SEQLEN"]                   # 192 is a multiple of 64, not of 128
    assert _call(lib, fn, N=160, qb=64, kb=64) == E["OMNI_ERR_SEQLEN"]
    assert _call(lib, fn, orig=0) == E["OMNI_ERR_SEQLEN"]
    assert _call(lib, fn, orig=129) == E["OMNI_ERR_SEQLEN"]
    assert _call(lib, fn, B=0) == E["OMNI_ERR_SHAPE"]
    assert _call(lib, fn, mb=0) == E["OMNI_ERR_SHAPE"]
    assert _call(lib, fn, B=70000) == E["OMNI_ERR_SHAPE"]
    assert _call(lib, fn, npart=-1) == E["OMNI_ERR_PARTIAL"]
    assert _call(lib, fn, npart=3) == E["OMNI_ERR_PARTIAL"]
    assert _call(lib, fn, N=128 * 1025, orig=128) == E["OMNI_ERR_TOO_LONG"]
    simple = 1 if fn.endswith("simple_sm100") else 0
    for D in (32, 64, 128):   # with 64-blocks the tables reach less far; the limit is what the library reports
        lim = lib.omni_attn_max_seqlen(D, 64, simple)
        assert 0 < lim < 128 * 1024 and lim % 128 == 0
        assert _call(lib, fn, N=lim + 64, orig=64, D=D, qb=64, kb=64) == E["OMNI_ERR_TOO_LONG"]
        assert lib.omni_attn_max_seqlen(D, 128, simple) == 128 * 1024
    base = _call.__defaults__
    buf = (ctypes.c_char * 64)()
    odd = (ctypes.addressof(buf) | 15) - 7  # not 16-byte aligned
    assert _call(lib, fn, q=odd) == E["OMNI_ERR_ALIGNMENT"]
    for code in E.values():
        assert isinstance(lib.omni_attn_error_string(code), bytes)


def test_validation_from_four_threads_at_once():
    """The entry points hold no unsynchronised first-use state: four host threads making their first
    calls together all get the documented codes."""
    import threading

    lib = ops.load_library()
    E = error_codes()
    go, got = threading.Barrier(4), [None] * 4

    def work(i):
        go.wait()
        got[i] = [_call(lib, q=None), _call(lib, D=96), _call(lib, N=100), lib.omni_attn_max_seqlen(128, 128, 0)]

    ts = [threading.Thread(target=work, args=(i,)) for i in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert all(g == [E["OMNI_ERR_NULL_POINTER"], E["OMNI_ERR_HEAD_DIM"], E["OMNI_ERR_SEQLEN"], 131072] for g in got)


def test_pack_validation():
    lib = ops.load_library()
    E = error_codes()
    assert lib.omni_attn_pack_partial_masks_blk_sm100(None, None, 2, 32, None) == E["OMNI_ERR_BLOCK_SIZE"]
    assert lib.omni_attn_pack_partial_masks_blk_sm100(None, None, 2, 64, None) == E["OMNI_ERR_NULL_POINTER"]
    assert lib.omni_attn_pack_partial_masks_sm100(None, None, 0, None) == 0
    assert lib.omni_attn_pack_partial_masks_sm100(None, None, 2, None) == E["OMNI_ERR_NULL_POINTER"]
    assert lib.omni_attn_pack_partial_masks_sm100(None, None, -1, None) == E["OMNI_ERR_PARTIAL"]


def test_operator_refuses_cpu_tensors():
    from omni_attention_b200 import create_causal_omni_block_mask, omni_attention

    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16)
    bm = create_causal_omni_block_mask(1, 1, 128, 128)
    with pytest.raises(ops.OmniAttnError):
        omni_attention(q, q, q, bm)
    with pytest.raises(ValueError):   # head_dim outside {32, 64, 128}
        omni_attention(torch.zeros(1, 1, 128, 96, dtype=torch.float16), torch.zeros(1, 1, 128, 96, dtype=torch.float16),
                       torch.zeros(1, 1, 128, 96, dtype=torch.float16), bm)
    bm.Q_BLOCK_SIZE = 32              # block sizes outside {64, 128}
    bm.KV_BLOCK_SIZE = 32
    with pytest.raises(ValueError):
        omni_attention(q, q, q, bm)


def _call_bwd(lib, fn="omni_attn_bwd_sm100", **kw):
    buf = (ctypes.c_char * 4096)()
    a = (ctypes.addressof(buf) + 15) & ~15
    d = dict(q=a, k=a, v=a, o=a, lse=a, do=a, dq=a, dk=a, dv=a, nb=a, idx=a, typ=a, pidx=None, pbool=None, pbits=None,
             B=1, H=1, N=128, orig=128, D=64, qb=128, kb=128, mb=1, npart=0, dtype=0, scale=0.0, stream=None, status=None,
             ws=a, ws_bytes=1 << 20)
    d.update(kw)
    args = [d["q"], d["k"], d["v"], d["o"], d["lse"], d["do"], d["dq"], d["dk"], d["dv"], d["nb"], d["idx"], d["typ"],
            d["pidx"], d["pbool"], d["pbits"], d["B"], d["H"], d["N"], d["orig"], d["D"], d["qb"], d["kb"], d["mb"],
            d["npart"], d["dtype"], d["scale"], d["stream"], d["status"], d["ws"], d["ws_bytes"]]
    if fn == "omni_attn_bwd_ex_sm100":
        args.append(d.get("softcap", 0.0))
    return getattr(lib, fn)(*args)


@pytest.mark.parametrize("fn", ["omni_attn_bwd_sm100", "omni_attn_bwd_ex_sm100"])
def test_backward_argument_validation_codes(fn):
    """The backward entry points check their arguments before anything touches the device."""
    lib = ops.load_library()
    E = error_codes()
    for name in ("q", "lse", "do", "dq", "dk", "dv", "typ", "ws"):
        assert _call_bwd(lib, fn, **{name: None}) == E["OMNI_ERR_NULL_POINTER"], name
    assert _call_bwd(lib, fn, dtype=3) == E["OMNI_ERR_DTYPE"]
    assert _call_bwd(lib, fn, D=48) == E["OMNI_ERR_HEAD_DIM"]
    assert _call_bwd(lib, fn, D=256) == E["OMNI_ERR_HEAD_DIM"]
    assert _call_bwd(lib, fn, qb=64, kb=64) == E["OMNI_ERR_BLOCK_SIZE"]
    assert _call_bwd(lib, fn, N=130) == E["OMNI_ERR_SEQLEN"]
    assert _call_bwd(lib, fn, orig=200) == E["OMNI_ERR_SEQLEN"]
    assert _call_bwd(lib, fn, H=0) == E["OMNI_ERR_SHAPE"]
    assert _call_bwd(lib, fn, npart=2) == E["OMNI_ERR_PARTIAL"]
    assert _call_bwd(lib, fn, N=128 * 1025, orig=128) == E["OMNI_ERR_TOO_LONG"]
    assert _call_bwd(lib, fn, ws_bytes=16) == E["OMNI_ERR_WORKSPACE"]
    base = (ctypes.addressof((ctypes.c_char * 64)()) + 15) & ~15
    assert _call_bwd(lib, fn, dq=base + 4) == E["OMNI_ERR_ALIGNMENT"]
    if fn == "omni_attn_bwd_ex_sm100":
        assert _call_bwd(lib, fn, softcap=-1.0) == E["OMNI_ERR_SOFTCAP"]
        assert _call_bwd(lib, fn, softcap=float("nan")) == E["OMNI_ERR_SOFTCAP"]
    # the workspace size the header promises: codes [BH, nq, nq] rounded to 256 bytes + delta [BH, N]
    assert lib.omni_attn_bwd_workspace_bytes(2, 3, 512) == ((6 * 4 * 4 * 4 + 255) // 256) * 256 + 6 * 512 * 4
    assert lib.omni_attn_bwd_workspace_bytes(2, 3, 500) == 0
