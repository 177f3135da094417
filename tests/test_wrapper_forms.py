"""The reference's five unmodified wrappers (omni-attn-mma/omni_attn_torch.py:517-1253) against this
repository's `omni_attn` module: what they pass, recorded once on a stand-in module
(tests/golden/record_wrapper_calls.py -> tests/golden/ref_wrapper_calls.json), must be what the module's
argument checks (omni_attention_b200/csrc/omni_attn_pybind.cc) accept. The GPU suite replays the same
recorded forms on the real module (tests/test_boundary_gpu.py)."""
import json
import os
import sys

import pytest

from conftest import GOLDEN_DIR, load_golden

REF_DIR = os.environ.get("OMNI_REFERENCE_DIR") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference", "omni-attn-mma"))
FORMS = json.load(open(os.path.join(GOLDEN_DIR, "ref_wrapper_calls.json")))


def test_fixture_is_what_the_reference_wrappers_do_today():
    if not os.path.exists(os.path.join(REF_DIR, "omni_attn_torch.py")):
        pytest.skip("reference checkout not present")
    sys.path.insert(0, GOLDEN_DIR)
    try:
        import record_wrapper_calls as rec
    finally:
        sys.path.remove(GOLDEN_DIR)
    assert rec.record(REF_DIR) == FORMS


def test_every_wrapper_and_block_shape_is_covered():
    wrappers = {f["wrapper"] for f in FORMS}
    assert wrappers == {"omni_attention_shared_kv", "omni_attention_simple", "omni_attention_cp_async",
                        "omni_attention_preftech", "omni_attention_shared_kv_swizzle"}
    blocks = {f["args"][7]["int"] for f in FORMS}
    dims = {f["args"][0]["tensor"]["shape"][3] for f in FORMS}
    assert blocks == {64, 128} and {32, 64} <= dims


@pytest.mark.parametrize("form", FORMS, ids=lambda f: f"{f['wrapper']}-{f['case']}")
def test_recorded_call_passes_the_modules_checks(form):
    """A restatement of forward_impl's checks in omni_attn_pybind.cc (minus `is_cuda`), applied to the
    recorded argument forms, plus: the function the wrapper asks the module for exists in it."""
    import omni_attention_b200 as pkg

    mod = pkg.install_reference_module()
    assert callable(getattr(mod, form["function"]))
    a = form["args"]
    assert len(a) == 13
    Q = a[0]["tensor"]
    assert Q["dtype"] in ("float16", "bfloat16") and len(Q["shape"]) == 4
    for t in a[1:4]:
        assert t["tensor"] == Q and Q["contiguous"]
    B, H, N, D = Q["shape"]
    qb, kb, n_orig = a[7]["int"], a[8]["int"], a[9]["int"]
    assert qb == kb and qb in (64, 128) and N % qb == 0 and D in (32, 64, 128)
    assert 0 < n_orig <= N and n_orig == form["n_orig"]
    nq = N // qb
    nb, idx, typ = (x["tensor"] for x in a[4:7])
    assert nb == {"dtype": "int32", "shape": [B, H, nq], "contiguous": True}
    assert idx["dtype"] == "int32" and idx["shape"][:3] == [B, H, nq] and idx["contiguous"] and typ == idx
    pidx, pool, has_partial = a[10]["tensor"], a[11]["tensor"], a[12]["bool"]
    g = load_golden(form["case"])
    assert has_partial == (g["bm"].partial_block_masks is not None)
    if has_partial:
        assert pidx == idx
        assert pool["dtype"] == "bool" and pool["shape"][1:] == [qb, kb] and pool["contiguous"]
    else:
        # placeholders the module must not look at: empty tensors (omni_attn_torch.py:660-661) or, from three
        # of the wrappers, an all -1 index tensor with an empty [0, blk, blk] pool (:766-779)
        assert pool["shape"][0] == 0
        assert pidx["shape"] in ([0], idx["shape"])
