import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
GOLDEN_CASES = ["ref_causal_n256_d64", "ref_fcp_n512_d64", "ref_fcp_n384_d128", "ref_interleaved_n512_d64"]
# the other block shape (64x64) and head_dim (32) of the reference's launchers
GOLDEN_CASES_64_32 = ["ref_fcp_n448_d64_blk64", "ref_fcp_n384_d32", "ref_interleaved_n512_d32_blk64",
                      "ref_fcp_n320_d128_blk64"]

# tolerances of the parity contract: 16-bit outputs atol 2e-2 / rtol 1e-2, log-sum-exp 1e-3
OUT_ATOL, OUT_RTOL, LSE_ATOL = 2e-2, 1e-2, 1e-3


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def load_golden(name):
    """Golden case written by tests/golden/make_golden.py -> dict of torch tensors + OmniBlockMask."""
    from omni_attention_b200.block_mask import OmniBlockMask

    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    t = lambda k: torch.from_numpy(z[k])
    Bq, Bk = int(z["Q_BLOCK_SIZE"]), int(z["KV_BLOCK_SIZE"])
    q_len, kv_len = int(z["q_len"]), int(z["kv_len"])
    pidx = pool = None
    if int(z["has_partial"]):
        pidx = t("partial_block_mask_indices")
        pool = torch.from_numpy(np.unpackbits(z["partial_block_masks"], axis=-1)[..., :Bk].astype(bool))
    bm = OmniBlockMask(t("kv_num_blocks"), t("kv_indices"), t("block_mask_types"), q_len, kv_len, Bq, Bk, pidx, pool)
    dense = torch.from_numpy(np.unpackbits(z["dense_mask"], axis=-1)[..., :kv_len].astype(bool))
    return {"q": t("q"), "k": t("k"), "v": t("v"), "out": t("out"), "lse": t("lse"), "bm": bm, "dense": dense}


def assert_parity(out, lse, ref_out, ref_lse, what=""):
    """Output within atol 2e-2 / rtol 1e-2 of the oracle, lse within 1e-3."""
    out = out.float().cpu()
    ref_out = ref_out.float().cpu()
    err = (out - ref_out).abs()
    tol = OUT_ATOL + OUT_RTOL * ref_out.abs()
    bad = err > tol
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} output elements out of tolerance, max abs err {float(err.max()):.4g}"
    if lse is not None:
        lerr = (lse.float().cpu() - ref_lse.float().cpu()).abs()
        assert float(lerr.max()) <= LSE_ATOL, f"{what}: lse max abs err {float(lerr.max()):.4g}"


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
