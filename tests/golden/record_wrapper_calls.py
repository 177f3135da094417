"""Records what the reference's five UNMODIFIED Python wrappers
(omni-attn-mma/omni_attn_torch.py:517-1253) pass to the `omni_attn` extension module, by running them
on CPU tensors against a recording stand-in for that module.

Usage (needs the reference checkout; the committed ref_wrapper_calls.json is its output):
    python tests/golden/record_wrapper_calls.py /path/to/reference/omni-attn-mma

Every wrapper pads, casts and marshals on the host and only then calls the module, so everything up to
the call runs without a GPU; `torch.cuda.synchronize`, which each wrapper calls right after, is
replaced by a no-op for the duration. The scenarios are golden cases of this directory, so that a
GPU test can rebuild exactly the recorded argument forms (dtypes, shapes, placeholders, scalars)
without the checkout and replay them on the real module.
"""
import json
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

# (golden case, unpadded length handed to the wrapper)
SCENARIOS = [
    ("ref_interleaved_n512_d64", 500),        # 128-blocks, PARTIAL pool, ragged length (padded by the wrapper)
    ("ref_causal_n256_d64", 256),             # no PARTIAL data: empty placeholder tensors
    ("ref_interleaved_n512_d32_blk64", 490),  # 64-blocks, head_dim 32, ragged
    ("ref_fcp_n448_d64_blk64", 448),          # 64-blocks, seven of them (448 is no multiple of 128)
]
WRAPPERS = ["omni_attention_shared_kv", "omni_attention_simple", "omni_attention_cp_async", "omni_attention_preftech",
            "omni_attention_shared_kv_swizzle"]
# names the wrappers import from the module (omni_attention_preftech asks for `omni_attn_preftech`,
# omni_attn_torch.py:978, a name the reference's own binding does not export)
MODULE_NAMES = ["omni_attn_mma_stages_split_q_shared_kv", "omni_attn_simple_kernel", "omni_attn_cp_async",
                "omni_attn_preftech_kernel", "omni_attn_preftech", "omni_attn_mma_stages_split_q_shared_kv_swizzle"]


def describe(a):
    if isinstance(a, torch.Tensor):
        return {"tensor": {"dtype": str(a.dtype).replace("torch.", ""), "shape": list(a.shape),
                           "contiguous": bool(a.is_contiguous())}}
    if isinstance(a, bool):
        return {"bool": a}
    if isinstance(a, int):
        return {"int": a}
    raise TypeError(type(a))


def record(ref_dir):
    from conftest import load_golden

    sys.path.insert(0, ref_dir)
    calls = []
    fake = types.ModuleType("omni_attn")
    for name in MODULE_NAMES:
        def fn(*args, _name=name):
            assert len(args) == 13, f"{_name}: {len(args)} positional arguments"
            calls.append((_name, args))
        setattr(fake, name, fn)
    saved_mod, saved_sync = sys.modules.get("omni_attn"), torch.cuda.synchronize
    sys.modules["omni_attn"] = fake
    torch.cuda.synchronize = lambda *a, **k: None
    try:
        import omni_attn_torch as ref  # the reference module, unmodified

        out = []
        for case, n_orig in SCENARIOS:
            g = load_golden(case)
            bm = g["bm"]
            rbm = ref.OmniBlockMask(kv_num_blocks=bm.kv_num_blocks, kv_indices=bm.kv_indices,
                                    block_mask_types=bm.block_mask_types, q_len=bm.q_len, kv_len=bm.kv_len,
                                    Q_BLOCK_SIZE=bm.Q_BLOCK_SIZE, KV_BLOCK_SIZE=bm.KV_BLOCK_SIZE,
                                    partial_block_mask_indices=bm.partial_block_mask_indices,
                                    partial_block_masks=bm.partial_block_masks)
            q, k, v = (g[x][:, :, :n_orig].float() for x in "qkv")
            for w in WRAPPERS:
                calls.clear()
                res = getattr(ref, w)(q, k, v, rbm)
                assert len(calls) == 1, f"{w}: {len(calls)} module calls"
                name, args = calls[0]
                assert tuple(res.shape) == (q.shape[0], q.shape[1], n_orig, q.shape[3])
                out.append({"wrapper": w, "function": name, "case": case, "n_orig": n_orig,
                            "args": [describe(a) for a in args]})
        return out
    finally:
        torch.cuda.synchronize = saved_sync
        if saved_mod is None:
            sys.modules.pop("omni_attn", None)
        else:
            sys.modules["omni_attn"] = saved_mod
        sys.modules.pop("omni_attn_torch", None)


if __name__ == "__main__":
    default = os.path.normpath(os.path.join(HERE, "..", "..", "..", "reference", "omni-attn-mma"))
    forms = record(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("OMNI_REFERENCE_DIR", default))
    with open(os.path.join(HERE, "ref_wrapper_calls.json"), "w") as f:
        json.dump(forms, f, indent=1)
    print(len(forms), "calls recorded")
