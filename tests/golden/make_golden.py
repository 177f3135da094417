"""Generates the golden vectors in this directory by RUNNING THE REFERENCE (its torch CPU path).

Usage (needs the reference checkout; the committed .npz files are its output):
    python tests/golden/make_golden.py /path/to/reference/omni-attn-mma

For each case the reference's own generator builds the block mask and dense mask
(generate_debug_data.generate_fixed_debug_F_C_P_data, generate_attn_data.generate_interleaved_mask,
omni_attn_torch.create_causal_omni_block_mask), the inputs are rounded to fp16 (the values a
kernel sees) and the expected output is the reference's
omni_attn_torch.naive_attention_with_dense_mask on those rounded values in fp32 with the score
mask from omni_attn_torch.to_score_mask. The log-sum-exp column is not a reference output (it
has none): it is torch.logsumexp of the same masked score tensor, stored for the LSE checks.

Stored per case: q, k, v (fp16), out (fp32), lse (fp32), kv_num_blocks / kv_indices /
block_mask_types / partial_block_mask_indices (int32), partial_block_masks and dense_mask
(bit-packed with numpy.packbits along the last axis), and the scalar metadata.
"""
import math
import os
import sys
import tempfile

import numpy as np
import torch


def main(ref_dir: str) -> None:
    sys.path.insert(0, ref_dir)
    import generate_attn_data as gad  # noqa: E402  (reference module)
    import generate_debug_data as gdd  # noqa: E402  (reference module)
    import omni_attn_torch as ref  # noqa: E402  (reference module)

    out_dir = os.path.dirname(os.path.abspath(__file__))
    tmp = tempfile.mkdtemp()

    def finish(name, Q, K, V, bm, dense_mask):
        q16, k16, v16 = Q.half(), K.half(), V.half()
        # the reference's own expansion must agree with the dense mask its generator produced
        expanded = bm.to_dense_mask()
        assert torch.equal(expanded, dense_mask), f"{name}: reference to_dense_mask != generator dense mask"
        score_mask = ref.to_score_mask(bm)
        out = ref.naive_attention_with_dense_mask(q16.float(), k16.float(), v16.float(), mask=score_mask)
        D = Q.shape[-1]
        scores = torch.matmul(q16.float(), k16.float().transpose(-2, -1)) * (1.0 / math.sqrt(D)) + score_mask
        lse = torch.logsumexp(scores, dim=-1)
        assert not torch.isnan(out).any(), f"{name}: a fully masked row"
        pidx = bm.partial_block_mask_indices
        pool = bm.partial_block_masks
        np.savez(
            os.path.join(out_dir, name + ".npz"),
            q=q16.numpy(), k=k16.numpy(), v=v16.numpy(), out=out.numpy(), lse=lse.numpy(),
            kv_num_blocks=bm.kv_num_blocks.to(torch.int32).numpy(),
            kv_indices=bm.kv_indices.to(torch.int32).numpy(),
            block_mask_types=bm.block_mask_types.to(torch.int32).numpy(),
            partial_block_mask_indices=(pidx.to(torch.int32).numpy() if pidx is not None else np.zeros(0, np.int32)),
            partial_block_masks=(np.packbits(pool.numpy(), axis=-1) if pool is not None else np.zeros(0, np.uint8)),
            dense_mask=np.packbits(dense_mask.numpy(), axis=-1),
            q_len=bm.q_len, kv_len=bm.kv_len, Q_BLOCK_SIZE=bm.Q_BLOCK_SIZE, KV_BLOCK_SIZE=bm.KV_BLOCK_SIZE,
            has_partial=int(pidx is not None and pool is not None),
        )
        types = bm.block_mask_types[0, 0]
        print(name, "saved; block types head 0:", types.tolist())

    # 1. causal, 2 heads, 256 tokens, D=64 (create_causal_omni_block_mask)
    torch.manual_seed(11)
    Q, K, V = (torch.randn(1, 2, 256, 64) for _ in range(3))
    bm = ref.create_causal_omni_block_mask(1, 2, 256, 256, 128, 128, device="cpu")
    finish("ref_causal_n256_d64", Q, K, V, bm, bm.to_dense_mask())

    # 2. random FULL / CAUSAL / PARTIAL blocks incl. CAUSAL below the diagonal, D=64
    d = gdd.generate_fixed_debug_F_C_P_data(B=1, H=2, seq_len=512, head_dim=64, device="cpu",
                                            output_file=os.path.join(tmp, "a.pt"), seed=5)
    finish("ref_fcp_n512_d64", d["Q_fp32"], d["K_fp32"], d["V_fp32"], d["omni_block_mask"], d["dense_mask"])

    # 3. same generator at D=128
    d = gdd.generate_fixed_debug_F_C_P_data(B=1, H=1, seq_len=384, head_dim=128, device="cpu",
                                            output_file=os.path.join(tmp, "b.pt"), seed=9)
    finish("ref_fcp_n384_d128", d["Q_fp32"], d["K_fp32"], d["V_fp32"], d["omni_block_mask"], d["dense_mask"])

    # 4. interleaved three-segment mask (block types derived from a dense mask), D=64
    d = gad.generate_interleaved_mask(B=1, H=2, seq_len=512, head_dim=64, device="cpu",
                                      output_file=os.path.join(tmp, "c.pt"), seed=3)
    finish("ref_interleaved_n512_d64", d["Q_fp32"], d["K_fp32"], d["V_fp32"], d["omni_block_mask"], d["dense_mask"])

    # 5.-8. the other block shape and head_dim of the reference's launchers (64x64 blocks, head_dim 32;
    # omni-attn-mma/mma/omni_attn_shared_kv.cu:725-741), from the same generators
    d = gdd.generate_fixed_debug_F_C_P_data(B=1, H=2, seq_len=448, head_dim=64, Q_BLOCK_SIZE=64, KV_BLOCK_SIZE=64,
                                            device="cpu", output_file=os.path.join(tmp, "d.pt"), seed=21)
    finish("ref_fcp_n448_d64_blk64", d["Q_fp32"], d["K_fp32"], d["V_fp32"], d["omni_block_mask"], d["dense_mask"])

    d = gdd.generate_fixed_debug_F_C_P_data(B=1, H=2, seq_len=384, head_dim=32, device="cpu",
                                            output_file=os.path.join(tmp, "e.pt"), seed=22)
    finish("ref_fcp_n384_d32", d["Q_fp32"], d["K_fp32"], d["V_fp32"], d["omni_block_mask"], d["dense_mask"])

    d = gad.generate_interleaved_mask(B=1, H=2, seq_len=512, head_dim=32, Q_BLOCK_SIZE=64, KV_BLOCK_SIZE=64,
                                      device="cpu", output_file=os.path.join(tmp, "f.pt"), seed=23)
    finish("ref_interleaved_n512_d32_blk64", d["Q_fp32"], d["K_fp32"], d["V_fp32"], d["omni_block_mask"],
           d["dense_mask"])

    d = gdd.generate_fixed_debug_F_C_P_data(B=1, H=1, seq_len=320, head_dim=128, Q_BLOCK_SIZE=64, KV_BLOCK_SIZE=64,
                                            device="cpu", output_file=os.path.join(tmp, "g.pt"), seed=24)
    finish("ref_fcp_n320_d128_blk64", d["Q_fp32"], d["K_fp32"], d["V_fp32"], d["omni_block_mask"], d["dense_mask"])

    # 9. the Transfusion model's attention core with its tanh soft-cap (transfusion_pytorch/transfusion.py:
    # 963-983), on case 4's inputs and dense mask, caps 50 (the model's default) and 4. The package cannot be
    # imported here (einx and others are missing), so the two pure-torch helpers the core uses, softclamp
    # (:298-299) and max_neg_value (:301-302), are taken out of its source file and executed; the remaining
    # lines of the core are torch operators written out below as they stand there (einx.where with the
    # pattern 'b i j, b h i j, -> b h i j' is torch.where with the mask broadcast over heads).
    import ast

    src = open(os.path.join(ref_dir, "..", "transfusion_pytorch", "transfusion.py")).read()
    helpers = {"torch": torch}
    for node in ast.parse(src).body:
        if isinstance(node, ast.FunctionDef) and node.name in ("softclamp", "max_neg_value"):
            exec(compile(ast.Module([node], []), "transfusion.py", "exec"), helpers)
    z = np.load(os.path.join(out_dir, "ref_interleaved_n512_d64.npz"))
    q, k, v = (torch.from_numpy(z[n]).float() for n in "qkv")
    attn_mask = torch.from_numpy(np.unpackbits(z["dense_mask"], axis=-1)[..., :512].astype(bool))[:, 0]   # [b, i, j]
    scale = 64 ** -0.5
    res = {}
    for cap in (50.0, 4.0):
        sim = torch.einsum("bhid,bhjd->bhij", q * scale, k)
        sim = helpers["softclamp"](sim, cap)
        sim = torch.where(attn_mask[:, None], sim, torch.full_like(sim, helpers["max_neg_value"](sim)))
        attn = sim.softmax(dim=-1)
        res[f"out_cap{int(cap)}"] = torch.einsum("bhij,bhjd->bhid", attn, v).numpy()
        res[f"lse_cap{int(cap)}"] = torch.logsumexp(sim, dim=-1).numpy()
    np.savez(os.path.join(out_dir, "ref_softcap_interleaved_n512_d64.npz"), **res)
    print("ref_softcap_interleaved_n512_d64 saved (inputs and mask: ref_interleaved_n512_d64)")


if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    default = os.path.normpath(os.path.join(here, "..", "..", "..", "reference", "omni-attn-mma"))
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("OMNI_REFERENCE_DIR", default))
