"""The slot the kernels fill in the Transfusion model (transfusion_pytorch/transfusion.py:891-1005): the
soft-capped attention core against goldens written from the reference's own softclamp, and
``patch_attention`` on a module with the reference Attention's attributes against the oracle's
restatement of that module's forward.

Tolerances (conftest.py): output atol 2e-2 / rtol 1e-2, log-sum-exp 1e-3.
"""
import os

import numpy as np
import pytest
import torch
from torch import nn

from conftest import GOLDEN_DIR, assert_parity, load_golden
from omni_attention_b200.block_mask import create_omni_block_mask_from_modality_positions
from omni_attention_b200.ops import omni_attention
from omni_attention_b200.transfusion import patch_attention, transfusion_block_mask, unpatch_attention
from oracle import omni_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cap", [50, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_softcap_core_against_the_reference_core_golden(cuda_device, cap, dtype):
    g = load_golden("ref_interleaved_n512_d64")
    z = np.load(os.path.join(GOLDEN_DIR, "ref_softcap_interleaved_n512_d64.npz"))
    q, k, v = (g[x].to(dtype) for x in "qkv")
    if dtype == torch.float16:
        ref_out, ref_lse = torch.from_numpy(z[f"out_cap{cap}"]), torch.from_numpy(z[f"lse_cap{cap}"])
    else:   # bf16 inputs: the pinned oracle on the rounded values
        ref_out, ref_lse = orc.attention_dense_mask(q.float(), k.float(), v.float(), orc.to_score_mask(g["dense"]),
                                                    softcap=float(cap))
    dev = cuda_device
    out, lse = omni_attention(q.to(dev), k.to(dev), v.to(dev), g["bm"], return_lse=True, check_status=True, softcap=float(cap))
    assert_parity(out, lse, ref_out, ref_lse, f"softcap {cap} {dtype}")


class AttentionLike(nn.Module):
    """A module with the attribute surface of the reference's Attention (transfusion.py:837-897): the
    same projections and parameters under the same names, written with plain reshapes."""

    def __init__(self, dim, dim_head, heads, softcap_value=50.0, gate_values=True, learned_mix=True):
        super().__init__()
        self.heads, self.dim_head = heads, dim_head
        self.scale = dim_head ** -0.5
        self.softcap_value = softcap_value
        self.laser, self.laser_softclamp_value = False, 15.0
        self.qk = nn.Linear(dim, 2 * heads * dim_head, bias=False)
        self.vproj = nn.Linear(dim, heads * dim_head, bias=False)
        self.mix = nn.Linear(dim, heads) if learned_mix else None
        self.gates = nn.Linear(dim, heads, bias=False) if gate_values else None
        self.out = nn.Linear(heads * dim_head, dim, bias=False)
        self.dropout = nn.Dropout(0.0)
        self.to_gates = (lambda x: self.gates(x).transpose(1, 2).unsqueeze(-1)) if gate_values else None

    def to_qk(self, x):
        b, n, _ = x.shape
        t = self.qk(x).view(b, n, 2, self.heads, self.dim_head).permute(2, 0, 3, 1, 4)
        return t[0], t[1]

    def to_v(self, x):
        b, n, _ = x.shape
        return self.vproj(x).view(b, n, self.heads, self.dim_head).transpose(1, 2)

    def to_learned_value_residual(self, x):
        if self.mix is None:
            return 0.5
        return self.mix(x).sigmoid().transpose(1, 2).unsqueeze(-1)

    def to_out(self, o):
        b, h, n, d = o.shape
        return self.out(o.transpose(1, 2).reshape(b, n, h * d))

    def forward(self, x, attn_mask=None, rotary_emb=None, cache=None, causal=False, block_mask=None,
                return_kv_cache=False, return_values=False, value_residual=None):
        raise AssertionError("the original forward must not run for a call that brings an OmniBlockMask")


@pytest.mark.parametrize("dim_head,softcap", [(64, 50.0), (128, 4.0)])
def test_patch_attention_against_the_oracles_attention_forward(cuda_device, dim_head, softcap):
    torch.manual_seed(5)
    dev = cuda_device
    b, n, dim, heads = 2, 700, 256, 4
    mod = AttentionLike(dim, dim_head, heads, softcap_value=softcap)
    x = torch.randn(b, n, dim)
    value_residual = torch.randn(b, heads, n, dim_head)
    mp = torch.tensor([[[1, 60, 200], [1, 400, 130]], [[1, 0, 128], [1, 300, 257]]], dtype=torch.int32)
    attn_mask = orc.naive_attn_mask(n, mp)                                         # [b, i, j], the model's dense mask
    expect = orc.transfusion_attention_forward(mod, x, attn_mask=attn_mask, value_residual=value_residual)

    gpu = patch_attention(AttentionLike(dim, dim_head, heads, softcap_value=softcap)).to(dev)
    gpu.load_state_dict(mod.state_dict())
    gpu = gpu.half()
    bm = transfusion_block_mask(mp.to(dev), heads, n)
    got, values = gpu(x.to(dev).half(), block_mask=bm, value_residual=value_residual.to(dev).half(), return_values=True)
    assert got.shape == expect.shape and values.shape == (b, heads, n, dim_head)
    assert_parity(got, None, expect.detach(), None, f"patched attention d={dim_head}")
    # without an OmniBlockMask the call goes to the module's own forward
    with pytest.raises(AssertionError, match="original forward"):
        gpu(x.to(dev).half())
    unpatch_attention(gpu)
    assert not hasattr(gpu, "_omni_original_forward")


def test_patch_attention_trains(cuda_device):
    """Gradients flow through the patched core (backward kernels) into the module's parameters."""
    torch.manual_seed(6)
    dev = cuda_device
    b, n, dim, heads, dh = 1, 384, 128, 2, 64
    mod = AttentionLike(dim, dh, heads, gate_values=False, learned_mix=False)
    x = torch.randn(b, n, dim)
    mp = torch.tensor([[[1, 100, 150]]], dtype=torch.int32)
    attn_mask = orc.naive_attn_mask(n, mp)
    ref = orc.transfusion_attention_forward(mod, x, attn_mask=attn_mask)
    ref.square().sum().backward()
    want = mod.qk.weight.grad.clone()

    gpu = patch_attention(AttentionLike(dim, dh, heads, gate_values=False, learned_mix=False)).to(dev)
    gpu.load_state_dict(mod.state_dict())
    bm = create_omni_block_mask_from_modality_positions(mp.to(dev), b, heads, n, n, 128, 128, dev)
    out = gpu(x.to(dev), block_mask=bm)             # fp32 module: the core runs on bf16 copies
    out.float().square().sum().backward()
    got = gpu.qk.weight.grad.float().cpu()
    assert float((got - want).abs().max()) <= 3e-2 * float(want.abs().max())
