"""The slot the operator fills in the Transfusion model: the attention core of
``transfusion_pytorch.transfusion.Attention.forward`` (transfusion_pytorch/transfusion.py:953-983) and
the mask hook of ``Transformer.forward`` (:1108-1125).

``patch_attention(module)`` puts the kernels into a model: it replaces the ``forward`` of an attention
module that has the reference ``Attention``'s attributes with one that runs the same projections, value
residual, rotary, gates and output projection through the module's own sub-modules and hands the core
to ``transfusion_attention_core`` whenever the call brings an ``OmniBlockMask``.

In the reference model the core is either ``flex_attention(q, k, v, block_mask=...,
score_mod=softcap_score_mod(softcap_value))`` (:953-961) or, without FlexAttention, scaled q k^T ->
``softclamp`` (tanh soft-cap, :298-299, :967) -> mask -> softmax -> @ v (:963-983), both on
``[b, h, n, d]`` tensors produced by the projections' ``Rearrange`` (:858-866). The two functions
below are drop-ins for exactly those two places; nothing else of the model is rebuilt here.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .block_mask import OmniBlockMask, create_omni_block_mask_from_modality_positions
from .ops import omni_attention, omni_attention_autograd


def transfusion_block_mask(modality_positions: Tensor, heads: int, seq_len: int, device=None) -> OmniBlockMask:
    """Mask for a batch of interleaved sequences: ``modality_positions`` [b, m, 3] = (type, offset,
    length), the tensor ``modality_positions_to_tensor`` produces (:369-381). Built once per forward,
    like the model's own mask (:1108-1125); on a CUDA device it is built on the GPU."""
    device = modality_positions.device if device is None else device
    return create_omni_block_mask_from_modality_positions(modality_positions, modality_positions.shape[0], heads,
                                                          seq_len, seq_len, 128, 128, device)


def transfusion_attention_core(q: Tensor, k: Tensor, v: Tensor, block_mask: OmniBlockMask,
                               softcap_value: float = 50.0, scale: Optional[float] = None) -> Tensor:
    """``out = softmax(mask(softcap * tanh(q k^T * scale / softcap))) v`` on [b, h, n, d] CUDA tensors
    (fp16 / bf16, d in {64, 128}); ``scale`` defaults to d ** -0.5 (:851) and ``softcap_value`` to the
    model's 50 (:844); 0 switches the soft-cap off as in the model (:958)."""
    cap = softcap_value if softcap_value > 0 else None
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return omni_attention_autograd(q, k, v, block_mask, scale=scale, softcap=cap)   # training: backward kernels
    return omni_attention(q, k, v, block_mask, scale=scale, softcap=cap)


def _attention_forward_with_omni_core(module, original_forward):
    """The replacement ``forward``: the reference's argument list (transfusion_pytorch/transfusion.py:899-
    910) and, for a call with ``block_mask`` an OmniBlockMask and no kv cache, the reference's steps
    around the core (:921-950 before it, :987-1003 after it) on the module's own sub-modules, with the
    core itself (:953-983) computed by the kernels. Every other call (decoding with a cache, a dense
    ``attn_mask``, ``causal=True``, a flex BlockMask) goes to the module's original forward untouched."""

    def forward(x, attn_mask=None, rotary_emb=None, cache=None, causal=False, block_mask=None,
                return_kv_cache=False, return_values=False, value_residual=None):
        if not isinstance(block_mask, OmniBlockMask) or cache is not None or attn_mask is not None or causal:
            return original_forward(x, attn_mask=attn_mask, rotary_emb=rotary_emb, cache=cache, causal=causal,
                                    block_mask=block_mask, return_kv_cache=return_kv_cache, return_values=return_values,
                                    value_residual=value_residual)
        q, k = module.to_qk(x)
        v = module.to_v(x)
        orig_v = v
        if value_residual is not None:
            mix = module.to_learned_value_residual(x)
            v = v * mix + value_residual * (1.0 - mix)
        kv_cache = torch.stack((k, v)) if return_kv_cache else None
        if rotary_emb is not None:
            rotate = getattr(module, "apply_rotary", None)
            if rotate is None:
                raise ValueError("rotary_emb given: set module.apply_rotary(rotary_emb, t) to the model's rotary function "
                                 "(transfusion_pytorch/transfusion.py:941-942 calls apply_rotary_emb(rotary_emb, t, freqs_seq_dim=-2))")
            q, k = rotate(rotary_emb, q), rotate(rotary_emb, k)
        if getattr(module, "laser", False):
            v = ((v / module.laser_softclamp_value).tanh() * module.laser_softclamp_value).exp()
        dtype = q.dtype
        if dtype not in (torch.float16, torch.bfloat16):   # the kernels compute on 16-bit operands
            q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
        out = transfusion_attention_core(q.contiguous(), k.contiguous(), v.contiguous(), block_mask,
                                         softcap_value=float(module.softcap_value), scale=float(module.scale)).to(dtype)
        if getattr(module, "laser", False):
            out = out.log()
        if getattr(module, "to_gates", None) is not None:
            out = out * module.to_gates(x).sigmoid()
        out = module.to_out(out)
        if return_values:
            out = (out, orig_v)
        if not return_kv_cache:
            return out
        return out, kv_cache

    return forward


def patch_attention(module):
    """Swap the attention core of ``module`` for the kernels. ``module`` is the reference's
    ``transfusion_pytorch.transfusion.Attention`` or anything with the same attributes: ``to_qk`` (x ->
    q, k as [b, h, n, d]), ``to_v``, ``to_out``, ``scale``, ``softcap_value`` and, optionally,
    ``to_gates``, ``to_learned_value_residual``, ``laser`` / ``laser_softclamp_value``. Attention dropout
    is not applied by the kernels: a module whose ``dropout.p`` is non-zero in training mode is refused.
    The mask arrives through the ``block_mask`` argument the reference's forward already has, as an
    OmniBlockMask (``transfusion_block_mask``). Returns the module; ``unpatch_attention`` undoes it."""
    for name in ("to_qk", "to_v", "to_out", "scale", "softcap_value"):
        if not hasattr(module, name):
            raise TypeError(f"patch_attention: the module has no attribute {name!r}")
    drop = getattr(module, "dropout", None)
    if drop is not None and getattr(drop, "p", 0.0) > 0.0 and getattr(module, "training", False):
        raise ValueError("patch_attention: attention dropout is not supported by the kernels (set dropout to 0 or eval())")
    if hasattr(module, "_omni_original_forward"):
        return module
    module._omni_original_forward = module.forward
    module.forward = _attention_forward_with_omni_core(module, module._omni_original_forward)
    return module


def unpatch_attention(module):
    if hasattr(module, "_omni_original_forward"):
        module.forward = module._omni_original_forward
        del module._omni_original_forward
    return module
