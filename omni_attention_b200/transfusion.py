"""The slot the operator fills in the Transfusion model: the attention core of
``transfusion_pytorch.transfusion.Attention.forward`` (transfusion_pytorch/transfusion.py:953-983) and
the mask hook of ``Transformer.forward`` (:1108-1125).

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
