"""omni_attention_b200: block-mask ("omni") attention for NVIDIA B200 (sm_100a), forward and backward.

Public surface (mirrors the reference's operator module omni-attn-mma/omni_attn_torch.py):
  BlockMaskType, OmniBlockMask, build_partial_block_data, create_causal_omni_block_mask  - mask metadata
  omni_attention(q, k, v, block_mask, scale=None, return_lse=False)                        - the operator
  omni_attention_autograd(q, k, v, block_mask, scale=None)   - the same, differentiable (backward kernels;
                                                               the reference has no backward)
  install_reference_module()  - makes the `omni_attn` extension module (the reference's five pybind entry
                                points) importable, so the reference's own wrappers run on these kernels
"""
from .block_mask import (BlockMaskType, OmniBlockMask, block_mask_from_dense, block_mask_from_row_limits,
                         build_partial_block_data, create_causal_omni_block_mask,
                         create_omni_block_mask_from_modality_positions, dense_mask_from_blocks,
                         omni_block_mask_from_flex_block_mask, retile_block_mask,
                         row_limits_from_modality_positions)
from .ops import (OmniAttnError, omni_attention, omni_attention_autograd, omni_attention_backward_out,
                  omni_attention_forward_out, pack_partial_masks)

__all__ = [
    "BlockMaskType", "OmniBlockMask", "block_mask_from_dense", "block_mask_from_row_limits",
    "build_partial_block_data", "create_causal_omni_block_mask", "create_omni_block_mask_from_modality_positions",
    "dense_mask_from_blocks", "omni_block_mask_from_flex_block_mask", "retile_block_mask",
    "row_limits_from_modality_positions", "OmniAttnError", "omni_attention", "omni_attention_forward_out",
    "omni_attention_autograd", "omni_attention_backward_out",
    "pack_partial_masks", "install_reference_module",
]


def install_reference_module():
    """Import the in-tree `omni_attn` pybind module and register it in sys.modules under that name
    (the name omni-attn-mma/omni_attn_torch.py:539 imports)."""
    import importlib.util
    import os
    import sys
    import sysconfig

    import torch  # noqa: F401  (the extension links against libtorch)

    if "omni_attn" in sys.modules:
        return sys.modules["omni_attn"]
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "omni_attn" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
    if not os.path.exists(path):
        raise ImportError(f"{path} not found: build it with `python -m omni_attention_b200.build`")
    spec = importlib.util.spec_from_file_location("omni_attn", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["omni_attn"] = mod
    return mod
