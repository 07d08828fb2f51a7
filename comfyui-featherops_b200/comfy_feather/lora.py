"""Un-merged (low-VRAM) LoRA patches applied after the quantised linear: y += (x A^T) B^T * strength.

Same contract as the reference's comfy_feather/lora.py:4-35: `weight_functions` are ComfyUI low-VRAM patch objects with
`.patches` and `.key`; each patch tuple is (strength_patch, adapter, strength_model, offset, function) and the adapter
carries `.weights = (lora_B [N,r], lora_A [r,K], alpha | None, ...)`.  Anything else is rejected.
"""

import torch.nn.functional as F

_UNSUPPORTED = "FeatherOps currently only supports basic LoRA"


def _lora_terms(patch_fn):
    if not (hasattr(patch_fn, "patches") and hasattr(patch_fn, "key")):
        raise NotImplementedError(_UNSUPPORTED)
    for strength_patch, adapter, strength_model, *_ in patch_fn.patches.get(patch_fn.key, []):
        weights = getattr(adapter, "weights", None)
        if weights is None:
            raise NotImplementedError(_UNSUPPORTED)
        lora_b, lora_a, alpha = weights[0], weights[1], weights[2]
        strength = strength_patch * strength_model
        if alpha is not None:
            strength *= alpha / lora_a.shape[0]
        yield lora_a, lora_b, strength


def apply_lora_patches(x, y, weight_functions):
    for patch_fn in weight_functions:
        for lora_a, lora_b, strength in _lora_terms(patch_fn):
            down = F.linear(x, lora_a.to(device=x.device, dtype=x.dtype))
            up = F.linear(down, lora_b.to(device=x.device, dtype=x.dtype))
            y += up * strength
    return y
