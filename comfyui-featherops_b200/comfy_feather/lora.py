"""Un-merged (low-VRAM) LoRA patches of the quantised linear: y += (x A^T) B^T * strength.

Same contract as the reference's comfy_feather/lora.py:4-35: `weight_functions` are ComfyUI low-VRAM patch objects with
`.patches` and `.key`; each patch tuple is (strength_patch, adapter, strength_model, offset, function) and the adapter
carries `.weights = (lora_B [N,r], lora_A [r,K], alpha | None, ...)`.  Anything else is rejected.

Two ways to apply them.  `apply_lora_patches` is the reference's: two GEMMs and a read-modify-write of the whole [M, N]
output per patch, after the linear.  `fused_lora_operands` prepares the operands that let the linear's own GEMM add the
term inside its accumulator (`scaled_mm_lora` in kernel/hip/hip_kernel.py): one skinny GEMM for the down-projections of
all patches, and the up-projection runs as a few extra k-blocks of the main kernel - the output is written once.
"""

import torch
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


# fewer tokens than this and the un-fused path is as good: the read-modify-write of M x N values is small, and up to 16
# tokens the linear runs the streaming kernel, which has no low-rank blocks
FUSED_LORA_MIN_TOKENS = 64
FUSED_LORA_MAX_RANK = 1024


def fused_lora_operands(x, weight_functions, weight_scale):
    """(t, lb_prepacked) for `scaled_mm_lora`, or None when there is no patch or fusing does not pay.

    x [M, K] fp16 / bf16 on the GPU (the activations the GEMM will see); weight_scale: fp32 one-element tensor, the scale of
    the quantised weight.  The GEMM computes (x W + t lb^T) * scale, so lb carries strength / scale; a power of two alpha
    moves t up and lb down so that both fit fp16 (|t| <= 16384), which both are whatever x's dtype - the kernel runs the
    low-rank blocks as fp16 x fp16 MMAs, so the term keeps 11 significant bits per operand also in a bf16 model:
        t  = (x A^T) * alpha                                [M, R]    A = all patches' lora_A stacked, R padded to a multiple of 64
        lb = B * strength / (scale * alpha), prepacked      [R/8, N, 8]
    Everything stays on the device (no synchronisation)."""
    terms = [t for patch_fn in weight_functions for t in _lora_terms(patch_fn)]
    if not terms or x.shape[0] < FUSED_LORA_MIN_TOKENS or not x.is_cuda or x.dtype not in (torch.float16, torch.bfloat16):
        return None
    rank = sum(a.shape[0] for a, _, _ in terms)
    if rank > FUSED_LORA_MAX_RANK:
        return None
    dev, dt = x.device, x.dtype
    a_cat = torch.cat([a.to(device=dev, dtype=dt) for a, _, _ in terms], dim=0)                                  # [R, K]
    b_cat = torch.cat([b.to(device=dev, dtype=torch.float32) * float(s) for _, b, s in terms], dim=1)             # [N, R] with the strengths
    pad = (-rank) % 64
    if pad:
        a_cat = F.pad(a_cat, (0, 0, 0, pad))
        b_cat = F.pad(b_cat, (0, pad))
    try:                                                                                                         # [M, R]: a plain library GEMM,
        down = torch.mm(x, a_cat.t(), out_dtype=torch.float32)                                                   # kept in fp32 where torch can
    except (TypeError, RuntimeError):
        down = F.linear(x, a_cat).float()
    amax = down.abs().amax().clamp_min(1e-30)
    alpha = torch.exp2(torch.floor(torch.log2(16384.0 / amax))).clamp(2.0 ** -24, 2.0 ** 24)                      # power of two: the scaling of t is exact
    t = (down * alpha).to(torch.float16).contiguous()
    lb = (b_cat / (weight_scale.to(device=dev, dtype=torch.float32).reshape(()) * alpha)).to(torch.float16)       # [N, R], one rounding
    n, r = lb.shape
    lb_prepacked = lb.view(n, r // 8, 8).permute(1, 0, 2).contiguous()                                           # [R/8, N, 8]
    return t, lb_prepacked
