"""`feather_ops(out_dtype, excluded_names)` -> a ComfyUI custom-operations class whose `Linear` keeps its weight as
prepacked fp8e5m2 and runs the sm_100a mixed-precision GEMM.

Same surface and behaviour as the reference's comfy_feather/ops.py:17-148 (state-dict loading with `weight_scale` /
legacy `scale_weight`, exclusion rules, `convert_weight` / `set_weight` for LoRA merging, un-merged LoRA patches),
with two differences in `forward`: the reference pads the token count up to a multiple of 16/32/64/128 with `F.pad`
(ops.py:126-139) because its kernel needs tile-divisible M; the B200 kernel handles ragged M itself, so no padded copy
is made and the rows beyond M never exist.  And the cast of the result back to the model's dtype (ops.py:103) is folded
into the GEMM's epilogue.
"""

import torch
import torch.nn.functional as F
from comfy.ops import cast_bias_weight, manual_cast, run_every_op, uncast_bias_weight
from torch import nn

from ..kernel.convert import bf16_to_fp16
from ..kernel.hip.hip_kernel import scaled_mm_b200, scaled_mm_lora
from .lora import apply_lora_patches, fused_lora_operands
from .quant import get_feather_plain_tensors, is_feather_quantized_weight, make_feather_quantized_weight, quantize_feather_weight


def _frozen(tensor):
    return nn.Parameter(tensor, requires_grad=False)


_STATE_KEYS = ("weight", "bias", "weight_scale", "scale_weight")       # `scale_weight` is the legacy name of `weight_scale`


class _FeatherLinear:
    """Methods of the `Linear` below; `excluded_names` and `out_dtype` are class attributes of the class `feather_ops` builds."""

    excluded_names = ()
    out_dtype = torch.bfloat16

    # ------------------------------------------------------------------ loading and LoRA merging
    def _keeps_plain_weight(self, prefix, weight):
        """True for layers that stay un-quantised: excluded by name, vectors, or K not a multiple of 16."""
        if any(name in prefix for name in self.excluded_names):
            return True
        if self.in_features == 1 or self.out_features == 1 or weight.ndim == 1:
            return True
        return self.in_features % 16 != 0

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        weight, bias, weight_scale, legacy_scale = (state_dict.pop(prefix + key, None) for key in _STATE_KEYS)
        if weight is None:
            missing_keys.append(prefix + "weight")
        else:
            self.is_quantized = not self._keeps_plain_weight(prefix, weight)
            if self.is_quantized:
                scale = weight_scale if weight_scale is not None else legacy_scale
                weight = make_feather_quantized_weight(weight, scale, self.out_dtype)
            elif self.in_features % 16 != 0:
                print(f"Warning: Not prepacked {prefix}weight {tuple(weight.shape)}")
            self.weight = _frozen(weight)
        self.bias = None if bias is None else _frozen(bias.to(self.out_dtype))

    def convert_weight(self, weight, inplace=False, **kwargs):
        """The weight a LoRA merge works on: the dequantised matrix of a quantised layer."""
        if self.is_quantized and not is_feather_quantized_weight(weight):
            raise TypeError(f"Expected Feather quantized weight, got {type(weight).__name__}")
        return weight.dequantize() if self.is_quantized else weight

    def set_weight(self, weight, inplace_update=False, seed=None, return_weight=False, **kwargs):
        """Takes the merged matrix back: requantised (scale recalculated) for a quantised layer."""
        merged = quantize_feather_weight(weight, seed=seed, inplace_ops=True) if self.is_quantized else weight.to(self.weight.dtype)
        if return_weight:
            return merged
        assert inplace_update is False
        self.weight = _frozen(merged)

    # ------------------------------------------------------------------ forward
    def forward(self, input: torch.Tensor) -> torch.Tensor:
        run_every_op()
        if not self.is_quantized:
            return self._forward_plain(input)
        lead = input.shape[:-1]
        x = input.reshape(-1, input.shape[-1])
        if x.shape[0] == 0:
            return x.new_empty(*lead, self.out_features)
        y, lora_done = self._forward_quantized(x, self.weight_function)
        if not lora_done:
            y = apply_lora_patches(x, y, self.weight_function)
        return y.view(*lead, y.shape[-1])

    def _forward_plain(self, x):
        weight, bias, offload_stream = cast_bias_weight(self, x, offloadable=True)
        try:
            return F.linear(x, weight, bias)
        finally:
            uncast_bias_weight(self, weight, bias, offload_stream)

    def _forward_quantized(self, x, lora_functions=()):
        """x [M,K] any float dtype -> ([M,N] in x's dtype, whether the LoRA patches are already in it), through the
        fp16/bf16 x e5m2 kernel.

        The reference casts the activations to fp16, runs the op and casts the result back (ops.py:88,103).  Here the
        cast back happens in the GEMM's epilogue: it stores x's dtype after rounding to `out_dtype` and adding the bias
        in `out_dtype`, exactly the two roundings of `op(...).to(dtype)`.  bf16 activations go through the library's
        cast kernel first (kernel/convert.py:bf16_to_fp16 in the reference: same bits as `x.to`): the GEMM can also
        multiply bf16 activations as they are (`scaled_mm_b200` with a bf16 `a`), but its weights then have to be
        upcast to bf16 as well, and cast + fp16 GEMM measured 6-14 % faster from 256 to 32768 tokens on the Wan shapes
        (and is the only form the streaming kernel for a handful of tokens takes).
        """
        dtype_orig = x.dtype
        x = x.contiguous()
        if x.dtype == torch.bfloat16 and x.is_cuda:
            x = bf16_to_fp16(x)
        elif x.dtype != torch.float16:
            x = x.to(torch.float16)
        final_dtype = dtype_orig if dtype_orig in (torch.float16, torch.bfloat16) else self.out_dtype

        # cast_bias_weight must not apply low-VRAM LoRA patches to the prepacked weight
        saved_weight_function = self.weight_function
        self.weight_function = []
        try:
            bias_dtype = self.bias.dtype if self.bias is not None else None
            weight, bias, offload_stream = cast_bias_weight(self, x, dtype=self.weight.dtype, bias_dtype=bias_dtype, offloadable=True)
            qdata, scale = get_feather_plain_tensors(weight)
            scale = scale.to(device=x.device, dtype=torch.float32)
            # un-merged LoRA patches: folded into this GEMM's accumulator when that pays (see lora.py), else added afterwards
            fused = fused_lora_operands(x, lora_functions, scale) if lora_functions else None
            if fused is not None:
                y = scaled_mm_lora(x, qdata, scale, bias, self.out_dtype, final_dtype, *fused)
            else:
                y = scaled_mm_b200(x, qdata, scale, bias, out_dtype=self.out_dtype, final_dtype=final_dtype)
            uncast_bias_weight(self, weight, bias, offload_stream)
        finally:
            self.weight_function = saved_weight_function
        y = y if y.dtype == dtype_orig else y.to(dtype_orig)
        return y, fused is not None


def feather_ops(out_dtype=torch.bfloat16, excluded_names=()):
    """The operations class ComfyUI instantiates the model with: `manual_cast` whose `Linear` is the quantised linear."""
    names, dtype = tuple(excluded_names), out_dtype

    class FeatherOps(manual_cast):
        _excluded_names, _out_dtype = names, dtype

        class Linear(_FeatherLinear, manual_cast.Linear):
            excluded_names = names
            out_dtype = dtype

            def __init__(self, *args, **kwargs):
                super().__init__(*args, **kwargs)
                self.is_quantized = False

    return FeatherOps
