"""`feather_ops(out_dtype, excluded_names)` -> a ComfyUI custom-operations class whose `Linear` keeps its weight as
prepacked fp8e5m2 and runs the sm_100a mixed-precision GEMM.

Same surface and behaviour as the reference's comfy_feather/ops.py:17-148 (state-dict loading with `weight_scale` /
legacy `scale_weight`, exclusion rules, `convert_weight` / `set_weight` for LoRA merging, un-merged LoRA patches),
with two differences in `forward`: the reference pads the token count up to a multiple of 16/32/64/128 with `F.pad`
(ops.py:126-139) because its kernel needs tile-divisible M; the B200 kernel handles ragged M itself, so no padded copy
is made and the rows beyond M never exist.  And the two dtype passes around the op (ops.py:88,103) are folded into the
GEMM launch for fp16 / bf16 inputs.
"""

import torch
import torch.nn.functional as F
from comfy.ops import cast_bias_weight, manual_cast, run_every_op, uncast_bias_weight
from torch import nn

from ..kernel.convert import bf16_to_fp16
from ..kernel.hip.hip_kernel import scaled_mm_b200, scaled_mm_lora
from .lora import apply_lora_patches, fused_lora_operands
from .quant import get_feather_plain_tensors, is_feather_quantized_weight, make_feather_quantized_weight, quantize_feather_weight


def feather_ops(out_dtype=torch.bfloat16, excluded_names=()):
    excluded_names = tuple(excluded_names)

    class FeatherOps(manual_cast):
        _excluded_names = excluded_names
        _out_dtype = out_dtype

        class Linear(manual_cast.Linear):
            def __init__(self, *args, **kwargs):
                super().__init__(*args, **kwargs)
                self.excluded_names = FeatherOps._excluded_names
                self.out_dtype = FeatherOps._out_dtype
                self.is_quantized = False

            def _keeps_plain_weight(self, prefix, weight):
                """True for layers that stay un-quantised: excluded by name, vectors, or K not a multiple of 16."""
                if any(name in prefix for name in self.excluded_names):
                    return True
                if self.in_features == 1 or self.out_features == 1 or weight.ndim == 1:
                    return True
                return self.in_features % 16 != 0

            def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
                weight = state_dict.pop(prefix + "weight", None)
                bias = state_dict.pop(prefix + "bias", None)
                weight_scale = state_dict.pop(prefix + "weight_scale", None)
                legacy_scale = state_dict.pop(prefix + "scale_weight", None)
                if weight_scale is None:
                    weight_scale = legacy_scale

                if weight is None:
                    missing_keys.append(prefix + "weight")
                elif self._keeps_plain_weight(prefix, weight):
                    if self.in_features % 16 != 0:
                        print(f"Warning: Not prepacked {prefix}weight {tuple(weight.shape)}")
                    self.is_quantized = False
                    self.weight = nn.Parameter(weight, requires_grad=False)
                else:
                    self.is_quantized = True
                    self.weight = nn.Parameter(make_feather_quantized_weight(weight, weight_scale, self.out_dtype), requires_grad=False)

                self.bias = nn.Parameter(bias.to(self.out_dtype), requires_grad=False) if bias is not None else None

            def convert_weight(self, weight, inplace=False, **kwargs):
                if not self.is_quantized:
                    return weight
                if not is_feather_quantized_weight(weight):
                    raise TypeError(f"Expected Feather quantized weight, got {type(weight).__name__}")
                return weight.dequantize()

            def set_weight(self, weight, inplace_update=False, seed=None, return_weight=False, **kwargs):
                if self.is_quantized:
                    weight = quantize_feather_weight(weight, seed=seed, inplace_ops=True)
                else:
                    weight = weight.to(self.weight.dtype)
                if return_weight:
                    return weight
                assert inplace_update is False
                self.weight = nn.Parameter(weight, requires_grad=False)

            def _forward_quantized(self, x, lora_functions=()):
                """x [M,K] any float dtype -> [M,N] in x's dtype, through the fp16/bf16 x e5m2 kernel.

                The reference casts the activations to fp16, runs the op and casts the result back (ops.py:88,103).  Here
                both casts happen inside the GEMM launch for 16-bit inputs: bf16 activations are multiplied as they are
                (bitwise the cast-first result for every value fp16 represents exactly; values beyond +-65504, which the
                cast would turn into inf, are multiplied unrounded), and the epilogue stores x's dtype after rounding to
                `out_dtype` and adding the bias in `out_dtype`, exactly the two roundings of `op(...).to(dtype)`.
                """
                dtype_orig = x.dtype
                x = x.contiguous()
                if x.dtype == torch.bfloat16 and x.is_cuda and x.shape[0] <= 16:
                    # a handful of tokens: the bandwidth-bound streaming kernel takes fp16, and the cast of M x K values is
                    # nothing (the library's cast kernel, kernel/convert.py:bf16_to_fp16 in the reference: same bits as `x.to`)
                    x = bf16_to_fp16(x)
                elif x.dtype not in (torch.float16, torch.bfloat16):
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

            def forward(self, input: torch.Tensor) -> torch.Tensor:
                x = input
                del input
                run_every_op()

                if not self.is_quantized:
                    weight, bias, offload_stream = cast_bias_weight(self, x, offloadable=True)
                    y = F.linear(x, weight, bias)
                    uncast_bias_weight(self, weight, bias, offload_stream)
                    return y

                batch_shape = x.shape[:-1]
                x = x.reshape(-1, x.shape[-1])
                if x.shape[0] == 0:
                    return x.new_empty(*batch_shape, self.out_features)

                y, lora_done = self._forward_quantized(x, self.weight_function)
                if not lora_done:
                    y = apply_lora_patches(x, y, self.weight_function)
                return y.view(*batch_shape, y.shape[-1])

    return FeatherOps
