"""bf16 -> fp16 conversion (reference: kernel/convert.py:24-34 `bf16_to_fp16`, a Triton kernel with RDNA inline asm).

Here it is a vectorised CUDA kernel in libfeather_b200; the result equals `x.to(torch.float16)` bit for bit
(round-to-nearest-even, overflow to inf).  Unlike the reference, an odd element count is accepted.
"""

import torch

from .b200 import native


def bf16_to_fp16(x: torch.Tensor) -> torch.Tensor:
    assert x.dtype == torch.bfloat16
    assert x.is_contiguous()
    return native.bf16_to_fp16(x)
