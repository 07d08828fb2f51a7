"""torch-on-CPU restatement of the reference's kernel/naive.py op sequence.  TEST INFRASTRUCTURE / TIMED CPU BASELINE ONLY.

This is the "reference's naive torch CPU path" that bench.py times on the host cores (its cpu_baseline leg and its
`--impl reference` arm) and that tests compare with the numpy oracle.  It is never imported by the shipped package.

It follows kernel/naive.py:13-41 step for step - unpack (K/16,N,16) -> (K,N), upcast both operands to fp16, matmul,
`* scale` in fp32, cast to the output dtype, `+ bias` in the output dtype - with one switch: `product="fp32"` keeps
the matmul result in fp32 (operands are still the fp16 values), because the verbatim fp16 matmul result overflows to inf
at amax/57344 weight scales (naive.py:20-23 rounds the unscaled product to fp16).  `product="fp16"` is verbatim.
Parity: pinned through tests/test_oracle_golden.py and tests/test_cpu_baseline_port.py against the fixtures produced by
the reference itself.
"""

import torch


def unpack_weight(b_prepacked):
    """(K/16, N, 16) -> (K, N).   naive.py:13-16"""
    kb, n, _ = b_prepacked.shape
    return b_prepacked.permute(0, 2, 1).reshape(kb * 16, n)


def scaled_mm_cpu(a, b_prepacked, scale, bias, out_dtype, product="fp32"):
    w = unpack_weight(b_prepacked).to(torch.float16)            # naive.py:22
    a = a.to(torch.float16)                                     # naive.py:21
    if product == "fp16":
        c = a @ w                                               # naive.py:23
    else:
        c = a.to(torch.float32) @ w.to(torch.float32)
    if scale is not None:
        c = c.to(torch.float32)
        c *= scale.to(torch.float32)                            # naive.py:24-28
    c = c.to(out_dtype)                                         # naive.py:34
    if bias is not None:
        c += bias.to(c.dtype)[None, :]                          # naive.py:35-40
    return c


def quantize_prepack_cpu(w):
    """fp32/bf16/fp16 (N,K) -> ((K/16,N,16) e5m2, fp32 scale): quant.py:52-74 + 11-13 with torch ops (timed baseline
    of the quantise+prepack step)."""
    scale = torch.amax(w.abs()).to(torch.float32) / 57344.0
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    if w.dtype == torch.float16:
        scale = 1.0 / torch.clamp(1.0 / scale, min=-65504.0, max=65504.0)
    q = (w * (1.0 / scale).to(w.dtype)).to(torch.float8_e5m2)
    n, k = q.shape
    return q.view(n, k // 16, 16).permute(1, 0, 2).contiguous(), scale
