"""Operator surface of the mixed-precision linear, same names and signatures as the reference's
kernel/hip/hip_kernel.py (the module path is kept so `comfy_feather/ops.py` and the reference's test and benchmark
scripts import it unchanged), routed to the sm_100a library instead of the HIP extension.

    scaled_mm_hip(a, b_prepacked, scale, bias, out_dtype)                      hip_kernel.py:136-167
    scaled_mm_hip_configured(a, b_prepacked, scale, bias, out_dtype, *cfg5)    hip_kernel.py:12-58
    _CONFIGS                                                                   hip_kernel.py:60-93
    prepack_b_for_scaled_mm(b)                                                 hip_kernel.py:170-171
    torch.ops.feather_ops.scaled_mm(a, b, scale, bias, c, 5 ints, b_dtype)     hip_kernel.cu:746-767

    torch.ops.feather_ops_internal.scaled_mm_autotuned(...)                    hip_kernel.py:95-133 (the op torch.compile sees)

Differences a caller can observe: the five tile integers are accepted and ignored (the kernel variant is chosen from
the shape, so there is no first-call autotune pause and nothing for inductor to tune); M does not have to be a multiple of
any tile (ragged token counts are handled in the kernel); fp8e4m3fn weights are upcast exactly (subnormals and NaN codes
included; the reference's kernel approximates them, hip_kernel.cu:83-99).

One addition: `scaled_mm_b200(a, b_prepacked, scale, bias, out_dtype, final_dtype)` takes bf16 activations as they are
and can store the other 16-bit dtype, which removes the two elementwise passes the reference's `FeatherOps.Linear.forward`
runs around the GEMM (comfy_feather/ops.py:88,103).
"""

import torch

from ..b200 import native

# The reference's 28 tile configs, kept so scripts that iterate `_CONFIGS` keep working.  (warps_m, warps_n,
# unroll_k, repeat_m, repeat_n); every entry maps to the same shape-driven variant here.
_CONFIGS = sorted(
    [
        (1, 1, 2, 1, 2), (1, 1, 4, 1, 2), (1, 2, 2, 1, 2), (1, 2, 4, 1, 2), (1, 4, 2, 1, 2), (1, 4, 4, 1, 2), (1, 8, 2, 1, 2),
        (1, 8, 4, 1, 2), (1, 1, 2, 2, 2), (1, 1, 4, 2, 2), (1, 1, 2, 4, 4), (1, 1, 4, 4, 4), (1, 2, 2, 2, 2), (1, 2, 4, 2, 2),
        (2, 1, 2, 2, 2), (2, 1, 4, 2, 2), (1, 4, 2, 4, 2), (1, 4, 4, 4, 2), (1, 8, 2, 8, 2), (1, 8, 4, 8, 2), (2, 2, 2, 4, 4),
        (2, 2, 4, 4, 4), (2, 4, 2, 4, 2), (2, 4, 4, 4, 2), (2, 4, 2, 4, 4), (2, 4, 4, 4, 4), (4, 2, 2, 2, 4), (4, 2, 4, 2, 4),
    ],
    key=lambda x: (x[0], x[1], x[3], x[4], x[2]),
)  # fmt: skip


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _validate(a, b_prepacked, scale, bias, c, b_dtype, allow_bf16_a=False, bias_dtype=None):
    """Argument checks of the reference op (hip_kernel.cu:648-730), minus tile divisibility of M and N.

    Written as plain `if` statements so that a message is only formatted when its check fails: this runs on every call and
    a small-M GEMM takes less time on the GPU than thirty formatted strings take on the host."""
    if not (a.is_cuda):
        raise RuntimeError("a must be a CUDA tensor")
    if not (b_prepacked.is_cuda):
        raise RuntimeError("b_prepacked must be a CUDA tensor")
    if not (c.is_cuda):
        raise RuntimeError("c must be a CUDA tensor")
    if not (b_prepacked.device == a.device):
        raise RuntimeError("b_prepacked must be on the same device as a")
    if not (c.device == a.device):
        raise RuntimeError("c must be on the same device as a")
    if not (a.dtype == torch.float16 or (allow_bf16_a and a.dtype == torch.bfloat16)):
        raise RuntimeError("a must be float16")
    if not (c.dtype in (torch.float16, torch.bfloat16)):
        raise RuntimeError("c must be float16 or bfloat16")
    if not (b_dtype in (0, 1)):
        raise RuntimeError("b_dtype must be 0 (fp8e4m3) or 1 (fp8e5m2)")
    if b_dtype == 1 and not (b_prepacked.dtype == torch.float8_e5m2):
        raise RuntimeError("b_prepacked must be float8_e5m2 when b_dtype=1")
    if b_dtype == 0 and not (b_prepacked.dtype == torch.float8_e4m3fn):
        raise RuntimeError("b_prepacked must be float8_e4m3fn when b_dtype=0")
    if not (a.dim() == 2):
        raise RuntimeError("a must be 2D")
    if not (b_prepacked.dim() == 3):
        raise RuntimeError("b_prepacked must be 3D (K/16, N, 16)")
    if not (c.dim() == 2):
        raise RuntimeError("c must be 2D")
    M, K = a.shape
    N = b_prepacked.shape[1]
    if not (K % 16 == 0):
        raise RuntimeError("K must be divisible by 16")
    if not (b_prepacked.shape[0] == K // 16):
        raise RuntimeError(f"b_prepacked.shape[0] must equal K/16 ({K // 16})")
    if not (b_prepacked.shape[2] == 16):
        raise RuntimeError("b_prepacked.shape[2] must be 16")
    if not (c.shape[0] == M):
        raise RuntimeError("c.shape[0] must equal M")
    if not (c.shape[1] == N):
        raise RuntimeError("c.shape[1] must equal N")
    if not (a.stride(0) == K or M <= 1):
        raise RuntimeError(f"a.stride(0) must equal K ({K})")
    if not (a.stride(1) == 1):
        raise RuntimeError("a.stride(1) must be 1")
    if not (b_prepacked.stride(0) == N * 16 or K == 16):
        raise RuntimeError(f"b_prepacked.stride(0) must equal N*16 ({N * 16})")
    if not (b_prepacked.stride(1) == 16):
        raise RuntimeError("b_prepacked.stride(1) must be 16")
    if not (b_prepacked.stride(2) == 1):
        raise RuntimeError("b_prepacked.stride(2) must be 1")
    if not (c.stride(0) >= N or M <= 1):
        raise RuntimeError(f"c.stride(0) must be at least N ({N})")
    if not (c.stride(1) == 1):
        raise RuntimeError("c.stride(1) must be 1")
    if scale is not None:
        if not (scale.is_cuda):
            raise RuntimeError("scale must be a CUDA tensor")
        if not (scale.device == a.device):
            raise RuntimeError("scale must be on the same device as a")
        if not (scale.dtype == torch.float32):
            raise RuntimeError("scale must be float32")
        if not (scale.numel() == 1):
            raise RuntimeError("scale must have one element")
    if bias is not None:
        if not (bias.is_cuda):
            raise RuntimeError("bias must be a CUDA tensor")
        if not (bias.device == a.device):
            raise RuntimeError("bias must be on the same device as a")
        if not (bias.dtype == (c.dtype if bias_dtype is None else bias_dtype)):
            raise RuntimeError("bias must have the same dtype as c" if bias_dtype is None else "bias must have the out dtype")
        if not (bias.numel() == N):
            raise RuntimeError("bias must have N elements")
        if not (bias.is_contiguous()):
            raise RuntimeError("bias must be contiguous")
    if not (a.data_ptr() % 16 == 0):
        raise RuntimeError("a data pointer must be 16-byte aligned")
    if not (b_prepacked.data_ptr() % 16 == 0):
        raise RuntimeError("b_prepacked data pointer must be 16-byte aligned")


# ------------------------------------------------------------------------------------------------
# torch.ops.feather_ops.scaled_mm: same schema as the reference's stable-ABI op (out-parameter convention).
# ------------------------------------------------------------------------------------------------
_lib_def = torch.library.Library("feather_ops", "DEF")
_lib_def.define(
    "scaled_mm(Tensor a, Tensor b_prepacked, Tensor? scale, Tensor? bias, Tensor(a!) c, int block_warps_m, int block_warps_n, "
    "int unroll_k, int repeat_m, int repeat_n, int b_dtype) -> ()"
)


def _scaled_mm_cuda(a, b_prepacked, scale, bias, c, block_warps_m, block_warps_n, unroll_k, repeat_m, repeat_n, b_dtype):
    _validate(a, b_prepacked, scale, bias, c, b_dtype)
    if a.shape[0] == 0:
        return
    if b_dtype == 1:
        native.scaled_mm_into(a, b_prepacked, scale, bias, c)
    else:
        native.scaled_mm_typed_into(a, b_prepacked, scale, bias, c)


_lib_impl = torch.library.Library("feather_ops", "IMPL")
_lib_impl.impl("scaled_mm", _scaled_mm_cuda, "CUDA")


def _scaled_mm_meta(a, b_prepacked, scale, bias, c, block_warps_m, block_warps_n, unroll_k, repeat_m, repeat_n, b_dtype):
    return None


_lib_impl.impl("scaled_mm", _scaled_mm_meta, "Meta")


@torch.library.custom_op("feather_ops_internal::scaled_mm_configured", mutates_args=())
def _configured_op(
    a: torch.Tensor,
    b_prepacked: torch.Tensor,
    scale: torch.Tensor | None,
    bias: torch.Tensor | None,
    out_dtype: torch.dtype,
    block_warps_m: int,
    block_warps_n: int,
    unroll_k: int,
    repeat_m: int,
    repeat_n: int,
) -> torch.Tensor:
    out = torch.empty((a.shape[0], b_prepacked.shape[1]), device=a.device, dtype=out_dtype)
    torch.ops.feather_ops.scaled_mm.default(
        a, b_prepacked, scale, bias, out, block_warps_m, block_warps_n, unroll_k, repeat_m, repeat_n,
        0 if b_prepacked.dtype == torch.float8_e4m3fn else 1,
    )  # fmt: skip
    return out


@_configured_op.register_fake
def _(a, b_prepacked, scale, bias, out_dtype, block_warps_m, block_warps_n, unroll_k, repeat_m, repeat_n):
    return torch.empty((a.shape[0], b_prepacked.shape[1]), device=a.device, dtype=out_dtype)


scaled_mm_hip_configured = _configured_op


# The op the reference hands to torch.compile (hip_kernel.py:95-133): scale and bias always tensors plus two flags, the five
# tile integers optional.  The reference registers it with inductor's custom-op autotuning over its 28 tile configs; here
# the variant follows from the shape inside the library, so there is nothing to tune and the op forwards to the configured
# op.  Kept so graphs and scripts that name `feather_ops_internal::scaled_mm_autotuned` keep working.
@torch.library.custom_op("feather_ops_internal::scaled_mm_autotuned", mutates_args=())
def _autotuned_op(
    a: torch.Tensor,
    b_prepacked: torch.Tensor,
    scale: torch.Tensor,
    bias: torch.Tensor,
    out_dtype: torch.dtype,
    has_scale: bool,
    has_bias: bool,
    block_warps_m: int = 0,
    block_warps_n: int = 0,
    unroll_k: int = 0,
    repeat_m: int = 0,
    repeat_n: int = 0,
) -> torch.Tensor:
    return _configured_op(a, b_prepacked, scale if has_scale else None, bias if has_bias else None, out_dtype, *_DEFAULT_CFG)


@_autotuned_op.register_fake
def _(a, b_prepacked, scale, bias, out_dtype, has_scale, has_bias, block_warps_m=0, block_warps_n=0, unroll_k=0, repeat_m=0, repeat_n=0):
    return torch.empty((a.shape[0], b_prepacked.shape[1]), device=a.device, dtype=out_dtype)


# bf16 or fp16 activations in, either 16-bit dtype out: one launch, no elementwise pass before or after it.
def _typed_impl(a, b_prepacked, scale, bias, out_dtype, final_dtype):
    if final_dtype not in (torch.float16, torch.bfloat16) or out_dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("out_dtype and final_dtype must be float16 or bfloat16")
    out = torch.empty((a.shape[0], b_prepacked.shape[1]), device=a.device, dtype=final_dtype)
    _validate(a, b_prepacked, scale, bias, out, 0 if b_prepacked.dtype == torch.float8_e4m3fn else 1, allow_bf16_a=True, bias_dtype=out_dtype)
    if a.shape[0] != 0:
        native.scaled_mm_typed_into(a, b_prepacked, scale, bias, out, out_dtype=out_dtype)
    return out


@torch.library.custom_op("feather_ops_internal::scaled_mm_b200", mutates_args=())
def _typed_op(
    a: torch.Tensor,
    b_prepacked: torch.Tensor,
    scale: torch.Tensor | None,
    bias: torch.Tensor | None,
    out_dtype: torch.dtype,
    final_dtype: torch.dtype,
) -> torch.Tensor:
    return _typed_impl(a, b_prepacked, scale, bias, out_dtype, final_dtype)


@_typed_op.register_fake
def _(a, b_prepacked, scale, bias, out_dtype, final_dtype):
    return torch.empty((a.shape[0], b_prepacked.shape[1]), device=a.device, dtype=final_dtype)


def scaled_mm_b200(a, b_prepacked, scale, bias, out_dtype, final_dtype=None):
    """`scaled_mm_hip` with the casts around it folded in: `a` may be bf16 (multiplied as it is; equals casting it to fp16
    first for every value fp16 represents exactly), and the result is stored as `final_dtype` (default `out_dtype`) after
    the rounding to `out_dtype` and the bias add in `out_dtype` - the bits `scaled_mm_hip(...).to(final_dtype)` gives."""
    final_dtype = out_dtype if final_dtype is None else final_dtype
    if torch.compiler.is_compiling():
        return _typed_op(a, b_prepacked, scale, bias, out_dtype, final_dtype)
    return _typed_impl(a, b_prepacked, scale, bias, out_dtype, final_dtype)

_DEFAULT_CFG = (1, 8, 4, 8, 2)


def scaled_mm_hip(
    a: torch.Tensor,
    b_prepacked: torch.Tensor,
    scale: torch.Tensor | None,
    bias: torch.Tensor | None,
    out_dtype: torch.dtype,
) -> torch.Tensor:
    """C = cvt((a @ up(b_prepacked)) * scale) + bias.  a fp16 [M,K]; b_prepacked e5m2 [K/16,N,16]; returns [M,N].

    Under torch.compile the call stays one opaque custom op (with a fake implementation for shape inference);
    in eager mode it validates, allocates the output and launches, with no autotune step.
    """
    if torch.compiler.is_compiling():
        # the op name the reference's compiled graphs carry (hip_kernel.py:143-152)
        return _autotuned_op(a, b_prepacked, scale if scale is not None else a, bias if bias is not None else a, out_dtype,
                             scale is not None, bias is not None)
    out = torch.empty((a.shape[0], b_prepacked.shape[1]), device=a.device, dtype=out_dtype)
    _scaled_mm_cuda(a, b_prepacked, scale, bias, out, *_DEFAULT_CFG, 0 if b_prepacked.dtype == torch.float8_e4m3fn else 1)
    return out


def scaled_mm_lora(a, b_prepacked, scale, bias, out_dtype, final_dtype, t, lb_prepacked):
    """`scaled_mm_b200` with an un-merged LoRA term folded into the accumulator: returns
    cast(cvt((a @ up(b) + t @ lb^T) * scale) + bias).  t and lb_prepacked come from comfy_feather/lora.py:fused_lora_operands."""
    final_dtype = out_dtype if final_dtype is None else final_dtype
    if final_dtype not in (torch.float16, torch.bfloat16) or out_dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("out_dtype and final_dtype must be float16 or bfloat16")
    out = torch.empty((a.shape[0], b_prepacked.shape[1]), device=a.device, dtype=final_dtype)
    _validate(a, b_prepacked, scale, bias, out, 1, allow_bf16_a=True, bias_dtype=out_dtype)
    if a.shape[0] != 0:
        native.scaled_mm_lora_into(a, b_prepacked, scale, bias, out, t, lb_prepacked, out_dtype=out_dtype)
    return out


def prepack_b_for_scaled_mm(b: torch.Tensor) -> torch.Tensor:
    """(K, N) -> (K/16, N, 16): out[kb, n, j] = b[16*kb + j, n]."""
    if b.dim() != 2 or b.shape[0] % 16 != 0:
        raise RuntimeError("b must be 2D (K, N) with K divisible by 16")
    if b.element_size() != 1:
        raise RuntimeError("prepack_b_for_scaled_mm expects an 8-bit weight tensor")
    return native.prepack_bytes(b.contiguous(), src_is_kn=True)
