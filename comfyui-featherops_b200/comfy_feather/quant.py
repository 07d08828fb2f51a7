"""Feather weight format: per-tensor-scaled fp8e5m2, prepacked to (K/16, N, 16).

Same public surface as the reference's comfy_feather/quant.py (names, arguments, return values, error messages), with
the arithmetic done by the CUDA kernels of libfeather_b200 instead of torch elementwise ops:

    prepack_transpose / unprepack_transpose           quant.py:11-19
    FeatherFP8E5M2PackedParams                        quant.py:22-49
    quantize_fp8e5m2_scaled                           quant.py:52-74
    FeatherFP8E5M2PackedLayout                        quant.py:77-113
    make_feather_quantized_weight                     quant.py:116-136
    quantize_feather_weight                           quant.py:139-146
    is_feather_quantized_weight / get_feather_plain_tensors   quant.py:149-156

The results are bit-identical to the reference for round-to-nearest-even (seed None or 0).  With seed > 0 the
rounding itself is ComfyUI's `comfy.float.stochastic_rounding`, exactly as in the reference; only the prepack runs here.

There is no CPU implementation: a tensor that lives in host memory (a checkpoint being loaded) is copied to the
current CUDA device, processed there and the result is returned on the tensor's original device.
"""

from dataclasses import dataclass, fields, replace

import comfy.float
import torch
from comfy.quant_ops import QuantizedLayout, QuantizedTensor, register_layout_class

from ..kernel.b200 import native

FEATHER_FP8E5M2_LAYOUT = "FeatherFP8E5M2PackedLayout"

_QUANT_SRC_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _compute_device(t):
    """Device the kernels run on for tensor `t`: its own if CUDA, else the current CUDA device."""
    if t.is_cuda:
        return t.device
    if not torch.cuda.is_available():
        raise native.FeatherNativeError("FeatherOps B200 needs a CUDA device: quantise/prepack has no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


# (N, K) -> (K/16, N, 16)
def prepack_transpose(x):
    if x.ndim != 2 or x.shape[1] % 16 != 0:
        raise ValueError(f"Feather FP8 packed weights require a 2D tensor with K divisible by 16, got {tuple(x.shape)}")
    if x.element_size() != 1:
        raise TypeError(f"prepack_transpose expects an 8-bit tensor, got {x.dtype}")
    dev = _compute_device(x)
    out = native.prepack_bytes(x.to(dev).contiguous())
    return out.to(x.device)


# (K/16, N, 16) -> (N, K)
def unprepack_transpose(x):
    if x.ndim != 3 or x.shape[2] != 16:
        raise ValueError(f"expected a (K/16, N, 16) tensor, got {tuple(x.shape)}")
    dev = _compute_device(x)
    out = native.unprepack_bytes(x.to(dev).contiguous())
    return out.to(x.device)


@dataclass(frozen=True)
class FeatherFP8E5M2PackedParams:
    """What a packed weight carries beside its bytes.  `QuantizedTensor` moves, clones and overwrites it through the three
    methods below (the contract of the reference's class, comfy_feather/quant.py:22-49); `scale` is the only tensor."""

    scale: torch.Tensor
    orig_dtype: torch.dtype
    orig_shape: tuple[int, ...]

    _TENSORS = ("scale",)

    def _with_tensors(self, fn):
        return replace(self, **{name: fn(getattr(self, name)) for name in self._TENSORS})

    def to_device(self, device):
        return self._with_tensors(lambda t: t.to(device=device))

    def clone(self):
        return self._with_tensors(torch.Tensor.clone)

    def copy_from(self, src, non_blocking=False):
        for f in fields(self):
            if f.name in self._TENSORS:
                getattr(self, f.name).copy_(getattr(src, f.name), non_blocking=non_blocking)
            else:
                object.__setattr__(self, f.name, getattr(src, f.name))            # frozen dataclass: the plain fields are replaced


def _quantize_and_prepack(x, scale, seed, inplace_ops, premul=None):
    """Shared body of quantize_fp8e5m2_scaled + prepack_transpose.  Returns (prepacked qdata, fp32 scale) on x's device."""
    if x.ndim != 2:
        raise ValueError(f"Feather FP8 packed weights require a 2D tensor, got {x.ndim}D")
    if x.shape[1] % 16 != 0:
        raise ValueError(f"Feather FP8 packed weights require K divisible by 16, got {tuple(x.shape)}")
    if x.dtype not in _QUANT_SRC_DTYPES:
        raise TypeError(f"cannot quantise a {x.dtype} weight (expected float32, bfloat16 or float16)")
    dev = _compute_device(x)
    recalc = scale is None or (isinstance(scale, str) and scale == "recalculate")
    given = None
    if not recalc:
        given = (scale if isinstance(scale, torch.Tensor) else torch.tensor(scale)).to(device=dev, dtype=torch.float32)

    if seed is not None and seed > 0:
        # Stochastic rounding is ComfyUI's own routine (reference: quant.py:70-71); the scale rule and the
        # dtype-rounded multiply stay as in quant.py:53-66.  Only the (N,K)->(K/16,N,16) move runs natively.
        xs = x.to(dev)
        if recalc:
            given = torch.amax(xs.abs()).to(dtype=torch.float32) / torch.finfo(torch.float8_e5m2).max
            given = torch.where(given == 0, torch.ones_like(given), given)
            if xs.dtype not in {torch.float32, torch.bfloat16}:
                info = torch.finfo(xs.dtype)
                given = 1.0 / torch.clamp(1.0 / given, min=info.min, max=info.max)
        inv = (1.0 / given).to(dtype=xs.dtype)
        if inplace_ops and xs is x:
            xs *= inv
        else:
            xs = xs * inv
        q = comfy.float.stochastic_rounding(xs, dtype=torch.float8_e5m2, seed=seed)
        qdata = native.prepack_bytes(q.contiguous())
        return qdata.to(x.device), given.float().to(x.device)

    xs = x.to(dev).contiguous()
    pm = premul.to(device=dev, dtype=torch.float32) if premul is not None else None
    qdata, out_scale = native.quantize_prepack(xs, scale=given, premul=pm)
    if inplace_ops and x.is_cuda:
        # The reference leaves x scaled by 1/scale when inplace_ops is set (quant.py:65-66); callers only use that
        # mode on temporaries, but keep the side effect so the tensor they hold matches what the reference leaves.
        x *= (1.0 / out_scale).to(dtype=x.dtype)
    return qdata.to(x.device), out_scale.to(x.device)


def quantize_fp8e5m2_scaled(x, scale="recalculate", seed=None, inplace_ops=False):
    """x (N,K) -> (e5m2 tensor (N,K), fp32 scale).  Layout-neutral form kept for callers of the reference function."""
    qdata, out_scale = _quantize_and_prepack(x, scale, seed, inplace_ops)
    return unprepack_transpose(qdata), out_scale.float()


class FeatherFP8E5M2PackedLayout(QuantizedLayout):
    Params = FeatherFP8E5M2PackedParams

    @classmethod
    def quantize(cls, tensor, scale="recalculate", stochastic_rounding=0, inplace_ops=False):
        if tensor.ndim != 2:
            raise ValueError(f"Feather FP8 packed weights require a 2D tensor, got {tensor.ndim}D")
        if tensor.shape[1] % 16 != 0:
            raise ValueError(f"Feather FP8 packed weights require K divisible by 16, got {tensor.shape}")
        orig_dtype = tensor.dtype
        orig_shape = tuple(tensor.shape)
        qdata, scale = _quantize_and_prepack(tensor, scale, stochastic_rounding, inplace_ops)
        params = cls.Params(scale=scale.float(), orig_dtype=orig_dtype, orig_shape=orig_shape)
        return qdata, params

    @classmethod
    def dequantize(cls, qdata, params):
        dev = _compute_device(qdata)
        scale = params.scale.to(device=dev, dtype=torch.float32).reshape(1)
        out = native.dequantize(qdata.to(dev).contiguous(), scale, params.orig_dtype)
        return out.to(qdata.device)

    @classmethod
    def get_plain_tensors(cls, qtensor):
        return qtensor._qdata, qtensor._params.scale

    @classmethod
    def state_dict_tensors(cls, qdata, params):
        return {
            "": unprepack_transpose(qdata),
            "_scale": params.scale,
        }


def make_feather_quantized_weight(weight, scale, orig_dtype):
    """Loader path: an e5m2 checkpoint weight is only prepacked (its scale kept); any other dtype is taken to fp32,
    multiplied by the checkpoint scale and re-quantised with a recalculated scale."""
    if weight.ndim != 2:
        raise ValueError(f"Feather FP8 packed weights require a 2D tensor, got {weight.ndim}D")

    if scale is None:
        scale = torch.ones((), device=weight.device, dtype=torch.float32)
    else:
        scale = scale.to(device=weight.device, dtype=torch.float32)

    if weight.dtype == torch.float8_e5m2:
        qdata = prepack_transpose(weight)
    else:
        # fp32 source with the checkpoint scale folded in by the kernel (fp32 multiply, then amax, then quantise)
        qdata, scale = _quantize_and_prepack(weight.to(torch.float32), "recalculate", None, False, premul=scale.reshape(1))

    params = FeatherFP8E5M2PackedLayout.Params(scale=scale, orig_dtype=orig_dtype, orig_shape=tuple(weight.shape))
    return QuantizedTensor(qdata, FEATHER_FP8E5M2_LAYOUT, params)


def quantize_feather_weight(weight, seed=None, inplace_ops=False):
    qdata, params = FeatherFP8E5M2PackedLayout.quantize(weight, scale="recalculate", stochastic_rounding=seed, inplace_ops=inplace_ops)
    return QuantizedTensor(qdata, FEATHER_FP8E5M2_LAYOUT, params)


def is_feather_quantized_weight(weight):
    return isinstance(weight, QuantizedTensor) and weight._layout_cls == FEATHER_FP8E5M2_LAYOUT


def get_feather_plain_tensors(weight):
    if not is_feather_quantized_weight(weight):
        raise TypeError(f"Expected {FEATHER_FP8E5M2_LAYOUT}, got {type(weight).__name__}")
    return FeatherFP8E5M2PackedLayout.get_plain_tensors(weight)


register_layout_class(FEATHER_FP8E5M2_LAYOUT, FeatherFP8E5M2PackedLayout)
