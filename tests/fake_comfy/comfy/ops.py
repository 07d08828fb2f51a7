import torch
from torch import nn

_run_every_op_calls = 0


def run_every_op():
    global _run_every_op_calls
    _run_every_op_calls += 1


class disable_weight_init:
    class Linear(nn.Linear):
        comfy_cast_weights = False

        def __init__(self, in_features, out_features, bias=True, device=None, dtype=None):
            # like ComfyUI: no weight initialisation work
            nn.Module.__init__(self)
            self.in_features = in_features
            self.out_features = out_features
            self.weight = nn.Parameter(torch.empty((out_features, in_features), device=device, dtype=dtype), requires_grad=False)
            self.bias = nn.Parameter(torch.empty((out_features,), device=device, dtype=dtype), requires_grad=False) if bias else None
            self.weight_function = []
            self.bias_function = []

        def reset_parameters(self):
            return None


class manual_cast(disable_weight_init):
    class Linear(disable_weight_init.Linear):
        comfy_cast_weights = True


def cast_bias_weight(s, input=None, dtype=None, device=None, bias_dtype=None, offloadable=False, compute_dtype=None, want_requant=False):
    """Moves weight/bias to the input's device (and dtype for plain tensors).  Returns (weight, bias, offload_stream)."""
    if input is not None:
        if device is None:
            device = input.device
        if dtype is None:
            dtype = input.dtype
        if bias_dtype is None:
            bias_dtype = dtype
    weight = s.weight
    is_quantized = hasattr(weight, "_qdata")
    if is_quantized:
        # the wrapper's own .device is not reliable after nn.Module.to(); look at the packed data
        if weight._qdata.device != torch.device(device):
            weight = type(weight)(weight._qdata.to(device), weight._layout_cls, weight._params.to_device(device))
    else:
        weight = weight.to(device=device, dtype=dtype)
    for fn in getattr(s, "weight_function", []):
        weight = fn(weight)
    bias = None
    if s.bias is not None:
        bias = s.bias.to(device=device, dtype=bias_dtype)
        for fn in getattr(s, "bias_function", []):
            bias = fn(bias)
    return weight, bias, None


def uncast_bias_weight(s, weight, bias, offload_stream):
    return None
