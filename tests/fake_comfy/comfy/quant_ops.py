import torch

_LAYOUTS = {}


class QuantizedLayout:
    pass


def register_layout_class(name, cls):
    _LAYOUTS[name] = cls


class QuantizedTensor(torch.Tensor):
    """Wrapper tensor subclass: looks like a tensor of the original shape/dtype, carries packed data + params."""

    @staticmethod
    def __new__(cls, qdata, layout_cls, params):
        return torch.Tensor._make_wrapper_subclass(
            cls, tuple(params.orig_shape), dtype=params.orig_dtype, device=qdata.device, requires_grad=False
        )

    def __init__(self, qdata, layout_cls, params):
        self._qdata = qdata
        self._layout_cls = layout_cls
        self._params = params

    @property
    def params(self):
        return self._params

    def dequantize(self):
        return _LAYOUTS[self._layout_cls].dequantize(self._qdata, self._params)

    def __repr__(self):
        return f"QuantizedTensor(layout={self._layout_cls}, shape={tuple(self.shape)})"

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        name = func.overloadpacket.__name__
        self = args[0]
        if name in ("detach", "alias"):
            return QuantizedTensor(self._qdata, self._layout_cls, self._params)
        if name == "clone":
            return QuantizedTensor(self._qdata.clone(), self._layout_cls, self._params.clone())
        if name == "_to_copy":
            device = kwargs.get("device", None)
            if device is None:
                return QuantizedTensor(self._qdata, self._layout_cls, self._params)
            return QuantizedTensor(self._qdata.to(device), self._layout_cls, self._params.to_device(device))
        raise NotImplementedError(f"fake QuantizedTensor does not implement {func}")
