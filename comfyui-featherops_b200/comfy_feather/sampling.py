"""Keeps the model that is being sampled resident: while a sampler runs, ComfyUI's `free_memory` is asked to keep the
active Feather model loaded (reference: comfy_feather/sampling.py:64-83 `install_sampling_model_pin`).  Host-side
bookkeeping only; no kernels."""

import comfy.model_management
from comfy.patcher_extension import WrappersMP

_STATE = "_feather_b200_pin_state"
_WRAPPER_KEY = "feather_sampling_model_pin"


def _state():
    st = getattr(comfy.model_management, _STATE, None)
    if st is None:
        st = {"pins": {}, "original": None}
        setattr(comfy.model_management, _STATE, st)
    return st


def _wrap_free_memory():
    st = _state()
    if st["original"] is not None:
        return
    st["original"] = comfy.model_management.free_memory

    def free_memory_keeping_pins(memory_required, device, keep_loaded=None, *args, **kwargs):
        keep = list(keep_loaded or [])
        pins = _state()["pins"]
        if pins:
            have = {id(x) for x in keep}
            for loaded in comfy.model_management.current_loaded_models:
                if loaded.model is not None and id(loaded.model) in pins and id(loaded) not in have:
                    keep.append(loaded)
                    have.add(id(loaded))
        return st["original"](memory_required, device, keep, *args, **kwargs)

    comfy.model_management.free_memory = free_memory_keeping_pins


def install_sampling_model_pin(model_patcher):
    if getattr(model_patcher, "_feather_sampling_model_pin", False):
        return
    _wrap_free_memory()

    def pinned_outer_sample(executor, *args, **kwargs):
        patcher = getattr(executor.class_obj, "model_patcher", model_patcher)
        pins = _state()["pins"]
        pins[id(patcher)] = pins.get(id(patcher), 0) + 1
        try:
            return executor(*args, **kwargs)
        finally:
            pins[id(patcher)] -= 1
            if pins[id(patcher)] <= 0:
                del pins[id(patcher)]

    model_patcher.add_wrapper_with_key(WrappersMP.OUTER_SAMPLE, _WRAPPER_KEY, pinned_outer_sample)
    model_patcher._feather_sampling_model_pin = True
