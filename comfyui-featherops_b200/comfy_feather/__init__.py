"""Node registration: the class and display names ComfyUI shows are the reference's (comfy_feather/__init__.py:1-9)."""

from . import loader

_NODES = ((loader.FeatherUNetLoader, "Load Diffusion Model (Feather)"),)

NODE_CLASS_MAPPINGS = {cls.__name__: cls for cls, _ in _NODES}
NODE_DISPLAY_NAME_MAPPINGS = {cls.__name__: title for cls, title in _NODES}
