"""FeatherOps for B200: fp16 activations @ prepacked fp8e5m2 weights on sm_100a, behind the operator surface of
woct0rdho/ComfyUI-FeatherOps (`comfy_feather/ops.py`, `kernel/hip/hip_kernel.py`).

As a ComfyUI custom node this directory exports NODE_CLASS_MAPPINGS (reference: __init__.py:1, comfy_feather/__init__.py:1-9).
Outside ComfyUI (tests, benchmarks) the node classes are not importable, and the mappings stay empty.
"""

NODE_CLASS_MAPPINGS = {}
NODE_DISPLAY_NAME_MAPPINGS = {}

try:  # ComfyUI present: register the loader node
    import folder_paths  # noqa: F401

    from .comfy_feather import NODE_CLASS_MAPPINGS, NODE_DISPLAY_NAME_MAPPINGS  # noqa: F401
except ImportError:
    pass
