"""Minimal stand-in for the parts of ComfyUI the FeatherOps plugin touches, for tests only.

ComfyUI itself is not available offline; the surface below follows the plugin's call sites and the reference's
typings/ stubs (typings/comfy/*.pyi).  It carries no ComfyUI code.
"""
