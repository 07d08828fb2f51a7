"""numpy <-> torch helpers for the tests (bf16 travels as uint16 bit patterns, e5m2 as uint8)."""

import numpy as np
import torch

TORCH_DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "e5m2": torch.float8_e5m2}


def to_torch(x, dtype, device="cpu"):
    x = np.ascontiguousarray(x)
    if dtype == "fp32":
        t = torch.from_numpy(x.astype(np.float32))
    elif dtype == "fp16":
        t = torch.from_numpy(x.astype(np.float16))
    elif dtype == "bf16":
        t = torch.from_numpy(x.astype(np.uint16).view(np.int16)).view(torch.bfloat16)
    elif dtype == "e5m2":
        t = torch.from_numpy(x.astype(np.uint8)).view(torch.float8_e5m2)
    else:
        raise ValueError(dtype)
    return t.to(device)


def from_torch(t):
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float8_e5m2:
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def assert_gemm_close(got, ref, out_dtype, fo, what=""):
    """The GEMM gate: |err| <= 1e-2 * rms(out) once the one-ulp rounding-boundary flips any two fp32-accumulating
    implementations show are set aside (they exceed 1e-2*rms by construction for bf16), Frobenius-relative error
    <= 1e-3, and inf/NaN in the same places."""
    rep = fo.error_report(got, ref, out_dtype)
    assert rep["nonfinite_agree"], (what, rep)
    assert rep["max_excess_over_1ulp"] <= 1e-2 * max(rep["rms"], 1e-30), (what, rep)
    assert rep["fro_rel"] <= 1e-3, (what, rep)
    if out_dtype == "fp16":
        assert rep["max_abs"] <= 1e-2 * max(rep["rms"], 1e-30), (what, rep)
    return rep
