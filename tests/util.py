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


def assert_gemm_close(got, ref, out_dtype, fo, what="", has_bias=True, bias=None):
    """The GEMM gate: |err| <= 1e-2 * rms(out) once the one-ulp rounding-boundary flips any two fp32-accumulating
    implementations show are set aside (they exceed 1e-2*rms by construction for bf16), Frobenius-relative error
    <= 1e-3, and inf/NaN in the same places.

    The flips themselves are bounded too, so a wrong rounding mode cannot hide under the Frobenius bound: the number of
    elements whose bits differ from the oracle's stays below 1e-3 of the output for bf16 (the reference's own naive.py
    against the oracle shows 1e-4 at 256 x 1024 x 1024) and 8e-3 for fp16 (its ulp is 8 times finer against the same
    fp32 summation noise), and without a bias every differing element is exactly one ulp away (a bias add can cancel
    and turn one ulp of the product into several of the sum).  `bias` (float32 values of the bias that was added, optional):
    one ulp is then measured at the pre-bias magnitude where that is larger.  The count is printed (pytest -s shows it)."""
    rep = fo.error_report(got, ref, out_dtype, bias=bias)
    size = int(np.asarray(got).size)
    limit = (1e-3 if out_dtype == "bf16" else 8e-3) * size + 4
    print(f"[gemm gate] {what}: {rep['mismatches']} of {size} elements differ from the oracle (limit {limit:.0f}), max {rep['max_ulp']} ulp, "
          f"fro_rel {rep['fro_rel']:.2e}")
    assert rep["nonfinite_agree"], (what, rep)
    assert rep["max_excess_over_1ulp"] <= 1e-2 * max(rep["rms"], 1e-30), (what, rep)
    assert rep["fro_rel"] <= 1e-3, (what, rep)
    assert rep["mismatches"] <= limit, (what, rep)
    if not has_bias:
        assert rep["max_ulp"] <= 1, (what, rep)
    if out_dtype == "fp16":
        assert rep["max_abs"] <= 1e-2 * max(rep["rms"], 1e-30), (what, rep)
    return rep
