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


def assert_gemm_close(got, ref, out_dtype, fo, what="", bias=None, has_bias=None):
    """The GEMM gate.  `bias`: the bias that was added, as the storage array of `out_dtype` (or float32 values), or None.

    1. |err| <= 1e-2 * rms(out) once rounding-boundary flips are set aside: two correct fp32-accumulating evaluations round a
       value that sits on a boundary of the output dtype to different neighbours, and one bf16 ulp at |out| >= 2 rms already
       exceeds 1e-2 * rms, so the literal bound cannot hold for bf16 by any implementation.  Without a bias the allowance is
       one ulp of the oracle's value; with a bias two ulps at the larger of the pre- and post-bias magnitudes (the flip
       happens before the add and the second rounding can widen it; see error_report).
    2. Without a bias, what is left after the one-ulp allowance must be fp32 summation noise: <= 1e-4 * rms.  (A count of
       ulps cannot be bounded: where a sum cancels to nearly zero its ulp shrinks below the noise of the fp32 additions.)
    3. The number of elements whose bits differ from the oracle's (which rounds the exact sum once) is bounded: the chance
       of a flip is about (fp32 summation noise) / (output ulp), i.e. some 1e-3 for bf16 at K = 5120 and 3e-2 for fp16 at
       K = 12288 (measured), so at most 1 % of the elements for bf16 and 8 % for fp16.  A wrong rounding mode (truncation,
       say) flips about half of all elements and fails this by a wide margin.  The count is printed (pytest -s shows it).
    4. Frobenius-relative error <= 1e-3; inf/NaN in the same places; for fp16 also the literal max|err| <= 1e-2 * rms.
    """
    if bias is not None and np.asarray(bias).dtype != np.float32:
        bias = fo.to_f32(bias, out_dtype)
    if has_bias is None:
        has_bias = bias is not None
    rep = fo.error_report(got, ref, out_dtype, bias=bias)
    size = int(np.asarray(got).size)
    limit = (1e-2 if out_dtype == "bf16" else 8e-2) * size + 4
    print(f"[gemm gate] {what}: {rep['mismatches']} of {size} elements differ from the oracle (limit {limit:.0f}), max {rep['max_ulp']} ulp, "
          f"beyond the ulp allowance {rep['max_excess_over_1ulp']:.2e}, fro_rel {rep['fro_rel']:.2e}, rms {rep['rms']:.3g}")
    rms = max(rep["rms"], 1e-30)
    assert rep["nonfinite_agree"], (what, rep)
    assert rep["max_excess_over_1ulp"] <= (1e-2 if has_bias else 1e-4) * rms, (what, rep)
    assert rep["fro_rel"] <= 1e-3, (what, rep)
    assert rep["mismatches"] <= limit, (what, rep)
    if out_dtype == "fp16":
        assert rep["max_abs"] <= 1e-2 * rms, (what, rep)
    return rep
