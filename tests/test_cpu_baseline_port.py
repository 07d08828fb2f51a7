"""CPU: the torch restatement that bench.py times as the CPU baseline agrees with the fixtures and the numpy oracle."""

import numpy as np
import pytest
import torch

from oracle import feather_oracle as fo
from oracle import naive_torch
from tests.golden import cases
from tests.util import TORCH_DT, from_torch, to_torch


@pytest.mark.parametrize("name", list(cases.GEMM_REF_CASES))
def test_verbatim_mode_matches_reference_fixture(golden, name):
    c = cases.gemm_ref_case(name)
    out = naive_torch.scaled_mm_cpu(
        to_torch(c["a"], "fp16"), to_torch(c["b_prepacked"], "e5m2"), torch.tensor(float(c["scale"])), to_torch(c["bias"], c["out_dtype"]),
        TORCH_DT[c["out_dtype"]], product="fp16",
    )
    assert np.array_equal(from_torch(out), golden[f"gemm/{name}/out"])


@pytest.mark.parametrize("name", list(cases.GEMM_BENCH_CASES))
def test_fp32_mode_matches_fixture_and_oracle(golden, name):
    c = cases.gemm_bench_case(name)
    out = naive_torch.scaled_mm_cpu(
        to_torch(c["a"], "fp16"), to_torch(c["b_prepacked"], "e5m2"), torch.tensor(float(c["scale"])),
        to_torch(c["bias"], c["out_dtype"]) if c["bias"] is not None else None, TORCH_DT[c["out_dtype"]],
    )
    got = from_torch(out)
    rows = golden[f"gemm/{name}/rows"]
    assert np.array_equal(got[rows], golden[f"gemm/{name}/out_rows"])
    rep = fo.error_report(got, fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"]), c["out_dtype"])
    assert rep["max_excess_over_1ulp"] <= 1e-5 * rep["rms"], rep


def test_quantize_port_matches_oracle():
    c = cases.quant_case("q_fp32_normal")
    q, s = naive_torch.quantize_prepack_cpu(to_torch(c["x"], "fp32"))
    rq, rs = fo.layout_quantize(c["x"], "fp32")
    assert np.array_equal(from_torch(q), rq) and np.float32(s.item()) == rs
