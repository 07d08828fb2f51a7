"""CPU: the numpy oracle against the fixtures produced by the reference's own code (tests/golden/make_golden.py)."""

import hashlib

import numpy as np
import pytest

from oracle import feather_oracle as fo
from tests.golden import cases


def sha(x):
    return hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest()


@pytest.mark.parametrize("name", list(cases.GEMM_REF_CASES))
def test_gemm_reference_distribution(golden, name):
    """Verbatim kernel/naive.py output (fp16 product) on the reference's test distribution."""
    c = cases.gemm_ref_case(name)
    ref = golden[f"gemm/{name}/out"]
    mine = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product="fp16")
    rep = fo.error_report(mine, ref, c["out_dtype"])
    # the fp16 rounding of the product depends on torch's summation order: allow a handful of one-step flips
    assert rep["nonfinite_agree"] and rep["fro_rel"] <= 1e-5 and rep["mismatches"] <= ref.size // 1000, rep
    # and the fp32-product math (what the kernel computes) passes the reference's own gate, test_scaled_mm_hip.py:26-30
    mine32 = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product="fp32")
    rep32 = fo.error_report(mine32, ref, c["out_dtype"])
    assert rep32["fro_rel"] <= 0.01 and rep32["max_abs"] <= (2.0 if c["out_dtype"] == "fp16" else 16.0), rep32


@pytest.mark.parametrize("name", list(cases.GEMM_BENCH_CASES))
def test_gemm_benchmark_distribution(golden, name):
    c = cases.gemm_bench_case(name)
    rows = golden[f"gemm/{name}/rows"]
    ref = golden[f"gemm/{name}/out_rows"]
    assert np.float32(golden[f"gemm/{name}/scale"]) == c["scale"]
    mine = fo.scaled_mm(c["a"][rows], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product="fp32")
    rep = fo.error_report(mine, ref, c["out_dtype"])
    assert rep["nonfinite_agree"] and rep["max_excess_over_1ulp"] <= 1e-5 * rep["rms"] and rep["fro_rel"] < 1e-3, rep


def test_verbatim_naive_overflows_on_benchmark_distribution(golden):
    """Why the fp32-product oracle exists: kernel/naive.py:20-23 rounds the unscaled product to fp16."""
    assert int(golden["gemm/config1_256x1024x1024_bf16/verbatim_inf_count"]) > 10000
    c = cases.gemm_bench_case("config1_256x1024x1024_bf16")
    mine = fo.scaled_mm(c["a"][:16], c["b_prepacked"], c["scale"], None, "bf16", product="fp16")
    assert np.isinf(fo.to_f32(mine, "bf16")).sum() > 100


@pytest.mark.parametrize("name", cases.QUANT_CASES)
def test_quantize_prepack(golden, name):
    c = cases.quant_case(name)
    if c["path"] == "layout":
        q, s = fo.layout_quantize(c["x"], c["dtype"])
    else:
        q, s = fo.make_feather_quantized_weight(c["x"], c["dtype"], c["scale"])
    assert np.array_equal(cases.canonical_e5m2(q), cases.canonical_e5m2(golden[f"quant/{name}/qdata"]))
    assert np.float32(s).view(np.uint32) == np.float32(golden[f"quant/{name}/scale"]).view(np.uint32)
    for od in ("fp32", "bf16", "fp16"):
        deq = fo.layout_dequantize(golden[f"quant/{name}/qdata"], golden[f"quant/{name}/scale"], od)
        assert sha(np.nan_to_num(fo.to_f32(deq, od), nan=12345.0)) == str(golden[f"quant/{name}/dequant_{od}_sha"])


def test_fp16_clamp_branch_is_exercised():
    """quant.py:56-58: for fp16 sources with amax < 0.875, 1/scale is clamped to 65504."""
    c = cases.quant_case("q_fp16_clamped")
    _, s = fo.layout_quantize(c["x"], "fp16")
    assert s == np.float32(1.0) / np.float32(65504.0)
    amax = np.abs(c["x"].astype(np.float32)).max()
    assert s != np.float32(amax / np.float32(57344.0))


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("scale", cases.EXHAUSTIVE_SCALES)
def test_exhaustive_cast(golden, dtype, scale):
    pats = cases.exhaustive_patterns(dtype)
    with np.errstate(all="ignore"):
        q, _ = fo.quantize_fp8e5m2_scaled(pats, dtype, scale=scale)
    assert sha(cases.canonical_e5m2(q)) == str(golden[f"exhaustive/{dtype}/{scale!r}/sha"])


def test_fp32_random_bit_patterns(golden):
    rng = np.random.default_rng(77)
    pats32 = rng.integers(0, 2 ** 32, size=(8192, 16), dtype=np.uint64).astype(np.uint32).view(np.float32)
    with np.errstate(all="ignore"):
        q, _ = fo.quantize_fp8e5m2_scaled(pats32, "fp32", scale=1.0)
    assert sha(cases.canonical_e5m2(q)) == str(golden["exhaustive/fp32/random_bits/sha"])


def test_e5m2_upcast_is_a_byte_shift(golden):
    codes = np.arange(256, dtype=np.uint8).reshape(16, 16)
    assert np.array_equal((codes.astype(np.uint16) << 8), golden["codes/e5m2_to_fp16_bits"] | 0) or np.array_equal(
        np.where(np.isnan(fo.e5m2_bits_to_f32(codes)), 0, codes.astype(np.uint16) << 8),
        np.where(np.isnan(fo.e5m2_bits_to_f32(codes)), 0, golden["codes/e5m2_to_fp16_bits"]),
    )


def test_prepack_round_trip_and_layouts():
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, size=(24, 64), dtype=np.uint8)
    p = fo.prepack_transpose(x)
    assert p.shape == (4, 24, 16)
    assert p[2, 7, 5] == x[7, 2 * 16 + 5]
    assert np.array_equal(fo.unprepack_transpose(p), x)
    assert np.array_equal(fo.prepack_b_for_scaled_mm(np.ascontiguousarray(x.T)), p)


def test_bf16_to_fp16(golden):
    pats = cases.exhaustive_patterns("bf16")
    with np.errstate(all="ignore"):
        mine = fo.from_f32(fo.bf16_bits_to_f32(pats), "fp16")
    nan_mask = np.isnan(mine)
    assert sha(np.where(nan_mask, np.uint16(0x7E00), mine.view(np.uint16))) == str(golden["convert/bf16_to_fp16_sha"])


@pytest.mark.parametrize("name", list(cases.GEMM_E4M3_CASES))
def test_gemm_e4m3_weights(golden, name):
    """fp8e4m3fn weights: the oracle against verbatim kernel/naive.py run on a float8_e4m3fn tensor."""
    c = cases.gemm_e4m3_case(name)
    ref = golden[f"gemm/{name}/out"]
    mine = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product="fp16", b_format="e4m3")
    rep = fo.error_report(mine, ref, c["out_dtype"])
    assert rep["nonfinite_agree"] and rep["fro_rel"] <= 1e-5 and rep["mismatches"] <= max(ref.size // 1000, 2), rep
    if "all_codes" in name:      # one product per output: nothing depends on a summation order
        finite = ~np.isnan(fo.to_f32(ref, c["out_dtype"]))
        assert np.array_equal(mine[finite], ref[finite]) and (~finite).sum() == 2 * ref.shape[0]


def test_e4m3_decode_table():
    import torch

    codes = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    got = fo.e4m3_bits_to_f32(codes)
    assert np.array_equal(np.isnan(want), np.isnan(got)) and np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])
    assert np.isnan(got[[0x7F, 0xFF]]).all() and got[0x7E] == 448.0 and got[0x01] == 2.0 ** -9


def test_oracle_operand_and_result_types():
    """bf16 activations multiplied as they are equal cast-first where the cast is exact; the final cast is one more rounding."""
    rng = np.random.default_rng(0)
    a32 = rng.standard_normal((8, 64), dtype=np.float32)
    a_bf = fo.from_f32(a32, "bf16")
    w = (rng.standard_normal((32, 64), dtype=np.float32) / 8).astype(np.float32)
    bq, s = fo.make_feather_quantized_weight(w, "fp32", None)
    direct = fo.scaled_mm(a_bf, bq, s, None, "bf16", a_format="bf16")
    cast_first = fo.scaled_mm(a_bf, bq, s, None, "bf16", a_format="bf16_cast_first")
    as_fp16 = fo.scaled_mm(fo.to_f32(a_bf, "bf16").astype(np.float16), bq, s, None, "bf16")
    assert np.array_equal(cast_first, as_fp16)
    assert fo.error_report(direct, cast_first, "bf16")["max_ulp"] <= 1           # randn may hold a few values below 2^-14
    y16 = fo.scaled_mm(fo.to_f32(a_bf, "bf16").astype(np.float16), bq, s, None, "fp16")
    y16_as_bf = fo.scaled_mm(fo.to_f32(a_bf, "bf16").astype(np.float16), bq, s, None, "fp16", final_dtype="bf16")
    assert np.array_equal(y16_as_bf, fo.from_f32(fo.to_f32(y16, "fp16"), "bf16"))
