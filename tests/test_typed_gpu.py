"""GPU: the operand and result types around the fp16 x e5m2 core, through `feather_scaled_mm_typed` and the operator:
fp8e4m3fn weights (exact upcast), bf16 activations multiplied without a cast pass, and the other 16-bit dtype stored straight
from the epilogue.  Checkers: the fixtures made by the reference's kernel/naive.py, the numpy oracle, and - for the two fused
casts - the library's own cast-first / cast-after results, which must match bit for bit wherever the casts are exact."""

import importlib

import numpy as np
import pytest
import torch

from oracle import feather_oracle as fo
from tests.golden import cases
from tests.util import TORCH_DT, assert_gemm_close, from_torch, to_torch

pytestmark = pytest.mark.gpu


def _weights(rng, N, K):
    w = (rng.standard_normal((N, K), dtype=np.float32) / np.float32(np.sqrt(K))).astype(np.float32)
    return fo.make_feather_quantized_weight(w, "fp32", None)


@pytest.mark.parametrize("name", list(cases.GEMM_E4M3_CASES))
def test_e4m3_weights_against_the_reference_fixture(golden, hip_kernel, native, cuda_dev, name):
    """fp8e4m3fn weights through the reference's operator surface (`scaled_mm_hip`, b_dtype 0).  The all-codes case has one
    product per output, so nothing but the upcast and the roundings is in play: bit for bit the reference's naive.py."""
    c = cases.gemm_e4m3_case(name)
    a = to_torch(c["a"], "fp16", cuda_dev)
    b_pp = torch.from_numpy(c["b_prepacked"]).to(cuda_dev).view(torch.float8_e4m3fn)
    scale = torch.tensor(float(c["scale"]), dtype=torch.float32, device=cuda_dev)
    bias = to_torch(c["bias"], c["out_dtype"], cuda_dev)
    out = hip_kernel.scaled_mm_hip(a, b_pp, scale, bias, TORCH_DT[c["out_dtype"]])
    native.check_device_status(cuda_dev)
    got = from_torch(out)
    fixture = golden[f"gemm/{name}/out"]
    if "all_codes" in name:
        nan = np.isnan(fo.to_f32(fixture, c["out_dtype"]))
        assert nan[:, [127, 255]].all() and nan.sum() == 2 * fixture.shape[0]
        assert np.array_equal(np.isnan(fo.to_f32(got, c["out_dtype"])), nan)
        assert np.array_equal(got[~nan], fixture[~nan])
    else:
        rep = fo.error_report(got, fixture, c["out_dtype"])
        assert rep["fro_rel"] <= 0.01 and rep["max_abs"] <= 16.0, rep                      # the reference's own gate (test_scaled_mm_hip.py:26-30)
        ref32 = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], b_format="e4m3")
        assert_gemm_close(got, ref32, c["out_dtype"], fo, name, bias=fo.to_f32(c["bias"], c["out_dtype"]))


@pytest.mark.parametrize("M,N,K", [(300, 520, 1040), (64, 256, 512), (2100, 1024, 2048)])
def test_bf16_activations_equal_cast_first_where_the_cast_is_exact(native, cuda_dev, M, N, K):
    """bf16 activations that fp16 represents exactly (all of them with 2^-14 <= |x| <= 65504, and zero): multiplying them as
    bf16 gives bit for bit what casting them to fp16 first gives, for both output dtypes, with and without the final cast."""
    rng = np.random.default_rng(M + N)
    bq, s = _weights(rng, N, K)
    x = torch.from_numpy(rng.standard_normal((M, K), dtype=np.float32) * 3).to(torch.bfloat16)
    x = torch.where(x.abs() < 2.0 ** -14, torch.zeros_like(x), x).to(cuda_dev)
    assert torch.equal(x.to(torch.float16).to(torch.bfloat16), x)
    B = to_torch(bq, "e5m2", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    for out_dtype, final in ((torch.bfloat16, torch.bfloat16), (torch.float16, torch.bfloat16), (torch.float16, torch.float16), (torch.bfloat16, torch.float16)):
        bias = torch.from_numpy(rng.standard_normal((N,), dtype=np.float32)).to(cuda_dev).to(out_dtype)
        ref = torch.empty((M, N), dtype=out_dtype, device=cuda_dev)
        native.scaled_mm_into(native.bf16_to_fp16(x), B, S, bias, ref, variant=native.make_variant(kernel=native.KERNEL_TMEM))
        got = torch.full((M, N), float("nan"), dtype=final, device=cuda_dev)
        native.scaled_mm_typed_into(x, B, S, bias, got, out_dtype=out_dtype, variant=native.make_variant(kernel=native.KERNEL_TMEM))
        native.check_device_status(cuda_dev)
        assert torch.equal(got.view(torch.int16), ref.to(final).view(torch.int16)), (out_dtype, final)
    # and against the oracle, which multiplies the bf16 values as they are
    ref_np = fo.scaled_mm(from_torch(x), bq, s, None, "bf16", a_format="bf16")
    got = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_dev)
    native.scaled_mm_typed_into(x, B, S, None, got)
    assert_gemm_close(from_torch(got), ref_np, "bf16", fo, f"bf16 activations {(M, N, K)}")


def test_bf16_activations_outside_the_fp16_range(native, cuda_dev):
    """Where the cast is not exact the two paths differ by design: |x| > 65504 becomes inf under cast-first (naive.py:21) and
    poisons its output row, while the bf16 product is finite and equals the oracle on the unrounded values; tiny values keep
    the bits fp16 subnormals would drop."""
    rng = np.random.default_rng(7)
    M, N, K = 64, 256, 512
    bq, s = _weights(rng, N, K)
    x = torch.from_numpy(rng.standard_normal((M, K), dtype=np.float32)).to(torch.bfloat16)
    x[3, 5] = 1.0e5
    x[9, :] *= 2.0 ** -20
    x = x.to(cuda_dev)
    B = to_torch(bq, "e5m2", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    got = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_dev)
    native.scaled_mm_typed_into(x, B, S, None, got)
    native.check_device_status(cuda_dev)
    assert_gemm_close(from_torch(got), fo.scaled_mm(from_torch(x), bq, s, None, "bf16", a_format="bf16"), "bf16", fo, "unrounded bf16")
    cast_first = fo.to_f32(fo.scaled_mm(from_torch(x), bq, s, None, "bf16", a_format="bf16_cast_first"), "bf16")
    assert not np.isfinite(cast_first[3]).all() and torch.isfinite(got[3].float()).all()


@pytest.mark.parametrize("M", [8, 16, 200])
def test_final_cast_in_every_kernel(native, cuda_dev, M):
    """`final_dtype` is honoured by the streaming kernel (M <= 16), the split-K reduction and the staged epilogue alike."""
    rng = np.random.default_rng(M)
    N, K = 520, 2048
    bq, s = _weights(rng, N, K)
    a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    A, B = to_torch(a, "fp16", cuda_dev), to_torch(bq, "e5m2", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    variants = [None, native.make_variant(16 if M <= 16 else 128, 1, 4, 2, 0), native.make_variant(kernel=native.KERNEL_TMEM)]
    for out_dtype, final in ((torch.float16, torch.bfloat16), (torch.bfloat16, torch.float16)):
        bias = torch.from_numpy(rng.standard_normal((N,), dtype=np.float32)).to(cuda_dev).to(out_dtype)
        for v in variants:
            ref = torch.empty((M, N), dtype=out_dtype, device=cuda_dev)
            native.scaled_mm_into(A, B, S, bias, ref, variant=v)
            got = torch.full((M, N), float("nan"), dtype=final, device=cuda_dev)
            native.scaled_mm_typed_into(A, B, S, bias, got, out_dtype=out_dtype, variant=v)
            native.check_device_status(cuda_dev)
            assert torch.equal(got.view(torch.int16), ref.to(final).view(torch.int16)), (M, out_dtype, final, v.as_tuple() if v else None)
        ref_np = fo.scaled_mm(a, bq, s, from_torch(bias), "bf16" if out_dtype == torch.bfloat16 else "fp16",
                              final_dtype="bf16" if final == torch.bfloat16 else "fp16")
        rep = fo.error_report(from_torch(got), ref_np, "bf16" if final == torch.bfloat16 else "fp16")
        assert rep["nonfinite_agree"] and rep["fro_rel"] <= 2e-3, rep


def test_operator_linear_folds_both_casts(pkg, native, hip_kernel, cuda_dev):
    """`FeatherOps.Linear` with out_dtype fp16 in a bf16 model (the Wan configuration of the loader): the reference computes
    `scaled_mm_hip(x.to(fp16), ..., fp16).to(bf16)` (ops.py:88-103); the operator here issues one launch and must give
    those bits."""
    ops_mod = importlib.import_module("feather_b200.comfy_feather.ops")
    g = torch.Generator().manual_seed(11)
    N, K = 640, 1024
    w = torch.randn((N, K), generator=g) / K ** 0.5
    bias = torch.randn((N,), generator=g) * 0.1
    Ops = ops_mod.feather_ops(out_dtype=torch.float16)
    lin = Ops.Linear(K, N, bias=True)
    lin._load_from_state_dict({"l.weight": w.clone(), "l.bias": bias.clone()}, "l.", {}, True, [], [], [])
    lin = lin.to(cuda_dev)
    for T in (8, 300):
        x = torch.randn((2, T, K), generator=g).to(torch.bfloat16).to(cuda_dev)
        y = lin(x)
        native.check_device_status(cuda_dev)
        assert y.dtype == torch.bfloat16 and y.shape == (2, T, N)
        ref = hip_kernel.scaled_mm_hip(x.reshape(-1, K).to(torch.float16), lin.weight._qdata.to(cuda_dev), lin.weight._params.scale.to(cuda_dev).reshape(1).float(),
                                       lin.bias.to(cuda_dev), torch.float16).to(torch.bfloat16)
        assert torch.equal(y.reshape(-1, N).view(torch.int16), ref.view(torch.int16)), T
