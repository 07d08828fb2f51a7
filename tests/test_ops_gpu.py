"""GPU: the FeatherOps.Linear operator (comfy_feather/ops.py surface) under the test double of `comfy`, against the
oracle: state-dict loading, forward, LoRA merge round trip, un-merged LoRA patches, checkpoint round trip."""

import importlib

import numpy as np
import pytest
import torch

from oracle import feather_oracle as fo
from tests.util import TORCH_DT, assert_gemm_close, from_torch, to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops_mod(pkg):
    return importlib.import_module("feather_b200.comfy_feather.ops")


@pytest.fixture(scope="module")
def quant_mod(pkg):
    return importlib.import_module("feather_b200.comfy_feather.quant")


def _make_linear(ops_mod, K, N, out_dtype, state, prefix="blocks.0.ffn.", excluded=()):
    Ops = ops_mod.feather_ops(out_dtype=out_dtype, excluded_names=excluded)
    lin = Ops.Linear(K, N, bias="bias" in state)
    missing, unexpected, errors = [], [], []
    sd = {prefix + k: v for k, v in state.items()}
    lin._load_from_state_dict(sd, prefix, {}, True, missing, unexpected, errors)
    assert not missing and not sd
    return lin


@pytest.mark.parametrize("src_dtype", ["fp32", "bf16", "fp16"])
@pytest.mark.parametrize("out_dtype", ["bf16", "fp16"])
def test_load_and_forward(ops_mod, cuda_dev, src_dtype, out_dtype):
    rng = np.random.default_rng(3)
    K, N, M = 256, 384, 77
    w = fo.from_f32((rng.standard_normal((N, K), dtype=np.float32) / 16).astype(np.float32), src_dtype)
    bias = rng.standard_normal((N,), dtype=np.float32)
    x = rng.standard_normal((3, M, K), dtype=np.float32).astype(np.float16)
    lin = _make_linear(ops_mod, K, N, TORCH_DT[out_dtype], {"weight": to_torch(w, src_dtype), "bias": torch.from_numpy(bias)})
    assert lin.is_quantized and lin.bias.dtype == TORCH_DT[out_dtype]
    lin = lin.to(cuda_dev)
    y = lin(to_torch(x, "fp16", cuda_dev))
    assert y.shape == (3, M, N) and y.dtype == torch.float16
    q_ref, s_ref = fo.make_feather_quantized_weight(w, src_dtype, None)
    assert np.array_equal(from_torch(lin.weight._qdata), q_ref)
    ref = fo.scaled_mm(x.reshape(-1, K), q_ref, s_ref, fo.from_f32(bias, out_dtype), out_dtype)
    ref16 = fo.from_f32(fo.to_f32(ref, out_dtype), "fp16")        # y.to(dtype_orig)
    assert_gemm_close(from_torch(y.reshape(-1, N)), ref16, "fp16", fo, bias=bias)


def test_e5m2_checkpoint_with_scale_keys(ops_mod, cuda_dev):
    rng = np.random.default_rng(4)
    K, N = 128, 64
    codes = rng.integers(0, 0x7B, size=(N, K), dtype=np.uint8)
    for key in ("weight_scale", "scale_weight"):
        lin = _make_linear(ops_mod, K, N, torch.bfloat16, {"weight": to_torch(codes, "e5m2"), key: torch.tensor(0.0123)})
        assert lin.is_quantized and lin.bias is None
        assert np.array_equal(from_torch(lin.weight._qdata), fo.prepack_transpose(codes))
        assert float(lin.weight._params.scale) == pytest.approx(0.0123)
        x = rng.standard_normal((5, K), dtype=np.float32).astype(np.float16)
        y = lin.to(cuda_dev)(to_torch(x, "fp16", cuda_dev).to(torch.bfloat16))
        assert y.dtype == torch.bfloat16
        xb = fo.to_f32(from_torch(to_torch(x, "fp16").to(torch.bfloat16)), "bf16").astype(np.float16)
        ref = fo.scaled_mm(xb, fo.prepack_transpose(codes), np.float32(0.0123), None, "bf16")
        assert_gemm_close(from_torch(y), ref, "bf16", fo)


def test_layers_that_stay_plain(ops_mod, cuda_dev):
    w = torch.randn(32, 64)
    lin = _make_linear(ops_mod, 64, 32, torch.bfloat16, {"weight": w}, prefix="head.proj.", excluded=("head",))
    assert not lin.is_quantized and torch.equal(lin.weight, w)
    lin2 = _make_linear(ops_mod, 24, 32, torch.bfloat16, {"weight": torch.randn(32, 24)})       # K % 16 != 0
    assert not lin2.is_quantized
    lin3 = _make_linear(ops_mod, 64, 1, torch.bfloat16, {"weight": torch.randn(1, 64)})
    assert not lin3.is_quantized
    x = torch.randn(4, 64, device=cuda_dev)
    assert torch.allclose(lin.to(cuda_dev)(x), x @ w.to(cuda_dev).t(), atol=1e-4)


def test_missing_weight_and_empty_input(ops_mod, cuda_dev):
    Ops = ops_mod.feather_ops()
    lin = Ops.Linear(64, 32, bias=False)
    missing = []
    lin._load_from_state_dict({}, "a.", {}, True, missing, [], [])
    assert missing == ["a.weight"]
    lin = _make_linear(ops_mod, 64, 32, torch.float16, {"weight": torch.randn(32, 64)}).to(cuda_dev)
    y = lin(torch.zeros((2, 0, 64), dtype=torch.float16, device=cuda_dev))
    assert y.shape == (2, 0, 32)


def test_lora_merge_round_trip(ops_mod, quant_mod, cuda_dev):
    """ModelPatcher path: convert_weight (dequantise) -> add a delta -> set_weight (re-quantise, recalculated scale)."""
    rng = np.random.default_rng(6)
    K, N = 128, 96
    w = (rng.standard_normal((N, K), dtype=np.float32) / 11).astype(np.float32)
    lin = _make_linear(ops_mod, K, N, torch.bfloat16, {"weight": torch.from_numpy(w)}).to(cuda_dev)
    q0, s0 = fo.make_feather_quantized_weight(w, "fp32", None)
    deq = lin.convert_weight(lin.weight).to(cuda_dev)      # the packed data stays where the checkpoint was loaded (host)
    assert deq.dtype == torch.bfloat16 and deq.shape == (N, K)
    assert np.array_equal(from_torch(deq), fo.layout_dequantize(q0, s0, "bf16"))
    delta = fo.f32_to_bf16_bits((rng.standard_normal((N, K), dtype=np.float32) / 50).astype(np.float32))
    merged = deq + to_torch(delta, "bf16", cuda_dev)
    merged_np = from_torch(merged)
    new_w = lin.set_weight(merged.clone(), seed=0, return_weight=True)
    assert quant_mod.is_feather_quantized_weight(new_w)
    q1, s1 = fo.layout_quantize(merged_np, "bf16")
    assert np.array_equal(from_torch(new_w._qdata), q1) and np.float32(new_w._params.scale.item()) == s1
    lin.set_weight(merged.clone(), seed=None)
    assert np.array_equal(from_torch(lin.weight._qdata), q1)
    # stochastic rounding goes through comfy.float (test double here): every code is a neighbour of the exact value
    sr = lin.set_weight(merged.clone(), seed=1234, return_weight=True)
    codes_sr = fo.e5m2_bits_to_f32(fo.unprepack_transpose(from_torch(sr._qdata)))
    codes_rn = fo.e5m2_bits_to_f32(fo.unprepack_transpose(q1))
    exact = fo.to_f32(merged_np, "bf16") / np.float32(sr._params.scale.item())
    assert np.all(np.abs(codes_sr - exact) <= np.abs(codes_rn - exact) * 2 + np.abs(exact) * 0.26 + 1e-3)
    assert (codes_sr != codes_rn).any()


def test_unmerged_lora_patches(ops_mod, pkg, cuda_dev):
    lora = importlib.import_module("feather_b200.comfy_feather.lora")
    rng = np.random.default_rng(7)
    K, N, M, r = 128, 64, 20, 8
    w = (rng.standard_normal((N, K), dtype=np.float32) / 11).astype(np.float32)
    lin = _make_linear(ops_mod, K, N, torch.float16, {"weight": torch.from_numpy(w)}).to(cuda_dev)

    class Adapter:
        def __init__(self, b, a, alpha):
            self.weights = (b, a, alpha, None, None, None)

    class PatchFn:
        key = "blocks.0.ffn.weight"

        def __init__(self, patches):
            self.patches = {self.key: patches}

    A = torch.randn(r, K) / 10
    B = torch.randn(N, r) / 10
    x = torch.randn(M, K, device=cuda_dev, dtype=torch.float16)
    base = lin(x).float()
    lin.weight_function = [PatchFn([(0.8, Adapter(B, A, 4.0), 1.5, None, None)])]
    y = lin(x).float()
    delta = fo.lora_delta(x.float().cpu().numpy(), A.numpy(), B.numpy(), 0.8 * 1.5 * 4.0 / r)
    assert np.allclose((y - base).cpu().numpy(), delta, atol=2e-2, rtol=2e-2)
    assert lin.weight_function, "weight_function must be restored after the call"
    lin.weight_function = [object()]
    with pytest.raises(NotImplementedError, match="basic LoRA"):
        lin(x)
    with pytest.raises(NotImplementedError, match="basic LoRA"):
        lora.apply_lora_patches(x, base, [PatchFn([(1.0, object(), 1.0, None, None)])])


def test_state_dict_round_trip(quant_mod, cuda_dev):
    """state_dict_tensors emits un-prepacked (N,K) e5m2 + scale; loading that checkpoint reproduces the same bytes."""
    w = torch.randn(80, 160, device=cuda_dev) / 9
    qt = quant_mod.quantize_feather_weight(w)
    sd = quant_mod.FeatherFP8E5M2PackedLayout.state_dict_tensors(qt._qdata, qt._params)
    assert sd[""].shape == (80, 160) and sd[""].dtype == torch.float8_e5m2
    again = quant_mod.make_feather_quantized_weight(sd[""], sd["_scale"], torch.bfloat16)
    assert torch.equal(again._qdata.view(torch.uint8), qt._qdata.view(torch.uint8))
    assert again._params.scale.item() == qt._params.scale.item()
    p = qt._params.clone().to_device("cpu")
    assert p.scale.device.type == "cpu" and p.orig_shape == (80, 160)


def test_quant_surface_errors_and_host_tensors(quant_mod, cuda_dev):
    with pytest.raises(ValueError, match="2D tensor"):
        quant_mod.FeatherFP8E5M2PackedLayout.quantize(torch.zeros(4, 4, 16))
    with pytest.raises(ValueError, match="K divisible by 16"):
        quant_mod.FeatherFP8E5M2PackedLayout.quantize(torch.zeros(4, 24))
    with pytest.raises(TypeError, match="Expected FeatherFP8E5M2PackedLayout"):
        quant_mod.get_feather_plain_tensors(torch.zeros(2))
    # host tensors are staged through the GPU and come back on the host
    w = torch.randn(32, 64)
    q, params = quant_mod.FeatherFP8E5M2PackedLayout.quantize(w)
    assert q.device.type == "cpu" and q.shape == (4, 32, 16)
    rq, rs = fo.layout_quantize(w.numpy(), "fp32")
    assert np.array_equal(from_torch(q), rq) and np.float32(params.scale.item()) == rs
    e, s = quant_mod.quantize_fp8e5m2_scaled(w)
    assert e.shape == (32, 64) and np.array_equal(from_torch(e), fo.unprepack_transpose(rq))


def test_torch_compile_fullgraph(hip_kernel, native, cuda_dev):
    """The op stays one opaque node under torch.compile(fullgraph=True) (reference:
    test_scaled_mm_hip_autotune_compile.py:42-102), including a bf16 3-D input cast in-graph and scale=None."""
    K, N = 256, 128
    b = torch.randint(0, 0x70, (K // 16, N, 16), dtype=torch.uint8, device=cuda_dev).view(torch.float8_e5m2)
    scale = torch.tensor(0.01, device=cuda_dev)

    def fn(x, b, scale):
        x2 = x.reshape(-1, x.shape[-1]).to(torch.float16)
        return hip_kernel.scaled_mm_hip(x2, b, scale, None, torch.float16)

    x = torch.randn(2, 16, K, device=cuda_dev, dtype=torch.bfloat16)
    eager = fn(x, b, scale)
    compiled = torch.compile(fn, fullgraph=True)(x, b, scale)
    native.check_device_status(cuda_dev)
    assert torch.equal(eager, compiled)
    none_scale = torch.compile(lambda x, b: hip_kernel.scaled_mm_hip(x, b, None, None, torch.float16), fullgraph=True)(eager.new_zeros(16, K), b)
    assert none_scale.shape == (16, N)
