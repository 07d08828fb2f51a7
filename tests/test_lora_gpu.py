"""GPU: un-merged LoRA patches folded into the GEMM's accumulator (`feather_scaled_mm_lora`), against the oracle (the float64
sum of the quantised linear and the patches, rounded once) and against the reference's way of applying them (two GEMMs and an
add to the rounded output per patch, comfy_feather/lora.py:4-35), which differs by its roundings only."""

import importlib

import numpy as np
import pytest
import torch

from oracle import feather_oracle as fo
from tests.util import from_torch, to_torch

pytestmark = pytest.mark.gpu


class _Adapter:
    def __init__(self, b, a, alpha):
        self.weights = (b, a, alpha, None, None, None)


class _PatchFn:
    key = "w"

    def __init__(self, patches):
        self.patches = {self.key: patches}


def _gate(got, ref, dtype, what, fro_limit):
    """The GEMM gate's tolerance with room for the term's own 16-bit operands: |err| <= 1e-2 * rms beyond two ulps."""
    rep = fo.error_report(got, ref, dtype)
    print(f"[lora] {what}: {rep}")
    ulp = 2.0 ** (-7 if dtype == "bf16" else -10)
    r = fo.to_f32(ref, dtype).astype(np.float64)
    err = np.abs(fo.to_f32(got, dtype).astype(np.float64) - r)
    excess = float(np.max(err - 2.0 * ulp * np.maximum(np.abs(r), 1e-30)))
    assert rep["nonfinite_agree"] and rep["fro_rel"] <= fro_limit and excess <= 1e-2 * rep["rms"], (what, rep, excess)


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("M,N,K,ranks", [(300, 520, 1040, (16,)), (700, 1024, 2048, (64, 32)), (128, 256, 512, (8, 4, 100))])
def test_fused_lora_against_the_oracle(pkg, native, hip_kernel, cuda_dev, dtype, M, N, K, ranks):
    lora = importlib.import_module("feather_b200.comfy_feather.lora")
    rng = np.random.default_rng(M + N + sum(ranks))
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    x = torch.from_numpy(rng.standard_normal((M, K), dtype=np.float32)).to(tdt)
    w = (rng.standard_normal((N, K), dtype=np.float32) / np.float32(np.sqrt(K))).astype(np.float32)
    bq, s = fo.make_feather_quantized_weight(w, "fp32", None)
    bias = fo.from_f32(rng.standard_normal((N,), dtype=np.float32), dtype)
    terms, patches = [], []
    for r in ranks:
        A = (rng.standard_normal((r, K), dtype=np.float32) / np.float32(np.sqrt(K))).astype(np.float32)
        Bm = (rng.standard_normal((N, r), dtype=np.float32) / np.float32(np.sqrt(r))).astype(np.float32)
        sp, sm, alpha = 0.8, 1.25, float(2 * r)
        terms.append((A, Bm, sp * sm * alpha / r))
        patches.append((sp, _Adapter(torch.from_numpy(Bm), torch.from_numpy(A), alpha), sm, None, None))
    X = x.to(cuda_dev)
    B = to_torch(bq, "e5m2", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    Bi = to_torch(bias, dtype, cuda_dev)
    fused = lora.fused_lora_operands(X, [_PatchFn(patches)], S)
    assert fused is not None and fused[0].shape[1] % 64 == 0
    y = hip_kernel.scaled_mm_lora(X, B, S, Bi, tdt, tdt, *fused)
    native.check_device_status(cuda_dev)
    a_np = from_torch(x)
    ref = fo.scaled_mm_lora(a_np, bq, s, bias, dtype, terms, a_format=dtype)
    # the term's operands t and lb are fp16 also in a bf16 model (the down-projection is kept in fp32 until it is scaled)
    _gate(from_torch(y), ref, dtype, f"{(M, N, K, ranks)} {dtype}", fro_limit=2e-3 if dtype == "fp16" else 4e-3)
    # the linear alone must be untouched by the extra blocks: zero LoRA matrices give the plain result bit for bit
    zero = [_PatchFn([(1.0, _Adapter(torch.zeros(N, 8), torch.zeros(8, K), None), 1.0, None, None)])]
    t0, lb0 = lora.fused_lora_operands(X, zero, S)
    plain = hip_kernel.scaled_mm_b200(X, B, S, Bi, tdt, tdt)
    with_zero = hip_kernel.scaled_mm_lora(X, B, S, Bi, tdt, tdt, t0, lb0)
    assert torch.equal(plain.view(torch.int16), with_zero.view(torch.int16))


def test_operator_linear_fuses_unmerged_patches(pkg, native, cuda_dev):
    """`FeatherOps.Linear` with low-VRAM LoRA patches: from 64 tokens on the patches ride inside the GEMM; the result stays within
    rounding of the reference's sequence (linear, then y += (x A^T) B^T * strength per patch), and fewer tokens take that sequence."""
    ops_mod = importlib.import_module("feather_b200.comfy_feather.ops")
    lora = importlib.import_module("feather_b200.comfy_feather.lora")
    g = torch.Generator().manual_seed(5)
    K, N, r = 1024, 640, 16
    w = torch.randn((N, K), generator=g) / K ** 0.5
    bias = torch.randn((N,), generator=g) * 0.1
    Ops = ops_mod.feather_ops(out_dtype=torch.bfloat16)
    lin = Ops.Linear(K, N, bias=True)
    lin._load_from_state_dict({"l.weight": w.clone(), "l.bias": bias.clone()}, "l.", {}, True, [], [], [])
    lin = lin.to(cuda_dev)
    A = torch.randn((r, K), generator=g) / K ** 0.5
    Bm = torch.randn((N, r), generator=g) / r ** 0.5
    patch = [_PatchFn([(0.7, _Adapter(Bm, A, 8.0), 1.0, None, None)])]
    for T in (512, 20):
        x = torch.randn((T, K), generator=g).to(torch.bfloat16).to(cuda_dev)
        lin.weight_function = []
        base = lin(x)
        lin.weight_function = patch
        y = lin(x)
        native.check_device_status(cuda_dev)
        assert lin.weight_function is patch
        unfused = lora.apply_lora_patches(x, base.clone(), patch)
        delta = fo.lora_delta(x.float().cpu().numpy(), A.numpy(), Bm.numpy(), 0.7 * 8.0 / r)
        rms = float(np.sqrt(np.mean(delta ** 2)))
        assert rms > 0.1                                                       # the patch is not negligible
        got = (y.float() - base.float()).cpu().numpy()
        assert np.abs(got - delta).max() <= 0.05 * max(rms, 1.0) + 2.0 ** -6 * float(base.float().abs().max())
        assert float((y.float() - unfused.float()).abs().max()) <= 2.0 ** -5 * float(unfused.float().abs().max())
        if T < lora.FUSED_LORA_MIN_TOKENS:
            assert torch.equal(y.view(torch.int16), unfused.view(torch.int16))
