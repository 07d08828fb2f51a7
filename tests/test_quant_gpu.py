"""GPU parity tests of quantise + prepack and its inverses: bit-exact against the oracle and the reference fixtures."""

import numpy as np
import pytest
import torch

from oracle import feather_oracle as fo
from tests.golden import cases
from tests.util import TORCH_DT, from_torch, to_torch

pytestmark = pytest.mark.gpu


def _gpu_quant(native, dev, c):
    if c["dtype"] == "e5m2":
        return from_torch(native.prepack_bytes(to_torch(c["x"], "e5m2", dev))), np.float32(c["scale"])
    if c["path"] == "layout":
        q, s = native.quantize_prepack(to_torch(c["x"], c["dtype"], dev))
    else:
        pm = torch.tensor([float(c["scale"])], dtype=torch.float32, device=dev) if c["scale"] is not None else None
        q, s = native.quantize_prepack(to_torch(c["x"], c["dtype"], dev).float(), premul=pm)
    return from_torch(q), np.float32(s.item())


@pytest.mark.parametrize("name", cases.QUANT_CASES)
def test_quantize_prepack_bit_exact(golden, native, cuda_dev, name):
    c = cases.quant_case(name)
    q, s = _gpu_quant(native, cuda_dev, c)
    assert np.array_equal(cases.canonical_e5m2(q), cases.canonical_e5m2(golden[f"quant/{name}/qdata"]))
    assert s.view(np.uint32) == np.float32(golden[f"quant/{name}/scale"]).view(np.uint32)
    # inverses on the same bytes
    qd = to_torch(q, "e5m2", cuda_dev)
    assert np.array_equal(from_torch(native.unprepack_bytes(qd)), fo.unprepack_transpose(q))
    sc = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    for od in ("fp32", "bf16", "fp16"):
        got = fo.to_f32(from_torch(native.dequantize(qd, sc, TORCH_DT[od])), od)
        ref = fo.to_f32(fo.layout_dequantize(q, s, od), od)
        assert np.array_equal(np.isnan(got), np.isnan(ref))
        assert np.array_equal(np.nan_to_num(got, nan=0.0), np.nan_to_num(ref, nan=0.0))


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("scale", cases.EXHAUSTIVE_SCALES)
def test_exhaustive_16bit_patterns(native, cuda_dev, dtype, scale):
    pats = cases.exhaustive_patterns(dtype)
    q, _ = native.quantize_prepack(to_torch(pats, dtype, cuda_dev), scale=torch.tensor(scale, dtype=torch.float32, device=cuda_dev))
    with np.errstate(all="ignore"):
        ref, _ = fo.layout_quantize(pats, dtype, scale=scale)
    assert np.array_equal(cases.canonical_e5m2(from_torch(q)), cases.canonical_e5m2(ref))


def test_fp32_random_bit_patterns(native, cuda_dev):
    rng = np.random.default_rng(77)
    pats32 = rng.integers(0, 2 ** 32, size=(8192, 16), dtype=np.uint64).astype(np.uint32).view(np.float32)
    q, _ = native.quantize_prepack(to_torch(pats32, "fp32", cuda_dev), scale=torch.tensor(1.0, device=cuda_dev))
    with np.errstate(all="ignore"):
        ref, _ = fo.layout_quantize(pats32, "fp32", scale=1.0)
    assert np.array_equal(cases.canonical_e5m2(from_torch(q)), cases.canonical_e5m2(ref))


def test_fp32_rounding_boundaries(native, cuda_dev):
    """Every e5m2 code, every midpoint between neighbouring codes (the round-to-nearest-even ties) and the fp32 values
    just below and above each, both signs; includes the subnormal codes and the 57344 / 61440 / 65536 overflow edge."""
    codes = np.arange(0, 0x7D, dtype=np.uint16)                      # 0 .. inf
    vals = (codes << 8).view(np.float16).astype(np.float32)          # e5m2 code -> value (top byte of fp16)
    vals[-1] = 65536.0                                               # where inf would sit if e5m2 continued
    mid = ((vals[:-1].astype(np.float64) + vals[1:].astype(np.float64)) / 2).astype(np.float32)
    pts = np.concatenate([vals, mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(np.inf)),
                          np.nextafter(vals[1:], np.float32(0)), np.nextafter(vals, np.float32(np.inf))])
    pts = np.concatenate([pts, -pts]).astype(np.float32)
    pad = (-pts.size) % 64
    pats32 = np.concatenate([pts, np.zeros(pad, np.float32)]).reshape(-1, 64)
    q, _ = native.quantize_prepack(to_torch(pats32, "fp32", cuda_dev), scale=torch.tensor(1.0, device=cuda_dev))
    with np.errstate(all="ignore"):
        ref, _ = fo.layout_quantize(pats32, "fp32", scale=1.0)
    assert np.array_equal(cases.canonical_e5m2(from_torch(q)), cases.canonical_e5m2(ref))


def test_prepack_kn_matches_reference_helper(hip_kernel, cuda_dev):
    b = torch.randint(0, 256, (160, 72), dtype=torch.uint8, device=cuda_dev)
    got = from_torch(hip_kernel.prepack_b_for_scaled_mm(b.view(torch.float8_e5m2)))
    assert np.array_equal(got, fo.prepack_b_for_scaled_mm(from_torch(b)))


def test_bf16_to_fp16_all_patterns(golden, native, cuda_dev):
    """kernel/convert.py contract (test_convert.py:11-15: max diff < 1e-5 vs x.to(float16)); here bit-exact on every pattern."""
    pats = cases.exhaustive_patterns("bf16")
    got = from_torch(native.bf16_to_fp16(to_torch(pats, "bf16", cuda_dev)))
    with np.errstate(all="ignore"):
        ref = fo.from_f32(fo.bf16_bits_to_f32(pats), "fp16")
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(np.where(nan, 0, got.view(np.uint16)), np.where(nan, 0, ref.view(np.uint16)))
    odd = torch.randn(1003, device=cuda_dev).to(torch.bfloat16)     # length not a multiple of 8
    assert torch.equal(native.bf16_to_fp16(odd), odd.to(torch.float16))


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_full_size_round_trips(native, cuda_dev, dtype):
    """Wan ffn weight (13824 x 5120): properties that need no oracle at this size.  prepack/unprepack are inverse
    permutations; quantising the dequantised weight with the same scale reproduces the codes (idempotence)."""
    N, K = 13824, 5120
    g = torch.Generator(device=cuda_dev).manual_seed(1)
    w = (torch.randn((N, K), generator=g, device=cuda_dev) / K ** 0.5).to(TORCH_DT[dtype])
    q, s = native.quantize_prepack(w)
    up = native.unprepack_bytes(q)
    assert torch.equal(native.prepack_bytes(up).view(torch.uint8), q.view(torch.uint8))
    # each code is the RTNE of w/scale: check on a slab against the oracle
    slab = slice(4000, 4064)
    ref_q, ref_s = fo.quantize_fp8e5m2_scaled(from_torch(w[slab]), dtype, scale=np.float32(s.item()))
    assert np.array_equal(from_torch(up[slab]), ref_q)
    amax = w.abs().max().float()
    assert np.float32(s.item()) == np.float32(np.float32(amax.item()) / np.float32(57344.0))
    deq = native.dequantize(q, s.reshape(1), torch.float32)
    q2, s2 = native.quantize_prepack(deq, scale=s)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and s2.item() == s.item()
