"""Seeded synthetic inputs shared by the fixture generator (make_golden.py, which needs the reference checkout) and by the
tests (which do not).  Everything is generated with numpy's PCG64 so the same arrays come out on any machine.

Storage conventions as in oracle/feather_oracle.py: fp16 = float16 arrays, bf16 = uint16 bit patterns, e5m2 = uint8.
"""

import os
import sys

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from oracle import feather_oracle as fo  # noqa: E402

# ------------------------------------------------------------------------------------------------
# GEMM cases on the reference's own test distribution (test_scaled_mm_hip.py:10-13):
#   a = randn -> fp16, b = randn(K,N) -> e5m2, scale = 2.34, bias = randn(N) in the out dtype.
# Verbatim kernel/naive.py is finite here, so its output is the fixture.
# ------------------------------------------------------------------------------------------------
GEMM_REF_CASES = {
    # name: (M, N, K, out_dtype, seed)
    "ref_16x128x128_fp16": (16, 128, 128, "fp16", 11),
    "ref_16x128x128_bf16": (16, 128, 128, "bf16", 12),
    "ref_64x128x512_fp16": (64, 128, 512, "fp16", 13),
    "ref_64x128x512_bf16": (64, 128, 512, "bf16", 14),
    "ref_128x256x128_fp16": (128, 256, 128, "fp16", 15),
    "ref_100x72x80_bf16": (100, 72, 80, "bf16", 16),     # ragged: nothing is a multiple of a tile
}


def gemm_ref_case(name):
    M, N, K, out_dtype, seed = GEMM_REF_CASES[name]
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    b_kn = fo.f32_to_e5m2_bits(rng.standard_normal((K, N), dtype=np.float32))
    bias = fo.from_f32(rng.standard_normal((N,), dtype=np.float32), out_dtype)
    return {
        "a": a,
        "b_kn": b_kn,
        "b_prepacked": fo.prepack_b_for_scaled_mm(b_kn),
        "scale": np.float32(2.34),
        "bias": bias,
        "out_dtype": out_dtype,
    }


# ------------------------------------------------------------------------------------------------
# GEMM cases with fp8e4m3fn weights (kernel/naive.py handles them through the same `b.to(float16)`; the reference's kernel
# has an approximate e4m3 upcast, hip_kernel.cu:83-99).  Weights are drawn as byte codes, so no fp32 -> e4m3 cast is involved.
# ------------------------------------------------------------------------------------------------
GEMM_E4M3_CASES = {
    # name: (M, N, K, out_dtype, seed)
    "e4m3_48x256x256_bf16": (48, 256, 256, "bf16", 41),        # random finite codes
    "e4m3_all_codes_fp16": (8, 256, 16, "fp16", 42),           # column n multiplies by code n alone: every value, subnormals and the two NaN codes
}


def gemm_e4m3_case(name):
    M, N, K, out_dtype, seed = GEMM_E4M3_CASES[name]
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    if "all_codes" in name:
        b_kn = np.zeros((K, N), dtype=np.uint8)
        b_kn[0, :] = np.arange(256, dtype=np.uint8)
        scale = np.float32(0.5)
    else:
        b_kn = rng.integers(0, 256, size=(K, N), dtype=np.uint8)
        b_kn = np.where((b_kn & 0x7F) == 0x7F, np.uint8(0x3A), b_kn).astype(np.uint8)      # no NaN codes here
        scale = np.float32(2.0 ** -6)
    bias = fo.from_f32(rng.standard_normal((N,), dtype=np.float32), out_dtype)
    return {"a": a, "b_kn": b_kn, "b_prepacked": fo.prepack_b_for_scaled_mm(b_kn), "scale": scale, "bias": bias, "out_dtype": out_dtype}


# ------------------------------------------------------------------------------------------------
# GEMM cases on the benchmark distribution: A ~ N(0,1) fp16, W ~ N(0, 1/sqrt(K)) quantised through the loader path
# (fp32 in, scale = amax/57344).  Verbatim naive.py overflows fp16 here; the fixture is the same op sequence with an
# fp32 product, evaluated with torch in make_golden.py.
# ------------------------------------------------------------------------------------------------
GEMM_BENCH_CASES = {
    # name: (M, N, K, out_dtype, with_bias, seed)
    "config1_256x1024x1024_bf16": (256, 1024, 1024, "bf16", False, 0),
    "bench_48x384x320_fp16": (48, 384, 320, "fp16", True, 21),
    "bench_1x256x512_bf16": (1, 256, 512, "bf16", False, 22),
}


def gemm_bench_case(name):
    M, N, K, out_dtype, with_bias, seed = GEMM_BENCH_CASES[name]
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((N, K), dtype=np.float32) / np.float32(np.sqrt(K))).astype(np.float32)
    b_prepacked, scale = fo.make_feather_quantized_weight(w, "fp32", None)
    bias = fo.from_f32(rng.standard_normal((N,), dtype=np.float32), out_dtype) if with_bias else None
    return {"a": a, "w": w, "b_prepacked": b_prepacked, "scale": scale, "bias": bias, "out_dtype": out_dtype}


# ------------------------------------------------------------------------------------------------
# quantise + prepack cases
# ------------------------------------------------------------------------------------------------
def _weights(rng, n, k, std):
    return (rng.standard_normal((n, k), dtype=np.float32) * np.float32(std)).astype(np.float32)


def quant_case(name):
    """Returns dict(x=storage array, dtype=..., path='layout'|'loader', scale=given checkpoint scale or None)."""
    rng = np.random.default_rng(abs(hash_name(name)))
    if name == "q_fp32_normal":
        return {"x": _weights(rng, 96, 256, 0.03), "dtype": "fp32", "path": "layout", "scale": None}
    if name == "q_bf16_normal":
        return {"x": fo.f32_to_bf16_bits(_weights(rng, 64, 128, 0.05)), "dtype": "bf16", "path": "layout", "scale": None}
    if name == "q_fp16_clamped":       # amax < 0.875: 1/scale is clamped to 65504 (quant.py:56-58)
        return {"x": _weights(rng, 64, 128, 0.03).astype(np.float16), "dtype": "fp16", "path": "layout", "scale": None}
    if name == "q_fp16_large":         # amax > 0.875: no clamp
        return {"x": _weights(rng, 40, 64, 30.0).astype(np.float16), "dtype": "fp16", "path": "layout", "scale": None}
    if name == "q_fp32_zeros":         # scale 0 -> 1 (quant.py:55)
        return {"x": np.zeros((32, 32), dtype=np.float32), "dtype": "fp32", "path": "layout", "scale": None}
    if name == "q_fp32_edges":
        x = _weights(rng, 32, 64, 1.0)
        x[0, :8] = [57344.0, -57344.0, 61439.0, 61440.0, 65535.0, 1e-8, -1e-8, 0.0]
        x[1, :8] = [np.inf, -np.inf, 3.0e38, -3.0e38, 1.5e-5, 2.0 ** -16, 2.0 ** -17, -(2.0 ** -17)]
        return {"x": x, "dtype": "fp32", "path": "layout", "scale": None}
    if name == "q_fp32_tiny":          # everything lands in the e5m2 subnormal range except the amax element
        x = _weights(rng, 32, 48, 1e-6)
        x[3, 5] = 1.0
        return {"x": x, "dtype": "fp32", "path": "layout", "scale": None}
    if name == "q_bf16_ragged":        # N not a multiple of the kernel tile, K = 16
        return {"x": fo.f32_to_bf16_bits(_weights(rng, 37, 16, 2.0)), "dtype": "bf16", "path": "layout", "scale": None}
    if name == "loader_fp32_scaled":   # loader path: weight.float() * checkpoint_scale, recalculated scale (quant.py:128-129)
        return {"x": _weights(rng, 64, 128, 40.0), "dtype": "fp32", "path": "loader", "scale": np.float32(0.0123)}
    if name == "loader_fp16_noscale":  # loader upcasts fp16 to fp32 first, so no fp16 clamp
        return {"x": _weights(rng, 64, 128, 0.03).astype(np.float16), "dtype": "fp16", "path": "loader", "scale": None}
    if name == "loader_bf16_scaled":
        return {"x": fo.f32_to_bf16_bits(_weights(rng, 48, 96, 3.0)), "dtype": "bf16", "path": "loader", "scale": np.float32(0.5)}
    if name == "loader_e5m2_passthrough":   # already-quantised checkpoint: prepack only, keep scale (quant.py:125-126)
        x = rng.integers(0, 256, size=(80, 160), dtype=np.uint8)
        return {"x": x, "dtype": "e5m2", "path": "loader", "scale": np.float32(0.00037)}
    raise KeyError(name)


QUANT_CASES = [
    "q_fp32_normal", "q_bf16_normal", "q_fp16_clamped", "q_fp16_large", "q_fp32_zeros", "q_fp32_edges", "q_fp32_tiny",
    "q_bf16_ragged", "loader_fp32_scaled", "loader_fp16_noscale", "loader_bf16_scaled", "loader_e5m2_passthrough",
]  # fmt: skip


def hash_name(name):
    h = 0
    for ch in name:
        h = (h * 131 + ord(ch)) % 2147483647
    return h


# exhaustive cast sweeps: every 16-bit pattern of the source dtype with a given (not recalculated) scale
EXHAUSTIVE_SCALES = [1.0, 0.37, 2.0 ** -10, 1536.0]


def exhaustive_patterns(dtype):
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16).reshape(4096, 16)
    if dtype == "fp16":
        return bits.view(np.float16)
    if dtype == "bf16":
        return bits
    raise ValueError(dtype)


def canonical_e5m2(bits):
    """NaN payload/sign is not part of the contract: map every e5m2 NaN (0x7D-0x7F, 0xFD-0xFF) to 0x7F."""
    b = np.asarray(bits, dtype=np.uint8)
    is_nan = (b & 0x7F) > 0x7C
    return np.where(is_nan, np.uint8(0x7F), b)
