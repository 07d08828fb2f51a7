"""CPU oracle for the FeatherOps mixed-precision linear path.  TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference's algorithm (woct0rdho/ComfyUI-FeatherOps), used as the checker by tests/,
by __graft_entry__.smoke() and by bench.py's cpu_baseline leg.  Nothing in the shipped package imports it, and it is
never the thing that is measured or shipped as the product.

Parity status: PINNED.  tests/golden/make_golden.py runs the reference's own kernel/naive.py and
comfy_feather/quant.py (imported from a checkout of the reference) on the seeded inputs of tests/golden/cases.py,
asserts this oracle reproduces them, and stores the reference outputs as fixtures; tests/test_oracle_golden.py re-checks
the oracle against those fixtures without the reference present.

Each function cites the reference file:line it restates.  Arrays: fp16 tensors are numpy float16; bf16 tensors are
uint16 bit patterns (numpy has no bf16); e5m2 tensors are uint8 bit patterns; fp32 is float32.
"""

import numpy as np

E5M2_MAX = np.float32(57344.0)     # torch.finfo(torch.float8_e5m2).max
FP16_MAX = np.float32(65504.0)


# ------------------------------------------------------------------------------------------------
# dtype helpers
# ------------------------------------------------------------------------------------------------
def bf16_bits_to_f32(bits):
    """uint16 bf16 patterns -> float32 (exact)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(x):
    """float32 -> bf16 bit patterns, round-to-nearest-even, NaN -> 0x7FC0 (what torch's fp32->bf16 cast does)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)
    out = rounded.astype(np.uint16)
    return np.where(np.isnan(x), np.uint16(0x7FC0), out)


def e5m2_bits_to_f32(bits):
    """uint8 e5m2 patterns -> float32 (exact): an e5m2 value is the top byte of the fp16 with the same value.

    This is the upcast the GEMM applies to weights (reference: hip_kernel.cu:105-112, naive.py:22 `b.to(float16)`)."""
    b = np.asarray(bits, dtype=np.uint8)
    return (b.astype(np.uint16) << np.uint16(8)).view(np.float16).astype(np.float32)


def e4m3_bits_to_f32(bits):
    """uint8 fp8e4m3fn patterns -> float32 (exact).  Sign, 4 exponent bits (bias 7), 3 mantissa bits; exponent field 0 is
    subnormal (m * 2^-9); 0x7F / 0xFF are NaN and there is no infinity.  This is `b.to(torch.float16)` of naive.py:22 for a
    float8_e4m3fn weight (the reference's kernel approximates it, hip_kernel.cu:83-99; naive.py is exact)."""
    b = np.asarray(bits, dtype=np.uint8).astype(np.int32)
    e, m = (b >> 3) & 0xF, b & 0x7
    mag = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float64)))
    mag = np.where((b & 0x7F) == 0x7F, np.nan, mag)
    return np.where(b & 0x80, -mag, mag).astype(np.float32)


def f32_to_e5m2_bits(x):
    """float32 -> e5m2 bit patterns: round-to-nearest-even, overflow to inf (no saturation), NaN -> sign|0x7F.

    This is the cast `x.to(torch.float8_e5m2)` performs (reference call site: quant.py:73)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    sign = ((u >> np.uint32(24)) & np.uint32(0x80)).astype(np.uint8)
    a = u & np.uint32(0x7FFFFFFF)
    out = np.zeros(x.shape, dtype=np.uint32)
    big = a >= np.uint32(0x47800000)                       # >= 65536, inf, NaN
    out = np.where(big, np.where(a > np.uint32(0x7F800000), np.uint32(0x7F), np.uint32(0x7C)), out)
    small = a < np.uint32(0x38800000)                      # < 2^-14: e5m2 subnormals, spacing 2^-16
    with np.errstate(invalid="ignore", over="ignore"):
        sub = np.rint(a.view(np.float32).astype(np.float64) * 65536.0)   # rint = ties-to-even
    sub = np.where(small, sub, 0.0).astype(np.uint32)
    out = np.where(small, sub, out)
    mid = ~big & ~small
    am = np.where(mid, a, np.uint32(0x38800000))
    am = am + np.uint32(0x000FFFFF) + ((am >> np.uint32(21)) & np.uint32(1))
    norm = (am >> np.uint32(21)) - np.uint32(112 << 2)
    out = np.where(mid, norm, out)
    return out.astype(np.uint8) | sign


def to_f32(x, dtype):
    """Values of a tensor stored as `dtype` ('fp32' | 'bf16' | 'fp16') as float32."""
    if dtype == "fp32":
        return np.asarray(x, dtype=np.float32)
    if dtype == "fp16":
        return np.asarray(x, dtype=np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(x)
    raise ValueError(dtype)


def round_to(x, dtype):
    """Round float32 values to `dtype` (RTNE) and return them as float32 again."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "fp32":
        return x
    if dtype == "fp16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits(x))
    raise ValueError(dtype)


def from_f32(x, dtype):
    """float32 -> storage array of `dtype` (RTNE)."""
    if dtype == "fp32":
        return np.asarray(x, dtype=np.float32)
    if dtype == "fp16":
        with np.errstate(over="ignore"):
            return np.asarray(x, dtype=np.float32).astype(np.float16)
    if dtype == "bf16":
        return f32_to_bf16_bits(x)
    raise ValueError(dtype)


# ------------------------------------------------------------------------------------------------
# weight layout  (quant.py:11-19, hip_kernel.py:170-171)
# ------------------------------------------------------------------------------------------------
def prepack_transpose(x):
    """(N, K) -> (K/16, N, 16): out[kb, n, j] = x[n, 16 kb + j].   quant.py:11-13"""
    n, k = x.shape
    return np.ascontiguousarray(x.reshape(n, k // 16, 16).transpose(1, 0, 2))


def unprepack_transpose(x):
    """(K/16, N, 16) -> (N, K).   quant.py:17-19"""
    kb, n, _ = x.shape
    return np.ascontiguousarray(x.transpose(1, 0, 2).reshape(n, kb * 16))


def prepack_b_for_scaled_mm(b):
    """(K, N) -> (K/16, N, 16): out[kb, n, j] = b[16 kb + j, n].   hip_kernel.py:170-171"""
    k, n = b.shape
    return np.ascontiguousarray(b.reshape(k // 16, 16, n).transpose(0, 2, 1))


# ------------------------------------------------------------------------------------------------
# quantise  (quant.py:52-74, 77-96, 116-136)
# ------------------------------------------------------------------------------------------------
def compute_scale(x_f32, dtype):
    """amax|x| / 57344 in fp32; 0 -> 1; for fp16 sources 1/scale is clamped to the fp16 range.   quant.py:53-58"""
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        amax = np.max(np.abs(np.asarray(x_f32, dtype=np.float32))).astype(np.float32)
        scale = np.float32(amax / E5M2_MAX)
        if scale == 0:
            scale = np.float32(1.0)
        if dtype not in ("fp32", "bf16"):
            inv = np.float32(np.float32(1.0) / scale)
            inv = np.float32(np.clip(inv, -FP16_MAX, FP16_MAX))
            scale = np.float32(np.float32(1.0) / inv)
    return np.float32(scale)


def quantize_fp8e5m2_scaled(x, dtype, scale=None):
    """x (storage array of `dtype`, shape (N,K)) -> (e5m2 bits (N,K), fp32 scale).   quant.py:52-74, seed None/0 branch

    inv_scale = (1/scale) rounded to x's dtype; the product x*inv_scale is rounded to x's dtype; then RTNE to e5m2."""
    xf = to_f32(x, dtype)
    scale = compute_scale(xf, dtype) if scale is None else np.float32(scale)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        inv = round_to(np.float32(np.float32(1.0) / scale), dtype)
        y = round_to(xf * np.float32(inv), dtype)
    return f32_to_e5m2_bits(y), scale


def layout_quantize(x, dtype, scale=None):
    """FeatherFP8E5M2PackedLayout.quantize: quantise then prepack.   quant.py:80-96"""
    if x.ndim != 2:
        raise ValueError(f"Feather FP8 packed weights require a 2D tensor, got {x.ndim}D")
    if x.shape[1] % 16 != 0:
        raise ValueError(f"Feather FP8 packed weights require K divisible by 16, got {tuple(x.shape)}")
    q, s = quantize_fp8e5m2_scaled(x, dtype, scale)
    return prepack_transpose(q), s


def make_feather_quantized_weight(weight, dtype, scale=None):
    """Loader path.   quant.py:116-136
    e5m2 checkpoints (dtype == 'e5m2') are only prepacked and keep the given scale; anything else is upcast to fp32,
    multiplied by the checkpoint scale and re-quantised with a recalculated scale."""
    s = np.float32(1.0) if scale is None else np.float32(scale)
    if dtype == "e5m2":
        return prepack_transpose(np.asarray(weight, dtype=np.uint8)), s
    with np.errstate(invalid="ignore", over="ignore"):
        wf = (to_f32(weight, dtype) * s).astype(np.float32)
    q, s2 = quantize_fp8e5m2_scaled(wf, "fp32", None)
    return prepack_transpose(q), s2


def layout_dequantize(qdata, scale, orig_dtype):
    """FeatherFP8E5M2PackedLayout.dequantize: unprepack -> fp32 * scale -> orig dtype.   quant.py:98-102"""
    w = e5m2_bits_to_f32(unprepack_transpose(qdata))
    with np.errstate(invalid="ignore", over="ignore"):
        return from_f32((w * np.float32(scale)).astype(np.float32), orig_dtype)


# ------------------------------------------------------------------------------------------------
# GEMM  (naive.py:4-41)
# ------------------------------------------------------------------------------------------------
def scaled_mm(a, b_prepacked, scale, bias, out_dtype, product="fp32", b_format="e5m2", a_format="fp16", final_dtype=None):
    """out = cvt((a @ up(b)) * scale) + bias, the math of kernel/naive.py:13-41 with b_prepacked=True.

    a            float16 (M,K); with a_format='bf16' uint16 bf16 patterns that are multiplied as they are (the typed entry
                 point's semantics; naive.py:21 would cast them to fp16 first, which `a_format='bf16_cast_first'` does)
    b_prepacked  uint8 weight bits (K/16, N, 16), e5m2 or (b_format='e4m3') fp8e4m3fn
    scale        float or None;  bias: storage array of out_dtype, shape (N,), or None
    out_dtype    'fp16' | 'bf16'
    product      'fp32': the product keeps fp32 precision before `* scale` (what a fp32-accumulating kernel computes;
                         evaluated here in float64 and rounded once to fp32);
                 'fp16': the product is rounded to fp16 first, as naive.py:20-23 does verbatim (it overflows to inf
                         once |a @ b| exceeds 65504, which happens at amax/57344 scales).
    final_dtype  None, or the 16-bit dtype the result is cast to afterwards (`y.to(dtype)`, comfy_feather/ops.py:103)
    Returns the storage array of final_dtype or out_dtype, shape (M,N).
    """
    kb, n, _ = b_prepacked.shape
    w_bits = b_prepacked.transpose(0, 2, 1).reshape(kb * 16, n)                    # naive.py:13-16
    w = e5m2_bits_to_f32(w_bits) if b_format == "e5m2" else e4m3_bits_to_f32(w_bits)
    if a_format == "fp16":
        a64 = np.asarray(a, dtype=np.float16).astype(np.float64)
    elif a_format == "bf16":
        a64 = bf16_bits_to_f32(a).astype(np.float64)
    elif a_format == "bf16_cast_first":
        with np.errstate(over="ignore"):
            a64 = bf16_bits_to_f32(a).astype(np.float16).astype(np.float64)          # naive.py:21
    else:
        raise ValueError(a_format)
    with np.errstate(invalid="ignore", over="ignore"):
        acc = (a64 @ w.astype(np.float64)).astype(np.float32)
        if product == "fp16":
            acc = acc.astype(np.float16).astype(np.float32)                       # naive.py:20-23
        elif product != "fp32":
            raise ValueError(product)
        if scale is not None:
            acc = (acc * np.float32(scale)).astype(np.float32)                    # naive.py:24-28
        out = round_to(acc, out_dtype)                                            # naive.py:34
        if bias is not None:
            out = round_to(out + to_f32(bias, out_dtype)[None, :], out_dtype)     # naive.py:35-40
        if final_dtype is not None and final_dtype != out_dtype:
            return from_f32(round_to(out, final_dtype), final_dtype)
    return from_f32(out, out_dtype)


def scaled_mm_lora(a, b_prepacked, scale, bias, out_dtype, terms, a_format="fp16", final_dtype=None):
    """The linear with un-merged LoRA terms added before the rounding: cvt((a @ up(b)) * scale + sum_p (a A_p^T) B_p^T s_p) + bias.
    `terms` is a list of (lora_a [r,K], lora_b [N,r], strength) as float arrays.  This is what folding the patches of
    comfy_feather/lora.py:4-35 into the GEMM computes; the reference adds each patch to the rounded output instead, so the two
    differ by roundings only.  Evaluated in float64, rounded once."""
    kb, n, _ = b_prepacked.shape
    w = e5m2_bits_to_f32(b_prepacked.transpose(0, 2, 1).reshape(kb * 16, n)).astype(np.float64)
    a64 = np.asarray(a, dtype=np.float16).astype(np.float64) if a_format == "fp16" else bf16_bits_to_f32(a).astype(np.float64)
    acc = a64 @ w
    if scale is not None:
        acc = acc * float(scale)
    for lora_a, lora_b, strength in terms:
        acc = acc + ((a64 @ np.asarray(lora_a, dtype=np.float64).T) @ np.asarray(lora_b, dtype=np.float64).T) * float(strength)
    with np.errstate(invalid="ignore", over="ignore"):
        out = round_to(acc.astype(np.float32), out_dtype)
        if bias is not None:
            out = round_to(out + to_f32(bias, out_dtype)[None, :], out_dtype)
        if final_dtype is not None and final_dtype != out_dtype:
            return from_f32(round_to(out, final_dtype), final_dtype)
    return from_f32(out, out_dtype)


def lora_delta(x_f32, lora_a, lora_b, lora_scale):
    """(x A^T) B^T * s in float64: the un-merged LoRA term of comfy_feather/lora.py:30-33 (checker for its tests)."""
    t = np.asarray(x_f32, dtype=np.float64) @ np.asarray(lora_a, dtype=np.float64).T
    return (t @ np.asarray(lora_b, dtype=np.float64).T) * float(lora_scale)


# ------------------------------------------------------------------------------------------------
# comparison helpers shared by the tests
# ------------------------------------------------------------------------------------------------
def ulp_distance_16(x_bits, y_bits):
    """Distance in representable values between two 16-bit float patterns of the same format (sign-magnitude aware)."""
    def key(b):
        b = np.asarray(b).view(np.uint16).astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    return np.abs(key(x_bits) - key(y_bits))


def error_report(out, ref, out_dtype, bias=None):
    """max|err|, rms(ref), Frobenius-relative error and max ulp distance between two outputs of `out_dtype`.

    `bias` (the [N] bias that was added, as float32 values): the output is cvt(acc * scale) + bias with the rounding BEFORE
    the bias add (naive.py:34-40) and a second rounding after it.  A one-ulp rounding-boundary flip of the first rounding has
    the size of an ulp of the pre-bias value (which can be twice the ulp of the final value when the add crosses a binade
    downwards), and the second rounding can send the two candidates to neighbours that are one more ulp apart.  With `bias`
    given, the allowance is therefore two ulps, taken at the larger of the pre- and post-bias magnitudes."""
    o = to_f32(out, out_dtype).astype(np.float64)
    r = to_f32(ref, out_dtype).astype(np.float64)
    finite = np.isfinite(r) & np.isfinite(o)
    with np.errstate(invalid="ignore"):
        same_nonfinite = np.array_equal(np.isnan(r), np.isnan(o)) and np.array_equal(np.where(np.isinf(r), np.sign(r), 0.0), np.where(np.isinf(o), np.sign(o), 0.0))
    with np.errstate(invalid="ignore"):
        d = np.where(finite, o - r, 0.0)
    rms = float(np.sqrt(np.mean(np.where(finite, r, 0.0) ** 2)))
    fro = float(np.linalg.norm(d) / max(np.linalg.norm(np.where(finite, r, 0.0)), 1e-6))
    ob = np.asarray(out).view(np.uint16)
    rb = np.asarray(ref).view(np.uint16)
    ulp = int(np.max(np.where(finite, ulp_distance_16(ob, rb), 0))) if ob.size else 0
    # error beyond one unit in the last place of the reference value (two correct fp32-accumulating evaluations can
    # round a value sitting on a rounding boundary to different neighbours)
    mant = 10 if out_dtype == "fp16" else 7
    with np.errstate(divide="ignore"):
        mag = np.abs(np.where(finite, r, 1.0))
        if bias is not None:
            mag = np.maximum(mag, np.abs(np.where(finite, r - np.asarray(bias, dtype=np.float64)[None, :], 1.0)))
        ulp_at = np.where(mag != 0, 2.0 ** (np.floor(np.log2(np.maximum(mag, 1e-300))) - mant), 0.0) * (2.0 if bias is not None else 1.0)
    excess = float(np.max(np.where(finite, np.abs(d) - ulp_at, 0.0))) if d.size else 0.0
    return {
        "max_excess_over_1ulp": max(excess, 0.0),
        "max_abs": float(np.max(np.abs(d))) if d.size else 0.0,
        "rms": rms,
        "fro_rel": fro,
        "max_ulp": ulp,
        "mismatches": int(np.sum(np.where(finite, ob != rb, False))),
        "nonfinite_agree": bool(same_nonfinite),
    }
