"""Generates tests/golden/golden.npz by running the REFERENCE's own code on the seeded inputs of cases.py.

Needs a checkout of woct0rdho/ComfyUI-FeatherOps (default: a directory named `reference` beside this repository, override
with FEATHER_REFERENCE_DIR) and torch on CPU.  The reference modules are imported by file path (never copied): kernel/naive.py as is, comfy_feather/quant.py under the
test double of the `comfy` package in tests/fake_comfy.  While generating, it also asserts that the numpy oracle
(oracle/feather_oracle.py) reproduces every reference output, which is what pins the oracle.

    python tests/golden/make_golden.py
"""

import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "fake_comfy"))

from oracle import feather_oracle as fo  # noqa: E402
from tests.golden import cases  # noqa: E402

REF = os.environ.get("FEATHER_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference"))


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


naive = load_by_path("ref_naive", os.path.join(REF, "kernel", "naive.py"))
quant = load_by_path("ref_quant", os.path.join(REF, "comfy_feather", "quant.py"))

TORCH_DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "e5m2": torch.float8_e5m2}


def to_torch(x, dtype):
    x = np.ascontiguousarray(x)
    if dtype == "fp32":
        return torch.from_numpy(x.astype(np.float32))
    if dtype == "fp16":
        return torch.from_numpy(x.astype(np.float16))
    if dtype == "bf16":
        return torch.from_numpy(x.astype(np.uint16).view(np.int16)).view(torch.bfloat16)
    if dtype == "e5m2":
        return torch.from_numpy(x.astype(np.uint8)).view(torch.float8_e5m2)
    raise ValueError(dtype)


def from_torch(t):
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float8_e5m2:
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def sha(x):
    return hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest()


def main():
    torch.manual_seed(0)
    out = {}
    report = []

    # ---- GEMM, reference test distribution: verbatim scaled_mm_naive ---------------------------------------
    for name in cases.GEMM_REF_CASES:
        c = cases.gemm_ref_case(name)
        a = to_torch(c["a"], "fp16")
        b_kn = to_torch(c["b_kn"], "e5m2")
        # the e5m2 bits came from the oracle's cast: the reference's cast must agree
        rng = np.random.default_rng(cases.GEMM_REF_CASES[name][4])
        rng.standard_normal(c["a"].shape, dtype=np.float32)
        b_f32 = rng.standard_normal(c["b_kn"].shape, dtype=np.float32)
        assert np.array_equal(from_torch(torch.from_numpy(b_f32).to(torch.float8_e5m2)), c["b_kn"]), name
        b_pp = to_torch(c["b_prepacked"], "e5m2")
        scale = torch.tensor(float(c["scale"]), dtype=torch.float32)
        bias = to_torch(c["bias"], c["out_dtype"])
        ref = naive.scaled_mm_naive(a, b_pp, scale, bias, TORCH_DT[c["out_dtype"]], b_prepacked=True)
        ref_unpacked = naive.scaled_mm_naive(a, b_kn, scale, bias, TORCH_DT[c["out_dtype"]], b_prepacked=False)
        assert torch.equal(ref.view(torch.int16), ref_unpacked.view(torch.int16)), "prepack_b_for_scaled_mm restatement"
        ref_np = from_torch(ref)
        out[f"gemm/{name}/out"] = ref_np
        for product in ("fp16", "fp32"):
            mine = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product=product)
            rep = fo.error_report(mine, ref_np, c["out_dtype"])
            report.append((name, product, rep))
            assert rep["nonfinite_agree"]
            assert rep["fro_rel"] <= 0.01, (name, product, rep)

    # ---- GEMM with fp8e4m3fn weights: verbatim scaled_mm_naive on a float8_e4m3fn tensor ------------------------------
    codes = torch.arange(256, dtype=torch.uint8)
    assert np.array_equal(np.nan_to_num(codes.view(torch.float8_e4m3fn).float().numpy(), nan=12345.0),
                          np.nan_to_num(fo.e4m3_bits_to_f32(codes.numpy()), nan=12345.0)), "e4m3 decode restatement"
    for name in cases.GEMM_E4M3_CASES:
        c = cases.gemm_e4m3_case(name)
        a = to_torch(c["a"], "fp16")
        b_pp = torch.from_numpy(c["b_prepacked"]).view(torch.float8_e4m3fn)
        scale = torch.tensor(float(c["scale"]), dtype=torch.float32)
        bias = to_torch(c["bias"], c["out_dtype"])
        ref_np = from_torch(naive.scaled_mm_naive(a, b_pp, scale, bias, TORCH_DT[c["out_dtype"]], b_prepacked=True))
        out[f"gemm/{name}/out"] = ref_np
        for product in ("fp16", "fp32"):
            mine = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product=product, b_format="e4m3")
            rep = fo.error_report(mine, ref_np, c["out_dtype"])
            report.append((name, product, rep))
            assert rep["nonfinite_agree"] and rep["fro_rel"] <= 0.01, (name, product, rep)

    # ---- GEMM, benchmark distribution: verbatim naive overflows; fixture = same ops with an fp32 product ---------
    for name in cases.GEMM_BENCH_CASES:
        c = cases.gemm_bench_case(name)
        a = to_torch(c["a"], "fp16")
        b_pp = to_torch(c["b_prepacked"], "e5m2")
        scale = torch.tensor(float(c["scale"]), dtype=torch.float32)
        bias = to_torch(c["bias"], c["out_dtype"]) if c["bias"] is not None else None
        verb = naive.scaled_mm_naive(a, b_pp, scale, bias, TORCH_DT[c["out_dtype"]], b_prepacked=True)
        n_inf = int(torch.isinf(verb.float()).sum())
        out[f"gemm/{name}/verbatim_inf_count"] = np.int64(n_inf)
        # the reference's op order (naive.py:13-40) with the product kept in fp32
        kb, N, _ = b_pp.shape
        b = b_pp.permute(0, 2, 1).reshape(kb * 16, N)
        prod = a.to(torch.float16).float() @ b.to(torch.float16).float()
        prod *= scale
        ref = prod.to(TORCH_DT[c["out_dtype"]])
        if bias is not None:
            ref += bias[None, :]
        ref_np = from_torch(ref)
        # keep the fixture small: first and last 8 rows (or everything when M <= 16)
        M = ref_np.shape[0]
        rows = np.arange(M) if M <= 16 else np.concatenate([np.arange(8), np.arange(M - 8, M)])
        out[f"gemm/{name}/rows"] = rows.astype(np.int64)
        out[f"gemm/{name}/out_rows"] = ref_np[rows]
        out[f"gemm/{name}/scale"] = np.float32(c["scale"])
        mine = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product="fp32")
        rep = fo.error_report(mine, ref_np, c["out_dtype"])
        report.append((name, "fp32", rep))
        # two fp32-accumulating evaluations may differ by one ulp of the out dtype on a few elements
        assert rep["max_excess_over_1ulp"] <= 1e-5 * rep["rms"] and rep["fro_rel"] < 1e-3, (name, rep)
        # and the weight itself must be the reference's loader-path quantisation, bit for bit
        qt = quant.make_feather_quantized_weight(torch.from_numpy(c["w"]), None, TORCH_DT[c["out_dtype"]])
        assert np.array_equal(from_torch(qt._qdata), c["b_prepacked"]), name
        assert np.float32(qt._params.scale.item()) == c["scale"], name

    # ---- quantise + prepack ---------------------------------------------------------------------
    for name in cases.QUANT_CASES:
        c = cases.quant_case(name)
        x = to_torch(c["x"], c["dtype"])
        if c["path"] == "layout":
            q, params = quant.FeatherFP8E5M2PackedLayout.quantize(x.clone())
            s = params.scale
            mq, ms = fo.layout_quantize(c["x"], c["dtype"])
        else:
            given = None if c["scale"] is None else torch.tensor(float(c["scale"]), dtype=torch.float32)
            qt = quant.make_feather_quantized_weight(x.clone(), given, torch.bfloat16)
            q, s = qt._qdata, qt._params.scale
            mq, ms = fo.make_feather_quantized_weight(c["x"], c["dtype"], c["scale"])
        q_np = from_torch(q)
        s_np = np.float32(s.item())
        assert np.array_equal(cases.canonical_e5m2(q_np), cases.canonical_e5m2(mq)), (name, int((q_np != mq).sum()))
        assert s_np.view(np.uint32) == np.float32(ms).view(np.uint32) or (np.isnan(s_np) and np.isnan(ms)), (name, s_np, ms)
        out[f"quant/{name}/qdata"] = q_np
        out[f"quant/{name}/scale"] = s_np
        # inverse directions on the same data
        params = quant.FeatherFP8E5M2PackedLayout.Params(scale=s.float(), orig_dtype=torch.float32, orig_shape=tuple(x.shape))
        for od in ("fp32", "bf16", "fp16"):
            p2 = quant.FeatherFP8E5M2PackedLayout.Params(scale=s.float(), orig_dtype=TORCH_DT[od], orig_shape=tuple(x.shape))
            deq = from_torch(quant.FeatherFP8E5M2PackedLayout.dequantize(q, p2))
            mine = fo.layout_dequantize(q_np, s_np, od)
            same = np.array_equal(np.asarray(deq).view(np.uint8), np.asarray(mine).view(np.uint8)) or np.allclose(
                fo.to_f32(deq, od), fo.to_f32(mine, od), rtol=0, atol=0, equal_nan=True
            )
            assert same, (name, od)
            out[f"quant/{name}/dequant_{od}_sha"] = np.array(sha(np.nan_to_num(fo.to_f32(deq, od), nan=12345.0)))
        sd = quant.FeatherFP8E5M2PackedLayout.state_dict_tensors(q, params)
        assert np.array_equal(from_torch(sd[""].contiguous()), fo.unprepack_transpose(q_np)), name

    # ---- exhaustive cast sweeps -------------------------------------------------------------------------
    for dtype in ("fp16", "bf16"):
        pats = cases.exhaustive_patterns(dtype)
        x = to_torch(pats, dtype)
        for sc in cases.EXHAUSTIVE_SCALES:
            with np.errstate(all="ignore"):
                q, s = quant.quantize_fp8e5m2_scaled(x.clone(), scale=sc)
                mq, ms = fo.quantize_fp8e5m2_scaled(pats, dtype, scale=sc)
            q_np = cases.canonical_e5m2(from_torch(q))
            assert np.array_equal(q_np, cases.canonical_e5m2(mq)), (dtype, sc, int((q_np != cases.canonical_e5m2(mq)).sum()))
            out[f"exhaustive/{dtype}/{sc!r}/sha"] = np.array(sha(q_np))
    # fp32: a dense sample of bit patterns around every e5m2 rounding boundary plus random patterns
    rng = np.random.default_rng(77)
    pats32 = rng.integers(0, 2 ** 32, size=(8192, 16), dtype=np.uint64).astype(np.uint32).view(np.float32)
    q, s = quant.quantize_fp8e5m2_scaled(torch.from_numpy(pats32.copy()), scale=1.0)
    mq, _ = fo.quantize_fp8e5m2_scaled(pats32, "fp32", scale=1.0)
    assert np.array_equal(cases.canonical_e5m2(from_torch(q)), cases.canonical_e5m2(mq))
    out["exhaustive/fp32/random_bits/sha"] = np.array(sha(cases.canonical_e5m2(from_torch(q))))

    # ---- dequantise: all 256 codes ------------------------------------------------------------------
    codes = np.arange(256, dtype=np.uint8).reshape(16, 16)
    up = from_torch(to_torch(codes, "e5m2").to(torch.float16))
    assert np.array_equal(np.nan_to_num(up.astype(np.float32), nan=7.0), np.nan_to_num(fo.e5m2_bits_to_f32(codes), nan=7.0))
    out["codes/e5m2_to_fp16_bits"] = up.view(np.uint16)

    # ---- bf16 -> fp16 (kernel/convert.py contract: equals x.to(float16), test_convert.py:11-15) --------------
    pats = cases.exhaustive_patterns("bf16")
    conv = from_torch(to_torch(pats, "bf16").to(torch.float16))
    mine = fo.from_f32(fo.bf16_bits_to_f32(pats), "fp16")
    a_, b_ = conv.view(np.uint16), mine.view(np.uint16)
    nan_mask = np.isnan(conv)
    assert np.array_equal(np.where(nan_mask, 0, a_), np.where(nan_mask, 0, b_)) and np.array_equal(nan_mask, np.isnan(mine))
    out["convert/bf16_to_fp16_sha"] = np.array(sha(np.where(nan_mask, np.uint16(0x7E00), a_)))

    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({os.path.getsize(path) / 1024:.1f} KiB, {len(out)} arrays)")
    for name, product, rep in report:
        print(f"  {name:32s} product={product}: max_abs={rep['max_abs']:.4g} rms={rep['rms']:.4g} fro={rep['fro_rel']:.3g} "
              f"max_ulp={rep['max_ulp']} mismatches={rep['mismatches']}")


if __name__ == "__main__":
    main()
