"""CPU: the C-ABI library loads without a GPU and exports every symbol include/feather_b200.h declares; argument
validation that needs no device returns error codes instead of faulting."""

import ctypes
import importlib.util
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "feather_b200.h")).read()
    return re.findall(r"FEATHER_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)


def test_header_declares_the_documented_entry_points():
    syms = _declared_symbols()
    assert "launch_scaled_mm" in syms and "feather_scaled_mm_ex" in syms and "feather_quantize_prepack" in syms
    assert len(syms) == len(set(syms)) >= 11


def test_library_exports_every_declared_symbol(native):
    lib = native.load_library()
    for sym in _declared_symbols():
        assert hasattr(lib, sym), sym
    assert set(_declared_symbols()) == set(native.EXPORTED_SYMBOLS)
    assert lib.feather_version() >= 100


def test_every_declaration_cites_the_reference():
    text = open(os.path.join(ROOT, "include", "feather_b200.h")).read()
    for block in re.split(r"\n\s*\n", text):
        if re.search(r"^FEATHER_API ", block, re.M) and "feather_last_error_string" not in block and "feather_version" not in block:
            # an entry point either cites the reference interface it replaces or says that it has none
            assert re.search(r"\w+\.(py|cu|md|cpp):\d+", block) or "no counterpart in the reference" in block.lower(), block[:120]


def test_bad_arguments_return_codes_without_a_device(native):
    lib = native.load_library()
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)   # never dereferenced: the checks fail first
    assert lib.feather_scaled_mm_ex(null, one, null, null, one, 16, 16, 16, 16, 0, None, null, 0, null, null) == 1
    assert b"null" in lib.feather_last_error_string()
    assert lib.feather_scaled_mm_ex(one, one, null, null, one, 16, 16, 24, 16, 0, None, null, 0, null, null) == 1
    assert b"divisible by 16" in lib.feather_last_error_string()
    assert lib.feather_scaled_mm_ex(one, one, null, null, one, 16, 16, 16, 8, 0, None, null, 0, null, null) == 1
    assert lib.feather_scaled_mm_ex(one, one, null, null, one, 16, 16, 16, 16, 7, None, null, 0, null, null) == 1
    assert lib.feather_scaled_mm_ex(ctypes.c_void_p(8), one, null, null, one, 16, 16, 16, 16, 0, None, null, 0, null, null) == 1
    assert b"16-byte aligned" in lib.feather_last_error_string()
    assert lib.launch_scaled_mm(one, one, null, null, one, 16, 16, 16, 0, 0, 1, 8, 4, 8, 2, 0, 0, null) == 0   # e4m3 rejected
    assert lib.feather_quantize_prepack(one, 0, null, 16, 24, 1, one, one, one, null) == 1
    assert lib.feather_quantize_prepack(one, 9, null, 16, 16, 1, one, one, one, null) == 1
    assert lib.feather_quantize_prepack(one, 1, one, 16, 16, 1, one, one, one, null) == 1        # premul needs fp32
    assert lib.feather_prepack_bytes(null, 16, 16, 0, one, null) == 1
    assert lib.feather_unprepack_bytes(one, 16, 0, one, null) == 1
    assert lib.feather_dequantize(one, one, 16, 16, 5, one, null) in (1, 4)
    assert lib.feather_bf16_to_fp16(one, one, -1, null) == 1
    assert lib.feather_bf16_to_fp16(null, null, 0, null) == 0
    assert lib.feather_copy_block(null, 64, one, 64, 32, 4, null) == 1
    assert lib.feather_copy_block(one, 16, one, 64, 32, 4, null) == 1                            # pitch smaller than the width
    assert b"pitch" in lib.feather_last_error_string()
    assert lib.feather_copy_block(one, 64, one, 64, 0, 4, null) == 0                             # nothing to copy
    ptrs = (ctypes.c_void_p * 1)(16)
    assert lib.feather_reduce_partials(one, 0, 16, 64, null, null, 0, ptrs, 1, 64, 1, null) == 1    # n_src out of range
    assert lib.feather_reduce_partials(one, 2, 16, 60, null, null, 0, ptrs, 1, 64, 1, null) == 1    # N not a multiple of 8


def test_missing_library_fails_loudly(native, monkeypatch):
    monkeypatch.setattr(native, "_lib", None)
    monkeypatch.setattr(native, "LIB_PATH", os.path.join(ROOT, "does_not_exist.so"))
    with pytest.raises(native.FeatherNativeError, match="no fallback"):
        native.load_library()


def test_cpu_tensors_are_rejected(native):
    import torch

    a = torch.zeros((16, 16), dtype=torch.float16)
    b = torch.zeros((1, 16, 16), dtype=torch.uint8).view(torch.float8_e5m2)
    c = torch.zeros((16, 16), dtype=torch.float16)
    with pytest.raises(native.FeatherNativeError, match="no CPU path"):
        native.scaled_mm_into(a, b, None, None, c)
    with pytest.raises(native.FeatherNativeError, match="no CPU path"):
        native.quantize_prepack(torch.zeros((16, 16)))


def test_header_compiles_as_c_and_the_c_harness_builds(tmp_path):
    """include/feather_b200.h is a C header (C99, pedantic, no CUDA include needed), and the plain-C timing program in
    cbench/ compiles and links against it and the library (the counterpart of the reference's cpp_benchmarks/
    benchmark_scaled_mm_hip.cpp, which declares the launcher itself, :27-45)."""
    import shutil
    import subprocess

    cc = shutil.which("cc") or shutil.which("gcc")
    if cc is None:
        pytest.skip("no C compiler")
    probe = tmp_path / "probe.c"
    probe.write_text('#include "feather_b200.h"\nint main(void) { feather_mm_variant v = {0}; return (int)sizeof(v) - 28 + (int)FEATHER_OK; }\n')
    res = subprocess.run([cc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(probe)],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout
    spec = importlib.util.spec_from_file_location("feather_b200_build", os.path.join(ROOT, "comfyui-featherops_b200", "build.py"))
    builder = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(builder)
    try:
        binary = builder.build_cbench()
    except RuntimeError as e:
        if "nvcc not found" in str(e):
            pytest.skip("no CUDA toolkit")
        raise
    assert os.path.exists(binary)
