"""GPU: `feather_scaled_mm_static`, the entry point for callers that cannot allocate device memory.

Some users of the library are not allowed to call cudaMalloc when they need a GEMM: code that runs while a CUDA graph is
being captured, host callbacks, plugins that only ever receive pointers from a framework's allocator.  For them the
split-K scratch lives in a fixed array inside the library.  This file checks, through the C ABI, that the entry point
gives exactly what the ordinary one gives (same variant, so the same additions in the same order: bitwise equal), on two
calls in a row (the array keeps the first call's contents), and that a shape which needs more scratch than the array
holds is refused with a clear message.  The file name sorts last so a run that stops at the first failure has already
run every other test.
"""

import numpy as np
import pytest
import torch

from oracle import feather_oracle as fo
from tests.util import assert_gemm_close, from_torch, to_torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((N, K), dtype=np.float32) / np.float32(np.sqrt(K))).astype(np.float32)
    bq, s = fo.make_feather_quantized_weight(w, "fp32", None)
    bias = fo.from_f32(rng.standard_normal((N,), dtype=np.float32), "bf16")
    return a, bq, s, bias


def test_static_scratch_entry_matches_workspace_entry_twice(native, cuda_dev):
    variant = native.make_variant(16, 1, 4, 2, 0)                      # split-K: the variant that uses scratch
    assert native.workspace_bytes(16, 512, 2048, variant) > 0
    for call, (M, N, K) in enumerate([(16, 512, 2048), (9, 384, 4096)]):
        a, bq, s, bias = _case(M, N, K, seed=100 + call)
        A, B = to_torch(a, "fp16", cuda_dev), to_torch(bq, "e5m2", cuda_dev)
        S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
        Bi = to_torch(bias, "bf16", cuda_dev)
        ref = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
        native.scaled_mm_into(A, B, S, Bi, ref, variant=variant)
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
        native.scaled_mm_static_into(A, B, S, Bi, got, variant=variant)
        native.check_device_status(cuda_dev)
        assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), f"call {call}"
        assert_gemm_close(from_torch(got), fo.scaled_mm(a, bq, s, bias, "bf16"), "bf16", fo, f"call {call}", bias=bias)


def test_static_scratch_entry_with_library_chosen_variant(native, cuda_dev):
    """No variant passed: the entry point makes the choice feather_scaled_mm_ex makes with an 8 MiB workspace.  Up to 16
    tokens that is the streaming kernel (no scratch); at (128, 4096, 8192) the library's unconstrained choice is a 4-way
    K split that needs more than the array holds, and the entry point must shrink it, not refuse."""
    limit = native.static_scratch_bytes()
    for M, N, K in ((16, 5120, 2048), (8, 1024, 4096), (128, 4096, 8192), (64, 5120, 5120)):
        a, bq, s, bias = _case(M, N, K, seed=7 + M)
        A, B = to_torch(a, "fp16", cuda_dev), to_torch(bq, "e5m2", cuda_dev)
        S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
        same_choice = native.choose_variant(M, N, K, workspace_bytes=limit)
        if M == 128:
            assert native.workspace_bytes(M, N, K) > limit >= native.workspace_bytes(M, N, K, same_choice) > 0
        for _ in range(2):
            got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
            native.scaled_mm_static_into(A, B, S, None, got)
            ref = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
            native.scaled_mm_into(A, B, S, None, ref, variant=None if M <= 16 else same_choice)
            native.check_device_status(cuda_dev)
            assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), (M, N, K)
        assert_gemm_close(from_torch(got), fo.scaled_mm(a, bq, s, None, "bf16"), "bf16", fo, f"{(M, N, K)}")


def test_static_scratch_entry_rejects_oversized_requests(native, cuda_dev):
    limit = native.static_scratch_bytes()
    assert limit == 8 << 20
    variant = native.make_variant(128, 1, 8, 2, 0)
    M, N, K = 128, 4096, 8192
    assert native.workspace_bytes(M, N, K, variant) > limit
    A = torch.zeros((M, K), dtype=torch.float16, device=cuda_dev)
    B = torch.zeros((K // 16, N, 16), dtype=torch.uint8, device=cuda_dev).view(torch.float8_e5m2)
    C = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_dev)
    with pytest.raises(native.FeatherNativeError, match="built-in scratch holds"):
        native.scaled_mm_static_into(A, B, None, None, C, variant=variant)
