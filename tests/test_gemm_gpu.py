"""GPU parity tests of the mixed-precision GEMM, through the operator surface and the C ABI.

Checker: the numpy oracle (fp32-product math of kernel/naive.py) and the fixtures made by the reference's own
kernel/naive.py.  Tolerances: north-star gate max|err| <= 1e-2 * rms(out) (one-ulp rounding-boundary flips set aside
for bf16, see tests/util.py), plus the reference's own gate (fro <= 0.01, max_abs <= 2 fp16 / 16 bf16,
test_scaled_mm_hip.py:26-30) against verbatim naive.py output.
"""

import numpy as np
import pytest
import torch

from oracle import feather_oracle as fo
from tests.golden import cases
from tests.util import TORCH_DT, assert_gemm_close, from_torch, to_torch

pytestmark = pytest.mark.gpu


def _run(native, dev, a, bq, scale, bias, out_dtype, variant=None):
    A = to_torch(a, "fp16", dev)
    B = to_torch(bq, "e5m2", dev)
    S = torch.tensor([float(scale)], dtype=torch.float32, device=dev) if scale is not None else None
    Bi = to_torch(bias, out_dtype, dev) if bias is not None else None
    C = torch.full((a.shape[0], bq.shape[1]), float("nan"), dtype=TORCH_DT[out_dtype], device=dev)
    native.scaled_mm_into(A, B, S, Bi, C, variant=native.make_variant(*variant) if variant else None)
    native.check_device_status(dev)
    return from_torch(C)


def _synthetic(M, N, K, out_dtype, seed, bias=True):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((N, K), dtype=np.float32) / np.float32(np.sqrt(K))).astype(np.float32)
    bq, s = fo.make_feather_quantized_weight(w, "fp32", None)
    b = fo.from_f32(rng.standard_normal((N,), dtype=np.float32), out_dtype) if bias else None
    return a, bq, s, b


@pytest.mark.parametrize("name", list(cases.GEMM_REF_CASES))
def test_reference_distribution_through_operator(golden, hip_kernel, native, cuda_dev, name):
    """The reference's own test recipe (test_scaled_mm_hip.py:9-32): prepack_b_for_scaled_mm + scaled_mm_hip_configured
    against scaled_mm_naive, on its distribution, with its tolerances; here naive's output is the stored fixture."""
    c = cases.gemm_ref_case(name)
    a = to_torch(c["a"], "fp16", cuda_dev)
    b_kn = to_torch(c["b_kn"], "e5m2", cuda_dev)
    scale = torch.tensor(float(c["scale"]), dtype=torch.float32, device=cuda_dev)
    bias = to_torch(c["bias"], c["out_dtype"], cuda_dev)
    b_pp = hip_kernel.prepack_b_for_scaled_mm(b_kn)
    assert np.array_equal(from_torch(b_pp), c["b_prepacked"])
    for cfg in (hip_kernel._CONFIGS[0], hip_kernel._CONFIGS[-1], (1, 8, 4, 8, 2)):
        out = hip_kernel.scaled_mm_hip_configured(a, b_pp, scale, bias, TORCH_DT[c["out_dtype"]], *cfg)
        native.check_device_status(cuda_dev)
        got = from_torch(out)
        rep = fo.error_report(got, golden[f"gemm/{name}/out"], c["out_dtype"])
        assert rep["fro_rel"] <= 0.01 and rep["max_abs"] <= (2.0 if c["out_dtype"] == "fp16" else 16.0), rep
        ref32 = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product="fp32")
        assert_gemm_close(got, ref32, c["out_dtype"], fo, name, bias=c["bias"])


@pytest.mark.parametrize("name", list(cases.GEMM_BENCH_CASES))
def test_benchmark_distribution(golden, hip_kernel, native, cuda_dev, name):
    c = cases.gemm_bench_case(name)
    out = hip_kernel.scaled_mm_hip(
        to_torch(c["a"], "fp16", cuda_dev),
        to_torch(c["b_prepacked"], "e5m2", cuda_dev),
        torch.tensor(float(c["scale"]), dtype=torch.float32, device=cuda_dev),
        to_torch(c["bias"], c["out_dtype"], cuda_dev) if c["bias"] is not None else None,
        TORCH_DT[c["out_dtype"]],
    )
    native.check_device_status(cuda_dev)
    got = from_torch(out)
    rows = golden[f"gemm/{name}/rows"]
    assert_gemm_close(got[rows], golden[f"gemm/{name}/out_rows"], c["out_dtype"], fo, name + " vs fixture", bias=c["bias"])
    ref = fo.scaled_mm(c["a"], c["b_prepacked"], c["scale"], c["bias"], c["out_dtype"], product="fp32")
    assert_gemm_close(got, ref, c["out_dtype"], fo, name + " vs oracle", bias=c["bias"])


# (M, N, K, out_dtype, (tokens_tile, cta_pair, split_k, transform_groups, max_ctas[, kernel, staging]), bias, scale)
VARIANT_CASES = [
    (16, 128, 64, "fp16", (16, 1, 1, 2, 0), False, True),
    (16, 128, 128, "fp16", (16, 1, 1, 1, 0), True, True),
    (128, 128, 512, "fp16", (128, 1, 1, 2, 0), True, True),
    (256, 128, 512, "bf16", (256, 1, 1, 2, 0), True, True),
    (100, 72, 80, "bf16", (128, 1, 1, 2, 0), True, True),          # ragged in every dimension
    (1, 256, 512, "bf16", (16, 1, 1, 2, 0), False, True),           # a single token
    (33, 200, 48, "fp16", (64, 1, 1, 2, 0), True, True),            # K = 48: last k-block three quarters empty
    (33, 200, 48, "fp16", (32, 1, 1, 2, 0), True, False),           # no scale
    (7, 8, 16, "fp16", (16, 1, 1, 2, 0), True, True),               # smallest legal K, tiny N
    (700, 640, 2048, "bf16", (256, 1, 1, 2, 0), True, True),
    (700, 640, 2048, "fp16", (128, 1, 1, 2, 8), True, True),        # persistent: 8 CTAs walk 30 tiles
    (520, 384, 1024, "fp16", (256, 1, 1, 1, 2), False, True),
    (16, 256, 2048, "bf16", (16, 1, 4, 2, 0), True, True),          # split-K
    (128, 384, 4096, "fp16", (128, 1, 8, 2, 0), True, True),
    (40, 1000, 1040, "fp16", (64, 1, 3, 2, 5), True, True),         # split-K, uneven slices, few CTAs
    (32, 256, 128, "fp16", (32, 2, 1, 2, 0), False, True),          # CTA pairs
    (256, 256, 512, "fp16", (256, 2, 1, 2, 0), True, True),
    (700, 640, 2048, "bf16", (256, 2, 1, 2, 0), True, True),
    (700, 640, 2048, "bf16", (192, 2, 1, 2, 0), True, True),        # 192-token tiles: two accumulators in TMEM
    (1000, 384, 1024, "fp16", (192, 1, 1, 2, 3), True, True),
    (300, 520, 512, "bf16", (128, 1, 1, 2, 0), True, True),          # N % 8 == 0 but not a multiple of the tile
    (90, 250, 256, "fp16", (128, 1, 1, 2, 0), True, True),           # N % 8 != 0: rows not 16-byte aligned, plain-store epilogue
    (700, 600, 2048, "fp16", (128, 2, 1, 1, 8), True, True),        # pairs, N not a multiple of 256
    (64, 512, 4096, "fp16", (64, 2, 4, 2, 0), True, True),          # pairs + split-K
    (3000, 1024, 512, "bf16", (256, 2, 1, 2, 8, 0, 2), True, True),  # two staging buffers per epilogue group: 4 CTA pairs walk 48 tiles, ragged last token tile
    (1500, 520, 256, "fp16", (256, 2, 1, 1, 4, 0, 2), True, True),  # the same with one transform group, N not a multiple of the tile
    (16, 5120, 1024, "bf16", None, True, True),                     # library-chosen variant
    (300, 1024, 1024, "bf16", None, False, True),
]


@pytest.mark.parametrize("M,N,K,out_dtype,variant,bias,scale", VARIANT_CASES)
def test_variants_against_oracle(native, cuda_dev, M, N, K, out_dtype, variant, bias, scale):
    a, bq, s, b = _synthetic(M, N, K, out_dtype, seed=M * 7 + N * 3 + K, bias=bias)
    got = _run(native, cuda_dev, a, bq, s if scale else None, b, out_dtype, variant)
    ref = fo.scaled_mm(a, bq, s if scale else None, b, out_dtype, product="fp32")
    assert_gemm_close(got, ref, out_dtype, fo, f"{(M, N, K, variant)}", bias=b)


STREAM_CASES = [
    # (M, N, K, out_dtype, bias)
    (1, 256, 512, "bf16", False),
    (1, 13824, 1024, "bf16", True),
    (5, 72, 48, "fp16", True),            # N not a multiple of the 8-column strip group, K = 3 k16-blocks for 16 warps
    (16, 200, 1040, "fp16", True),
    (16, 8, 16, "bf16", True),            # one strip, one k16-block
    (17, 1000, 2048, "bf16", True),       # three groups of eight tokens, the library's choice for a small weight
    (24, 520, 4096, "fp16", True),
    (25, 1000, 2048, "bf16", True),       # four groups: on request only
    (32, 5120, 1024, "fp16", False),
    (20, 13824, 5120, "bf16", False),     # a large weight at 17-24 tokens stays with the tensor-memory kernel
    (9, 13824, 320, "bf16", True),
    (8, 5120, 2048, "bf16", True),        # up to 8 tokens: the weights-as-rows variant
    (3, 104, 64, "fp16", True),
    (7, 24, 16, "fp16", False),
]


@pytest.mark.parametrize("M,N,K,out_dtype,bias", STREAM_CASES)
def test_streaming_kernel_against_oracle(native, cuda_dev, M, N, K, out_dtype, bias):
    """The register-streaming kernel (at most 32 tokens), forced, and as the library's own choice: up to 16 tokens always, up to
    24 tokens for weights of at most 32 MB."""
    a, bq, s, b = _synthetic(M, N, K, out_dtype, seed=M * 11 + N + K, bias=bias)
    ref = fo.scaled_mm(a, bq, s, b, out_dtype, product="fp32")
    forced = _run(native, cuda_dev, a, bq, s, b, out_dtype, (0, 0, 0, 0, 0, native.KERNEL_STREAM))
    assert_gemm_close(forced, ref, out_dtype, fo, f"forced {(M, N, K)}", bias=b)
    auto = _run(native, cuda_dev, a, bq, s, b, out_dtype, None)
    if M <= 16 or (M <= 24 and N * K <= 32 << 20):     # elsewhere the tensor-memory kernel measured faster
        assert np.array_equal(auto, forced)
        assert native.choose_variant(M, N, K).kernel == native.KERNEL_STREAM
    else:
        assert_gemm_close(auto, ref, out_dtype, fo, f"auto {(M, N, K)}", bias=b)
        assert native.choose_variant(M, N, K).kernel == native.KERNEL_TMEM
    tmem = _run(native, cuda_dev, a, bq, s, b, out_dtype, (0, 0, 0, 0, 0, native.KERNEL_TMEM))
    assert_gemm_close(tmem, ref, out_dtype, fo, f"tensor-memory kernel {(M, N, K)}", bias=b)


@pytest.mark.parametrize("M,N,K", [(1, 5120, 13824), (8, 5120, 4096), (16, 5120, 13824), (12, 2048, 8192), (24, 1024, 4096)])
def test_streaming_kernel_k_split_across_ctas(native, cuda_dev, M, N, K):
    """Few weight columns and a long K: the streaming kernel shares a group of strips between several CTAs, each over a slice
    of K, through the workspace (partials added in slice order by the last CTA to arrive).  Against the oracle, bitwise
    repeatable, equal to the forced choice, and the tile counters are back at zero."""
    a, bq, s, b = _synthetic(M, N, K, "bf16", seed=M + N + K)
    ref = fo.scaled_mm(a, bq, s, b, "bf16", product="fp32")
    stream = (0, 0, 0, 0, 0, native.KERNEL_STREAM)
    runs = [_run(native, cuda_dev, a, bq, s, b, "bf16", stream) for _ in range(3)]
    assert_gemm_close(runs[0], ref, "bf16", fo, f"{(M, N, K)}", bias=b)
    assert all(np.array_equal(r, runs[0]) for r in runs[1:])
    ws = native.workspace_for(cuda_dev)
    assert int(ws[:65536].view(torch.int32).abs().sum().item()) == 0
    assert native.workspace_bytes(M, N, K) <= ws.numel()


def test_streaming_kernel_rejects_many_tokens(native, cuda_dev):
    a, bq, s, b = _synthetic(40, 64, 64, "bf16", seed=2)
    with pytest.raises(native.FeatherNativeError, match="at most 32 tokens"):
        _run(native, cuda_dev, a, bq, s, b, "bf16", (0, 0, 0, 0, 0, native.KERNEL_STREAM))


def test_split_k_workspace_is_reusable(native, cuda_dev):
    """Back-to-back split-K launches on one workspace: the tile counters must be back at zero after each."""
    a, bq, s, b = _synthetic(48, 384, 2048, "bf16", seed=3)
    ref = fo.scaled_mm(a, bq, s, b, "bf16", product="fp32")
    for _ in range(3):
        got = _run(native, cuda_dev, a, bq, s, b, "bf16", (64, 1, 4, 2, 0))
        assert_gemm_close(got, ref, "bf16", fo, bias=b)
    # the tile counters occupy the first 64 KiB of the workspace
    ws = native.workspace_for(cuda_dev)
    assert int(ws[:65536].view(torch.int32).abs().sum().item()) == 0


def test_split_k_launches_of_different_tile_counts_share_a_workspace(native, cuda_dev):
    """A launch with few tiles followed by one with many: the second one's counters must not see the first one's partials."""
    a, bq, s, b = _synthetic(16, 256, 2048, "bf16", seed=31)
    got = _run(native, cuda_dev, a, bq, s, b, "bf16", (16, 1, 4, 2, 0))
    assert_gemm_close(got, fo.scaled_mm(a, bq, s, b, "bf16"), "bf16", fo, bias=b)
    a, bq, s, b = _synthetic(16, 13824, 1024, "bf16", seed=32)
    got = _run(native, cuda_dev, a, bq, s, b, "bf16", (16, 1, 4, 2, 0))
    assert_gemm_close(got, fo.scaled_mm(a, bq, s, b, "bf16"), "bf16", fo, bias=b)


def test_split_k_on_two_streams_does_not_share_a_workspace(native, cuda_dev):
    """Split-K launches on two streams of one device may overlap on the GPU; each stream has a workspace of its own, so
    neither sees the other's tile counters or partial sums."""
    shapes = [(48, 5120, 4096, (64, 1, 4, 2, 0)), (16, 13824, 2048, (16, 1, 4, 2, 0))]
    streams = [torch.cuda.Stream(cuda_dev) for _ in shapes]
    work = []
    for (M, N, K, variant), st in zip(shapes, streams):
        a, bq, s, b = _synthetic(M, N, K, "bf16", seed=M + N + K)
        A, B = to_torch(a, "fp16", cuda_dev), to_torch(bq, "e5m2", cuda_dev)
        S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
        Bi = to_torch(b, "bf16", cuda_dev)
        C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
        work.append((st, A, B, S, Bi, C, native.make_variant(*variant), fo.scaled_mm(a, bq, s, b, "bf16")))
    torch.cuda.synchronize()
    for _ in range(20):                                   # interleaved launches, nothing orders one stream after the other
        for st, A, B, S, Bi, C, v, _ in work:
            with torch.cuda.stream(st):
                native.scaled_mm_into(A, B, S, Bi, C, variant=v)
    torch.cuda.synchronize()
    native.check_device_status(cuda_dev)
    ws = {native.workspace_for(cuda_dev, st.cuda_stream).data_ptr() for st, *_ in work}
    assert len(ws) == 2
    for st, A, B, S, Bi, C, v, ref in work:
        assert_gemm_close(from_torch(C), ref, "bf16", fo, f"stream {st.cuda_stream:#x}", has_bias=True)


def test_tile_variants_agree_bitwise(native, cuda_dev):
    """Without split-K, variants with the same number of MMA issuers add the k-blocks of an output element in the same
    order: tiles of 192 or 256 tokens in one chain, narrower tiles as (even k-blocks) + (odd k-blocks).  CTA pairs, the
    number of transform groups and the tile width inside a class change nothing, and neither does a repeat."""
    a, bq, s, b = _synthetic(300, 512, 1536, "bf16", seed=9)
    one_issuer = [_run(native, cuda_dev, a, bq, s, b, "bf16", v) for v in ((256, 1, 1, 2, 0), (256, 2, 1, 2, 0), (192, 1, 1, 1, 0), (256, 1, 1, 2, 0))]
    two_issuers = [_run(native, cuda_dev, a, bq, s, b, "bf16", v) for v in ((128, 1, 1, 1, 0), (64, 1, 1, 2, 0), (128, 2, 1, 2, 0), (16, 1, 1, 2, 0), (128, 1, 1, 1, 0))]
    for outs in (one_issuer, two_issuers):
        for o in outs[1:]:
            assert np.array_equal(o, outs[0])
    assert_gemm_close(two_issuers[0], fo.scaled_mm(a, bq, s, b, "bf16"), "bf16", fo, bias=b)


def test_empty_and_edge_shapes(hip_kernel, native, cuda_dev):
    b = torch.zeros((4, 64, 16), dtype=torch.uint8, device=cuda_dev).view(torch.float8_e5m2)
    a0 = torch.zeros((0, 64), dtype=torch.float16, device=cuda_dev)
    out = hip_kernel.scaled_mm_hip(a0, b, None, None, torch.float16)
    assert out.shape == (0, 64)
    # zero activations: output is exactly the bias
    a = torch.zeros((5, 64), dtype=torch.float16, device=cuda_dev)
    bias = torch.randn(64, device=cuda_dev).to(torch.bfloat16)
    w = torch.randint(0, 0x7B, (4, 64, 16), dtype=torch.uint8, device=cuda_dev).view(torch.float8_e5m2)
    out = hip_kernel.scaled_mm_hip(a, w, torch.tensor(3.0, device=cuda_dev), bias, torch.bfloat16)
    native.check_device_status(cuda_dev)
    assert torch.equal(out, bias[None, :].expand(5, 64))


def test_argument_checks(hip_kernel, cuda_dev):
    """Same preconditions and messages as the reference op (hip_kernel.cu:648-730)."""
    a = torch.zeros((16, 64), dtype=torch.float16, device=cuda_dev)
    b = torch.zeros((4, 32, 16), dtype=torch.uint8, device=cuda_dev).view(torch.float8_e5m2)
    c = torch.empty((16, 32), dtype=torch.float16, device=cuda_dev)
    op = torch.ops.feather_ops.scaled_mm
    cfg = (1, 8, 4, 8, 2)
    with pytest.raises(RuntimeError, match="a must be float16"):
        op(a.float(), b, None, None, c, *cfg, 1)
    with pytest.raises(RuntimeError, match="b_prepacked.shape\\[0\\] must equal K/16"):
        op(a, b[:3], None, None, c, *cfg, 1)
    with pytest.raises(RuntimeError, match="scale must be float32"):
        op(a, b, torch.ones(1, dtype=torch.float16, device=cuda_dev), None, c, *cfg, 1)
    with pytest.raises(RuntimeError, match="bias must have N elements"):
        op(a, b, None, torch.zeros(31, dtype=torch.float16, device=cuda_dev), c, *cfg, 1)
    with pytest.raises(RuntimeError, match="bias must have the same dtype as c"):
        op(a, b, None, torch.zeros(32, dtype=torch.bfloat16, device=cuda_dev), c, *cfg, 1)
    with pytest.raises(RuntimeError, match="c.shape\\[1\\] must equal N"):
        op(a, b, None, None, c[:, :16], *cfg, 1)
    with pytest.raises(RuntimeError, match="float8_e5m2 when b_dtype=1"):
        op(a, b.view(torch.uint8).view(torch.float8_e4m3fn), None, None, c, *cfg, 1)
    with pytest.raises(RuntimeError, match="float8_e4m3fn when b_dtype=0"):
        op(a, b, None, None, c, *cfg, 0)
    with pytest.raises(RuntimeError, match="b_dtype must be 0"):
        op(a, b, None, None, c, *cfg, 2)
    with pytest.raises(RuntimeError, match="a.stride\\(0\\) must equal K"):
        op(torch.zeros((64, 16), dtype=torch.float16, device=cuda_dev).t(), b, None, None, c, *cfg, 1)


def test_reference_c_abi_signature(native, cuda_dev):
    """`launch_scaled_mm` keeps the reference's argument order (hip_kernel.cu:564-582) and returns 1 / 0 like its bool."""
    a, bq, s, b = _synthetic(64, 256, 512, "fp16", seed=5)
    A, B = to_torch(a, "fp16", cuda_dev), to_torch(bq, "e5m2", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    Bi = to_torch(b, "fp16", cuda_dev)
    C = torch.empty((64, 256), dtype=torch.float16, device=cuda_dev)
    assert native.launch_scaled_mm_reference_abi(A, B, S, Bi, C) == 1
    torch.cuda.synchronize()
    assert_gemm_close(from_torch(C), fo.scaled_mm(a, bq, s, b, "fp16"), "fp16", fo, bias=b)
    assert native.launch_scaled_mm_reference_abi(A, B, S, Bi, C, b_dtype=2) == 0      # neither e4m3 (0) nor e5m2 (1): refused like an unknown config
    # a handful of tokens through the same signature: the streaming kernel (this entry point has no workspace to split K through)
    C8 = torch.empty((8, 256), dtype=torch.float16, device=cuda_dev)
    assert native.launch_scaled_mm_reference_abi(A[:8].contiguous(), B, S, Bi, C8) == 1
    torch.cuda.synchronize()
    stream8 = torch.empty_like(C8)
    native.scaled_mm_into(A[:8].contiguous(), B, S, Bi, stream8, variant=native.make_variant(kernel=native.KERNEL_STREAM))
    assert torch.equal(C8, stream8)
    assert_gemm_close(from_torch(C8), fo.scaled_mm(a[:8], bq, s, b, "fp16"), "fp16", fo, bias=b)


def test_column_shard_writes_in_place(native, cuda_dev):
    """Two weight shards along N write their column blocks of one [M,N] buffer; the result is bitwise the unsharded one."""
    a, bq, s, b = _synthetic(200, 512, 1024, "bf16", seed=8)
    full = _run(native, cuda_dev, a, bq, s, b, "bf16")
    A = to_torch(a, "fp16", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    C = torch.zeros((200, 512), dtype=torch.bfloat16, device=cuda_dev)
    for r in range(2):
        Bs = to_torch(np.ascontiguousarray(bq[:, r * 256:(r + 1) * 256, :]), "e5m2", cuda_dev)
        bias_s = to_torch(b[r * 256:(r + 1) * 256], "bf16", cuda_dev)
        native.scaled_mm_into(A, Bs, S, bias_s, C[:, r * 256:(r + 1) * 256])
    native.check_device_status(cuda_dev)
    assert np.array_equal(from_torch(C), full)


@pytest.mark.parametrize("M,N,K,g", [(700, 13824, 1024, 8), (700, 5120, 1024, 8), (300, 13824, 512, 4)])
def test_ragged_column_shards_reproduce_the_full_output(native, cuda_dev, M, N, K, g):
    """The column shards of 4 and 8 ranks (1728, 640, 3456 columns: not multiples of the 256-column pair tile, so the last
    pair stores a clipped block and its second CTA may have nothing to store), written in place through the fused-exchange
    entry point with one destination: bitwise the unsharded output."""
    torch.manual_seed(0)
    A = torch.randn(M, K, device=cuda_dev, dtype=torch.float16)
    B = torch.randint(0, 0x7B, (K // 16, N, 16), dtype=torch.uint8, device=cuda_dev).view(torch.float8_e5m2)
    S = torch.full((1,), 1e-2, device=cuda_dev)
    bias = torch.randn(N, device=cuda_dev).to(torch.bfloat16)
    full = torch.empty(M, N, device=cuda_dev, dtype=torch.bfloat16)
    native.scaled_mm_into(A, B, S, bias, full)
    sharded = torch.full((M, N), float("nan"), device=cuda_dev, dtype=torch.bfloat16)
    n = N // g
    for r in range(g):
        Br = B[:, r * n:(r + 1) * n, :].contiguous()
        native.scaled_mm_multi_into(A, Br, S, bias[r * n:(r + 1) * n].contiguous(), [sharded[:, r * n:(r + 1) * n]])
    native.check_device_status(cuda_dev)
    assert torch.equal(full.view(torch.int16), sharded.view(torch.int16))


def test_multi_destination_epilogue_on_one_gpu(native, cuda_dev):
    """The fused-exchange launch with all destinations on one GPU: every buffer receives the block, bitwise equal to the
    ordinary launch; column ranges of a wider buffer are written in place and nothing else is touched."""
    a, bq, s, b = _synthetic(300, 256, 1024, "bf16", seed=12)
    single = _run(native, cuda_dev, a, bq, s, b, "bf16", (256, 2, 1, 2, 0))
    A, B = to_torch(a, "fp16", cuda_dev), to_torch(bq, "e5m2", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    Bi = to_torch(b, "bf16", cuda_dev)
    wide = [torch.full((300, 768), 7.0, dtype=torch.bfloat16, device=cuda_dev) for _ in range(3)]
    native.scaled_mm_multi_into(A, B, S, Bi, [w[:, 256:512] for w in wide])
    native.check_device_status(cuda_dev)
    for w in wide:
        assert np.array_equal(from_torch(w[:, 256:512]), single)
        assert bool((w[:, :256] == 7.0).all()) and bool((w[:, 512:] == 7.0).all())
    with pytest.raises(native.FeatherNativeError, match="16-byte aligned rows"):
        odd = [torch.empty((300, 250), dtype=torch.bfloat16, device=cuda_dev) for _ in range(2)]
        a2, bq2, s2, _ = _synthetic(300, 250, 64, "bf16", seed=1, bias=False)
        native.scaled_mm_multi_into(to_torch(a2, "fp16", cuda_dev), to_torch(bq2, "e5m2", cuda_dev), None, None, odd)


@pytest.mark.parametrize("variant", [(256, 2, 1, 2, 8), (256, 2, 1, 1, 6), None])
def test_many_tiles_to_several_destinations_on_one_gpu(native, cuda_dev, variant):
    """256-token pair tiles stored to several destinations (here all on one GPU; across GPUs those stores cross NVLink): a few
    CTA pairs walk many tiles through the two staging buffers of each epilogue group, the last token tile and the last column
    tile are ragged; every buffer must hold the single-destination result bit for bit and nothing outside its column range."""
    a, bq, s, b = _synthetic(3000, 904, 512, "bf16", seed=77)
    single = _run(native, cuda_dev, a, bq, s, b, "bf16", (256, 2, 1, 2, 0))
    A, B = to_torch(a, "fp16", cuda_dev), to_torch(bq, "e5m2", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    Bi = to_torch(b, "bf16", cuda_dev)
    wide = [torch.full((3000, 1800), 7.0, dtype=torch.bfloat16, device=cuda_dev) for _ in range(4)]
    for _ in range(2):
        native.scaled_mm_multi_into(A, B, S, Bi, [w[:, 448:448 + 904] for w in wide], variant=native.make_variant(*variant) if variant else None)
    native.check_device_status(cuda_dev)
    for w in wide:
        assert np.array_equal(from_torch(w[:, 448:448 + 904]), single)
        assert bool((w[:, :448] == 7.0).all()) and bool((w[:, 448 + 904:] == 7.0).all())


@pytest.mark.parametrize("K,N", [(5120, 13824), (13824, 5120), (5120, 5120)])
def test_full_size_wan_shapes_properties(native, cuda_dev, K, N):
    """M = 32768 Wan-14B linears.  The CPU oracle cannot do 4.6 TFLOP in seconds, so: rows sampled across the whole
    output against the oracle, and exact properties that hold at any size (scaling A by 2 doubles the output bit for bit;
    permuting token rows permutes output rows)."""
    M = 32768
    g = torch.Generator(device=cuda_dev).manual_seed(K + N)
    A = torch.randn((M, K), generator=g, device=cuda_dev, dtype=torch.float32).to(torch.float16)
    w = torch.randn((N, K), generator=g, device=cuda_dev, dtype=torch.float32) / K ** 0.5
    B, S = native.quantize_prepack(w)
    del w
    S = S.reshape(1)
    C = torch.empty((M, N), dtype=torch.bfloat16, device=cuda_dev)
    native.scaled_mm_into(A, B, S, None, C)
    native.check_device_status(cuda_dev)
    rows = np.unique(np.concatenate([np.arange(0, M, 4099), [M - 1, 255, 256, M - 257]]))
    ref = fo.scaled_mm(from_torch(A[rows]), from_torch(B), np.float32(S.item()), None, "bf16", product="fp32")
    assert_gemm_close(from_torch(C[rows]), ref, "bf16", fo, "sampled rows")
    # linearity in powers of two is exact (no overflow at this scale)
    C2 = torch.empty_like(C)
    native.scaled_mm_into(A * 2, B, S, None, C2)
    assert torch.equal(C2.view(torch.int16), (C.float() * 2).to(torch.bfloat16).view(torch.int16))
    # row permutation
    perm = torch.randperm(M, generator=g, device=cuda_dev)
    native.scaled_mm_into(A[perm].contiguous(), B, S, None, C2)
    native.check_device_status(cuda_dev)
    assert torch.equal(C2.view(torch.int16), C[perm].view(torch.int16))


@pytest.mark.parametrize("M", [1, 16, 128])
@pytest.mark.parametrize("K,N", [(5120, 13824), (13824, 5120)])
def test_small_m_sweep(native, cuda_dev, M, K, N):
    """The bandwidth-bound sweep of the benchmark, full K and N, checked in full against the oracle."""
    a, bq, s, _ = _synthetic(M, N, K, "bf16", seed=M + K, bias=False)
    got = _run(native, cuda_dev, a, bq, s, None, "bf16")
    assert_gemm_close(got, fo.scaled_mm(a, bq, s, None, "bf16"), "bf16", fo, f"M={M}")


@pytest.mark.parametrize("K,N", [(3072, 3072), (3072, 9216), (3072, 12288), (12288, 3072)])
def test_qwen_image_shapes(native, cuda_dev, K, N):
    """M = 4352 (4096 image + 256 text tokens), fp16 out; 64 sampled rows against the oracle."""
    M = 4352
    a, bq, s, _ = _synthetic(M, N, K, "fp16", seed=K + N, bias=False)
    got = _run(native, cuda_dev, a, bq, s, None, "fp16")
    rows = np.arange(0, M, 68)
    assert_gemm_close(got[rows], fo.scaled_mm(a[rows], bq, s, None, "fp16"), "fp16", fo, f"{K}x{N}")


@pytest.mark.parametrize("args", [["300", "520", "1040", "--bias", "--check", "--iters", "5"], ["16", "1024", "2048", "--fp16", "--check", "--iters", "5"],
                                  ["64", "5120", "2048", "--ex", "--check", "--iters", "5"]])
def test_c_harness_runs_without_python_in_the_loop(args):
    """cbench/bench_scaled_mm: a plain C process that links the library, launches through `launch_scaled_mm` (reference argument
    order) or `feather_scaled_mm_ex`, times with events and checks sampled outputs against a host sum."""
    import importlib.util
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("feather_b200_build", os.path.join(root, "comfyui-featherops_b200", "build.py"))
    builder = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(builder)
    binary = builder.CBENCH_BIN if os.path.exists(builder.CBENCH_BIN) else builder.build_cbench()
    res = subprocess.run([binary, *args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    print(res.stdout)
    assert res.returncode == 0, res.stdout
    assert "TFLOPS" in res.stdout and "-> ok" in res.stdout
