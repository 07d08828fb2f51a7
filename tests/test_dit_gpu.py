"""GPU: the 4-block Wan-like DiT forward whose linears are all Feather e5m2 linears, against a CPU forward whose linears
are the oracle (torch restatement of the reference's kernel/naive.py with an fp32 product).

Two checks per case.  (1) Every linear, on exactly the fp16 input the CUDA forward gave it (captured by a hook), against the
oracle with the GEMM gate of tests/util.py.  (2) The whole forward against the CPU forward: RMSNorm, attention and GELU run
in bf16 through different kernels on the two devices, so this is a tolerance, stated here: Frobenius-relative error <= 3e-2
after 4 blocks (2 blocks for the narrow case) and no element further than 0.25 * rms(out).
"""

import importlib

import numpy as np
import pytest
import torch

from oracle import feather_oracle as fo
from oracle import naive_torch
from tests.dit_cpu import CpuOracleFactory
from tests.util import assert_gemm_close, from_torch

pytestmark = pytest.mark.gpu


def _models(pkg, cuda_dev, cfg_kwargs, mode="all_gather", seed=1):
    dit = importlib.import_module("feather_b200.kernel.b200.dit")
    cfg = dit.DitConfig(**cfg_kwargs)
    gpu = dit.FeatherDiT(cfg, device=cuda_dev, mode=mode, seed=seed, init_device=torch.device("cpu"))
    cpu = dit.FeatherDiT(cfg, device=torch.device("cpu"), mode=mode, seed=seed, init_device=torch.device("cpu"), linear_factory=CpuOracleFactory())
    return cfg, gpu, cpu


@pytest.mark.parametrize("cfg_kwargs,tokens", [
    (dict(hidden=1024, heads=8, head_dim=128, ffn=2816, blocks=2), 520),           # narrow, ragged token count
    (dict(hidden=5120, heads=40, head_dim=128, ffn=13824, blocks=4), 512),        # the benchmark's widths at a reduced token count
])
def test_forward_against_cpu_forward_with_oracle_linears(pkg, native, cuda_dev, cfg_kwargs, tokens):
    cfg, gpu, cpu = _models(pkg, cuda_dev, cfg_kwargs)
    x = torch.randn((tokens, cfg.hidden), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    seen = []
    y_gpu = gpu(x.to(cuda_dev), hook=lambda name, i, a16, y: seen.append((name, i, a16.cpu(), y.cpu())))
    native.check_device_status(cuda_dev)
    assert len(seen) == 6 * cfg.blocks
    # (1) every linear on the very input the CUDA forward fed it
    for name, i, a16, y in seen:
        lin = cpu.blocks[i][name]
        ref = naive_torch.scaled_mm_cpu(a16, lin.q, lin.s, lin.b, torch.bfloat16)
        assert_gemm_close(from_torch(y), from_torch(ref), "bf16", fo, f"block {i} {name}", bias=lin.b.float().numpy())
    # (2) end to end
    y_cpu = cpu(x)
    got, ref = y_gpu.float().cpu(), y_cpu.float()
    rms = float(ref.pow(2).mean().sqrt())
    fro = float((got - ref).norm() / ref.norm())
    worst = float((got - ref).abs().max())
    print(f"[dit] {cfg_kwargs} T={tokens}: fro_rel {fro:.3e}, max|err| {worst:.3e}, rms {rms:.3e}")
    assert torch.isfinite(got).all()
    assert fro <= 3e-2 and worst <= 0.25 * rms, (fro, worst, rms)


def test_pairs_mode_on_one_gpu_is_the_same_forward(pkg, native, cuda_dev):
    """With one rank the tensor-parallel pairs degenerate to plain linears with the residual added after the bias, in the
    same order as the all-gather mode: bitwise equal."""
    cfg_kwargs = dict(hidden=1024, heads=8, head_dim=128, ffn=2816, blocks=2)
    cfg, a, _ = _models(pkg, cuda_dev, cfg_kwargs, mode="all_gather")
    _, b, _ = _models(pkg, cuda_dev, cfg_kwargs, mode="pairs")
    x = torch.randn((384, cfg.hidden), generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).to(cuda_dev)
    ya, yb = a(x), b(x)
    native.check_device_status(cuda_dev)
    assert torch.equal(ya.view(torch.int16), yb.view(torch.int16))


def test_tokens_mode_on_one_gpu_is_the_same_forward(pkg, native, cuda_dev):
    """With one rank the token-sharded mode runs the same linears on all rows and attention on all queries: bitwise equal."""
    cfg_kwargs = dict(hidden=1024, heads=8, head_dim=128, ffn=2816, blocks=2)
    cfg, a, _ = _models(pkg, cuda_dev, cfg_kwargs, mode="all_gather")
    _, b, _ = _models(pkg, cuda_dev, cfg_kwargs, mode="tokens")
    x = torch.randn((384, cfg.hidden), generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).to(cuda_dev)
    ya, yb = a(x), b(x)
    native.check_device_status(cuda_dev)
    assert torch.equal(ya.view(torch.int16), yb.view(torch.int16))


def test_harness_linear_is_the_operator_linear(pkg, native, cuda_dev):
    """A linear of the harness gives bit for bit what `FeatherOps.Linear` (the ComfyUI operator, here under the test double
    of `comfy`) gives for the same fp32 weight, bias and bf16 input."""
    ops_mod = importlib.import_module("feather_b200.comfy_feather.ops")
    dit = importlib.import_module("feather_b200.kernel.b200.dit")
    g = torch.Generator().manual_seed(3)
    N, K, T = 384, 512, 200
    w = torch.randn((N, K), generator=g) / K ** 0.5
    bias = torch.randn((N,), generator=g) * 0.1
    x = torch.randn((T, K), generator=g).to(torch.bfloat16).to(cuda_dev)
    factory = dit.CudaLinearFactory(0, 1, cuda_dev)
    y_harness = factory.column(w, bias)(factory.to_fp16(x), torch.bfloat16)
    Ops = ops_mod.feather_ops(out_dtype=torch.bfloat16)
    lin = Ops.Linear(K, N, bias=True)
    lin._load_from_state_dict({"l.weight": w.clone(), "l.bias": bias.clone()}, "l.", {}, True, [], [], [])
    y_op = lin.to(cuda_dev)(x)
    native.check_device_status(cuda_dev)
    assert torch.equal(y_op.view(torch.int16), y_harness.view(torch.int16))


@pytest.mark.parametrize("M,N,K,g", [(512, 640, 2048, 4), (256, 520, 1024, 8), (2048, 5120, 1024, 8)])
def test_row_parallel_pieces_on_one_gpu(native, cuda_dev, M, N, K, g):
    """The row-parallel linear's two kernels with all g "ranks" played by one GPU: each rank's GEMM over its K slice scatters
    its bf16 partial of token rows [d*M/g, (d+1)*M/g) into slot `rank` of owner d's buffer; each owner then adds its g
    partials in fp32, adds the bias and a residual, and writes its rows into every rank's output.  Checked against the
    oracle's full-K result (+ residual) with the GEMM gate: K is split, so this is a tolerance, not bitwise - but all
    "ranks" must hold identical bits."""
    rng = np.random.default_rng(M + N + K)
    a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((N, K), dtype=np.float32) / np.float32(np.sqrt(K))).astype(np.float32)
    bq, s = fo.make_feather_quantized_weight(w, "fp32", None)
    bias = fo.from_f32(rng.standard_normal((N,), dtype=np.float32), "bf16")
    from tests.util import to_torch

    A, B = to_torch(a, "fp16", cuda_dev), to_torch(bq, "e5m2", cuda_dev)
    S = torch.tensor([float(s)], dtype=torch.float32, device=cuda_dev)
    Bi = to_torch(bias, "bf16", cuda_dev)
    res = torch.randn((M, N), device=cuda_dev).to(torch.bfloat16)
    rows, kl = M // g, K // g
    partials = [torch.full((g, rows, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev) for _ in range(g)]     # per owner
    for r in range(g):
        native.scaled_mm_scatter_into(A[:, r * kl:(r + 1) * kl].contiguous(), B[r * kl // 16:(r + 1) * kl // 16].contiguous(), S,
                                      [partials[d][r] for d in range(g)], rows)
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev) for _ in range(g)]
    plain = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda_dev)
    for d in range(g):
        native.reduce_partials_into(partials[d], Bi, res[d * rows:(d + 1) * rows], [o[d * rows:(d + 1) * rows] for o in outs])
        native.reduce_partials_into(partials[d], None, None, [plain[d * rows:(d + 1) * rows]])
    native.check_device_status(cuda_dev)
    for o in outs[1:]:
        assert torch.equal(o.view(torch.int16), outs[0].view(torch.int16))
    # the reduce kernel, bit for bit: fp32 sum of the g partials in rank order, one rounding, + bias, + residual in bf16
    stacked = torch.cat(partials, dim=1)                                       # [g sources, M, N]: owner d's rows are rows d*rows..
    acc = torch.zeros((M, N), dtype=torch.float32, device=cuda_dev)
    for src in range(g):
        acc += stacked[src].float()
    emulated = acc.to(torch.bfloat16)
    assert torch.equal(plain.view(torch.int16), emulated.view(torch.int16))
    emulated = (emulated + Bi) + res
    assert torch.equal(outs[0].view(torch.int16), emulated.view(torch.int16))
    # every partial is an ordinary GEMM over a K slice, and their sum is the full result within the gate: K is split, so the
    # g roundings of the partials (each a fraction 1/sqrt(g) of the output's size) come on top of the final one
    p0 = fo.scaled_mm(a[:, :kl], bq[: kl // 16], s, None, "bf16", product="fp32")
    assert_gemm_close(from_torch(stacked[0]), p0, "bf16", fo, "partial of rank 0")
    ref_full = fo.scaled_mm(a, bq, s, None, "bf16", product="fp32")
    rep = fo.error_report(from_torch(plain), ref_full, "bf16")
    print(f"[row-parallel] {(M, N, K, g)}: {rep}")
    assert rep["nonfinite_agree"] and rep["fro_rel"] <= 3e-3 and rep["max_excess_over_1ulp"] <= 1e-2 * rep["rms"], rep
