#!/usr/bin/env python3
"""Benchmark of the FeatherOps mixed-precision linear on B200: TFLOPS of fp16 @ prepacked fp8e5m2 GEMMs at Wan-14B shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W]            our arm (CUDA kernels through the C ABI)
    python bench.py --impl reference ...                           the reference's naive torch path on the host cores

A step is one pass over the workload's linears (default: the three Wan-2.1-14B shapes at M = 32768 tokens, bf16 out).
One JSON line is printed by rank 0.  For N > 1 (launched with torch.distributed.run) every GEMM is sharded by weight
columns across the ranks and its output exchanged.  `--exchange copy_engine` (default for this workload, whose linears are
independent): the GEMM writes its column block and copy engines push it to the peers on a second stream under the next
linear's GEMM.  `--exchange peer_store` (default for the DiT, where the next operation needs the output at once): the GEMM's
own epilogue TMA-stores every finished block into all ranks' output buffers over NVLink.  The line reports the step with the
other of the two as `exchange.alternative`.  `--exchange all_gather` is the NCCL all-gather baseline.
After the warm-up, and outside the timed region, every rank compares rows of each exchanged output bit for bit with an
unsharded GEMM of the same rows (`exchange_check` in the line; a mismatch fails the run).

The N = 1 line also carries `small_m`: GB/s of the bandwidth-bound shapes (M in {1, 16, 128}), CUDA-graph replay.

Other workloads (not the driver's line): --workload qwen | smallm | quant | dit, or --shape M,N,K for a single GEMM.
`--workload dit` is the 4-block Wan-like DiT forward (32768 tokens) whose linears are all Feather linears; `--dit-mode pairs`
runs it as tensor-parallel pairs (column-parallel -> row-parallel) instead of an all-gather after every linear, `--dit-mode
tokens` with token rows sharded and weights replicated (no exchange in the linears, keys and values all-gathered per block).
"""

import argparse
import importlib
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, [(K, N), ...], out dtype)
    "wan": (32768, [(5120, 5120), (5120, 13824), (13824, 5120)], "bf16"),
    "qwen": (4352, [(3072, 3072), (3072, 9216), (3072, 12288), (12288, 3072)], "fp16"),
}
TORCH_DT = {"bf16": torch.bfloat16, "fp16": torch.float16}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples that arrived between t_begin and t_end (time.perf_counter values; the driver publishes a new
        reading about every 100 ms, so a short region holds few distinct ones); of all samples when no window is given."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        window = [(t, l) for t, l in self.lines if (t_begin is None or t >= t_begin) and (t_end is None or t <= t_end + 0.03)]
        if not window:                       # a region shorter than the sampling period: take the readings nearest to it
            window = self.lines[-2:]
        for _, line in window:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                pw.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_mhz_min": min(sm), "sm_max_mhz": max(mx), "power_w_max": max(pw), "samples": len(sm),
                "reasons": sorted(reasons)}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="wan", choices=["wan", "qwen", "smallm", "quant", "dit", "lora"])
    ap.add_argument("--dit-mode", default="all_gather", choices=["all_gather", "pairs", "tokens"])
    ap.add_argument("--tokens", type=int, default=32768, help="dit: token count")
    ap.add_argument("--blocks", type=int, default=4, help="dit: transformer blocks")
    ap.add_argument("--no-small-m", action="store_true", help="skip the small_m sub-record of the default N = 1 line")
    ap.add_argument("--a-dtype", default="fp16", choices=["fp16", "bf16"], help="one GPU: activation dtype (bf16 goes through feather_scaled_mm_typed)")
    ap.add_argument("--shape", default=None, help="M,N,K: time a single GEMM instead of a workload")
    ap.add_argument("--variant", default=None, help="tokens_tile,cta_pair,split_k,transform_groups,max_ctas (0 = auto)")
    ap.add_argument("--out-dtype", default=None, choices=["bf16", "fp16"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample-rows", type=int, default=2048)
    ap.add_argument("--exchange", default=None, choices=["copy_engine", "peer_store", "all_gather"],
                    help="N > 1: copy engines push each finished column block to the peers on a second stream under the next linear's GEMM; "
                         "fused peer-store epilogue over symmetric memory; or NCCL all-gather + relayout")
    ap.add_argument("--no-alt-exchange", action="store_true", help="N > 1: do not also time the step with the other of copy_engine / peer_store")
    args = ap.parse_args()
    if args.exchange is None:
        args.exchange = "peer_store" if args.workload == "dit" else "copy_engine"
    return args


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


def shapes_for(args):
    if args.shape:
        M, N, K = (int(x) for x in args.shape.split(","))
        return M, [(K, N)], args.out_dtype or "bf16", f"custom M={M} N={N} K={K}"
    M, kn, dt = WORKLOADS[args.workload]
    return M, kn, args.out_dtype or dt, {"wan": "Wan-2.1-14B linears, M=32768 tokens, (K,N) in {(5120,5120),(5120,13824),(13824,5120)}",
                                          "qwen": "Qwen-Image MMDiT linears, M=4352"}[args.workload]


def config_for(args, M, kn_list, out_dtype, desc, world):
    """The `config` object of the JSON line; both arms print the same one for the same arguments."""
    step_mb = sum(2.0 * M * K + K * N + 2.0 * M * N for K, N in kn_list) / 1e6
    l2 = (f"one step touches {step_mb:.0f} MB over {len(kn_list)} linears "
          + ("(larger than the 126 MB L2, so no launch finds its inputs cached); no flush needed" if step_mb > 252
             else "(not larger than twice the 126 MB L2 and no flush between launches: a probe shape, not a bench line)"))
    if world == 1:
        par = "single GPU"
    elif args.exchange == "copy_engine":
        par = (f"weights sharded by output columns over {world} GPUs; each rank's GEMM writes its column block of the [M,N] output and copy engines "
               "push the block to every peer over NVLink on a second stream while the next linear's GEMM runs; one cross-rank barrier per linear on that stream")
    elif args.exchange == "peer_store":
        par = (f"weights sharded by output columns over {world} GPUs; each rank's epilogue TMA-stores its blocks into every rank's output "
               "over NVLink (fused exchange), one cross-rank barrier per linear")
    else:
        par = f"weights sharded by output columns over {world} GPUs; NCCL all-gather of the output + relayout"
    return {"workload": desc, "out_dtype": out_dtype, "l2": l2, "parallelism": par, "variant": args.variant or "auto"}


# ------------------------------------------------------------------------------------------------------
# CPU arm: the reference's naive torch path.  The reference's own kernel/naive.py is used when a copy of the reference is
# at hand ($FEATHER_REFERENCE_DIR or baseline/_ref); otherwise oracle/naive_torch.py, which restates it.
# ------------------------------------------------------------------------------------------------------
def find_reference_naive():
    """The reference's `scaled_mm_naive` loaded by path from its own kernel/naive.py, or None."""
    for base in (os.environ.get("FEATHER_REFERENCE_DIR"), os.path.join(ROOT, "baseline", "_ref")):
        if not base:
            continue
        path = os.path.join(base, "kernel", "naive.py")
        if os.path.exists(path):
            spec = importlib.util.spec_from_file_location("feather_reference_naive", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            return mod.scaled_mm_naive, path
    return None, None


def time_cpu_step(kn_list, out_dtype, rows, repeats=1, warm=True, reference_fn=None):
    from oracle import naive_torch

    torch.manual_seed(0)
    cases = []
    for K, N in kn_list:
        a = torch.randn(rows, K).to(torch.float16)
        w = torch.randn(N, K) / K ** 0.5
        b, s = naive_torch.quantize_prepack_cpu(w)
        cases.append((a, b, s))
    flops = sum(2.0 * rows * K * N for K, N in kn_list)

    def one(a, b, s):
        if reference_fn is not None:
            return reference_fn(a, b, s, None, TORCH_DT[out_dtype], b_prepacked=True)
        return naive_torch.scaled_mm_cpu(a, b, s, None, TORCH_DT[out_dtype])

    if warm:
        a, b, s = cases[0]
        one(a[:64], b, s)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        for a, b, s in cases:
            one(a, b, s)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return flops / t / 1e12, t, flops


def run_reference(args):
    world, rank, _ = dist_env()
    if rank != 0:
        return
    M, kn_list, out_dtype, desc = shapes_for(args)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    rows = min(args.cpu_sample_rows, M)
    ref_fn, ref_path = find_reference_naive()
    for _ in range(max(args.warmup, 1) - 1):
        time_cpu_step(kn_list, out_dtype, min(rows, 256), warm=False)
    reps = max(1, min(args.steps, 3))
    tflops, t, _ = time_cpu_step(kn_list, out_dtype, rows, repeats=reps)
    kind, extra = "port", {}
    sample = f"{rows} of {M} token rows of each linear per step (kernel/naive.py op sequence, fp32 product), median of {reps} steps"
    if ref_fn is not None:
        # the reference's own file, verbatim (its fp16 product overflows at this weight scale; the time is what counts here)
        v_ref, t_ref, _ = time_cpu_step(kn_list, out_dtype, min(rows, 512), repeats=1, reference_fn=ref_fn)
        extra = {"port_value": tflops, "reference_file": "kernel/naive.py (verbatim, fp16 product)", "reference_rows": min(rows, 512)}
        # the faster of the two stands as the baseline, so the GPU/CPU ratio is never flattered by a slow fp16 CPU matmul
        if v_ref >= tflops:
            tflops, t, rows_used, kind = v_ref, t_ref, min(rows, 512), "reference"
            sample = f"{rows_used} of {M} token rows of each linear, the reference's own kernel/naive.py loaded by path"
            rows = rows_used
    line = {
        "impl": "reference", "metric": "TFLOPS fp16@fp8e5m2 scaled_mm at Wan-14B shapes", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3 * (M / rows), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp16xfp8e5m2->fp32", "data": "synthetic",
        "config": config_for(args, M, kn_list, out_dtype, desc, args.gpus),
        "timing": "host wall clock on a bounded row sample; ms_per_step extrapolated linearly in M",
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample, **extra},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------
# Our arm
# ------------------------------------------------------------------------------------------------------
def run_ours(args):
    import __graft_entry__

    __graft_entry__.load_package()
    native = importlib.import_module("feather_b200.kernel.b200.native")
    hk = importlib.import_module("feather_b200.kernel.hip.hip_kernel")
    sharded = importlib.import_module("feather_b200.kernel.b200.sharded")
    import torch.distributed as dist

    world, rank, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU arm)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    native.load_library()

    if args.workload == "smallm" and not args.shape:
        rows = run_smallm(args, native, dev, Ms=(1, 8, 16, 64, 128))
        peaks = load_peaks()
        print(json.dumps({"metric": "GB/s fp16@fp8e5m2 scaled_mm at M<=128", "unit": "GB/s", "peak_hbm_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
                          "config": {"workload": "small-M sweep, 4 rotating weight copies (283 MB > L2); us = CUDA-graph replay, us_eager = per-call launches"},
                          "rows": rows}), flush=True)
        return
    if args.workload == "quant" and not args.shape:
        return run_quant(args, native, dev)
    if args.workload == "dit" and not args.shape:
        return run_dit(args, native, dev, world, rank, local)
    if args.workload == "lora" and not args.shape:
        return run_lora(args, native, hk, dev)

    M, kn_list, out_dtype, desc = shapes_for(args)
    odt = TORCH_DT[out_dtype]
    variant = native.make_variant(*[int(x) for x in args.variant.split(",")]) if args.variant else None

    g = torch.Generator(device=dev).manual_seed(0)
    layers = []
    for K, N in kn_list:
        a = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32).to(torch.float16)
        w = torch.randn((N, K), generator=g, device=dev, dtype=torch.float32) / K ** 0.5
        bq, s = native.quantize_prepack(w)      # loader path: fp32 in, scale = amax / 57344
        del w
        lin = sharded.ColumnShardedLinear(bq, s.reshape(1), None, rank, world, dev, exchange=args.exchange)
        layers.append((a, lin, K, N, bq if world > 1 else None))
    torch.cuda.synchronize()

    typed_outputs = None
    if args.a_dtype == "bf16":
        if world != 1:
            raise SystemExit("--a-dtype bf16 is a one-GPU option")
        layers = [(a.to(torch.bfloat16), lin, K, N, x) for a, lin, K, N, x in layers]
        typed_outputs = [torch.empty((M, N), dtype=odt, device=dev) for _, _, _, N, _ in layers]

    # The three linears of a step are independent, so with the copy-engine exchange nothing on the compute stream waits for a
    # transfer: the exchange of one linear runs under the GEMM of the next (and of the next step's first).  The timed region
    # ends only after the compute stream has waited for every exchange.
    deferred = world > 1 and args.exchange == "copy_engine"

    def step(events=None, linears=None):
        for li, (a, lin, K, N, _) in enumerate(layers):
            lin = linears[li] if linears is not None else lin
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record()
            if typed_outputs is not None:
                native.scaled_mm_typed_into(a, lin.b_local, lin.scale, None, typed_outputs[li], variant=variant)
            elif world > 1 and lin.exchange == "copy_engine":
                lin(a, odt, variant=variant, defer=True)
            else:
                lin(a, odt, variant=variant)
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                events.append((e0, e1))

    launches_per_step = sum(lin.launches_per_call for _, lin, _, _, _ in layers)
    if world > 1 and args.exchange == "copy_engine":
        # If the copy-engine route cannot run on this box (the strided peer copy is refused), every rank falls back to the fused
        # exchange together; the line then says so in `config.parallelism` and `exchange.mode`.
        failed = 0
        try:
            step()
            for _, lin, _, _, _ in layers:
                lin.wait_exchange()
        except native.FeatherNativeError as err:
            failed = 1
            print(f"[bench] copy-engine exchange unavailable on rank {rank}: {err}", file=sys.stderr, flush=True)
        flag = torch.tensor([failed], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag.item()):
            args.exchange = "peer_store"
            layers = [(a, lin.with_exchange("peer_store"), K, N, bq_full) for a, lin, K, N, bq_full in layers]
            deferred = False
    for _ in range(args.warmup):
        step()
    native.check_device_status(dev)

    # The exchanged outputs are checked before anything is timed: on every rank, rows of each [M, N] output against an unsharded
    # GEMM of the same rows on that rank (K is never split, so they must agree bit for bit); MIN over the ranks.
    exchange_check = None
    token_sharded = None
    e2e_rows = None
    if world > 1:
        rows_checked, equal = 0, True
        for a, lin, K, N, bq_full in layers:
            out = lin(a, odt, variant=variant)
            for r0 in sorted({(rank * (M // world)) & ~255, max(M - 300, 0), ((rank + 1) * 1000) % max(M - 256, 1)}):
                r1 = min(r0 + 256, M)
                ref = torch.empty((r1 - r0, N), dtype=odt, device=dev)
                # the same tile class as the sharded launch (the variant chosen for the full token count), so the k-blocks are added in the same order
                native.scaled_mm_into(a[r0:r1], bq_full, lin.scale, None, ref, variant=lin._variant(M, variant))
                equal = equal and torch.equal(out[r0:r1].view(torch.int16), ref.view(torch.int16))
                rows_checked += r1 - r0
        flag = torch.tensor([1 if equal else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        exchange_check = {"bitwise_equal": bool(flag.item()), "layers": len(layers), "rows": rows_checked, "ranks": world,
                          "what": "rows of every exchanged [M,N] output on every rank against an unsharded GEMM of the same rows on that rank"}
        # The same step sharded by token rows instead (weights whole on every rank, M/g rows each, nothing exchanged, every rank
        # ends with its rows of the outputs): the data-parallel form of the path, reported beside the column-sharded line.
        rows = M // world
        replicated = [(a[rank * rows:(rank + 1) * rows], sharded.ReplicatedLinear(bq_full, lin.scale, None, dev), torch.empty((rows, N), dtype=odt, device=dev))
                      for a, lin, K, N, bq_full in layers]
        for _ in range(args.warmup):
            for a_rows, rl, out in replicated:
                rl(a_rows, odt, total_rows=M, out=out)
        torch.cuda.synchronize()
        dist.barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(args.steps):
            for a_rows, rl, out in replicated:
                rl(a_rows, odt, total_rows=M, out=out)
        r1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([r0.elapsed_time(r1) / args.steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        token_sharded = {"ms_per_step": float(t.item()), "tflops": sum(2.0 * M * K * N for K, N in kn_list) / (float(t.item()) * 1e-3) / 1e12,
                         "note": f"token rows sharded ({rows} per rank), weights replicated, no exchange; each rank keeps its rows of the outputs"}
        e2e_rows = [(a_rows, sharded.ColumnShardedLinear(rl.b, rl.scale, None, 0, 1, dev), K, N, None) for (a_rows, rl, _), (_, _, K, N, _) in zip(replicated, layers)]
        del replicated
        for i in range(len(layers)):                       # the full weights were only needed for the check (and the token-sharded legs)
            layers[i] = layers[i][:4] + (None,)
        torch.cuda.empty_cache()
        if not exchange_check["bitwise_equal"]:
            if rank == 0:
                print(json.dumps({"error": "exchange_check failed: an exchanged output differs from the unsharded GEMM", "exchange_check": exchange_check}), flush=True)
            dist.destroy_process_group()
            raise SystemExit(3)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launch_events = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        step(launch_events if world == 1 else None)
    if deferred:
        for _, lin, _, _, _ in layers:
            lin.wait_exchange()
    e1.record()
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if rank == 0:
        time.sleep(0.12)                     # the reading that covers the end of the region is published up to 100 ms later
    clocks = sampler.stop(t_begin, t_end + 0.1) if rank == 0 else None
    native.check_device_status(dev)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    flops_step = sum(2.0 * M * K * N for K, N in kn_list)
    tflops = flops_step / (ms_per_step * 1e-3) / 1e12

    # per-GEMM kernel time on this rank (events on the launching stream): inside the timed region on one GPU (an event pair
    # around every launch), and as a short burst per shape, which is also what a sharded run reports for its local GEMMs
    per_shape = []
    burst_ms = 0.0
    for li, (a, lin, K, N, _) in enumerate(layers):
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, min(args.steps, 10))
        torch.cuda.synchronize()
        k0.record()
        for _ in range(reps):
            if typed_outputs is not None:
                native.scaled_mm_typed_into(a, lin.b_local, lin.scale, None, typed_outputs[li], variant=variant)
            else:
                lin.gemm_only(a, odt, variant=variant)
        k1.record()
        torch.cuda.synchronize()
        t_ms = k0.elapsed_time(k1) / reps
        burst_ms += t_ms
        row = {"K": K, "N": N, "ms_burst": round(t_ms, 4), "tflops_burst": round(2.0 * M * K * (N // world) / (t_ms * 1e-3) / 1e12, 1)}
        if launch_events:
            mine = [launch_events[i] for i in range(li, len(launch_events), len(layers))]
            t_in = sum(x.elapsed_time(y) for x, y in mine) / len(mine)
            row.update({"ms": round(t_in, 4), "tflops": round(2.0 * M * K * N / (t_in * 1e-3) / 1e12, 1)})
        per_shape.append(row)
    peaks = load_peaks()
    local_flops = flops_step / world
    achieved_burst = local_flops / (burst_ms * 1e-3) / 1e12
    if launch_events:
        in_step_ms = sum(x.elapsed_time(y) for x, y in launch_events) / args.steps
        achieved = local_flops / (in_step_ms * 1e-3) / 1e12
        achieved_how = "sum of the CUDA-event durations of the three GEMM launches inside the timed region, averaged over the timed steps"
    else:
        achieved = achieved_burst
        achieved_how = "local GEMMs of this rank timed without the exchange, 3-10 launches in a row per shape"
    timed_seconds = ms * 1e-3
    peak = peaks["tflops_sustained"] if timed_seconds >= 2.0 else peaks["tflops"]
    # DRAM traffic of the dominant launch (ffn-up): measured by ncu at M = 4096 (profiles/scaled_mm_kernel_m4096_n13824_k5120_full.md),
    # 1.23 x that launch's algorithmic bytes (weight tiles are re-read after output writes evicted them from L2); the ratio is
    # applied to the algorithmic bytes of this run's ffn-up launch, since both grow with the token count.
    alg_ffn_up = 2.0 * M * 5120 + 5120 * 13824 + 2.0 * M * 13824
    traffic = 1.23 * alg_ffn_up if (not args.shape and args.workload == "wan" and world == 1) else None
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
        "traffic_note": "dram read+write of the (5120,13824) launch: ncu measured 1.23 x the algorithmic bytes at M=4096 (profiles/scaled_mm_kernel_m4096_n13824_k5120_full.md); "
                        f"applied to this launch's algorithmic bytes {alg_ffn_up:.3e}",
        "kernel": "scaled_mm_kernel", "achieved_how": achieved_how, "achieved_burst": achieved_burst,
        "peak_source": f"{peaks['source']} cuBLAS bf16, {'sustained' if timed_seconds >= 2.0 else 'burst'}",
        "frac_of_burst": achieved / peaks["tflops"], "frac_of_sustained": achieved / peaks["tflops_sustained"],
        "frac_of_nominal_2250": achieved / 2250.0, "frac_step_of_burst": (tflops / world) / peaks["tflops"], "per_shape": per_shape,
    }

    exchange = None
    if world > 1 and args.exchange in ("peer_store", "copy_engine"):
        out_bytes = sum(lin.bytes_out_per_call(M) for _, lin, _, _, _ in layers)
        exchange = {"mode": args.exchange, "bytes_out_per_rank": out_bytes, "bytes_in_per_rank": out_bytes, "gbs_per_rank": out_bytes / (ms_per_step * 1e-3) / 1e9,
                    "nvlink_peer_copy_gbs": 770.0, "frac_of_peer_copy": out_bytes / (ms_per_step * 1e-3) / 1e9 / 770.0,
                    "note": "each rank sends its column block of every output to each peer and receives theirs; the step cannot be shorter than bytes_in / link bandwidth"}
        if not args.no_alt_exchange:
            # the same step with the other exchange, timed the same way (same weights, buffers of its own)
            other = "peer_store" if args.exchange == "copy_engine" else "copy_engine"
            alt = [lin.with_exchange(other) for _, lin, _, _, _ in layers]
            for _ in range(args.warmup):
                step(linears=alt)
            for lin in alt:
                lin.wait_exchange()
            torch.cuda.synchronize()
            dist.barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(args.steps):
                step(linears=alt)
            for lin in alt:
                lin.wait_exchange()
            a1.record()
            torch.cuda.synchronize()
            dist.barrier()
            t = torch.tensor([a0.elapsed_time(a1) / args.steps], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            exchange["alternative"] = {"mode": other, "ms_per_step": float(t.item()), "tflops": flops_step / (float(t.item()) * 1e-3) / 1e12}
            del alt
            native.check_device_status(dev)

    # end to end through the operator with host buffers: pinned H2D of the activations, D2H of the output, every step
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(layers, hk, native, odt, dev, world, rank, flops_step, steps=max(2, min(args.steps, 5)), variant=variant) if typed_outputs is None else None
        if e2e is not None and e2e_rows is not None:
            # Host buffers in, host buffers out needs no exchange at all when the ranks split the token rows: every rank uploads its
            # M/g rows, multiplies them with the whole weights and downloads its rows of the outputs - nothing crosses NVLink.
            # That is the end-to-end form of the job on N GPUs; the column-sharded one (all-gather of the uploaded rows, sharded
            # linear, exchange) is kept beside it.
            bound = bind_to_gpu_numa_node(dev)
            rows_leg = run_e2e(e2e_rows, hk, native, odt, dev, 1, rank, flops_step / world, steps=max(2, min(args.steps, 5)), variant=None, all_ranks=world)
            rows_leg["column_sharded"] = {k: e2e[k] for k in ("value", "note")}
            rows_leg["host_binding_rank0"] = bound
            e2e = rows_leg

    small_m = None
    if world == 1 and args.workload == "wan" and not args.shape and not args.no_small_m:
        small_m = {"unit": "GB/s", "peak_hbm_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
                   "how": "algorithmic bytes 2MK+KN+2MN over the CUDA-graph replay time per launch; 4 rotating weight copies (283 MB > L2)",
                   "rows": run_smallm(args, native, dev, Ms=(1, 16, 128), steps=20)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        rows = min(args.cpu_sample_rows, M)
        v, t, _ = time_cpu_step(kn_list, out_dtype, rows)
        cpu = {"value": v, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"{rows} of {M} token rows of each linear, one pass ({t:.1f} s), torch CPU restatement of kernel/naive.py with an fp32 product"}

    if rank == 0:
        line = {
            "metric": "TFLOPS fp16@fp8e5m2 scaled_mm at Wan-14B shapes", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp16xfp8e5m2->fp32", "data": "synthetic",
            "config": config_for(args, M, kn_list, out_dtype, desc, world),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        }
        if exchange_check is not None:
            line["exchange_check"] = exchange_check
        if exchange is not None:
            line["exchange"] = exchange
        if token_sharded is not None:
            line["token_sharded"] = token_sharded
        if small_m is not None:
            line["small_m"] = small_m
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def bind_to_gpu_numa_node(dev):
    """Runs this process on the cores of the NUMA node the GPU hangs off, so that the pinned host buffers allocated afterwards
    are first touched there and the copies do not cross the socket link.  Returns a short description, or None if the
    topology cannot be read (then nothing changes)."""
    try:
        props = torch.cuda.get_device_properties(dev)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return f"numa node {node}, {len(allowed)} cores"
    except (OSError, ValueError, AttributeError):
        return None


def run_e2e(layers, hk, native, odt, dev, world, rank, flops_step, steps, variant=None, all_ranks=1):
    """The same step with HOST activations and outputs: H2D + kernel + D2H inside the timed region, every step.

    One GPU: through the operator `scaled_mm_hip`, each linear in four row chunks on copy-in / GEMM / copy-out streams.
    Several GPUs, two forms.  Token rows split over the ranks (`all_ranks` > 1: this function runs on every rank over its own
    M/g rows with the whole weights, nothing is exchanged) is the line's `e2e`.  The column-sharded form (run_e2e_sharded:
    every rank uploads its M/g rows, the rows are all-gathered over NVLink, the sharded linear runs with its exchange, every
    rank downloads its M/g rows of the exchanged output) is reported beside it.  Either way the box as a whole moves every
    activation byte up and every output byte down, once, every step.
    """
    import torch.distributed as dist

    if world > 1:
        return run_e2e_sharded(layers, native, odt, dev, world, rank, flops_step, steps, variant)
    host = []
    h2d = d2h = 0
    for a, lin, K, N, _ in layers:
        ha = torch.empty(a.shape, dtype=a.dtype, pin_memory=True)
        ha.copy_(a)
        hc = torch.empty((a.shape[0], lin.n_local), dtype=odt, pin_memory=True)
        host.append((ha, hc))
        h2d += ha.numel() * ha.element_size()
        d2h += hc.numel() * hc.element_size()

    # Three streams: rows of the next chunk go up while the current chunk is multiplied and the previous chunk's result
    # goes down (PCIe is full duplex).  Every byte of every step still crosses the bus inside the timed region.
    s_in, s_mm, s_out = (torch.cuda.Stream(dev) for _ in range(3))
    chunks = 4
    staging = []
    for a, lin, K, N, _ in layers:
        rows = (a.shape[0] + chunks - 1) // chunks
        staging.append((rows, [torch.empty((rows, a.shape[1]), dtype=a.dtype, device=dev) for _ in range(2)]))
    mm_done = {}

    def e2e_step():
        for li, ((ha, hc), (a, lin, K, N, _)) in enumerate(zip(host, layers)):
            rows, bufs = staging[li]
            for c in range(chunks):
                r0, r1 = c * rows, min((c + 1) * rows, ha.shape[0])
                if r0 >= r1:
                    break
                slot = c % 2
                with torch.cuda.stream(s_in):
                    if (li, slot) in mm_done:
                        s_in.wait_event(mm_done[(li, slot)])          # the GEMM that read this staging buffer is done
                    da = bufs[slot][: r1 - r0]
                    da.copy_(ha[r0:r1], non_blocking=True)
                    ev_in = torch.cuda.Event()
                    ev_in.record(s_in)
                with torch.cuda.stream(s_mm):
                    s_mm.wait_event(ev_in)
                    out = hk.scaled_mm_hip(da, lin.b_local, lin.scale, lin.bias_local, odt)
                    ev_mm = torch.cuda.Event()
                    ev_mm.record(s_mm)
                    mm_done[(li, slot)] = ev_mm
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_mm)
                    hc[r0:r1].copy_(out, non_blocking=True)
                    out.record_stream(s_out)

    e2e_step()
    torch.cuda.synchronize()
    if all_ranks > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    native.check_device_status(dev)
    note = "weights stay resident on the GPU; activations come from and outputs return to pinned host memory every step, in 4 row chunks per linear on copy-in / GEMM / copy-out streams"
    if all_ranks > 1:
        # every rank ran this over its own M/g token rows (whole weights, no exchange): the slowest rank's time counts
        t = torch.tensor([dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        return {"value": flops_step * all_ranks * steps / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * all_ranks, "d2h_bytes_per_step": d2h * all_ranks,
                "h2d_bytes_per_step_per_rank": h2d, "d2h_bytes_per_step_per_rank": d2h,
                "note": f"token rows split over the {all_ranks} ranks, weights whole on every rank, no exchange; " + note + "; bytes are totals over the ranks"}
    return {"value": flops_step * steps / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "note": note}


def run_e2e_sharded(layers, native, odt, dev, world, rank, flops_step, steps, variant):
    import torch.distributed as dist

    host, dev_bufs = [], []
    h2d = d2h = 0
    for a, lin, K, N, _ in layers:
        M = a.shape[0]
        rows = M // world
        r0 = rank * rows
        ha = torch.empty((rows, K), dtype=a.dtype, pin_memory=True)
        ha.copy_(a[r0:r0 + rows])
        hc = torch.empty((rows, N), dtype=odt, pin_memory=True)
        host.append((ha, hc, r0, rows))
        dev_bufs.append((torch.empty((rows, K), dtype=a.dtype, device=dev), torch.empty((world * rows, K), dtype=a.dtype, device=dev)))
        h2d += ha.numel() * ha.element_size()
        d2h += hc.numel() * hc.element_size()
    s_in, s_mm, s_out = (torch.cuda.Stream(dev) for _ in range(3))
    done = {}

    def e2e_step():
        for li, ((ha, hc, r0, rows), (a, lin, K, N, _)) in enumerate(zip(host, layers)):
            mine, full = dev_bufs[li]
            with torch.cuda.stream(s_in):
                if li in done:
                    s_in.wait_event(done[li])                 # the GEMM that read `full` in the previous step is done
                mine.copy_(ha, non_blocking=True)
                dist.all_gather_into_tensor(full, mine)       # rank-major concatenation of row blocks = the [M, K] activations
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            with torch.cuda.stream(s_mm):
                s_mm.wait_event(ev_in)
                deferred = lin.exchange == "copy_engine"
                out = lin(full, odt, variant=variant, defer=True) if deferred else lin(full, odt, variant=variant)
                ev_mm = torch.cuda.Event()
                ev_mm.record(s_mm)
                done[li] = ev_mm
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_mm)
                if deferred:
                    lin.wait_exchange(s_out)                  # the download waits for the peers' blocks, the next GEMM does not
                hc.copy_(out[r0:r0 + rows], non_blocking=True)
                ev_out = torch.cuda.Event()
                ev_out.record(s_out)
            # the exchanged output is double-buffered inside the linear: its next overwrite is two calls away, and this copy is
            # ordered before it by making the GEMM stream wait for the copy
            s_mm.wait_event(ev_out)

    e2e_step()
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    native.check_device_status(dev)
    t = torch.tensor([dt], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t.item())
    return {"value": flops_step * steps / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
            "h2d_bytes_per_step_per_rank": h2d, "d2h_bytes_per_step_per_rank": d2h,
            "note": "weights stay resident; every step each rank uploads its M/g rows of every activation from pinned host memory, the rows are all-gathered over "
                    "NVLink (NCCL), the column-sharded linear runs with its exchange, and each rank downloads its M/g rows of the output; bytes are totals over the ranks"}


def run_smallm(args, native, dev, Ms=(1, 8, 16, 64, 128), steps=None):
    """Bandwidth-bound sweep: M x {(5120,13824),(13824,5120)}, GB/s of algorithmic bytes.  Four weight copies (> L2 in total)
    are rotated so the weight is read from HBM, not from L2.  Returns one row per (M, K, N)."""
    peaks = load_peaks()
    steps = steps if steps is not None else args.steps
    rows = []
    side = torch.cuda.Stream()          # one capture stream for every graph: the split-K workspace belongs to the (device, stream) pair
    for K, N in ((5120, 13824), (13824, 5120)):
        g = torch.Generator(device=dev).manual_seed(0)
        w = torch.randn((N, K), generator=g, device=dev) / K ** 0.5
        bq, s = native.quantize_prepack(w)
        del w
        copies = [bq] + [bq.clone() for _ in range(3)]
        s = s.reshape(1)
        for M in Ms:
            a = torch.randn((M, K), generator=g, device=dev).to(torch.float16)
            c = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            variant = native.make_variant(*[int(x) for x in args.variant.split(",")]) if (args.variant and args.workload == "smallm") else None

            def sweep():
                for b in copies:
                    native.scaled_mm_into(a, b, s, None, c, variant=variant)

            for _ in range(max(args.warmup, 3)):
                sweep()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                sweep()
            e1.record()
            torch.cuda.synchronize()
            us_eager = e0.elapsed_time(e1) * 1e3 / (steps * len(copies))
            # the same launches replayed from a CUDA graph: kernel time without the host's per-call cost
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                sweep()
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(5):
                        sweep()
            for _ in range(2):
                graph.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (steps * 5 * len(copies))
            nbytes = 2 * M * K + K * N + 2 * M * N + 4
            v = native.choose_variant(M, N, K)
            rows.append({"M": M, "K": K, "N": N, "us": round(us, 2), "us_eager": round(us_eager, 2), "gbs": round(nbytes / us / 1e3, 1),
                         "frac_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 3), "tflops": round(2.0 * M * N * K / us / 1e6, 2),
                         "kernel": {1: "tensor-memory", 2: "streaming"}.get(v.kernel, "auto"), "variant": v.as_tuple()})
            del graph
        del copies
    native.check_device_status(dev)
    torch.cuda.empty_cache()
    return rows


def run_dit(args, native, dev, world, rank, local):
    """The random-init 4-block Wan-like DiT forward (hidden 5120, 40 x 128 heads, FFN 13824 GELU, RMSNorm, torch SDPA, bf16
    compute) with every linear a Feather e5m2 linear; one forward per step.  Reports model TFLOP/s (linears + attention) and
    where the time goes (a second, instrumented pass with a device synchronisation around each part)."""
    import torch.distributed as dist

    dit = importlib.import_module("feather_b200.kernel.b200.dit")
    cfg = dit.DitConfig(blocks=args.blocks)
    T = args.tokens
    model = dit.FeatherDiT(cfg, rank=rank, world=world, device=dev, mode=args.dit_mode, exchange=args.exchange, seed=0)
    x = torch.randn((T, cfg.hidden), generator=torch.Generator(device=dev).manual_seed(1), device=dev).to(torch.bfloat16)
    torch.cuda.synchronize()
    for _ in range(max(args.warmup, 1)):
        y = model(x)
    native.check_device_status(dev)
    check = None
    if world > 1:
        # every rank must hold the same output; in all-gather mode it is also bitwise the one-rank forward (tests/test_multi_gpu.py)
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y.contiguous())
        same = all(torch.equal(t.view(torch.int16), gathered[0].view(torch.int16)) for t in gathered)
        check = {"identical_on_all_ranks": bool(same), "finite": bool(torch.isfinite(y.float()).all().item())}
        del gathered
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        y = model(x)
    e1.record()
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    native.check_device_status(dev)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps

    # where the time goes: the linears alone (their inputs captured by a hook, replayed back to back, exchange included)
    captured = []
    model(x, hook=lambda name, i, a16, out: captured.append((name, i, a16)) if i == 0 else None)
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    blk = model.blocks[0]
    if world > 1:
        dist.barrier()
    k0.record()
    for _ in range(3):
        for name, _, a16 in captured:
            kw = {"residual": x} if (args.dit_mode == "pairs" and name in ("o", "down")) else {}
            if args.dit_mode == "tokens":
                kw = {"total_rows": T}
            blk[name](a16, torch.bfloat16, **kw)
    k1.record()
    torch.cuda.synchronize()
    lin_ms_block = k0.elapsed_time(k1) / 3
    lin_flops = cfg.linear_flops(T)
    attn_flops = cfg.attention_flops(T)
    peaks = load_peaks()
    if rank == 0:
        total = (lin_flops + attn_flops) / (ms_per_step * 1e-3) / 1e12
        line = {
            "metric": "model TFLOP/s of the 4-block Wan-like DiT forward (Feather e5m2 linears + torch SDPA)", "value": total, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 activations; linears fp16xfp8e5m2->fp32->bf16", "data": "synthetic",
            "config": {"workload": f"{cfg.blocks}-block Wan-like DiT forward, {T} tokens, hidden {cfg.hidden}, {cfg.heads}x{cfg.head_dim} heads, FFN {cfg.ffn} GELU, RMSNorm, torch SDPA",
                       "mode": args.dit_mode, "exchange": {"all_gather": args.exchange, "pairs": "reduce-scatter fused into the row-parallel GEMM + reduce/all-gather kernel",
                                                                "tokens": "token rows sharded, weights replicated: no exchange in any linear; keys and values all-gathered per block by copy engines"}[args.dit_mode],
                       "l2": "activations of one block exceed the 126 MB L2 many times over; no flush needed"},
            "flops": {"linears": lin_flops, "attention": attn_flops},
            "linears": {"ms_per_block_with_exchange": lin_ms_block, "tflops_whole_job": lin_flops / cfg.blocks / (lin_ms_block * 1e-3) / 1e12,
                        "frac_of_g_x_burst_peak": lin_flops / cfg.blocks / (lin_ms_block * 1e-3) / 1e12 / (world * peaks["tflops"]),
                        "share_of_step": lin_ms_block * cfg.blocks / ms_per_step},
            "rank_check": check, "gpu_launches": sum(lin.launches_per_call for _, _, lin in model.linears()) * args.steps, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_lora(args, native, hk, dev):
    """Un-merged LoRA on the Wan ffn-up linear (M = 32768, K = 5120, N = 13824, bf16 model, rank 64): the patch folded into the
    GEMM's accumulator (`scaled_mm_lora`) against the reference's sequence (linear, two GEMMs, y += up * strength)."""
    # loaded by path: importing the comfy_feather package would pull in the ComfyUI loader node
    spec = importlib.util.spec_from_file_location("feather_b200_lora", os.path.join(ROOT, "comfyui-featherops_b200", "comfy_feather", "lora.py"))
    lora = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(lora)
    M, K, N, r = 32768, 5120, 13824, 64
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16)
    w = torch.randn((N, K), generator=g, device=dev) / K ** 0.5
    bq, s = native.quantize_prepack(w)
    s = s.reshape(1)
    del w
    A = torch.randn((r, K), generator=g, device=dev) / K ** 0.5
    B = torch.randn((N, r), generator=g, device=dev) / r ** 0.5

    class Adapter:
        weights = (B, A, float(r), None, None, None)

    class PatchFn:
        key = "w"
        patches = {"w": [(1.0, Adapter(), 1.0, None, None)]}

    patch = [PatchFn()]

    # what `FeatherOps.Linear` does with a bf16 input: the library's cast kernel, then the fp16 kernels (the cast is timed)
    def plain():
        return hk.scaled_mm_b200(native.bf16_to_fp16(x), bq, s, None, torch.bfloat16, torch.bfloat16)

    def unfused():
        return lora.apply_lora_patches(x, plain(), patch)

    def fused():
        x16 = native.bf16_to_fp16(x)
        t, lb = lora.fused_lora_operands(x16, patch, s)
        return hk.scaled_mm_lora(x16, bq, s, None, torch.bfloat16, torch.bfloat16, t, lb)

    rows = {}
    for name, fn in (("linear alone", plain), ("reference sequence (linear, 2 GEMMs, add)", unfused), ("folded into the GEMM (operands prepared every call)", fused)):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        rows[name] = round(e0.elapsed_time(e1) / args.steps, 4)
    diff = (fused().float() - unfused().float()).abs().max().item()
    native.check_device_status(dev)
    print(json.dumps({"metric": "ms per call, Wan ffn-up linear with one un-merged rank-64 LoRA patch, bf16 model", "unit": "ms", "M": M, "K": K, "N": N, "rank": r,
                      "ms": rows, "max_abs_difference_between_the_two": diff}), flush=True)


def run_quant(args, native, dev):
    """quantise + prepack of one Wan ffn weight (13824 x 5120): GB/s of one-pass bytes (read s*N*K, write N*K) and of the
    two-pass bytes the amax dependency imposes on a weight larger than L2 (read 2*s*N*K, write N*K)."""
    peaks = load_peaks()
    N, K = 13824, 5120
    rows = []
    for dt, size in ((torch.float32, 4), (torch.bfloat16, 2), (torch.float16, 2)):
        w = (torch.randn((N, K), device=dev) / K ** 0.5).to(dt)
        for _ in range(3):
            native.quantize_prepack(w)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            native.quantize_prepack(w)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        nbytes = (size + 1) * N * K          # one pass: what a weight that stays in L2 between the two kernels would cost
        nbytes2 = (2 * size + 1) * N * K     # two passes: amax over the whole weight must finish before any byte is quantised
        rows.append({"src": str(dt).replace("torch.", ""), "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 3),
                     "gbs_two_pass": round(nbytes2 / us / 1e3, 1), "frac_hbm_two_pass": round(nbytes2 / us / 1e3 / peaks["hbm_gbs"], 3)})
    print(json.dumps({"metric": "GB/s quantise+prepack (13824x5120)", "unit": "GB/s", "peak_hbm_gbs": peaks["hbm_gbs"], "rows": rows}), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
