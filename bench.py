#!/usr/bin/env python3
"""Benchmark of the FeatherOps mixed-precision linear on B200: TFLOPS of fp16 @ prepacked fp8e5m2 GEMMs at Wan-14B shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W]            our arm (CUDA kernels through the C ABI)
    python bench.py --impl reference ...                           the reference's naive torch path on the host cores

A step is one pass over the workload's linears (default: the three Wan-2.1-14B shapes at M = 32768 tokens, bf16 out).
One JSON line is printed by rank 0.  For N > 1 (launched with torch.distributed.run) every GEMM is sharded by weight
columns across the ranks and followed by an all-gather of the output over NCCL.

Other workloads (not the driver's line): --workload qwen | smallm | quant, or --shape M,N,K for a single GEMM.
"""

import argparse
import importlib
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
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
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
        busy = [c for c, p in zip(sm, pw) if p > 0.5 * max(pw)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "power_w_max": max(pw), "samples": len(sm), "reasons": sorted(reasons)}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="wan", choices=["wan", "qwen", "smallm", "quant"])
    ap.add_argument("--shape", default=None, help="M,N,K: time a single GEMM instead of a workload")
    ap.add_argument("--variant", default=None, help="tokens_tile,cta_pair,split_k,transform_groups,max_ctas (0 = auto)")
    ap.add_argument("--out-dtype", default=None, choices=["bf16", "fp16"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample-rows", type=int, default=2048)
    ap.add_argument("--exchange", default="peer_store", choices=["peer_store", "all_gather"],
                    help="N > 1: fused peer-store epilogue over symmetric memory, or NCCL all-gather + relayout")
    return ap.parse_args()


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


# ------------------------------------------------------------------------------------------------------
# CPU arm: the reference's naive torch path (oracle/naive_torch.py restates kernel/naive.py; fp32 product)
# ------------------------------------------------------------------------------------------------------
def time_cpu_step(kn_list, out_dtype, rows, repeats=1, warm=True):
    from oracle import naive_torch

    torch.manual_seed(0)
    cases = []
    for K, N in kn_list:
        a = torch.randn(rows, K).to(torch.float16)
        w = torch.randn(N, K) / K ** 0.5
        b, s = naive_torch.quantize_prepack_cpu(w)
        cases.append((a, b, s))
    flops = sum(2.0 * rows * K * N for K, N in kn_list)
    if warm:
        a, b, s = cases[0]
        naive_torch.scaled_mm_cpu(a[:64], b, s, None, TORCH_DT[out_dtype])
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        for a, b, s in cases:
            naive_torch.scaled_mm_cpu(a, b, s, None, TORCH_DT[out_dtype])
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
    for _ in range(max(args.warmup, 1) - 1):
        time_cpu_step(kn_list, out_dtype, min(rows, 256), warm=False)
    tflops, t, _ = time_cpu_step(kn_list, out_dtype, rows, repeats=max(1, min(args.steps, 3)))
    sample = f"{rows} of {M} token rows of each linear per step (kernel/naive.py op sequence, fp32 product), median of {max(1, min(args.steps, 3))} steps"
    line = {
        "impl": "reference", "metric": "TFLOPS fp16@fp8e5m2 scaled_mm at Wan-14B shapes", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3 * (M / rows), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp16xfp8e5m2->fp32", "data": "synthetic",
        "config": {"workload": desc, "out_dtype": out_dtype, "timing": "host wall clock on a bounded row sample; ms_per_step extrapolated linearly in M"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
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
        return run_smallm(args, native, dev)
    if args.workload == "quant" and not args.shape:
        return run_quant(args, native, dev)

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
        layers.append((a, lin, K, N))
    torch.cuda.synchronize()

    def step():
        for a, lin, K, N in layers:
            lin(a, odt, variant=variant)

    launches_per_step = sum(lin.launches_per_call for _, lin, _, _ in layers)
    for _ in range(args.warmup):
        step()
    native.check_device_status(dev)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    native.check_device_status(dev)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    flops_step = sum(2.0 * M * K * N for K, N in kn_list)
    # bytes one step touches (activations, weights, outputs of all its linears) against the 126 MB L2
    step_mb = sum(2.0 * M * K + K * N + 2.0 * M * N for K, N in kn_list) / 1e6
    l2_note = (f"one step touches {step_mb:.0f} MB over {len(kn_list)} linears "
               + ("(larger than the 126 MB L2, so no launch finds its inputs cached)" if step_mb > 252 else "(not larger than twice the 126 MB L2 and no flush between launches: a probe shape, not a bench line)"))
    tflops = flops_step / (ms_per_step * 1e-3) / 1e12

    # per-GEMM kernel time on this rank (events on the launching stream), for the roofline line
    gemm_ms = 0.0
    per_shape = []
    for a, lin, K, N in layers:
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, min(args.steps, 10))
        torch.cuda.synchronize()
        k0.record()
        for _ in range(reps):
            lin.gemm_only(a, odt, variant=variant)
        k1.record()
        torch.cuda.synchronize()
        t_ms = k0.elapsed_time(k1) / reps
        gemm_ms += t_ms
        per_shape.append({"K": K, "N": N, "ms": round(t_ms, 4), "tflops": round(2.0 * M * K * (N // world) / (t_ms * 1e-3) / 1e12, 1)})
    peaks = load_peaks()
    local_flops = flops_step / world
    achieved = local_flops / (gemm_ms * 1e-3) / 1e12
    timed_seconds = ms * 1e-3
    peak = peaks["tflops_sustained"] if timed_seconds >= 2.0 else peaks["tflops"]
    # DRAM bytes per launch of the dominant kernel from the ncu capture in profiles/ (278.9 MB at M = 4096, N = 13824,
    # K = 5120), scaled by the token count for the ffn-up launch of this run; null for other workloads.
    traffic = 278.9e6 * (M / 4096.0) if (not args.shape and args.workload == "wan" and world == 1) else None
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
        "traffic_note": "ncu dram read+write of the (5120,13824) launch at M=4096, scaled by M/4096; algorithmic bytes of that launch: 1.31e9",
        "kernel": "scaled_mm_kernel", "peak_source": f"{peaks['source']} cuBLAS bf16, {'sustained' if timed_seconds >= 2.0 else 'burst'}",
        "frac_of_burst": achieved / peaks["tflops"], "frac_of_sustained": achieved / peaks["tflops_sustained"],
        "frac_of_nominal_2250": achieved / 2250.0, "per_shape": per_shape,
    }

    # end to end through the operator with host buffers: pinned H2D of the activations, D2H of the output, every step
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(layers, hk, native, odt, dev, world, rank, flops_step, steps=max(2, min(args.steps, 5)))

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
            "config": {"workload": desc, "out_dtype": out_dtype, "l2": l2_note,
                       "parallelism": "single GPU" if world == 1 else (
                           f"weights sharded by output columns over {world} GPUs; " + ("each rank's epilogue TMA-stores its blocks into every rank's output over NVLink (fused exchange)"
                                                                                      if args.exchange == "peer_store" else "NCCL all-gather of the output + relayout")),
                       "variant": args.variant or "auto"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(layers, hk, native, odt, dev, world, rank, flops_step, steps):
    """Same step through `scaled_mm_hip` with HOST activations and outputs: H2D + kernel + D2H inside the timed region."""
    import torch.distributed as dist

    host = []
    h2d = d2h = 0
    for a, lin, K, N in layers:
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
    for a, lin, K, N in layers:
        rows = (a.shape[0] + chunks - 1) // chunks
        staging.append((rows, [torch.empty((rows, a.shape[1]), dtype=a.dtype, device=dev) for _ in range(2)]))
    mm_done = {}

    def e2e_step():
        for li, ((ha, hc), (a, lin, K, N)) in enumerate(zip(host, layers)):
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
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    native.check_device_status(dev)
    if world > 1:
        t = torch.tensor([dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    return {"value": flops_step * steps / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "note": "weights stay resident on the GPU; activations come from and outputs return to pinned host memory every step, in 4 row chunks per linear on copy-in / GEMM / copy-out streams"}


def run_smallm(args, native, dev):
    """Bandwidth-bound sweep: M in {1,16,128} x {(5120,13824),(13824,5120)}, GB/s of algorithmic bytes.  Four weight
    copies (> L2 in total) are rotated so the weight is read from HBM, not from L2."""
    peaks = load_peaks()
    rows = []
    for K, N in ((5120, 13824), (13824, 5120)):
        g = torch.Generator(device=dev).manual_seed(0)
        w = torch.randn((N, K), generator=g, device=dev) / K ** 0.5
        bq, s = native.quantize_prepack(w)
        del w
        copies = [bq] + [bq.clone() for _ in range(3)]
        s = s.reshape(1)
        for M in (1, 8, 16, 64, 128):
            a = torch.randn((M, K), generator=g, device=dev).to(torch.float16)
            c = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            variant = native.make_variant(*[int(x) for x in args.variant.split(",")]) if args.variant else None
            def sweep():
                for b in copies:
                    native.scaled_mm_into(a, b, s, None, c, variant=variant)

            for _ in range(max(args.warmup, 3)):
                sweep()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(args.steps):
                sweep()
            e1.record()
            torch.cuda.synchronize()
            us_eager = e0.elapsed_time(e1) * 1e3 / (args.steps * len(copies))
            # the same launches replayed from a CUDA graph: kernel time without the host's per-call cost
            graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
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
            for _ in range(args.steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (args.steps * 5 * len(copies))
            nbytes = 2 * M * K + K * N + 2 * M * N + 4
            v = native.choose_variant(M, N, K)
            rows.append({"M": M, "K": K, "N": N, "us": round(us, 2), "us_eager": round(us_eager, 2), "gbs": round(nbytes / us / 1e3, 1),
                         "frac_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 3), "tflops": round(2.0 * M * N * K / us / 1e6, 2),
                         "kernel": {1: "tensor-memory", 2: "streaming"}.get(v.kernel, "auto"), "variant": v.as_tuple()})
    native.check_device_status(dev)
    print(json.dumps({"metric": "GB/s fp16@fp8e5m2 scaled_mm at M<=128", "unit": "GB/s", "peak_hbm_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"],
                      "config": {"workload": "small-M sweep, 4 rotating weight copies (283 MB > L2); us = CUDA-graph replay, us_eager = per-call launches"}, "rows": rows}), flush=True)


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
