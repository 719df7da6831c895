"""Benchmark of the GPTQ-2D hot path on B200: seconds per 8192 x 8192 INT4 layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size 8192]

One step = quantize one synthetic 8192 x 8192 fp32 layer to INT4 (symmetric, per-row fp16 abs-max scales) from its
weights and its two Hessian factors G (output side) and H (input side): factor preparation ``ldl_of_inverse`` of both,
the per-row scales, and the two-sided GPTQ-2D sweep, all through the package's public calls (which reach the kernels
through the C ABI).  Steps are issued through ``layer_set.LayerPipeline``, as a layer-set job issues its matrices: the
factor preparation of a step runs beside the sweep of the step before, so the headline is the time per layer of a running
job with two layers in flight; ``config`` also reports one layer alone, and the sweep alone (the reference's own timing
unit, demo.ipynb:157).  ``e2e`` is the same with host buffers: G, H and W in from pinned memory and Z out, every step,
inside the timed region.  With N > 1 ranks (one per GPU, launched by torchrun) every rank quantizes its own layer: the
path shards by matrix and has no collective.
Rank 0 prints one JSON line.  ``--impl reference`` times the CPU restatement of the reference's PyTorch path
(``oracle/``) on the host cores instead, on a bounded sample scaled by the algorithmic work.
"""
from __future__ import annotations

import argparse
import ctypes
import functools
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "gptq-2d_b200"))
sys.path.insert(0, ROOT)

METRIC = "s per 8192x8192 INT4 GPTQ-2D layer"


def sweep_flops(m: int, n: int) -> float:
    return float(m) * n * (m + n - 2)


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        data["source"] = "measured"
        return data
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(sm_max), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_prep_sample(size: int):
    """Time the CPU oracle's ldl_of_inverse on one bounded sample; returns seconds."""
    import numpy as np
    from oracle import oracle

    rng = np.random.default_rng(1)
    x = (rng.standard_normal((2 * size, size)) * np.exp(rng.standard_normal(size))).astype(np.float32)
    gram = x.T @ x / (2 * size)
    gram += 0.01 * np.mean(np.diag(gram)) * np.eye(size, dtype=np.float32)
    oracle.lib()
    start = time.perf_counter()
    oracle.ldl_of_inverse(gram.astype(np.float32))
    return time.perf_counter() - start


def cpu_layer_estimate(args):
    """Seconds per full-size layer on the host: sweep sample and factor-preparation sample, each scaled by its work."""
    sweep_s, cores = cpu_sweep_sample(args.cpu_sample)
    sweep_factor = sweep_flops(args.size, args.size) / sweep_flops(args.cpu_sample, args.cpu_sample)
    prep_size = max(256, args.cpu_sample // 2)
    prep_s = cpu_prep_sample(prep_size)
    prep_factor = 2 * (args.size / prep_size) ** 3
    note = (f"oracle port (OpenMP): {args.cpu_sample}x{args.cpu_sample} INT4 sweep {sweep_s:.2f} s scaled x{sweep_factor:.1f} by m n (m + n - 2), "
            f"plus ldl_of_inverse at n={prep_size} {prep_s:.2f} s scaled x{prep_factor:.0f} (two factors, n^3)")
    return sweep_s * sweep_factor + prep_s * prep_factor, sweep_s + prep_s, cores, note


def cpu_sweep_sample(size: int, threads_hint: int | None = None):
    """Time the CPU oracle's sweep (the restated reference PyTorch path) on a bounded sample; returns (seconds, cores)."""
    import numpy as np
    from oracle import oracle

    rng = np.random.default_rng(0)
    w = (0.02 * rng.standard_normal((size, size))).astype(np.float32)
    l = np.tril(rng.standard_normal((size, size)) * (0.3 / np.sqrt(size)), -1).astype(np.float32)
    u = np.triu(rng.standard_normal((size, size)) * (0.3 / np.sqrt(size)), 1).astype(np.float32)
    scale = np.broadcast_to(oracle.absmax_scale(w, -8, 7, oracle.FP16), (size, size))
    zero = np.zeros((size, size), dtype=np.float32)
    oracle.lib()
    start = time.perf_counter()
    oracle.sweep(w, l, u, kind=oracle.Q_AFFINE, scale=scale, zero_point=zero, qmin=-8, qmax=7)
    return time.perf_counter() - start, os.cpu_count() or 1


def run_reference(args) -> None:
    """The reference arm: the oracle port of the reference's CPU path, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times, raw = [], []
    for step in range(args.warmup + args.steps):
        per_layer, sample_seconds, cores, note = cpu_layer_estimate(args)
        if step >= args.warmup:
            times.append(per_layer)
            raw.append(sample_seconds)
    per_layer = statistics.mean(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": per_layer, "unit": "s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(raw), "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.size}x{args.size} fp32 layer from W, G, H: ldl_of_inverse x2, INT4 symmetric per-row fp16 abs-max scales, two-sided sweep",
                   "sample": note},
        "cpu_baseline": {"value": per_layer, "unit": "s", "cores": cores, "kind": "port", "sample": note},
        "e2e": {"value": per_layer, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--size", type=int, default=8192)
    parser.add_argument("--cpu-sample", type=int, default=2048)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    import _abi
    import gptq_2d as G
    import quantizer_int as Q
    import kron_factors as K
    import synthetic

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path. Use --impl reference for the CPU arm.")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _abi.library()

    m = n = args.size
    # ---- untimed setup: one seeded layer per rank (weights and the two Hessian factors) ----
    w, g, h = synthetic.make_layer(m, n, seed=1000 + rank, device=device, samples=m)
    zero = torch.zeros(1, 1, device=device).expand(m, n)
    quantizer = functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7)

    def sweep_only(weights, l, u):
        scale = Q.int_abs_max_scale_triton(weights, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
        return G.gptq_2d(weights, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))

    import layer_set
    pipeline = layer_set.LayerPipeline(device)

    def step(weights, gram_out=g, gram_in=h):
        # the call a layer-set job makes per matrix: factor preparation on the pipeline's front stream (beside the sweep
        # of the step before), scales and sweep on the current stream
        return pipeline.quantize(weights, gram_out, gram_in)

    def single_layer(weights, gram_out=g, gram_in=h):
        l, u = K.feedback_factors_from_grams(gram_out, gram_in)
        return sweep_only(weights, l, u)

    l, u = K.ldl_of_inverse(g), K.ldl_of_inverse(h).T.contiguous()  # checked once: raises if a factor is not positive definite

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        z = step(w)
    barrier()
    launches_before = lib.g2d_launch_count()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        begin.record()
        for _ in range(args.steps):
            z = step(w)
        end.record()
        barrier()
    elapsed_ms = begin.elapsed_time(end)
    launches = lib.g2d_launch_count() - launches_before
    if world > 1:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = t.item()
    ms_per_step = elapsed_ms / args.steps
    # the sweep alone and the preparation alone, same events, outside the headline region
    parts = {}
    for name, fn in (("sweep", lambda: sweep_only(w, l, u)), ("prep", lambda: K.feedback_factors_from_grams(g, h)),
                     ("single_layer", lambda: single_layer(w))):
        fn()
        torch.cuda.synchronize()
        begin.record()
        for _ in range(args.steps):
            fn()
        end.record()
        torch.cuda.synchronize()
        parts[name] = begin.elapsed_time(end) / args.steps

    # ---- end to end through the public call with HOST buffers: H2D of W, L, U and D2H of Z inside the timed region ----
    host_w, host_l, host_u = (t.cpu().pin_memory() for t in (w, g, h))
    host_z = [torch.empty_like(host_w).pin_memory() for _ in range(2)]
    e2e_count = [0]

    def e2e_step():
        # host buffers in, host buffer out, every step: G and H then the factors on the front stream, W on a copy stream,
        # Z back on an output stream behind the sweep; two layers in flight
        e2e_count[0] += 1
        return pipeline.quantize_from_host(host_w, host_l, host_u, host_z[e2e_count[0] % 2])

    e2e_step()
    barrier()
    begin.record()
    for _ in range(args.steps):
        arrived = e2e_step()
    torch.cuda.current_stream(device).wait_event(arrived)  # the last result has reached the host buffer
    end.record()
    barrier()
    e2e_ms = begin.elapsed_time(end)
    if world > 1:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item()
    e2e_ms /= args.steps
    h2d = (host_w.numel() + host_l.numel() + host_u.numel()) * 4
    d2h = host_z[0].numel() * 4

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- per-kernel timing of the same step (separate profiled pass, CUDA events around every launch) ----
    y = w.clone()
    scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
    desc = _abi.SweepDesc()
    desc.dtype, desc.quant_kind, desc.batch, desc.m, desc.n = _abi.F32, _abi.Q_AFFINE, 1, m, n
    desc.y, desc.l, desc.u = y.data_ptr(), l.data_ptr(), u.data_ptr()
    desc.scale, desc.zero = scale.data_ptr(), zero.data_ptr()
    desc.scale_row_stride, desc.scale_col_stride, desc.zero_row_stride, desc.zero_col_stride = scale.stride(0), 0, 0, 0
    desc.qmin, desc.qmax = -8.0, 7.0
    size = ctypes.c_size_t()
    _abi.check(lib.g2d_sweep_workspace_bytes(ctypes.byref(desc), ctypes.byref(size)), "workspace")
    workspace = torch.empty(size.value, dtype=torch.uint8, device=device)
    desc.workspace, desc.workspace_bytes = workspace.data_ptr(), size.value
    prof = (ctypes.c_double * 9)()
    _abi.check(lib.g2d_sweep_fused_profile(ctypes.byref(desc), torch.cuda.current_stream().cuda_stream, prof), "profile")
    assert torch.equal(y, z), "the profiled pass must reproduce the timed result"
    tile_ms, near_ms, far_ms, tile_n, near_n, far_n, total_flops, near_flops, far_flops = list(prof)
    pk = peaks()
    tensor_peak = pk["bf16_tflops_sustained"] / 6.0  # fp32-faithful tensor roofline: TF32 = bf16 / 2, three TF32 products per fp32 product
    far_tflops = far_flops / (far_ms * 1e-3) / 1e12 if far_ms > 0 else 0.0
    roofline = {
        "bound": "tensor", "kernel": "macro_update_tc_kernel (tcgen05 kind::tf32, 3xTF32 split; far updates, running beside the tile launches)",
        "achieved": far_tflops, "peak": tensor_peak, "unit": "TFLOP/s", "frac": far_tflops / tensor_peak if tensor_peak else None,
        # dram bytes read + written of one far-update launch, from the ncu capture of a 4096 x 4096 run (149.7 MB for
        # 946 target macro tiles, profiles/macro_update_tc_kernel_far_4096.md), scaled by the target tiles of an average launch here
        "traffic": 149.7e6 / 946 * (far_flops / far_n / (2 * 2 * 128 * 128 * 512)) if far_n else None,
        "peak_basis": f"{pk['source']} bf16 sustained {pk['bf16_tflops_sustained']} TFLOP/s / 2 (TF32) / 3 (three tf32 products per fp32 product)",
        "launches": int(far_n), "avg_launch_ms": far_ms / far_n if far_n else None,
        "algorithmic_flops_per_launch": far_flops / far_n if far_n else None,
        "kernel_ms": {"tile_sweep": tile_ms, "near_update": near_ms, "far_update": far_ms},
        "kernel_launches": {"tile_sweep": int(tile_n), "near_update": int(near_n), "far_update": int(far_n)},
        "whole_sweep_tflops": sweep_flops(m, n) / (parts["sweep"] * 1e-3) / 1e12,
        "prep_tflops": 2 * (2 * float(n) ** 3 / 3) / (parts["prep"] * 1e-3) / 1e12,
        "timed_in": "separate profiled pass of the same step inside bench.py, one CUDA event pair per launch on the launching stream",
        # the critical path: one tile launch per tile anti-diagonal, each a chain of 7 x 31 dependent rounding stages;
        # bound by that latency, not by memory or arithmetic throughput
        "critical_path": {"kernel": "tile_sweep_kernel", "launches": int(tile_n), "avg_launch_us": 1e3 * tile_ms / tile_n if tile_n else None,
                          "bound": "latency"},
    }

    line = {
        "metric": METRIC, "value": ms_per_step / 1e3 / world, "unit": "s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {
            "workload": f"{m}x{n} fp32 layer from W, G, H: ldl_of_inverse x2, INT4 symmetric per-row fp16 abs-max scales, two-sided sweep (one layer per GPU per step)",
            "step": "kron_factors.feedback_factors_from_grams(G, H) (both factors in shared launches), int_abs_max_scale, gptq_2d (fused engine, pipelined schedule) through layer_set.LayerPipeline: the factor preparation of a step runs beside the sweep of the step before",
            "l2": "inputs larger than L2: W, G, H are 3 x %.0f MB" % (m * n * 4 / 1e6),
            "layers_in_flight": 2, "single_layer_ms": parts["single_layer"],
            "sweep_ms": parts["sweep"], "prep_ms": parts["prep"],
            "stages": m + n - 1, "sweep_us_per_stage": parts["sweep"] * 1e3 / (m + n - 1),
        },
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_ms / 1e3 / world, "unit": "s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches),
        "roofline": roofline,
    }
    if world == 1 and not args.no_cpu_baseline:
        per_layer, _, cores, note = cpu_layer_estimate(args)
        line["cpu_baseline"] = {"value": per_layer, "unit": "s", "cores": cores, "kind": "port", "sample": note}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
