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
After the timed steps every rank takes its share of a fixed subset of the 70B-shaped layer set (``--layer-set-blocks``
blocks of 7 matrices at full size, dealt out longest first, no collective on the data path): the second half of the
metric, reported under ``layer_set`` with the wall time over ranks.
Rank 0 prints one JSON line.  ``--impl reference`` times the reference's PyTorch path on the host cores instead, on a
bounded sample scaled by the algorithmic work: the reference's own ``gptq_2d_torch`` and ``ldl_of_inverse`` when a copy
of the reference is importable from ``baseline/_ref``, else the CPU restatement under ``oracle/`` (OpenMP sweep, LAPACK
factorisation); the line says which.
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

def metric(size: int) -> str:
    return f"s per {size}x{size} INT4 GPTQ-2D layer"


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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs.  The sampler is started before
    the warm-up steps (nvidia-smi needs a few hundred milliseconds to print its first line, about as long as ten
    steps take) and every line is stamped on arrival; the summary keeps the lines that arrived inside the timed region."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.stamps, self.proc = index, [], [], None

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
            self.stamps.append(time.monotonic())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, window=None) -> dict:
        """`window`: (start, end) on the time.monotonic clock; without a line inside it, the first line after it counts
        (the GPU goes on working on the per-part timings then)."""
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        lines = list(zip(self.stamps, self.lines))
        if window is not None:
            inside = [line for stamp, line in lines if window[0] <= stamp <= window[1] + 0.05]
            if not inside:
                inside = [line for stamp, line in lines if stamp > window[1]][:1]
            chosen = inside
        else:
            chosen = [line for _, line in lines]
        for line in chosen:
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


def host_threads() -> int:
    """Use every host core for the CPU arm, whatever a launcher put into OMP_NUM_THREADS (torchrun sets it to 1)."""
    cores = os.cpu_count() or 1
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        pass
    try:
        import torch

        torch.set_num_threads(cores)
    except Exception:
        pass
    return cores


def reference_modules():
    """The reference's own modules when a copy is importable from baseline/_ref (not part of this repository), else None."""
    path = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(path, "gptq_2d.py")):
        return None
    import importlib.util

    loaded = {}
    try:
        for name in ("quantizer_int", "gptq_2d", "gptq_2d_reference"):
            spec = importlib.util.spec_from_file_location(f"_reference_{name}", os.path.join(path, f"{name}.py"))
            module = importlib.util.module_from_spec(spec)
            saved = sys.modules.get(name)
            if name == "gptq_2d":
                sys.modules["quantizer_int"] = loaded["quantizer_int"]  # the reference imports its sibling by this name
            spec.loader.exec_module(module)
            loaded[name] = module
            if name == "gptq_2d":
                sys.modules.pop("quantizer_int", None)
            if saved is not None:
                sys.modules[name] = saved
    except Exception:
        return None
    return loaded


def cpu_inputs(size: int):
    import numpy as np
    from oracle import oracle

    rng = np.random.default_rng(0)
    w = (0.02 * rng.standard_normal((size, size))).astype(np.float32)
    l = np.tril(rng.standard_normal((size, size)) * (0.3 / np.sqrt(size)), -1).astype(np.float32)
    u = np.triu(rng.standard_normal((size, size)) * (0.3 / np.sqrt(size)), 1).astype(np.float32)
    scale = np.ascontiguousarray(np.broadcast_to(oracle.absmax_scale(w, -8, 7, oracle.FP16), (size, size)))
    return w, l, u, scale


def cpu_sweep_sample(size: int, reference) -> float:
    """Seconds of one size x size INT4 sweep on the host: the reference's gptq_2d_torch, or the oracle's restatement of it."""
    import numpy as np
    from oracle import oracle

    w, l, u, scale = cpu_inputs(size)
    zero = np.zeros((size, size), dtype=np.float32)
    if reference is not None:
        import torch

        quantizer = functools.partial(reference["quantizer_int"].affine_quantizer_torch, qmin=-8, qmax=7)
        tensors = [torch.from_numpy(a) for a in (w, l, u, scale, zero)]
        start = time.perf_counter()
        reference["gptq_2d"].gptq_2d_torch(tensors[0], tensors[1], tensors[2], quantizer=quantizer, quantizer_inputs=(tensors[3], tensors[4]))
        return time.perf_counter() - start
    oracle.lib()
    start = time.perf_counter()
    oracle.sweep(w, l, u, kind=oracle.Q_AFFINE, scale=scale, zero_point=zero, qmin=-8, qmax=7)
    return time.perf_counter() - start


def cpu_prep_sample(size: int, reference) -> float:
    """Seconds of one ldl_of_inverse at n = size on the host (float32): the reference's, or the oracle's LAPACK restatement."""
    import numpy as np
    from oracle import oracle

    gram = oracle.dyadic_gram(size, seed=1)
    if reference is not None:
        import torch

        tensor = torch.from_numpy(gram)
        start = time.perf_counter()
        reference["gptq_2d_reference"].ldl_of_inverse(tensor)
        return time.perf_counter() - start
    start = time.perf_counter()
    oracle.ldl_of_inverse_lapack(gram)
    return time.perf_counter() - start


def cpu_layer_estimate(args, sample: int, reference, threads: int) -> dict:
    """Seconds per full-size layer on the host: a sweep sample and a factor-preparation sample, each scaled by its work."""
    sweep_s = cpu_sweep_sample(sample, reference)
    sweep_factor = sweep_flops(args.size, args.size) / sweep_flops(sample, sample)
    prep_size = min(args.size, 4096)
    prep_s = cpu_prep_sample(prep_size, reference)
    prep_factor = 2 * (args.size / prep_size) ** 3
    what = ("the reference's gptq_2d_torch + ldl_of_inverse (PyTorch CPU, float32)" if reference is not None
            else "oracle port of the reference's PyTorch path (OpenMP sweep, LAPACK factorisation, float32)")
    note = (f"{what}, {threads} threads: {sample}x{sample} INT4 sweep {sweep_s:.2f} s scaled x{sweep_factor:.1f} by m n (m + n - 2) = {sweep_s * sweep_factor:.1f} s, "
            f"plus ldl_of_inverse at n={prep_size} {prep_s:.2f} s scaled x{prep_factor:.0f} (two factors, n^3) = {prep_s * prep_factor:.1f} s")
    return {"per_layer": sweep_s * sweep_factor + prep_s * prep_factor, "sample_seconds": sweep_s + prep_s, "note": note,
            "kind": "reference" if reference is not None else "port", "sweep_s": sweep_s * sweep_factor, "prep_s": prep_s * prep_factor}


def run_reference(args) -> None:
    """The reference arm: the reference's CPU path (or its oracle port), all host threads, a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    reference = reference_modules()
    # the sample is sized so that warm-up + steps end within a few minutes: the port takes about 10 s at 4096 and 1.2 s
    # at 2048 on 16 cores, the reference's PyTorch path about twice that
    budget = 200.0 / max(1, args.steps)
    sample = args.cpu_sample or (4096 if budget >= (24 if reference is not None else 12) else 2048)
    sample = min(sample, args.size)
    times, raw, last = [], [], None
    for step in range(args.warmup + args.steps):
        if step < args.warmup:
            cpu_sweep_sample(min(512, args.size), reference)  # untimed: library loads, thread pools
            cpu_prep_sample(min(256, args.size), reference)
            continue
        last = cpu_layer_estimate(args, sample, reference, threads)
        times.append(last["per_layer"])
        raw.append(last["sample_seconds"])
    per_layer = statistics.mean(times)
    line = {
        "impl": "reference", "metric": metric(args.size), "value": per_layer, "unit": "s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(raw), "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.size}x{args.size} fp32 layer from W, G, H: ldl_of_inverse x2, INT4 symmetric per-row fp16 abs-max scales, two-sided sweep",
                   "sample": last["note"], "sweep_s": last["sweep_s"], "prep_s": last["prep_s"]},
        "cpu_baseline": {"value": per_layer, "unit": "s", "cores": threads, "kind": last["kind"], "sample": last["note"]},
        "e2e": {"value": per_layer, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def measure_tf32_peak(device) -> dict:
    """Dense TF32 matrix-product throughput of this GPU through torch.matmul (cuBLAS), measured the way the bf16 figure of
    MEASURED_PEAKS.json was: 8192^3, best of 10 (burst) and back to back for about a second (sustained)."""
    import torch

    n = 8192
    a, b = torch.randn(n, n, device=device), torch.randn(n, n, device=device)
    before = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            a @ b
        best = float("inf")
        for _ in range(10):
            begin.record()
            a @ b
            end.record()
            torch.cuda.synchronize()
            best = min(best, begin.elapsed_time(end))
        count = max(10, int(1000.0 / best))
        begin.record()
        for _ in range(count):
            a @ b
        end.record()
        torch.cuda.synchronize()
        sustained = begin.elapsed_time(end) / count
    finally:
        torch.backends.cuda.matmul.allow_tf32 = before
    flops = 2.0 * n ** 3
    return {"burst_tflops": flops / best / 1e9, "sustained_tflops": flops / sustained / 1e9, "how": f"torch.matmul fp32 with TF32 allowed, {n}^3, best of 10 and {count} back to back"}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None, help="timed steps; default 20 (about 0.65 s, several clock samples) and 5 for --impl reference (whose step is seconds of CPU work)")
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--size", type=int, default=8192)
    parser.add_argument("--cpu-sample", type=int, default=0, help="side of the CPU arm's sweep sample; 0 chooses by the time budget")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-peak-probe", action="store_true", help="skip the TF32 matrix-product measurement (for runs under a profiler)")
    parser.add_argument("--layer-set-blocks", type=int, default=8, help="blocks of the 70B-shaped layer set run after the timed steps (0: none)")
    args = parser.parse_args()
    if args.steps is None:
        args.steps = 5 if args.impl == "reference" else 20
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

    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        for _ in range(args.warmup):
            z = step(w)
        barrier()
        launches_before = lib.g2d_launch_count()
        window_start = time.monotonic()
        begin.record()
        for _ in range(args.steps):
            z = step(w)
        end.record()
        barrier()
        window = (window_start, time.monotonic())
        launches = lib.g2d_launch_count() - launches_before
        for _ in range(3):  # keeps the GPU at work until the sampler has printed a line for certain
            if any(window[0] <= stamp for stamp in clocks.stamps):
                break
            z_extra = step(w)
            torch.cuda.synchronize()
            del z_extra
    elapsed_ms = begin.elapsed_time(end)
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

    # ---- end to end through the public call with HOST buffers, every step, inside the timed region.  Two transfer
    # formats: the compact one (the headline `e2e`: W and the packed lower triangles of the symmetric G and H in, packed
    # INT4 codes and fp16 row scales out) and plain float matrices both ways (`e2e_float_io`) ----
    import packed_codes as P

    host_w, host_g, host_h = (t.cpu().pin_memory() for t in (w, g, h))
    host_gp, host_hp = (P.pack_symmetric(t).pin_memory() for t in (host_g, host_h))
    host_z = [torch.empty_like(host_w).pin_memory() for _ in range(2)]
    host_codes = [torch.empty(m, (n * 4 + 7) // 8, dtype=torch.uint8).pin_memory() for _ in range(2)]
    host_scales = [torch.empty(m, dtype=torch.float16).pin_memory() for _ in range(2)]
    e2e_count = [0]

    def e2e_step_packed():
        # G and H triangles, their unpacking and the factors on the front stream, W on a copy stream, codes and scales
        # back on an output stream behind the sweep; two layers in flight
        e2e_count[0] += 1
        k = e2e_count[0] % 2
        return pipeline.quantize_from_host_packed(host_w, host_gp, host_hp, host_codes[k], host_scales[k])

    def e2e_step_float():
        e2e_count[0] += 1
        return pipeline.quantize_from_host(host_w, host_g, host_h, host_z[e2e_count[0] % 2])

    def time_e2e(one_step):
        one_step()
        barrier()
        begin.record()
        for _ in range(args.steps):
            arrived = one_step()
        torch.cuda.current_stream(device).wait_event(arrived)  # the last result has reached the host buffer
        end.record()
        barrier()
        ms = begin.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms / args.steps

    e2e_ms = time_e2e(e2e_step_packed)
    last = e2e_count[0] % 2  # the buffers the last packed step wrote (the device is idle: time_e2e ends with a synchronisation)
    decoded = P.unpack_codes(host_codes[last].to(device), host_scales[last].to(device).float()[:, None], torch.zeros((), device=device),
                             qmin=-8, bits=4, n=n)
    assert torch.equal(decoded, z), "the codes that reached the host must decode to the device-timed result"
    e2e_float_ms = time_e2e(e2e_step_float)
    h2d = host_w.numel() * 4 + (host_gp.numel() + host_hp.numel()) * 4
    d2h = host_codes[0].numel() + host_scales[0].numel() * 2
    h2d_float, d2h_float = (host_w.numel() + host_g.numel() + host_h.numel()) * 4, host_z[0].numel() * 4
    # what the asynchronous calls of the timed regions could not report: a factor that is not positive definite, or a
    # bounded wait inside a tensor-core kernel that ran out (raises)
    pipeline.check()
    del host_w, host_g, host_h, host_gp, host_hp, host_z

    # ---- the layer-set half of the metric: a fixed subset of the 70B-shaped set, partitioned by matrix over the ranks ----
    set_summary = None
    if args.layer_set_blocks > 0:
        def gather(obj):
            if world == 1:
                return [obj]
            out = [None] * world if rank == 0 else None
            dist.gather_object(obj, out, dst=0)
            return out

        layer_set.quantize_matrix({"block": -1, "name": "warm-up", "m": 384, "n": 512, "seed": 1}, device)
        set_pipeline = layer_set.LayerPipeline(device)
        set_summary = layer_set.run(layer_set.layer_list(args.layer_set_blocks), functools.partial(layer_set.quantize_matrix, device=device, pipeline=set_pipeline),
                                    rank=rank, world=world, gather=gather, barrier=barrier)
        set_pipeline.check()
        torch.cuda.empty_cache()

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
    # the same far-update kernel with the GPU to itself: one pass of the macro schedule (everything on one stream, so no
    # other kernel runs beside it); tells the kernel's own rate from what its low priority costs it in the pipelined schedule
    y_alone = w.clone()
    desc.y, desc.reserved = y_alone.data_ptr(), 2
    prof_alone = (ctypes.c_double * 9)()
    _abi.check(lib.g2d_sweep_fused_profile(ctypes.byref(desc), torch.cuda.current_stream().cuda_stream, prof_alone), "profile of the macro schedule")
    desc.y, desc.reserved = y.data_ptr(), 0
    alone_ms, alone_n, alone_flops = prof_alone[2], prof_alone[5], prof_alone[8]
    alone_tflops = alone_flops / (alone_ms * 1e-3) / 1e12 if alone_ms > 0 else 0.0
    del y_alone
    pk = peaks()
    tensor_peak = pk["bf16_tflops_sustained"] / 6.0  # fp32-faithful tensor roofline: TF32 = bf16 / 2, three TF32 products per fp32 product
    far_tflops = far_flops / (far_ms * 1e-3) / 1e12 if far_ms > 0 else 0.0
    near_tflops = near_flops / (near_ms * 1e-3) / 1e12 if near_ms > 0 else 0.0
    panel_tflops = (near_flops + far_flops) / ((near_ms + far_ms) * 1e-3) / 1e12 if near_ms + far_ms > 0 else 0.0
    tf32 = {"burst_tflops": None, "sustained_tflops": None, "how": "skipped"} if args.no_peak_probe else measure_tf32_peak(device)
    measured_peak = tf32["sustained_tflops"] / 3.0 if tf32["sustained_tflops"] else None
    rtn = torch.clamp(torch.round(w / scale), -8, 7) * scale
    objective_vs_rtn = synthetic.objective(z, w, g, h) / synthetic.objective(rtn, w, g, h)
    roofline = {
        "bound": "tensor", "kernel": "macro_update_tc_kernel (tcgen05 kind::tf32, 3xTF32 split; far updates: the lowest-priority stream of three, on the SMs that the tile launch of the moment leaves free)",
        "achieved": far_tflops, "peak": tensor_peak, "unit": "TFLOP/s", "frac": far_tflops / tensor_peak if tensor_peak else None,
        # DRAM bytes of one launch are not measured live: an ncu capture of this kernel at 4096 x 4096 read and wrote
        # 149.7 MB for 946 target macro tiles; that figure scaled by the target tiles of an average launch here
        "traffic": 149.7e6 / 946 * (far_flops / far_n / (2 * 2 * 128 * 128 * 512)) if far_n else None,
        "traffic_basis": "ncu capture at 4096 x 4096 (dram__bytes_read.sum + dram__bytes_write.sum of one launch), scaled by target macro tiles; not measured in this run",
        "peak_basis": f"{pk['source']} bf16 sustained {pk['bf16_tflops_sustained']} TFLOP/s / 2 (TF32) / 3 (three tf32 products per fp32 product)",
        "peak_measured_tf32": {**tf32, "fp32_faithful_peak": measured_peak, "frac_of_it": far_tflops / measured_peak if measured_peak else None},
        "near": {"kernel": "band_tc_kernel (tcgen05 kind::tf32, M 128 x N 64, rank-64 updates on a side stream)", "achieved": near_tflops,
                 "frac": near_tflops / tensor_peak if tensor_peak else None, "launches": int(near_n), "algorithmic_flops": near_flops},
        "panel_gemms": {"what": "near + far updates: their algorithmic flops over their summed stream time", "achieved": panel_tflops,
                        "frac": panel_tflops / tensor_peak if tensor_peak else None, "algorithmic_flops": near_flops + far_flops,
                        "share_of_sweep_flops": (near_flops + far_flops) / total_flops if total_flops else None},
        "far_kernel_alone": {"what": "the same kernel in the macro schedule of the same matrix: one stream, nothing beside it", "achieved": alone_tflops,
                             "frac": alone_tflops / tensor_peak if tensor_peak else None, "launches": int(alone_n),
                             "avg_launch_ms": alone_ms / alone_n if alone_n else None, "algorithmic_flops": alone_flops},
        "launches": int(far_n), "avg_launch_ms": far_ms / far_n if far_n else None,
        "algorithmic_flops_per_launch": far_flops / far_n if far_n else None,
        "kernel_ms": {"tile_sweep": tile_ms, "near_update": near_ms, "far_update": far_ms},
        "kernel_launches": {"tile_sweep": int(tile_n), "near_update": int(near_n), "far_update": int(far_n)},
        "whole_sweep_tflops": sweep_flops(m, n) / (parts["sweep"] * 1e-3) / 1e12,
        "prep_tflops": 2 * (2 * float(n) ** 3 / 3) / (parts["prep"] * 1e-3) / 1e12,
        "timed_in": "separate profiled pass of the same step inside bench.py, one CUDA event pair per launch on the launching stream",
        # the critical path: one tile launch per tile anti-diagonal, each a chain of 7 x 32 dependent rounding stages;
        # bound by that latency, not by memory or arithmetic throughput
        "critical_path": {"kernel": "tile_sweep_kernel", "launches": int(tile_n), "avg_launch_us": 1e3 * tile_ms / tile_n if tile_n else None,
                          "bound": "latency"},
    }

    line = {
        "metric": metric(args.size), "value": ms_per_step / 1e3 / world, "unit": "s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {
            "workload": f"{m}x{n} fp32 layer from W, G, H: ldl_of_inverse x2, INT4 symmetric per-row fp16 abs-max scales, two-sided sweep (one layer per GPU per step)",
            "step": "kron_factors.feedback_factors_from_grams(G, H) (both factors in shared launches), int_abs_max_scale, gptq_2d (fused engine, pipelined schedule) through layer_set.LayerPipeline: the factor preparation of a step runs beside the sweep of the step before",
            "l2": "inputs larger than L2: W, G, H are 3 x %.0f MB" % (m * n * 4 / 1e6),
            "layers_in_flight": 2, "single_layer_ms": parts["single_layer"],
            "sweep_ms": parts["sweep"], "prep_ms": parts["prep"],
            "stages": m + n - 1, "sweep_us_per_stage": parts["sweep"] * 1e3 / (m + n - 1),
            "objective_vs_round_to_nearest": objective_vs_rtn, "status": "factor pivots and kernel wait flags read after the timed regions: clean",
        },
        "clocks": clocks.summary(window),
        "e2e": {"value": e2e_ms / 1e3 / world, "unit": "s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "format": "LayerPipeline.quantize_from_host_packed: W float32, G and H as packed lower triangles in; INT4 codes and fp16 row scales out"},
        "e2e_float_io": {"value": e2e_float_ms / 1e3 / world, "unit": "s", "h2d_bytes_per_step": h2d_float, "d2h_bytes_per_step": d2h_float,
                         "format": "LayerPipeline.quantize_from_host: W, G, H as float32 matrices in, Z as a float32 matrix out"},
        "gpu_launches": int(launches),
        "roofline": roofline,
    }
    if set_summary is not None:
        blocks = args.layer_set_blocks
        line["layer_set"] = {
            "what": f"{blocks} blocks of the 70B-shaped set at full size ({set_summary['matrices']} matrices: q, o 8192^2; k, v 1024x8192; gate, up 28672x8192; down 8192x28672), "
                    "seeded inputs generated on the owning GPU inside the timed region, INT4, two layers in flight per GPU, longest-first partition, no data-path collective",
            "blocks": blocks, "matrices": set_summary["matrices"], "n_gpus": world, "wall_s": set_summary["wall_s"], "busy_s": set_summary["busy_s"],
            "scaling": "strong", "mean_ms_by_shape": set_summary["mean_ms_by_shape"],
            "extrapolated_80_blocks_s": set_summary["wall_s"] * 80.0 / blocks, "extrapolation": f"wall time x 80 / {blocks}: not measured",
            "all_finite": set_summary["all_finite"], "all_codes_in_range": set_summary["all_codes_in_range"],
            "objective_vs_round_to_nearest": set_summary["objective_vs_rtn"],
        }
    if world == 1 and not args.no_cpu_baseline:
        threads = host_threads()
        estimate = cpu_layer_estimate(args, min(args.size, args.cpu_sample or 4096), reference_modules(), threads)
        line["cpu_baseline"] = {"value": estimate["per_layer"], "unit": "s", "cores": threads, "kind": estimate["kind"], "sample": estimate["note"],
                                "sweep_s": estimate["sweep_s"], "prep_s": estimate["prep_s"]}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
