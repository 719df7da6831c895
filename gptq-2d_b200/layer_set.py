"""Quantize a whole set of layers, sharded by matrix across the GPUs of one node.

Every weight matrix with its own two Hessian factors is an independent problem, so a layer set is partitioned by
matrix: no kernel reads another GPU's memory and the only exchange is the gathering of per-matrix statistics at the
end.  One process per GPU (``torchrun`` sets RANK / WORLD_SIZE / LOCAL_RANK); matrices are dealt out longest first to
the least loaded rank, using the algorithmic work (sweep + factor preparation) as the cost.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 gptq-2d_b200/layer_set.py --blocks 80

The default set has the shapes of a 70B-parameter decoder (80 blocks x {q, o 8192 x 8192; k, v 1024 x 8192;
gate, up 28672 x 8192; down 8192 x 28672}) with seeded synthetic weights and Hessian factors (``synthetic.py``),
INT4 symmetric per-row scales.
"""
from __future__ import annotations

import argparse
import functools
import json
import os
import sys
import time
from collections.abc import Callable

MATRICES_70B = (
    ("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192),
    ("gate", 28672, 8192), ("up", 28672, 8192), ("down", 8192, 28672),
)


# Matrices of a decoder block that read the same activations and therefore share their input-side Hessian factor.
INPUT_GROUPS_70B = {"q": "attention input", "k": "attention input", "v": "attention input", "gate": "mlp input", "up": "mlp input"}


def layer_list(blocks: int = 80, divide: int = 1, matrices=MATRICES_70B, shared_inputs: bool = False) -> list[dict]:
    """The matrices of the set; ``divide`` shrinks every dimension (for tests and short runs).

    With ``shared_inputs`` the matrices of ``INPUT_GROUPS_70B`` carry a ``group`` key and a common ``input_seed``: one
    input-side factor (and one ``U``) serves the whole group, which then stays together on one rank."""
    items = []
    for block in range(blocks):
        for index, (name, m, n) in enumerate(matrices):
            item = {"block": block, "name": name, "m": m // divide, "n": n // divide, "seed": 7919 * block + 101 * index + 1}
            if shared_inputs and name in INPUT_GROUPS_70B:
                item["group"] = f"{block}:{INPUT_GROUPS_70B[name]}"
                item["input_seed"] = 15485863 + 7919 * block + (1 if name in ("gate", "up") else 0)
            items.append(item)
    return items


def work(m: int, n: int, input_factor_ready: bool = False) -> float:
    """Algorithmic flops of one matrix: sweep ``m n (m + n - 2)`` plus its factor preparations ``2 k^3 / 3`` each (the
    input-side one only where it is not shared with a matrix counted before)."""
    prep = float(m) ** 3 + (0.0 if input_factor_ready else float(n) ** 3)
    return float(m) * n * (m + n - 2) + 2.0 * prep / 3.0


def _units(items: list[dict]) -> list[list[dict]]:
    """The indivisible pieces of a set: single matrices, and the groups that share an input-side factor."""
    units: dict = {}
    for k, item in enumerate(items):
        units.setdefault(item.get("group", ("single", k)), []).append(item)
    return list(units.values())


def _unit_work(unit: list[dict]) -> float:
    return sum(work(item["m"], item["n"], input_factor_ready=k > 0) for k, item in enumerate(unit))


def partition(items: list[dict], world: int) -> list[list[dict]]:
    """Longest-processing-time-first assignment of the matrices to ``world`` ranks (deterministic).  Matrices that share
    an input-side factor are dealt out as one piece and stay next to each other in their rank's order."""
    shares: list[list[dict]] = [[] for _ in range(world)]
    load = [0.0] * world
    units = _units(items)
    order = sorted(range(len(units)), key=lambda k: (-_unit_work(units[k]), k))
    for k in order:
        rank = min(range(world), key=lambda r: (load[r], r))
        shares[rank].extend(units[k])
        load[rank] += _unit_work(units[k])
    return shares


class LayerPipeline:
    """Two layers of one GPU in flight: the factor preparation of a layer runs on a stream of its own ("front"), so it
    overlaps the sweep of the layer before it.  Both are chains of short dependent launches that leave most SMs idle,
    and the layers of a set are independent, so a set finishes in about the time of its sweeps alone.

    ``quantize`` takes inputs that are resident on the device; ``quantize_from_host`` takes pinned host tensors, moves
    them in on the front stream (the weights on a third one) and moves the result out behind the sweep.  Results come
    back in stream order of the caller's current stream.  INT4 symmetric per-row scales, as the layer-set benchmark."""

    def __init__(self, device, qmin: int = -8, qmax: int = 7):
        import torch

        self.device, self.qmin, self.qmax = device, qmin, qmax
        self.front = torch.cuda.Stream(device=device)
        self.copy = torch.cuda.Stream(device=device)
        self.out = torch.cuda.Stream(device=device)
        self.swept = [None, None]  # events: the sweeps of the last two layers have finished (the older bounds the run-ahead)
        self.slots = {}        # device buffers of quantize_from_host, two per shape
        self.count = 0
        self.shared = None     # (group, H, U, event) of the input-side factor that the current group of matrices shares

    def _sweep(self, w, l, u):
        import torch

        import gptq_2d as G
        import quantizer_int as Q

        m, n = w.shape
        scale = Q.int_abs_max_scale_triton(w, qmin=self.qmin, qmax=self.qmax, dtype=torch.float16).expand(m, n)
        zero = torch.zeros(1, 1, device=w.device, dtype=w.dtype).expand(m, n)
        quantizer = functools.partial(Q.affine_quantizer_triton, qmin=self.qmin, qmax=self.qmax)
        return G.gptq_2d(w, l, u, quantizer=quantizer, quantizer_inputs=(scale, zero))

    def _prepare(self, g, h, main):
        """Factors of (g, h) on the front stream; the caller's stream waits for them.  At most one layer ahead."""
        import torch

        import kron_factors as K

        with torch.cuda.stream(self.front):
            l, u = K.feedback_factors_from_grams(g, h)
            ready = torch.cuda.Event()
            ready.record(self.front)
        main.wait_event(ready)
        l.record_stream(main)
        u.record_stream(main)
        return l, u

    def _prepare_shared(self, g, group, input_factor, main):
        """The same for a matrix whose input-side factor is shared with its group: ``U`` is prepared once, by the
        group's first matrix (``input_factor()`` makes H, on the front stream), and kept for the others; only ``L``
        is prepared per matrix."""
        import torch

        import kron_factors as K

        with torch.cuda.stream(self.front):
            if self.shared is None or self.shared[0] != group:
                h = input_factor()
                l, u = K.feedback_factors_from_grams(g, h)
                self.shared = (group, h, u)
            else:
                _, h, u = self.shared
                l = K.ldl_of_inverse(g, check=False)
            ready = torch.cuda.Event()
            ready.record(self.front)
        main.wait_event(ready)
        for t in (l, u, h):
            t.record_stream(main)
        return l, u, h

    def _after_sweep(self, main):
        import torch

        event = torch.cuda.Event()
        event.record(main)
        self.swept = [self.swept[1], event]
        return event

    def check(self) -> None:
        """Wait for the device and raise if anything since the last check went wrong where the asynchronous calls could
        not tell: a Hessian factor that is not positive definite (``torch.linalg.LinAlgError``, as the reference's
        Cholesky raises) or a bounded wait that ran out inside a tensor-core kernel (``RuntimeError``)."""
        import _abi
        import kron_factors as K

        K.check_pending()
        _abi.check_status(self.device, "LayerPipeline")

    def _throttle(self):
        # the preparation of this layer may run beside the sweep of the layer before it, not further ahead
        if self.swept[0] is not None:
            self.front.wait_event(self.swept[0])

    def quantize(self, w, g, h, inputs_ready=None):
        """Quantize one layer whose inputs are on the device.  ``inputs_ready``: an event after which ``g`` and ``h`` may
        be read, or None when they were complete before the call (the front stream does not wait for the caller's)."""
        import torch

        main = torch.cuda.current_stream(self.device)
        self._throttle()
        if inputs_ready is not None:
            self.front.wait_event(inputs_ready)
        l, u = self._prepare(g, h, main)
        z = self._sweep(w, l, u)
        self._after_sweep(main)
        return z

    def quantize_from_host(self, host_w, host_g, host_h, host_z):
        """The same from pinned host tensors into a pinned host result; returns the event that marks ``host_z`` complete."""
        import torch

        main = torch.cuda.current_stream(self.device)
        key = (tuple(host_w.shape), host_w.dtype)
        if key not in self.slots:
            self.slots[key] = [{"w": torch.empty(host_w.shape, dtype=host_w.dtype, device=self.device),
                                "g": torch.empty(host_g.shape, dtype=host_g.dtype, device=self.device),
                                "h": torch.empty(host_h.shape, dtype=host_h.dtype, device=self.device),
                                "free": None} for _ in range(2)]
        slot = self.slots[key][self.count % 2]
        self.count += 1
        if slot["free"] is not None:  # the sweep that read this slot two layers ago has finished
            self.front.wait_event(slot["free"])
            self.copy.wait_event(slot["free"])
        self._throttle()
        with torch.cuda.stream(self.front):
            slot["g"].copy_(host_g, non_blocking=True)
            slot["h"].copy_(host_h, non_blocking=True)
        with torch.cuda.stream(self.copy):
            slot["w"].copy_(host_w, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(self.copy)
        l, u = self._prepare(slot["g"], slot["h"], main)
        main.wait_event(arrived)
        z = self._sweep(slot["w"], l, u)
        slot["free"] = self._after_sweep(main)
        self.out.wait_event(slot["free"])
        with torch.cuda.stream(self.out):  # behind the sweep, beside the next layer
            host_z.copy_(z, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.out)
        z.record_stream(self.out)
        return done

    def quantize_from_host_packed(self, host_w, host_g_packed, host_h_packed, host_codes, host_scales):
        """``quantize_from_host`` in the transfer format that moves the fewest bytes: the two symmetric Hessian factors
        come as packed lower triangles (``packed_codes.pack_symmetric``: half the bytes), and the result goes back as
        packed ``bits``-wide integer codes ``host_codes`` (uint8 ``[m, ceil(n bits / 8)]``) with the per-row scales
        ``host_scales`` (float16 ``[m]``) instead of dequantised floats.  Returns the event that marks both complete."""
        import torch

        import packed_codes as P
        import quantizer_int as Q

        main = torch.cuda.current_stream(self.device)
        m, n = host_w.shape
        bits = (self.qmax - self.qmin).bit_length()
        key = ("packed", m, n, host_w.dtype)
        if key not in self.slots:
            make = lambda *shape, dtype=host_w.dtype: torch.empty(*shape, dtype=dtype, device=self.device)
            self.slots[key] = [{"w": make(m, n), "gp": make(host_g_packed.numel()), "hp": make(host_h_packed.numel()), "g": make(m, m), "h": make(n, n),
                                "free": None} for _ in range(2)]
        slot = self.slots[key][self.count % 2]
        self.count += 1
        if slot["free"] is not None:  # the sweep that read this slot two layers ago has finished
            self.front.wait_event(slot["free"])
            self.copy.wait_event(slot["free"])
        self._throttle()
        with torch.cuda.stream(self.front):
            slot["gp"].copy_(host_g_packed, non_blocking=True)
            slot["hp"].copy_(host_h_packed, non_blocking=True)
            P.unpack_symmetric(slot["gp"], m, out=slot["g"])
            P.unpack_symmetric(slot["hp"], n, out=slot["h"])
        with torch.cuda.stream(self.copy):
            slot["w"].copy_(host_w, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(self.copy)
        l, u = self._prepare(slot["g"], slot["h"], main)
        main.wait_event(arrived)
        z = self._sweep(slot["w"], l, u)
        scale = Q.int_abs_max_scale_triton(slot["w"], qmin=self.qmin, qmax=self.qmax, dtype=torch.float16)
        codes = P.pack_codes(z, scale, torch.zeros((), device=self.device, dtype=z.dtype), qmin=self.qmin, bits=bits)
        scales16 = scale.reshape(m).to(torch.float16)
        slot["free"] = self._after_sweep(main)
        self.out.wait_event(slot["free"])
        with torch.cuda.stream(self.out):  # behind the sweep, beside the next layer
            host_codes.copy_(codes, non_blocking=True)
            host_scales.copy_(scales16, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.out)
        for t in (codes, scales16):
            t.record_stream(self.out)
        return done


def quantize_matrix(item: dict, device, pipeline: LayerPipeline | None = None):
    """Generate one seeded layer on ``device``, prepare its factors, quantize it to INT4; returns timings and checks.

    With a ``pipeline`` the layer is generated and its factors are prepared on the pipeline's front stream, beside the
    sweep of the layer before it; the statistics then stay on the device and the call returns a function that fetches
    them (calling it waits for this layer), so that the host can enqueue the next layer first."""
    import torch

    import _abi
    import gptq_2d as G
    import kron_factors as K
    import quantizer_int as Q
    import synthetic

    m, n = item["m"], item["n"]
    samples = min(8192, max(m, n))
    events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    if pipeline is not None and "group" in item:
        # the input-side factor H and its U come from the group's first matrix on this rank
        main = torch.cuda.current_stream(device)
        pipeline._throttle()
        with torch.cuda.stream(pipeline.front):
            w, g, _ = synthetic.make_layer(m, n, seed=item["seed"], device=device, samples=samples, without_input_factor=True)
            events[0].record(pipeline.front)
        make_h = lambda: synthetic.shared_input_factor(n, item["input_seed"], device, samples=samples)
        l, u, h = pipeline._prepare_shared(g, item["group"], make_h, main)
        for t in (w, g):
            t.record_stream(main)
        events[1].record(main)
        z = pipeline._sweep(w, l, u)
        pipeline._after_sweep(main)
        events[2].record(main)
        scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
    elif pipeline is None:
        w, g, h = synthetic.make_layer(m, n, seed=item["seed"], device=device, samples=samples, input_seed=item.get("input_seed"))
        events[0].record()
        l, u = K.feedback_factors_from_grams(g, h)
        events[1].record()
        scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
        zero = torch.zeros(1, 1, device=device, dtype=w.dtype).expand(m, n)
        z = G.gptq_2d(w, l, u, quantizer=functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7), quantizer_inputs=(scale, zero))
        events[2].record()
    else:
        main = torch.cuda.current_stream(device)
        pipeline._throttle()
        with torch.cuda.stream(pipeline.front):
            w, g, h = synthetic.make_layer(m, n, seed=item["seed"], device=device, samples=samples, input_seed=item.get("input_seed"))
            events[0].record(pipeline.front)
        l, u = pipeline._prepare(g, h, main)
        for t in (w, g, h):
            t.record_stream(main)
        events[1].record(main)
        z = pipeline._sweep(w, l, u)
        pipeline._after_sweep(main)
        events[2].record(main)
        scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
    codes = torch.round(z / scale)
    # Statistics stay on the device, packed into one float64 vector, and travel to pinned host memory on a stream of
    # their own behind this matrix only: the host can enqueue the next matrix before it reads them.  Folded in: what
    # the asynchronous calls could not report, the pivot flags of this matrix's factor preparation and the device's
    # status word (set when a bounded wait inside a tensor-core kernel ran out).
    factor_flags = K.last_flags()
    parts = [codes.min(), codes.max(), torch.isfinite(z).all(), codes.double().sum(),
             factor_flags.abs().max() if factor_flags is not None else torch.zeros((), device=device),
             _abi.status_word(device).abs().max()]
    if m * n <= 4096 * 4096:  # the objective needs two more products; keep it to the smaller matrices
        rtn = torch.clamp(torch.round(w / scale), -8, 7) * scale
        r, r0 = (z - w).double(), (rtn - w).double()
        parts += [((g.double() @ r) * (r @ h.double())).sum(), ((g.double() @ r0) * (r0 @ h.double())).sum()]
    on_device = torch.stack([p.double() for p in parts])
    ready = torch.cuda.Event()
    ready.record(torch.cuda.current_stream(device))
    on_host = torch.empty(on_device.shape, dtype=torch.float64).pin_memory()
    fetched = torch.cuda.Event()
    side = pipeline.out if pipeline is not None else torch.cuda.current_stream(device)
    side.wait_event(ready)
    with torch.cuda.stream(side):
        on_host.copy_(on_device, non_blocking=True)
        fetched.record(side)
    on_device.record_stream(side)

    def finish() -> dict:
        fetched.synchronize()  # this matrix only: the next one may already be running
        values = on_host.tolist()
        stats = {
            **item, "prep_ms": events[0].elapsed_time(events[1]) if pipeline is None else None,
            "sweep_ms": events[1].elapsed_time(events[2]),
            "codes_in_range": values[0] >= -8 and values[1] <= 7,
            "factors_ok": values[4] == 0, "waits_ok": values[5] == 0, "code_sum": values[3],
        }
        stats["finite"] = bool(values[2]) and stats["factors_ok"] and stats["waits_ok"]
        if len(values) > 6:
            stats["objective_vs_rtn"] = values[6] / values[7]
        return stats

    return finish() if pipeline is None else finish


def read_journal(path: str | None) -> dict:
    """Statistics of the matrices a previous run finished, keyed by (block, name); lines that do not parse (a run killed
    in the middle of a write) are dropped."""
    done: dict = {}
    if path and os.path.exists(path):
        with open(path) as f:
            for line in f:
                try:
                    stats = json.loads(line)
                    done[(stats["block"], stats["name"])] = stats
                except (ValueError, KeyError):
                    continue
    return done


def run(items: list[dict], process: Callable[[dict], dict], *, rank: int, world: int, gather: Callable | None = None,
        barrier: Callable | None = None, journal: str | None = None) -> dict | None:
    """Process this rank's share; rank 0 returns the summary of the whole set.  ``gather(obj)`` must return the list
    of every rank's object on rank 0 (None elsewhere); ``barrier()`` aligns the ranks before the clock starts.

    With a ``journal`` (a path; every rank appends to ``<journal>.<rank>``) each finished matrix is written down at
    once, and matrices that any rank's journal of an earlier run already holds are not processed again: a set that was
    interrupted resumes where it stopped, whatever the number of ranks of the new run."""
    share = partition(items, world)[rank]
    finished: dict = {}
    if journal:
        directory, prefix = os.path.split(journal)
        for name in sorted(os.listdir(directory or ".")):
            if name.startswith(prefix + "."):
                finished.update(read_journal(os.path.join(directory, name)))
    log = None
    if journal:
        mine = f"{journal}.{rank}"
        cut_off = False
        if os.path.exists(mine) and os.path.getsize(mine) > 0:
            with open(mine, "rb") as f:
                f.seek(-1, os.SEEK_END)
                cut_off = f.read(1) != b"\n"  # a run killed in the middle of a line
        log = open(mine, "a")
        if cut_off:
            log.write("\n")

    def settle(entry):  # statistics of a matrix: fetched (a pipelined process hands back a fetcher) and written down
        stats = entry() if callable(entry) else entry
        if log is not None:
            log.write(json.dumps(stats) + "\n")
            log.flush()
        return stats

    if barrier is not None:
        barrier()
    start = time.perf_counter()
    results, pending = [], None
    for item in share:
        key = (item["block"], item["name"])
        if key in finished:
            results.append({**finished[key], "resumed": True})
            continue
        entry = process(item)
        if pending is not None:  # one behind: the host has enqueued the next matrix before it waits for this one
            results.append(settle(pending))
        pending = entry
    if pending is not None:
        results.append(settle(pending))
    if log is not None:
        log.close()
    busy = time.perf_counter() - start
    if barrier is not None:
        barrier()
    wall = time.perf_counter() - start
    mine = {"rank": rank, "busy_s": busy, "wall_s": wall, "results": results}
    everyone = gather(mine) if gather is not None else [mine]
    if everyone is None:
        return None
    results = [r for part in everyone for r in part["results"]]
    done = {(r["block"], r["name"]) for r in results}
    assert len(results) == len(items) and done == {(i["block"], i["name"]) for i in items}, "every matrix exactly once"
    by_shape: dict[str, dict] = {}
    for r in results:
        entry = by_shape.setdefault(f"{r['m']}x{r['n']}", {"count": 0, "prep_ms": 0.0, "sweep_ms": 0.0})
        entry["count"] += 1
        entry["prep_ms"] += r.get("prep_ms") or 0.0
        entry["sweep_ms"] += r.get("sweep_ms") or 0.0
    for entry in by_shape.values():
        entry["prep_ms"] /= entry["count"]
        entry["sweep_ms"] /= entry["count"]
    return {
        "matrices": len(results), "n_gpus": world, "wall_s": max(p["wall_s"] for p in everyone),
        "busy_s": [p["busy_s"] for p in sorted(everyone, key=lambda p: p["rank"])],
        "mean_ms_by_shape": by_shape,
        "all_finite": all(r.get("finite", True) for r in results),
        "all_codes_in_range": all(r.get("codes_in_range", True) for r in results),
        "objective_vs_rtn": [r["objective_vs_rtn"] for r in results if "objective_vs_rtn" in r][:8],
        "weights": sum(r["m"] * r["n"] for r in results),
        "resumed": sum(1 for r in results if r.get("resumed")),
    }


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--blocks", type=int, default=80)
    parser.add_argument("--divide", type=int, default=1, help="shrink every dimension by this factor")
    parser.add_argument("--serial", action="store_true", help="one layer at a time (per-part timings) instead of two in flight")
    parser.add_argument("--shared-inputs", action="store_true",
                        help="q, k, v of a block share one input-side Hessian factor, and so do gate and up (prepared once per group)")
    parser.add_argument("--journal", default=None, help="path prefix of the per-rank journals: finished matrices are written down and skipped on a rerun")
    args = parser.parse_args()
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import torch
    import torch.distributed as dist

    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    gather = barrier = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

        def gather(obj):
            out = [None] * world if rank == 0 else None
            dist.gather_object(obj, out, dst=0)
            return out

        def barrier():
            dist.barrier()
            torch.cuda.synchronize()
    # one small matrix through every kernel first: the CUDA module loads on first use and would otherwise be charged
    # to the first (largest) matrix of every rank
    quantize_matrix({"block": -1, "name": "warm-up", "m": 384, "n": 512, "seed": 1}, device)
    pipeline = None if args.serial else LayerPipeline(device)
    summary = run(layer_list(args.blocks, args.divide, shared_inputs=args.shared_inputs), functools.partial(quantize_matrix, device=device, pipeline=pipeline), rank=rank,
                  world=world, gather=gather, barrier=barrier, journal=args.journal)
    if summary is not None:
        print(json.dumps(summary))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
