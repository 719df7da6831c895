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


def layer_list(blocks: int = 80, divide: int = 1, matrices=MATRICES_70B) -> list[dict]:
    """The matrices of the set; ``divide`` shrinks every dimension (for tests and short runs)."""
    items = []
    for block in range(blocks):
        for index, (name, m, n) in enumerate(matrices):
            items.append({"block": block, "name": name, "m": m // divide, "n": n // divide, "seed": 7919 * block + 101 * index + 1})
    return items


def work(m: int, n: int) -> float:
    """Algorithmic flops of one matrix: sweep ``m n (m + n - 2)`` plus both factor preparations ``2 k^3 / 3``."""
    return float(m) * n * (m + n - 2) + 2.0 * (float(m) ** 3 + float(n) ** 3) / 3.0


def partition(items: list[dict], world: int) -> list[list[dict]]:
    """Longest-processing-time-first assignment of the matrices to ``world`` ranks (deterministic)."""
    shares: list[list[dict]] = [[] for _ in range(world)]
    load = [0.0] * world
    order = sorted(range(len(items)), key=lambda k: (-work(items[k]["m"], items[k]["n"]), k))
    for k in order:
        rank = min(range(world), key=lambda r: (load[r], r))
        shares[rank].append(items[k])
        load[rank] += work(items[k]["m"], items[k]["n"])
    return shares


def quantize_matrix(item: dict, device) -> dict:
    """Generate one seeded layer on ``device``, prepare its factors, quantize it to INT4; returns timings and checks."""
    import torch

    import gptq_2d as G
    import kron_factors as K
    import quantizer_int as Q
    import synthetic

    m, n = item["m"], item["n"]
    w, g, h = synthetic.make_layer(m, n, seed=item["seed"], device=device, samples=min(8192, max(m, n)))
    events = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    events[0].record()
    l, u = K.feedback_factors_from_grams(g, h)
    events[1].record()
    scale = Q.int_abs_max_scale_triton(w, qmin=-8, qmax=7, dtype=torch.float16).expand(m, n)
    zero = torch.zeros(1, 1, device=device, dtype=w.dtype).expand(m, n)
    z = G.gptq_2d(w, l, u, quantizer=functools.partial(Q.affine_quantizer_triton, qmin=-8, qmax=7), quantizer_inputs=(scale, zero))
    events[2].record()
    torch.cuda.synchronize(device)
    codes = torch.round(z / scale)
    stats = {
        **item, "prep_ms": events[0].elapsed_time(events[1]), "sweep_ms": events[1].elapsed_time(events[2]),
        "codes_in_range": bool((codes.min() >= -8) & (codes.max() <= 7)), "finite": bool(torch.isfinite(z).all()),
        "code_sum": float(codes.double().sum().item()),
    }
    if m * n <= 4096 * 4096:  # the objective needs two more products; keep it to the smaller matrices
        rtn = torch.clamp(torch.round(w / scale), -8, 7) * scale
        stats["objective_vs_rtn"] = synthetic.objective(z, w, g, h) / synthetic.objective(rtn, w, g, h)
    return stats


def run(items: list[dict], process: Callable[[dict], dict], *, rank: int, world: int, gather: Callable | None = None,
        barrier: Callable | None = None) -> dict | None:
    """Process this rank's share; rank 0 returns the summary of the whole set.  ``gather(obj)`` must return the list
    of every rank's object on rank 0 (None elsewhere); ``barrier()`` aligns the ranks before the clock starts."""
    share = partition(items, world)[rank]
    if barrier is not None:
        barrier()
    start = time.perf_counter()
    results = [process(item) for item in share]
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
        entry["prep_ms"] += r.get("prep_ms", 0.0)
        entry["sweep_ms"] += r.get("sweep_ms", 0.0)
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
    }


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--blocks", type=int, default=80)
    parser.add_argument("--divide", type=int, default=1, help="shrink every dimension by this factor")
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
    summary = run(layer_list(args.blocks, args.divide), functools.partial(quantize_matrix, device=device), rank=rank, world=world,
                  gather=gather, barrier=barrier)
    if summary is not None:
        print(json.dumps(summary))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
