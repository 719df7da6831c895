"""Host logic of the by-matrix sharding, including a two-rank run over gloo on the CPU (no GPU work: the per-matrix
function is a stand-in)."""
import os
import tempfile

import torch.distributed as dist
import torch.multiprocessing as mp


def test_layer_list_and_partition():
    import layer_set

    items = layer_set.layer_list(80)
    assert len(items) == 560 and sum(i["m"] * i["n"] for i in items) == 80 * (2 * 8192 * 8192 + 2 * 1024 * 8192 + 3 * 28672 * 8192)
    assert len({i["seed"] for i in items}) == 560
    for world in (1, 2, 4, 8):
        shares = layer_set.partition(items, world)
        assert sorted((i["block"], i["name"]) for s in shares for i in s) == sorted((i["block"], i["name"]) for i in items)
        loads = [sum(layer_set.work(i["m"], i["n"]) for i in s) for s in shares]
        assert max(loads) / (sum(loads) / world) < 1.02  # longest-first dealing balances the algorithmic work
    assert layer_set.partition(items[:3], 8)[3:] == [[]] * 5


def test_shared_input_factors_stay_together():
    """q, k, v of a block share one input-side factor and gate, up another: a group is dealt out as one piece, its
    matrices follow each other on their rank, and its cost counts the shared factor once."""
    import layer_set

    items = layer_set.layer_list(6, shared_inputs=True)
    groups = {}
    for item in items:
        if "group" in item:
            groups.setdefault(item["group"], []).append(item)
    assert len(groups) == 12 and sorted(len(g) for g in groups.values()) == [2] * 6 + [3] * 6
    for members in groups.values():
        assert len({i["input_seed"] for i in members}) == 1 and len({i["n"] for i in members}) == 1
    assert all("group" not in i for i in items if i["name"] in ("o", "down"))
    assert abs(layer_set.work(1024, 8192, input_factor_ready=True) - (layer_set.work(1024, 8192) - 2 * 8192.0 ** 3 / 3)) < 1e3
    for world in (1, 2, 4):
        shares = layer_set.partition(items, world)
        assert sorted((i["block"], i["name"]) for s in shares for i in s) == sorted((i["block"], i["name"]) for i in items)
        for share in shares:
            names = [i.get("group") for i in share]
            for group in set(names) - {None}:
                where = [k for k, name in enumerate(names) if name == group]
                assert where == list(range(where[0], where[0] + len(groups[group])))  # whole and contiguous
    assert "group" not in layer_set.layer_list(1)[0]


def _rank(rank, world, store_path, out_path):
    import sys

    from conftest import PACKAGE
    sys.path.insert(0, PACKAGE)
    import layer_set

    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)

    def gather(obj):
        out = [None] * world if rank == 0 else None
        dist.gather_object(obj, out, dst=0)
        return out

    process = lambda item: {**item, "prep_ms": 1.0, "sweep_ms": float(item["m"]) / 1024, "finite": True, "codes_in_range": True, "rank": rank}
    summary = layer_set.run(layer_set.layer_list(3, divide=64), process, rank=rank, world=world, gather=gather, barrier=dist.barrier)
    if rank == 0:
        import json
        with open(out_path, "w") as f:
            json.dump(summary, f)
    else:
        assert summary is None
    dist.destroy_process_group()


def test_two_ranks_over_gloo():
    import json

    with tempfile.TemporaryDirectory() as tmp:
        store, out = os.path.join(tmp, "store"), os.path.join(tmp, "out.json")
        mp.spawn(_rank, args=(2, store, out), nprocs=2, join=True)
        summary = json.load(open(out))
    assert summary["matrices"] == 21 and summary["n_gpus"] == 2 and len(summary["busy_s"]) == 2
    assert summary["mean_ms_by_shape"]["448x128"]["count"] == 6 and summary["all_finite"]


def test_journal_resumes_an_interrupted_set():
    """A run that dies half way leaves a journal; the next run (here with another number of ranks) skips what is done."""
    import json

    import layer_set

    items = layer_set.layer_list(2, divide=64)
    calls = []

    def process(item, fail_after=None):
        if fail_after is not None and len(calls) >= fail_after:
            raise RuntimeError("interrupted")
        calls.append((item["block"], item["name"]))
        stats = {**item, "prep_ms": 1.0, "sweep_ms": 2.0, "finite": True, "codes_in_range": True}
        return lambda: stats  # as a pipelined process does: a fetcher

    with tempfile.TemporaryDirectory() as tmp:
        journal = os.path.join(tmp, "set.journal")
        try:
            layer_set.run(items, lambda item: process(item, fail_after=5), rank=0, world=1, journal=journal)
        except RuntimeError:
            pass
        # the fifth matrix was enqueued but never settled: four are written down
        assert len(layer_set.read_journal(journal + ".0")) == 4
        with open(journal + ".0", "a") as f:
            f.write('{"block": 1, "na')  # a line cut off by the kill
        calls.clear()
        stash = []

        def gather_for(rank):
            def gather(obj):
                if rank == 1:
                    stash.append(obj)
                    return None
                return [obj] + stash
            return gather

        assert layer_set.run(items, process, rank=1, world=2, journal=journal, gather=gather_for(1)) is None
        summary = layer_set.run(items, process, rank=0, world=2, journal=journal, gather=gather_for(0))
        assert len(calls) == len(items) - 4  # nothing done twice
        assert summary["matrices"] == len(items) and summary["resumed"] == 4
        done = {}
        for name in os.listdir(tmp):
            done.update(layer_set.read_journal(os.path.join(tmp, name)))
        assert set(done) == {(i["block"], i["name"]) for i in items}
        assert all(json.dumps(v) for v in done.values())
