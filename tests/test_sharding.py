"""Sharding and the final gather on two CPU ranks (gloo)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from poker2_b200 import sharding


def test_shard_bounds_cover_everything():
    for total in (0, 1, 7, 4096, 4099):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a1 - a0 >= b1 - b0 >= 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(123)
        full_values = torch.rand(total, 2, 16, generator=g)  # the unsharded answer, same on every rank
        full_exploit = torch.rand(total, generator=g)
        lo, hi = sharding.shard_bounds(total, rank, world)
        gathered = sharding.gather_rows(full_values[lo:hi].clone())
        stats = sharding.reduce_exploitability(full_exploit[lo:hi])
        ok = torch.equal(gathered, full_values)
        ok &= abs(stats["local_exploitability"] - full_exploit.double().mean().item()) < 1e-12
        ok &= stats["local_exploitability_min"] == full_exploit.double().min().item()
        ok &= stats["local_exploitability_max"] == full_exploit.double().max().item()
        ok &= stats["count"] == total
        with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as fh:
            fh.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_gather_matches_unsharded_order(tmp_path):
    for total in (8, 7):  # equal and ragged shards
        port = _free_port()
        mp.spawn(_worker, args=(2, port, total, str(tmp_path)), nprocs=2, join=True)
        for r in range(2):
            assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_single_process_is_identity():
    x = torch.arange(6.0).reshape(3, 2)
    assert sharding.gather_rows(x) is x
    stats = sharding.reduce_exploitability(torch.tensor([0.25, 0.75]))
    assert stats["local_exploitability"] == 0.5 and stats["count"] == 2


def _worker_mismatch(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        local = torch.zeros(3, 2, 16 if rank == 0 else 8)  # rank 1 holds rows of another width
        try:
            sharding.gather_rows(local)
            outcome = "gathered"
        except ValueError as e:
            outcome = "raised" if "disagree" in str(e) else "other"
        with open(os.path.join(result_dir, f"mismatch{rank}.txt"), "w") as fh:
            fh.write(outcome)
    finally:
        dist.destroy_process_group()


def test_shards_of_different_width_raise_on_every_rank(tmp_path):
    mp.spawn(_worker_mismatch, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"mismatch{r}.txt").read() == "raised"


def _worker_leaver(rank, world, port, result_dir):
    """Rank 1 leaves between steps, before the final gather; rank 0 must not wait for ever."""
    import datetime
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    full = torch.rand(4, 2, 16, generator=torch.Generator().manual_seed(5))
    lo, hi = sharding.shard_bounds(4, rank, world)
    first = sharding.gather_rows(full[lo:hi].clone())  # a step in which both ranks take part
    if rank == 1:
        os._exit(0)  # gone: no destroy, no further collective
    t0 = time.perf_counter()
    try:
        sharding.gather_rows(full[lo:hi].clone())
        outcome = "gathered"
    except Exception as e:  # the process group reports the missing peer (timeout or closed connection)
        outcome = f"raised {type(e).__name__}"
    waited = time.perf_counter() - t0
    with open(os.path.join(result_dir, "leaver0.txt"), "w") as fh:
        fh.write(f"{outcome}|{torch.equal(first, full)}|{waited:.1f}")
    os._exit(0)  # the group is broken; skip its teardown


def test_a_rank_that_leaves_before_the_gather_makes_the_others_raise(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker_leaver, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
        assert not p.is_alive()
    outcome, first_ok, waited = open(tmp_path / "leaver0.txt").read().split("|")
    assert outcome.startswith("raised") and first_ok == "True" and float(waited) < 30
