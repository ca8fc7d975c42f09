#!/usr/bin/env python
"""Headline benchmark: batched river subgame solving, 256 DCFR iterations.

One "step" solves B=4096 independent seeded river subgames per GPU (random boards,
Dirichlet(1) ranges over the unblocked combos, pot U{20..200}, stack U{100..1000}, bins
{fold, call, 0.5 pot, 1 pot, all-in}, at most 2 raises per street) with one launch of the
fused CFR kernel.  Metric: subgame-CFR-iterations per second over all GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

With N > 1 launch under torch.distributed.run; every rank solves its own B subgames (no
collective inside the solve) and the value targets are all-gathered at the end of a step.
`--impl reference` times the CPU restatement of the upstream evaluator (oracle/) on the
host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH = 4096
ITERATIONS = 256
BET_BINS = (0.5, 1.0)
MAX_RAISES = 2
MAX_DEPTH = 8
SEED = 2


def make_inputs(batch: int, seed: int):
    """Seeded synthetic subgames: boards [B,5] int64, ranges [B,2,1326] fp32, pot, stack."""
    g = torch.Generator().manual_seed(seed)
    boards = torch.rand(batch, 52, generator=g).argsort(dim=1)[:, :5]
    card_hit = torch.zeros(batch, 52, dtype=torch.bool)
    card_hit.scatter_(1, boards, True)
    c1, c2 = np.triu_indices(52, k=1)
    blocked = card_hit[:, torch.from_numpy(c1)] | card_hit[:, torch.from_numpy(c2)]
    ranges = torch.empty(batch, 2, 1326).exponential_(generator=g) * (~blocked)[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    pot = torch.randint(20, 201, (batch,), generator=g)
    stack = torch.randint(100, 1001, (batch,), generator=g)
    return boards, ranges, pot, stack


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def cpu_port_rate(n_roots: int, iterations: int, seed: int):
    """Times the CPU restatement of the upstream evaluator (oracle/cfr.py) on a bounded
    sample of the same workload; returns (subgame-iterations per second, seconds, cores)."""
    from oracle import cfr as ocfr
    from poker2_b200 import tree as ptree

    torch.set_num_threads(os.cpu_count() or 1)
    boards, ranges, pot, stack = make_inputs(n_roots, seed)
    trees = ptree.build_trees(ptree.root_states(pot.numpy(), stack.numpy()), list(BET_BINS), MAX_DEPTH,
                              max_raises=MAX_RAISES)
    o = ocfr.SubgameOracle(trees.oracle_dict(boards.numpy()), ranges, iterations=iterations)
    o.initialize()
    t0 = time.perf_counter()
    for t in range(iterations):
        o.iteration(t)
    dt = time.perf_counter() - t0
    return n_roots * iterations / dt, dt, torch.get_num_threads()


def run_reference_arm(args, rank: int):
    """The upstream implementation is pure Python and is not present on the benchmark
    machine; its CPU restatement (validated bit-for-bit against it) is what is timed."""
    if rank != 0:
        return
    n_roots, iters = 32, 6
    for _ in range(args.warmup):
        cpu_port_rate(4, 1, SEED)
    rates, secs = [], []
    for k in range(args.steps):
        r, dt, cores = cpu_port_rate(n_roots, iters, SEED + k)
        rates.append(n_roots * iters)
        secs.append(dt)
    value = sum(rates) / sum(secs)
    sample = f"{n_roots} subgames x {iters} iterations per step, torch CPU eager, all host threads"
    print(json.dumps({
        "impl": "reference", "metric": "subgame-CFR-iterations/sec", "value": value, "unit": "subgame-iterations/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(secs) / len(secs),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": value, "unit": "subgame-iterations/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "subgame-iterations/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config():
    return {"workload": f"batched river subgames, B={BATCH} per GPU, {ITERATIONS} DCFR(1.5,0,2) iterations, bins "
                        "{fold,call,0.5p,1p,all-in}, max 2 raises, pot U[20,200], stack U[100,1000]",
            "batch_per_gpu": BATCH, "iterations": ITERATIONS, "l2": "inputs larger than L2 (state > 3 GB per GPU)"}


def run_gpu_arm(args, rank: int, world: int, local_rank: int):
    import torch.distributed as dist

    from poker2_b200 import build, sharding, solver
    from poker2_b200 import tree as ptree

    build.build()
    device = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(device)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=device)

    boards, ranges, pot, stack = make_inputs(BATCH, SEED + rank)
    trees = ptree.build_trees(ptree.root_states(pot.numpy(), stack.numpy()), list(BET_BINS), MAX_DEPTH,
                              max_raises=MAX_RAISES)
    layout = solver.device_layout(trees, boards.numpy())
    sv = solver.SubgameSolver(layout, boards, device, exploitability=True)
    rb = solver.pad_rows(ranges.to(device)).contiguous()
    scal = solver.iteration_scalars(ITERATIONS)
    gathered = None

    def step():
        res = sv.solve(rb, scal)
        if distributed:  # the one exchange of the path: value targets and exploitability statistics
            sharding.gather_rows(res.root_values)
            sharding.reduce_exploitability(res.exploitability)
        return res

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    if distributed:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    ms_step = ms_total / args.steps
    units_per_step = world * BATCH * ITERATIONS
    value = units_per_step / (ms_step / 1e3)

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, solver, sv, boards, ranges, pot, stack, layout, scal, gathered, distributed, device,
                      units_per_step)
    finish_gpu_arm(args, rank, world, layout, ms_step, value, clocks, e2e, distributed)


def run_e2e(args, solver, sv, boards, ranges, pot, stack, layout, scal, gathered, distributed, device,
            units_per_step):
    import torch.distributed as dist

    # ---- end to end through the public call, host buffers in, host buffers out ----
    h_boards = boards.to(torch.int16).pin_memory()
    h_ranges = ranges.pin_memory()
    pinned = {}
    e2e_steps = max(1, min(args.steps, 3))

    def e2e_step():
        res, _ = solver.solve_subgames(h_boards, h_ranges, pot, stack, iterations=ITERATIONS, bet_bins=BET_BINS,
                                       max_depth=MAX_DEPTH, max_raises=MAX_RAISES, device=device, exploitability=True)
        from poker2_b200 import sharding

        if distributed:
            sharding.gather_rows(res.root_values)
        out = res.to_host(pinned)
        out["stats"] = sharding.reduce_exploitability(res.exploitability)  # one small D2H read
        return out

    sv.release()
    torch.cuda.empty_cache()
    out = e2e_step()  # warm-up: allocator and pinned buffers
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        out = e2e_step()
    torch.cuda.synchronize()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=device)
    if distributed:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_value = units_per_step * e2e_steps / float(e2e_s.item())
    h2d = h_boards.numel() * 2 + h_ranges.numel() * 4 + layout.nodes.nbytes + layout.subgames.nbytes + scal.nbytes
    d2h = sum(t.numel() * 4 for t in out.values() if torch.is_tensor(t)) + 4 * 8
    return {"value": e2e_value, "unit": "subgame-iterations/s", "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h), "steps": e2e_steps}


def finish_gpu_arm(args, rank, world, layout, ms_step, value, clocks, e2e, distributed):
    import torch.distributed as dist

    if rank == 0:
        nonroot = int(layout.rows - BATCH)
        alg_bytes = 16.0 * 1326 * nonroot * ITERATIONS  # regrets + average policy, read + write, per iteration
        peak, peak_kind = measured_peak_gbs()
        achieved = alg_bytes / (ms_step / 1e3) / 1e9
        # DRAM bytes per subgame-pass from the ncu capture of a small case (profiles/), scaled
        # to this launch by the number of subgame-passes (traffic grows in proportion)
        traffic = 2.532e6 * BATCH * (ITERATIONS + 2)
        line = {
            "metric": "subgame-CFR-iterations/sec", "value": value, "unit": "subgame-iterations/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload_config(), nodes_per_gpu=int(layout.rows),
                           mean_nodes_per_subgame=layout.rows / BATCH),
            "clocks": clocks, "gpu_launches": args.steps,
            "e2e": e2e,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_source": peak_kind,
                         "kernel": "cfr_solve_kernel", "algorithmic_bytes_per_launch": alg_bytes},
        }
        if world == 1 and not args.no_cpu_baseline:
            rate, dt, cores = cpu_port_rate(32, 8, SEED)
            line["cpu_baseline"] = {"value": rate, "unit": "subgame-iterations/s", "cores": cores, "kind": "port",
                                    "sample": f"32 subgames x 8 iterations ({dt:.1f} s), torch CPU eager restatement "
                                              "of the upstream evaluator"}
        print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


def main():
    global BATCH, ITERATIONS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--batch", type=int, default=BATCH, help="subgames per GPU (default: the headline 4096)")
    ap.add_argument("--iterations", type=int, default=ITERATIONS, help="DCFR iterations (default: 256)")
    args = ap.parse_args()
    BATCH, ITERATIONS = args.batch, args.iterations
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (poker2_b200 has no CPU path)")
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
