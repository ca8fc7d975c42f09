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
                                       max_depth=MAX_DEPTH, max_raises=MAX_RAISES, device=device, exploitability=True,
                                       device_tree=True)
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
    h2d = h_boards.numel() * 8 + h_ranges.numel() * 4 + BATCH * 64 + scal.nbytes  # boards, ranges, root records, scalars
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
        traffic = 2.76e6 * BATCH * (ITERATIONS + 2)
        line = {
            "metric": "subgame-CFR-iterations/sec", "value": value, "unit": "subgame-iterations/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload_config(), nodes_per_gpu=int(layout.rows),
                           mean_nodes_per_subgame=layout.rows / BATCH),
            "clocks": clocks, "gpu_launches": 2 * args.steps,  # per step: record check + solver kernel
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


def _time_ms(fn, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_micro(args):
    """Rules / showdown micro-benchmark: 2^26 seven-card hands ranked to int32; 4096 river
    boards (x `--micro-board-factor` so that the working set exceeds L2) with two Dirichlet(1)
    ranges each, fp32 showdown values for both players."""
    from poker2_b200 import _lib, build, showdown

    build.build()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    g = torch.Generator(device=device).manual_seed(1)
    n_hands = 1 << args.micro_log2_hands
    chunks = []
    for _ in range(16):
        r = torch.rand((n_hands // 16, 52), device=device, generator=g)
        chunks.append(r.argsort(dim=1)[:, :7].to(torch.int16))
    cards = torch.cat(chunks)
    del chunks
    out = torch.empty(n_hands, dtype=torch.int32, device=device)
    sampler = ClockSampler(0)
    sampler.start()
    ms_rank = _time_ms(lambda: _lib.call("p2b_rank7_cards", _lib.ptr(cards), n_hands, _lib.ptr(out),
                                         _lib.stream_ptr(device)), max(args.steps, 5), max(args.warmup, 3))
    del cards, out
    m = 4096 * args.micro_board_factor
    boards = torch.rand((m, 52), device=device, generator=g).argsort(dim=1)[:, :5].contiguous()
    hit = torch.zeros(m, 52, dtype=torch.bool, device=device)
    hit.scatter_(1, boards, True)
    c1, c2 = np.triu_indices(52, k=1)
    blocked = hit[:, torch.from_numpy(c1).to(device)] | hit[:, torch.from_numpy(c2).to(device)]
    bel = torch.empty(m, 2, 1326, device=device).exponential_(generator=g) * (~blocked)[:, None, :]
    bel = (bel / bel.sum(-1, keepdim=True)).contiguous()
    pot = torch.ones((m, 2), dtype=torch.int64, device=device)
    scale = torch.ones(m, device=device)
    vals = torch.empty_like(bel)
    holder = {}

    def both():
        holder["t"] = showdown.BoardTables(boards)
        showdown.showdown_values(holder["t"], bel, pot, scale, out=vals)

    ms_both = _time_ms(both, max(args.steps, 5), max(args.warmup, 3))
    tabs = showdown.BoardTables(boards)
    ms_eval = _time_ms(lambda: showdown.showdown_values(tabs, bel, pot, scale, out=vals), max(args.steps, 5),
                       max(args.warmup, 3))
    # step-level kernels (the fused_cfr_triton call signatures) on 100,000 rows of 1326
    from poker2_b200 import fused_cfr

    del bel, vals, tabs
    rows_s, H = 100_000, 1326
    R = torch.randn(rows_s, H, device=device, generator=g)
    W = torch.rand(rows_s, H, device=device, generator=g)
    inst = torch.randn(rows_s, H, device=device, generator=g)
    out_s = torch.empty(rows_s, H, device=device)
    pos_s = inst.abs()
    uni = torch.full((rows_s, H), 0.2, device=device)
    ok = torch.rand(rows_s // 2, H, device=device, generator=g) > 0.18
    prob = ok.float() / ok.float().sum(-1, keepdim=True)
    bel2 = torch.rand(rows_s // 2, 2, H, device=device, generator=g)

    class _Discounted:
        name = "discounted"

    nel = rows_s * H
    steps_s, warm_s = max(args.steps, 5), max(args.warmup, 3)
    step_ops = {}
    for name, nbytes, fn in [
        ("dcfr_update", 20 * nel, lambda: fused_cfr.fused_dcfr_update_(R, W, inst, 5, _Discounted, 1.5, 0.0, False)),
        ("regret_matching_divide", 16 * nel, lambda: fused_cfr.fused_regret_matching_divide_(pos_s, W, uni, out_s)),
        ("block_normalize", 8 * nel + 5 * nel // 2, lambda: fused_cfr.fused_block_and_normalize_beliefs_(bel2, ok, prob)),
        ("unblocked_mass", 8 * nel, lambda: fused_cfr.unblocked_mass_triton(R)),
    ]:
        ms = _time_ms(fn, steps_s, warm_s)
        step_ops[name] = {"ms": ms, "achieved_gbs": nbytes / ms * 1e-6}
    clocks = sampler.stop()
    peak, peak_kind = measured_peak_gbs()
    for v in step_ops.values():
        v["frac"] = v["achieved_gbs"] / peak
    rank_gbs = n_hands * 18 / ms_rank * 1e-6
    both_gbs = m * 26520 / ms_both * 1e-6
    eval_gbs = m * 21216 / ms_eval * 1e-6
    line = {
        "metric": "showdown evals/sec", "value": 2 * m / (ms_both / 1e3), "unit": "evals/s", "n_gpus": 1,
        "steps": max(args.steps, 5), "warmup": max(args.warmup, 3), "ms_per_step": ms_both, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"rules/showdown microbench: {m} river boards x 2 Dirichlet(1) ranges, tables built "
                               f"per board then evaluated; 2^{args.micro_log2_hands} 7-card hands ranked",
                   "l2": "inputs larger than L2"},
        "clocks": clocks, "gpu_launches": 2 * max(args.steps, 5),
        "roofline": {"bound": "hbm", "achieved": both_gbs, "peak": peak, "unit": "GB/s", "frac": both_gbs / peak,
                     "traffic": None, "peak_source": peak_kind, "kernel": "board_setup_kernel + showdown_eval_kernel",
                     "algorithmic_bytes_per_board": 26520},
        "showdown_eval_only": {"evals_per_s": 2 * m / (ms_eval / 1e3), "ms": ms_eval, "achieved_gbs": eval_gbs,
                               "frac": eval_gbs / peak, "algorithmic_bytes_per_board": 21216},
        "rank7": {"hands_per_s": n_hands / (ms_rank / 1e3), "ms": ms_rank, "achieved_gbs": rank_gbs,
                  "frac": rank_gbs / peak, "algorithmic_bytes_per_hand": 18},
        "step_ops": step_ops,
    }
    print(json.dumps(line))


def make_street_inputs(batch: int, n_board: int, seed: int, alpha: float):
    g = torch.Generator().manual_seed(seed)
    boards = torch.rand(batch, 52, generator=g).argsort(dim=1)[:, :n_board]
    hit = torch.zeros(batch, 52, dtype=torch.bool)
    hit.scatter_(1, boards, True)
    c1, c2 = np.triu_indices(52, k=1)
    blocked = hit[:, torch.from_numpy(c1)] | hit[:, torch.from_numpy(c2)]
    if alpha == 1.0:
        gam = torch.empty(batch, 2, 1326).exponential_(generator=g)
    else:
        gam = torch._standard_gamma(torch.full((batch, 2, 1326), alpha), generator=g)
    ranges = gam * (~blocked)[:, None, :]
    ranges = ranges / ranges.sum(-1, keepdim=True)
    pot = torch.randint(20, 201, (batch,), generator=g)
    stack = torch.randint(100, 1001, (batch,), generator=g)
    return boards, ranges, pot, stack


def run_street(args, rank: int, world: int, local_rank: int):
    """Turn (B=1024, 128 iterations, leaves averaged over the 48 river cards) or flop
    (B=2048 per GPU, Dirichlet(0.5) ranges, 64 iterations, 49 turn cards) subgames whose
    leaves are valued by a random-init bf16 MLP (2x1326 + 52 + 3 -> 4 x 1536 GELU -> 2x1326)."""
    import torch.distributed as dist

    from poker2_b200 import build, leaf_eval, sharding, solver

    build.build()
    device = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(device)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=device)
    turn = args.workload == "turn"
    street, n_board = (2, 4) if turn else (1, 3)
    batch = args.batch if args.batch != 4096 else (1024 if turn else 2048)
    iterations = args.iterations if args.iterations != 256 else (128 if turn else 64)
    boards, ranges, pot, stack = make_street_inputs(batch, n_board, (3 if turn else 4) + rank, 1.0 if turn else 0.5)
    model = leaf_eval.ValueMLP(1536, 4, dtype=torch.bfloat16, seed=0).to(device)
    info = {}

    def step():
        res, trees, sv = solver.solve_subgames_with_model(
            boards, ranges, pot, stack, model, street=street, iterations=iterations, bet_bins=BET_BINS,
            max_depth=MAX_DEPTH, max_raises=MAX_RAISES, device=device, exploitability=True, chunk=args.leaf_chunk,
            device_tree=True)
        if distributed:
            sharding.gather_rows(res.root_values)
            sharding.reduce_exploitability(res.exploitability)
        info.update(launches=sv.launches, leaves=sv.layout.num_model_leaves, rows=sv.layout.rows)
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
    ms_step = float(ms.item()) / args.steps
    if rank == 0:
        cards_next = 52 - n_board
        print(json.dumps({
            "metric": "subgame-CFR-iterations/sec", "value": world * batch * iterations / (ms_step / 1e3),
            "unit": "subgame-iterations/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 solver state, bf16 leaf network", "data": "synthetic",
            "config": {"workload": f"batched {'turn' if turn else 'flop'} subgames, B={batch} per GPU, {iterations} "
                                   f"DCFR(1.5,0,2) iterations, leaves at the start of the next street valued by a "
                                   f"random-init bf16 MLP (2707 -> 4 x 1536 GELU -> 2652) averaged over the "
                                   f"{cards_next} next cards; tree build, host->device copies and the final "
                                   "exploitability pass inside the timed region",
                       "batch_per_gpu": batch, "iterations": iterations, "model_leaves_per_gpu": info["leaves"],
                       "network_samples_per_pass": info["leaves"] * cards_next, "nodes_per_gpu": info["rows"]},
            "clocks": clocks, "gpu_launches": info["launches"] * args.steps,
        }))
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
    ap.add_argument("--workload", default="river", choices=["river", "micro", "turn", "flop"],
                    help="river = the headline batched river solve; micro = rules/showdown micro-benchmark; "
                         "turn / flop = subgames with network-valued leaves")
    ap.add_argument("--micro-log2-hands", type=int, default=26)
    ap.add_argument("--micro-board-factor", type=int, default=4, help="boards = 4096 x this")
    ap.add_argument("--leaf-chunk", type=int, default=2048, help="leaves per network batch (x ~48 samples)")
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
    if args.workload == "micro":
        if rank == 0:
            run_micro(args)
        return
    if args.workload in ("turn", "flop"):
        run_street(args, rank, world, local_rank)
        return
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
