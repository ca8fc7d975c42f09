#!/usr/bin/env python
"""Headline benchmark: batched river subgame solving, 256 DCFR iterations.

One "step" solves B=4096 independent seeded river subgames per GPU (random boards,
Dirichlet(1) ranges over the unblocked combos, pot U{20..200}, stack U{100..1000}, bins
{fold, call, 0.5 pot, 1 pot, all-in}, at most 2 raises per street) with one launch of the
fused CFR kernel.  Metric: subgame-CFR-iterations per second over all GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

With N > 1 launch under torch.distributed.run; every rank solves its own B subgames (no
collective inside the solve) and the training targets are all-gathered at the end of a step.
`--impl reference` times the CPU restatement of the upstream evaluator (oracle/) on the
host cores instead.  The JSON line also carries: `roofline` (the iteration kernel, timed
alone with CUDA events on its stream), `micro` (showdown evals/s and 7-card ranks/s, the
second half of the metric), `without_weight_sums`, `strong` (N > 1: the SAME 4096 subgames
split over the ranks), `e2e` and, at N = 1, `cpu_baseline`.
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

# Per-build constants of the iteration kernel from its ncu capture on a small case (592 subgames x 16
# iterations; summary and command under profiles/): DRAM bytes moved and warp instructions executed
# per subgame-pass.  Both grow in proportion to the subgame-passes of a launch.
NCU_DRAM_BYTES_PER_SUBGAME_PASS = 3.07e6
NCU_WARP_INSTRUCTIONS_PER_SUBGAME_PASS = 0.968e6
NCU_CAPTURE = "ncu --set full on cfr_iter_kernel, 592 subgames x 16 iterations, scaled by subgame-passes"

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
    n_roots, iters = 32, 16
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
        "config": dict(workload_config(), workload=f"bounded sample of the batched river workload: {sample}; same tree "
                                                      "abstraction, ranges, pots and stacks as the B=4096 x 256 GPU arm",
                       batch_per_gpu=n_roots, iterations=iters, l2="not applicable: host run"),
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

    from poker2_b200 import _lib, build, sharding, solver
    from poker2_b200 import tree as ptree

    build.build()
    device = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(device)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=device)

    def iteration_kernel_ms() -> float:
        import ctypes

        out = ctypes.c_float(0.0)
        with torch.cuda.device(device):
            _lib.call("p2b_cfr_iteration_ms", ctypes.byref(out))
        return float(out.value)

    boards, ranges, pot, stack = make_inputs(BATCH, SEED + rank)
    trees = ptree.build_trees(ptree.root_states(pot.numpy(), stack.numpy()), list(BET_BINS), MAX_DEPTH,
                              max_raises=MAX_RAISES)
    layout = solver.device_layout(trees, boards.numpy())
    sv = solver.SubgameSolver(layout, boards, device, exploitability=True)
    rb = solver.pad_rows(ranges.to(device)).contiguous()
    scal = solver.iteration_scalars(ITERATIONS)
    gathered = None

    iter_ms = []

    def step(timed=False):
        res = sv.solve(rb, scal)
        if timed:  # duration of the iteration kernel alone (CUDA events around that launch, on its stream)
            iter_ms.append(iteration_kernel_ms())
        if distributed:  # the one exchange of the path: training targets and exploitability statistics
            sharding.gather_payload({"value_targets": res.root_values, "beliefs": rb})
            sharding.reduce_exploitability(res.exploitability)
        return res

    with torch.cuda.device(device):
        _lib.call("p2b_cfr_iteration_timing", 1)
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
        step(timed=True)
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
    extras = {"iteration_kernel_ms": sum(iter_ms) / len(iter_ms)}

    def guarded(name, fn):
        """An extra member must not cost the headline line: a failure is reported in its place."""
        try:
            extras[name] = fn()
        except Exception as exc:  # noqa: BLE001
            extras[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    if rank == 0 and not distributed and not args.no_extras:
        # the same step without the regret weight sums (they feed one statistic, cfr_evaluator.py:1642)
        sv.release()

        def without_weight_sums():
            sv2 = solver.SubgameSolver(layout, boards, device, exploitability=True, track_weight_sums=False)
            ms_nows = _time_ms(lambda: sv2.solve(rb, scal), 1, 1)
            sv2.release()
            return {"ms_per_step": ms_nows, "value": BATCH * ITERATIONS / (ms_nows / 1e3), "unit": "subgame-iterations/s"}

        guarded("without_weight_sums", without_weight_sums)
        torch.cuda.empty_cache()
        guarded("production_search_block", lambda: production_member(solver, layout, boards, rb, device))
        torch.cuda.empty_cache()
        guarded("micro", lambda: micro_member(device))
        if "micro" in extras and isinstance(extras["micro"], dict) and "showdown" in extras["micro"] and not args.no_cpu_baseline:
            guarded("micro_cpu", micro_cpu_baselines)
            if isinstance(extras.get("micro_cpu"), dict) and "showdown" in extras["micro_cpu"]:
                extras["micro"]["cpu_baseline"] = extras.pop("micro_cpu")
    if distributed and not args.no_extras:
        # every rank takes part in its collectives, so a failure here is not caught rank by rank
        extras["strong"] = run_strong(args, solver, sharding, rank, world, device)

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, solver, sv, boards, ranges, pot, stack, layout, scal, gathered, distributed, device,
                      units_per_step)
    finish_gpu_arm(args, rank, world, layout, ms_step, value, clocks, e2e, distributed, extras)


def production_member(solver, layout, boards, rb, device):
    """The same 4096 river subgames under the search block of the upstream production configuration
    (conf/config_rebel_cfr.yaml:78-94: discounted_plus with a delay of 80, exponent schedules alpha 2->4,
    beta -1->-2, gamma 5->0, 200 iterations of which a warm start of type `model` replaces the first 15,
    multiplier 10, zero-sum value targets), through the one-call solve.  The start policy stands in for the
    policy head's soft-max: a fixed random soft-max per (node, hand)."""
    T, ws, delay, mult = 200, 15, 80, 10.0
    kw = dict(cfr_type="discounted_plus", gamma=5.0, dcfr_delay=delay)
    scal = solver.iteration_scalars(T, alpha=2.0, alpha_final=4.0, beta=-1.0, beta_final=-2.0, gamma_final=0.0,
                                    warm_start_iterations=ws, **kw)
    first = solver.warm_start_mix_scalars(scal, warm_start_iterations=ws, **kw)
    sv = solver.SubgameSolver(layout, boards, device, exploitability=True)
    # start policy in the kernel's row order: soft-max of seeded logits over the siblings of every node
    g = torch.Generator(device=device).manual_seed(SEED)
    logits = torch.randn(layout.rows, 1326, device=device, generator=g)
    nodes = sv.nodes.view(torch.uint8).reshape(-1, 16)
    sub = sv.subgames.view(torch.int32).reshape(-1, 8)
    row_sub = torch.repeat_interleave(torch.arange(sub.shape[0], device=device), sub[:, 1].long())
    parent_row = sub[:, 0].long()[row_sub] + nodes[:, 0].long()  # node_begin + local parent index
    e = logits.exp()
    denom = torch.zeros_like(e).index_add_(0, parent_row, e)
    policy_rows = e / denom[parent_row]
    to_level = solver.layout_tensor(layout, "from_level_major", device)
    start_policy = policy_rows.index_select(0, to_level)  # the call takes the upstream node order
    del logits, e, denom, policy_rows

    def step():
        sv.solve(rb, scal, start_policy=start_policy, warm_start_iterations=ws, warm_start_multiplier=mult,
                 warm_start_scalars=first, enforce_zero_sum=True)

    ms = _time_ms(step, 1, 1)
    passes = T - ws + 1  # the warm start's own policy update and iterations 15..199
    sv.release()
    del start_policy
    torch.cuda.empty_cache()
    return {"workload": "B=4096 river subgames, discounted_plus (delay 80, alpha 2->4, beta -1->-2, gamma 5->0), 200 "
                        "iterations with a 15-iteration warm start of type model x 10, zero-sum targets",
            "ms_per_step": ms, "iteration_passes": passes, "value": BATCH * passes / (ms / 1e3),
            "unit": "subgame-iterations/s (passes actually run)"}


def run_strong(args, solver, sharding, rank, world, device):
    """Strong scaling: the SAME B subgames (seed of rank 0) split into contiguous blocks of roots,
    one per rank; device-timed like the main leg, maximum over the ranks."""
    import torch.distributed as dist
    from poker2_b200 import tree as ptree

    boards, ranges, pot, stack = make_inputs(BATCH, SEED)
    lo, hi = sharding.shard_bounds(BATCH, rank, world)
    trees = ptree.build_trees(ptree.root_states(pot[lo:hi].numpy(), stack[lo:hi].numpy()), list(BET_BINS), MAX_DEPTH,
                              max_raises=MAX_RAISES)
    layout = solver.device_layout(trees, boards[lo:hi].numpy())
    sv = solver.SubgameSolver(layout, boards[lo:hi], device, exploitability=True)
    rb = solver.pad_rows(ranges[lo:hi].to(device)).contiguous()
    scal = solver.iteration_scalars(ITERATIONS)

    def step():
        res = sv.solve(rb, scal)
        sharding.gather_payload({"value_targets": res.root_values, "beliefs": rb})
        sharding.reduce_exploitability(res.exploitability)

    step()
    torch.cuda.synchronize()
    dist.barrier()
    steps = max(1, min(args.steps, 3))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    sv.release()
    blocks = 2 * torch.cuda.get_device_properties(device).multi_processor_count
    return {"scaling": "strong", "subgames_total": BATCH, "subgames_per_gpu": hi - lo, "steps": steps,
            "ms_per_step": float(ms.item()), "value": BATCH * ITERATIONS / (float(ms.item()) / 1e3),
            "unit": "subgame-iterations/s",
            "waves_per_gpu": (hi - lo) / blocks,
            "note": f"{blocks} subgames are in flight per GPU (two thread blocks per SM); the last wave is partly empty"}


def run_e2e(args, solver, sv, boards, ranges, pot, stack, layout, scal, gathered, distributed, device,
            units_per_step):
    import torch.distributed as dist

    # ---- end to end through the public call, host buffers in, host buffers out ----
    h_boards = boards.to(torch.int16).pin_memory()
    h_ranges = ranges.pin_memory()
    e2e_steps = max(1, min(args.steps, 3))

    from poker2_b200 import sharding

    copy_stream = torch.cuda.Stream(device=device)
    pinned = [{}, {}]  # two sets of pinned buffers: the copy of step i runs under the solve of step i+1
    in_flight = []

    def e2e_step(i):
        res, _ = solver.solve_subgames(h_boards, h_ranges, pot, stack, iterations=ITERATIONS, bet_bins=BET_BINS,
                                       max_depth=MAX_DEPTH, max_raises=MAX_RAISES, device=device, exploitability=True,
                                       device_tree=True)
        if distributed:
            sharding.gather_payload({"value_targets": res.root_values})
        stats = sharding.reduce_exploitability(res.exploitability)  # one collective, one small D2H read
        out, done = res.to_host_async(pinned[i % 2], copy_stream)
        out["stats"] = stats
        in_flight.append((res, done))  # keeps the device buffers alive until their copy has finished
        while len(in_flight) > 1:  # the result of the step before is complete on the host before the next starts
            in_flight.pop(0)[1].synchronize()
        return out

    sv.release()
    torch.cuda.empty_cache()
    out = e2e_step(0)  # warm-up: allocator and pinned buffers
    in_flight.pop(0)[1].synchronize()
    out = e2e_step(1)
    in_flight.pop(0)[1].synchronize()
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        out = e2e_step(i)
    in_flight.pop(0)[1].synchronize()  # the last step's targets are on the host
    torch.cuda.synchronize()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=device)
    if distributed:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_value = units_per_step * e2e_steps / float(e2e_s.item())
    h2d = h_boards.numel() * 8 + h_ranges.numel() * 4 + BATCH * 64 + scal.nbytes  # boards, ranges, root records, scalars
    d2h = sum(t.numel() * 4 for t in out.values() if torch.is_tensor(t)) + 4 * 8
    return {"value": e2e_value, "unit": "subgame-iterations/s", "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h), "steps": e2e_steps}


def finish_gpu_arm(args, rank, world, layout, ms_step, value, clocks, e2e, distributed, extras):
    import torch.distributed as dist

    if rank == 0:
        nonroot = int(layout.rows - BATCH)
        alg_bytes = 16.0 * 1326 * nonroot * ITERATIONS  # regrets + average policy, read + write, per iteration
        peak, peak_kind = measured_peak_gbs()
        # the dominant kernel: all ITERATIONS passes of the batch run in one launch of cfr_iter_kernel,
        # timed alone with CUDA events on its stream (the start and final passes are separate launches)
        iter_ms = extras.pop("iteration_kernel_ms")
        achieved = alg_bytes / (iter_ms / 1e3) / 1e9
        passes = BATCH * ITERATIONS
        traffic = NCU_DRAM_BYTES_PER_SUBGAME_PASS * passes
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        sm_hz = 1e6 * (clocks.get("sm_mhz") or 1965.0) if clocks else 1.965e9
        issue_slots = (iter_ms / 1e3) * sms * 4 * sm_hz
        line = {
            "metric": "subgame-CFR-iterations/sec", "value": value, "unit": "subgame-iterations/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload_config(), nodes_per_gpu=int(layout.rows),
                           mean_nodes_per_subgame=layout.rows / BATCH),
            # per step: start pass, iteration passes, final pass, each a record check + a solver kernel
            "clocks": clocks, "gpu_launches": 6 * args.steps,
            "e2e": e2e,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "traffic_source": NCU_CAPTURE,
                         "peak_source": peak_kind, "kernel": "cfr_iter_kernel", "kernel_ms_per_launch": iter_ms,
                         "algorithmic_bytes_per_launch": alg_bytes,
                         # second roofline: issue slots (4 schedulers per SM, one warp instruction per cycle each)
                         "issue": {"warp_instructions_per_launch": NCU_WARP_INSTRUCTIONS_PER_SUBGAME_PASS * passes,
                                   "issue_slots_per_launch": issue_slots,
                                   "frac": NCU_WARP_INSTRUCTIONS_PER_SUBGAME_PASS * passes / issue_slots,
                                   "source": NCU_CAPTURE}},
        }
        line.update(extras)
        if world == 1 and not args.no_cpu_baseline:
            rate, dt, cores = cpu_port_rate(32, 32, SEED)
            line["cpu_baseline"] = {"value": rate, "unit": "subgame-iterations/s", "cores": cores, "kind": "port",
                                    "sample": f"32 subgames x 32 iterations ({dt:.1f} s), torch CPU eager restatement "
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


def micro_member(device, log2_hands: int = 26, board_factor: int = 4, seconds: float = 0.8) -> dict:
    """The second half of the metric inside the default run: showdown evals/s (board tables built per
    board, then both players evaluated; and evaluation alone) and 7-card ranks/s, each kernel repeated
    for about `seconds` so that the clock sampler sees the whole measurement."""
    from poker2_b200 import _lib, showdown

    g = torch.Generator(device=device).manual_seed(1)
    n_hands = 1 << log2_hands
    cards = torch.cat([torch.rand((n_hands // 16, 52), device=device, generator=g).argsort(dim=1)[:, :7].to(torch.int16)
                       for _ in range(16)])
    out = torch.empty(n_hands, dtype=torch.int32, device=device)
    m = 4096 * board_factor
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

    def rank():
        _lib.call("p2b_rank7_cards", _lib.ptr(cards), n_hands, _lib.ptr(out), _lib.stream_ptr(device))

    def both():
        holder["t"] = showdown.BoardTables(boards)
        showdown.showdown_values(holder["t"], bel, pot, scale, out=vals)

    tabs = showdown.BoardTables(boards)

    def evaluate():
        showdown.showdown_values(tabs, bel, pot, scale, out=vals)

    def timed(fn):
        once = _time_ms(fn, 3, 3)
        reps = max(5, int(seconds * 1e3 / max(once, 1e-3)))
        return _time_ms(fn, reps, 0), reps

    sampler = ClockSampler(device.index or 0)
    sampler.start()
    (ms_rank, n_rank), (ms_both, n_both), (ms_eval, n_eval) = timed(rank), timed(both), timed(evaluate)
    clocks = sampler.stop()
    peak, _ = measured_peak_gbs()
    rank_gbs, both_gbs, eval_gbs = n_hands * 18 / ms_rank * 1e-6, m * 26520 / ms_both * 1e-6, m * 21216 / ms_eval * 1e-6
    return {
        "workload": f"{m} river boards x 2 Dirichlet(1) ranges (larger than L2); 2^{log2_hands} seven-card hands",
        "showdown": {"evals_per_s": 2 * m / (ms_both / 1e3), "ms": ms_both, "launches_timed": 2 * n_both,
                     "kernels": "board_setup_kernel + showdown_eval_kernel", "algorithmic_bytes_per_board": 26520,
                     "achieved_gbs": both_gbs, "frac": both_gbs / peak},
        "showdown_eval_only": {"evals_per_s": 2 * m / (ms_eval / 1e3), "ms": ms_eval, "launches_timed": n_eval,
                               "algorithmic_bytes_per_board": 21216, "achieved_gbs": eval_gbs, "frac": eval_gbs / peak},
        "rank7": {"hands_per_s": n_hands / (ms_rank / 1e3), "ms": ms_rank, "launches_timed": n_rank,
                  "algorithmic_bytes_per_hand": 18, "achieved_gbs": rank_gbs, "frac": rank_gbs / peak},
        "clocks": clocks,
    }


def micro_cpu_baselines() -> dict:
    """The CPU restatements of the two micro-benchmark paths on bounded samples of the same inputs: the showdown
    oracle (torch CPU eager, the operations of upstream's `_showdown_value`, strength tables included) and the
    C restatement of the seven-card ranker (one core)."""
    from oracle import cards as ocards, rank7 as orank, showdown as oshow

    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(1)
    m = 1024
    boards = torch.rand((m, 52), generator=g).argsort(dim=1)[:, :5].numpy()
    bel = torch.empty(m, 2, 1326).exponential_(generator=g) * torch.from_numpy(ocards.allowed_mask(boards)).float()[:, None, :]
    bel = bel / bel.sum(-1, keepdim=True)
    pot, scale = np.ones((m, 2), dtype=np.int64), np.ones(m, dtype=np.float32)
    oshow.showdown_values(boards[:4], bel[:4], pot[:4], scale[:4])
    t0 = time.perf_counter()
    oshow.showdown_values(boards, bel, pot, scale)
    dt_sd = time.perf_counter() - t0
    n = 1 << 22
    hands = torch.rand((n // 16, 52), generator=g).argsort(dim=1)[:, :7].to(torch.int16).numpy()
    orank.rank7(hands[:1024])
    t0 = time.perf_counter()
    for _ in range(16):
        orank.rank7(hands)
    dt_rank = time.perf_counter() - t0
    return {"showdown": {"evals_per_s": 2 * m / dt_sd, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{m} boards, tables included ({dt_sd:.1f} s), torch CPU eager"},
            "rank7": {"hands_per_s": n / dt_rank, "cores": 1, "kind": "port",
                      "sample": f"2^22 hands ({dt_rank:.1f} s), C restatement, one core"}}


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
            device_tree=True, graph=args.graph)
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
                       "network_samples_per_pass": info["leaves"] * cards_next, "nodes_per_gpu": info["rows"],
                       "passes": "iteration passes replayed from one CUDA graph" if args.graph else "plain launches"},
            "clocks": clocks, "gpu_launches": info["launches"] * args.steps,
        }))
    if distributed:
        dist.destroy_process_group()


def run_production(args):
    """What the production configuration of the upstream repository asks of the evaluator per call
    (conf/config_rebel_cfr.yaml: 192 environments, bet sizes {0.5, 1.0}, depth 5, no raise cap, 200 iterations of
    discounted_plus with a delay of 80 and exponent schedules, a warm start of type `model` over the first 15):
    flop roots with deep stacks, so that the trees are the largest this configuration produces (up to 273
    nodes), leaves valued by a random-init bf16 MLP called once per leaf, through `evaluator.SubgameEvaluator`
    (initialize_subgame, evaluate_cfr with its leaf sampling and statistics, training_data)."""
    from poker2_b200 import build, evaluator, leaf_eval, tree as ptree

    build.build()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    batch = args.batch if args.batch != 4096 else 192
    iterations = args.iterations if args.iterations != 256 else 200
    boards3, ranges, _, _ = make_street_inputs(batch, 3, 7, 1.0)
    g = torch.Generator().manual_seed(8)
    pot = torch.randint(20, 900, (batch,), generator=g).numpy()
    stack = 1000 - pot // 2
    boards = torch.full((batch, 5), -1, dtype=torch.int64)
    boards[:, :3] = boards3
    roots = ptree.root_states(pot, stack, min_raise=10, street=1)
    env = evaluator.env_view(roots, boards.numpy())
    model = leaf_eval.ValueMLP(1536, 4, dtype=torch.bfloat16, seed=0).to(device)
    ws = min(15, max(iterations - 1, 0))
    info = {}

    def step():
        ev = evaluator.SubgameEvaluator(
            device, iterations=iterations, bet_bins=BET_BINS, max_depth=5, bb=10, cfr_type="discounted_plus", alpha=2.0,
            alpha_final=4.0, beta=-1.0, beta_final=-2.0, gamma=5.0, gamma_final=0.0, dcfr_delay=min(80, iterations // 2),
            warm_start_iterations=ws, warm_start_multiplier=10.0, enforce_zero_sum=True, model=model,
            chance_average=False, generator=torch.Generator(device=device).manual_seed(1))
        ev.initialize_subgame(env, torch.arange(batch), ranges)
        ev.evaluate_cfr()
        value_batch, _, policy_batch = ev.training_data()
        info.update(nodes=ev.trees.total_nodes, largest=int(np.bincount(ev.trees.root_of).max()),
                    leaves=ev.layout.num_model_leaves, launches=ev.solver.launches, rows=len(policy_batch),
                    exploitability=ev.stats["local_exploitability"])
        return float(value_batch.value_targets.float().sum().item())  # the read that ends the step

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    ms_step = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    passes = iterations - ws + 1 if ws else iterations
    print(json.dumps({
        "metric": "subgame-CFR-iterations/sec", "value": batch * passes / (ms_step / 1e3), "unit": "subgame-iterations/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 solver state, bf16 leaf network", "data": "synthetic",
        "config": {"workload": f"production-shaped evaluator call: {batch} flop roots (stack 1000, blinds 5/10), bet sizes "
                               f"{{0.5, 1.0}}, depth 5, no raise cap, {iterations} iterations discounted_plus with schedules, "
                               f"warm start {ws} x model ({passes} iteration passes), leaves valued by a random-init bf16 MLP "
                               "(2707 -> 4 x 1536 GELU -> 2652) once per leaf; tree build, leaf sampling, statistics and "
                               "training batches inside the timed region (host clock)",
                   "batch": batch, "iterations": iterations, "nodes": info["nodes"], "largest_tree": info["largest"],
                   "model_leaves": info["leaves"], "policy_rows": info["rows"],
                   "local_exploitability": info["exploitability"]},
        "clocks": clocks, "gpu_launches": info["launches"] * args.steps,
    }))


def main():
    global BATCH, ITERATIONS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the micro, without_weight_sums and strong members (profiling runs)")
    ap.add_argument("--batch", type=int, default=BATCH, help="subgames per GPU (default: the headline 4096)")
    ap.add_argument("--iterations", type=int, default=ITERATIONS, help="DCFR iterations (default: 256)")
    ap.add_argument("--workload", default="river", choices=["river", "micro", "turn", "flop", "production"],
                    help="river = the headline batched river solve; micro = rules/showdown micro-benchmark; "
                         "turn / flop = subgames with network-valued leaves; production = one evaluator call of the "
                         "upstream production configuration (192 flop roots, depth 5, no raise cap)")
    ap.add_argument("--micro-log2-hands", type=int, default=26)
    ap.add_argument("--micro-board-factor", type=int, default=4, help="boards = 4096 x this")
    ap.add_argument("--leaf-chunk", type=int, default=2048, help="leaves per network batch (x ~48 samples)")
    ap.add_argument("--graph", action="store_true",
                    help="turn / flop: replay the iteration passes (two sweeps and the leaf network) from one CUDA graph")
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
    if args.workload == "production":
        if rank == 0:
            run_production(args)
        return
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
