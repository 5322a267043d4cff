#!/usr/bin/env python
"""Benchmark of the fused recurrence hot path: fwd+bwd (B*T)/s on the headline workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

A "step" is one forward + BPTT backward (+ dR/db) of the whole workload
(LSTM bf16, B=8, T=1024, N=3, D=256, seeded synthetic inputs) with loss = sum(h) and
gradients for all four inputs. With N > 1 every rank runs the same-shaped workload on its own
batch shard (weak scaling over batch; no collective inside the time loop) and the weight
gradients dR/db are all-reduced over NCCL once per step (one flat buffer, one call). Before the
timed region every multi-GPU run checks, on a small shape, that this rank's shard reproduces the
same rows of the unsharded call, and that the all-reduced dR equals the unsharded dR.

Prints ONE JSON line (rank 0). `value` is timed with CUDA events with the inputs resident in
HBM; `e2e` goes through the public `flashrnn(...)` call with pinned HOST inputs: every step's
host->device copies (prefetched one step ahead on a side stream) and a device->host read of the loss
are inside the timed region.
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
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = "cfg2_lstm_bf16_B8_T1024_N3_D256"
METRIC = "fwd+bwd (B*T)/sec, LSTM bf16 B8 T1024 N3 D256"
CELL, B, T, N, D, SEED = "lstm", 8, 1024, 3, 256, 1
GR = 4
FLOP_FWD = 2 * GR * D * D * N * B * T          # R*h contraction of the forward kernel
FLOP_BWD = 2 * GR * D * D * N * B * T          # R^T*dg contraction of the backward kernel
FLOP_WGRAD = 2 * GR * D * D * N * B * T        # dR contraction
CPU_SAMPLE_T = 128                              # bounded CPU sample: same B, N, D, first 128 steps
REFERENCE_BUDGET_S = 150.0                      # wall-clock budget of the reference arm's timed steps
# dram__bytes_read.sum + dram__bytes_write.sum per launch on this workload. NOT measured by this run: quoted from
# the ncu capture summarised in the profile below (bench.py cannot run ncu on itself); re-capture when a kernel changes.
NCU_TRAFFIC_PROFILE = "profiles/recurrence_kernels_cfg2_lstm_bf16_B8_T1024_N3_D256.md"
NCU_TRAFFIC_BYTES = {"fwd": 52.0e6 + 62.5e6, "bwd": 152.7e6 + 32.9e6, "wgrad": 63.0e6 + 2.1e6}


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def config_dict(world: int) -> dict:
    """The workload description; identical in the GPU arm's and the reference arm's JSON line."""
    return {"workload": WORKLOAD, "cell": CELL, "B_per_gpu": B, "T": T, "N": N, "D": D,
            "sharding": "batch (weights replicated, dR+db summed by one all-reduce)" if world > 1 else "none",
            "l2": "GPU arm: 256 MiB written between timed steps (untimed)"}


def _host_threads() -> int:
    """All host cores, set explicitly: torchrun exports OMP_NUM_THREADS=1 to its children."""
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def _reference_callable():
    """(fn(wx, R, b, init) -> seconds for fwd + backward of sum(h), kind, description)."""
    from oracle.build_ref import load_reference

    ref = load_reference()
    if ref is not None:
        def run(wx, R, b, init):
            leaves = [t.detach().clone().requires_grad_(True) for t in (wx, R, b, init)]
            t0 = time.perf_counter()
            hist, _ = ref(*leaves, cell=CELL, numerics="fp32_state_bf16_mma")
            hist[0].sum().backward()
            return time.perf_counter() - t0

        return run, "reference", ("the reference's own flashrnn_torch(numerics='fp32_state_bf16_mma') + torch autograd "
                                  "(unmodified modules under oracle/_ref), fp32 originals of the inputs")
    from oracle import recurrence_port as port

    def run(wx, R, b, init):
        d_history = torch.zeros((2,) + tuple(wx.shape[:2]) + tuple(wx.shape[3:]))
        d_history[0] = 1.0
        t0 = time.perf_counter()
        port.forward_backward(wx, R, b, init, CELL, d_history, torch.zeros_like(init))
        return time.perf_counter() - t0

    return run, "port", "oracle port (oracle/_ref was not built: no reference checkout at build time), fwd + explicit BPTT"


def cpu_baseline(reps: int = 3):
    """The reference's CPU implementation on a bounded sample of the workload: the first CPU_SAMPLE_T steps,
    `reps` passes after one warm-up, median."""
    from flashrnn_b200.workloads import make_inputs

    cores = _host_threads()
    run, kind, what = _reference_callable()
    wx, R, b, initial = make_inputs(CELL, B, CPU_SAMPLE_T, N, D, SEED)
    run(wx[:, :8], R, b, initial)  # warm-up
    times = sorted(run(wx, R, b, initial) for _ in range(reps))
    dt = times[len(times) // 2]
    return {
        "value": B * CPU_SAMPLE_T / dt, "unit": "(B*T)/s", "cores": cores, "kind": kind,
        "sample": f"{what}; B={B} N={N} D={D}, first {CPU_SAMPLE_T} of {T} steps, median of {reps} passes "
                  f"({dt:.2f} s per pass)",
    }


def run_reference(args):
    """Reference arm: the reference's own CPU implementation on the FULL workload (all T steps, fwd + autograd
    backward of sum(h)), all host threads. A step takes seconds, so the arm runs as many of the requested steps as
    fit REFERENCE_BUDGET_S and prints the count it really ran; warm-up is one short call (the CPU path has no
    caches to warm beyond the first allocation)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from flashrnn_b200.workloads import make_inputs

    cores = _host_threads()
    run, kind, what = _reference_callable()
    wx, R, b, initial = make_inputs(CELL, B, T, N, D, SEED)
    run(wx[:, :16], R, b, initial)  # warm-up
    times, t_start = [], time.perf_counter()
    while len(times) < max(1, args.steps) and (not times or time.perf_counter() - t_start + times[-1] < REFERENCE_BUDGET_S):
        times.append(run(wx, R, b, initial))
    dt = sum(times) / len(times)
    value = B * T / dt
    base = {"value": value, "unit": "(B*T)/s", "cores": cores, "kind": kind,
            "sample": f"{what}; the full workload (T={T}), {len(times)} step(s) of {dt:.2f} s"}
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "(B*T)/s", "n_gpus": args.gpus,
        "steps": len(times), "steps_requested": args.steps, "warmup": 1, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 operands, f32 state/accumulate",
        "data": "synthetic", "config": config_dict(int(os.environ.get("WORLD_SIZE", "1"))),
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "(B*T)/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="time the resident step as eager launches only (default: also as a replayed CUDA graph)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra keys (wide head, head-sharded configuration); used for profiler runs")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the recurrence has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    from flashrnn_b200 import _lib, flashrnn, poll_errors
    from flashrnn_b200.sharding import flashrnn_sharded
    from flashrnn_b200.workloads import make_inputs

    _lib.load()
    shard_check = check_sharded_equals_unsharded(dev, dist, rank, world) if world > 1 else None
    # every rank holds its own batch shard of a global batch of world*B sequences
    wx32, R32, b32, init32 = make_inputs(CELL, B, T, N, D, SEED + rank)
    R32, b32 = make_inputs(CELL, B, T, N, D, SEED)[1:3]  # weights are replicated
    h_wx = wx32.to(torch.bfloat16).pin_memory()
    h_R, h_b, h_init = R32.pin_memory(), b32.pin_memory(), init32.pin_memory()
    h2d_bytes = sum(t.numel() * t.element_size() for t in (h_wx, h_R, h_b, h_init))
    d_wx, d_R, d_b, d_init = (t.to(dev) for t in (h_wx, h_R, h_b, h_init))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def call(leaves):
        # N > 1: this rank's batch shard; dR and db are summed over the ranks by ONE all-reduce inside backward
        if dist is not None:
            return flashrnn_sharded(*leaves, function=CELL, dtype="bfloat16", axis="batch")
        return flashrnn(*leaves, function=CELL, backend="b200", dtype="bfloat16")

    def step_resident():
        leaves = [t.detach().requires_grad_(True) for t in (d_wx, d_R, d_b, d_init)]
        hist, _ = call(leaves)
        hist[0].sum().backward()
        return leaves

    # End-to-end: every step copies its inputs from pinned host memory and copies the loss back to pinned host
    # memory. The input copy of step i+1 runs on a side stream while step i computes (what a prefetching data
    # loader does) and the host does not wait inside the loop (what a training loop that logs its loss
    # asynchronously does); all K input copies, K loss copies and the L2-evicting fill between steps are
    # inside the timed region, and every loss is checked after the final synchronisation.
    copy_stream = torch.cuda.Stream(device=dev)
    dev_sets = [[torch.empty_like(t, device=dev) for t in (h_wx, h_R, h_b, h_init)] for _ in range(2)]
    copy_done = [torch.cuda.Event(), torch.cuda.Event()]
    set_free = [torch.cuda.Event(), torch.cuda.Event()]  # the step that last read a device set has finished

    def start_copy(i):
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(set_free[i % 2])
            for dst, src in zip(dev_sets[i % 2], (h_wx, h_R, h_b, h_init)):
                dst.copy_(src, non_blocking=True)
            copy_done[i % 2].record(copy_stream)

    def run_e2e(steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        start_copy(0)
        losses = torch.zeros(steps, dtype=torch.float32).pin_memory()
        for i in range(steps):
            flush.fill_(1)
            torch.cuda.current_stream(dev).wait_event(copy_done[i % 2])
            if i + 1 < steps:
                start_copy(i + 1)
            leaves = [t.detach().requires_grad_(True) for t in dev_sets[i % 2]]
            hist, _ = call(leaves)
            loss = hist[0].sum()
            loss.backward()
            losses[i:i + 1].copy_(loss.detach().reshape(1), non_blocking=True)  # device -> host read of the result
            set_free[i % 2].record()
        e1.record()
        e1.synchronize()
        if not bool(torch.isfinite(losses).all()) or float(losses.abs().min()) == 0.0:
            raise RuntimeError(f"end-to-end loop produced an invalid loss: {losses.tolist()}")
        return e0.elapsed_time(e1), float(losses[-1])

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        # K steps are queued without a host wait in between, bracketed by the barriers outside; each step
        # has its own pair of events so that the L2-evicting fill between two steps stays outside the sum
        pairs = []
        for _ in range(steps):
            flush.fill_(1)  # evict L2 between timed iterations (untimed)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            pairs.append((e0, e1))
        torch.cuda.synchronize()
        return sum(e0.elapsed_time(e1) for e0, e1 in pairs)

    def step_local():
        # N > 1: this rank's shard WITHOUT the all-reduce; it follows each replay as an eager NCCL call on the same buffers
        leaves = [t.detach().requires_grad_(True) for t in (d_wx, d_R, d_b, d_init)]
        hist, _ = flashrnn(*leaves, function=CELL, backend="b200", dtype="bfloat16")
        hist[0].sum().backward()
        return leaves

    def capture_step():
        """The resident step (forward, loss, backward, dR/db) recorded once into a CUDA graph: the same launches on the
        same buffers without the host work between them. With N > 1 the all-reduce of dR+db stays an eager call after
        every replay (a collective inside the capture hung the two-GPU run). Returns a callable or None if refused."""
        if args.no_graph:
            return None
        try:
            body = step_resident if dist is None else step_local
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                body()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):   # other threads (NCCL's watchdog) may query events
                held = body()

            def replay():
                graph.replay()
                if dist is not None:
                    from flashrnn_b200.sharding import allreduce_weight_grads
                    allreduce_weight_grads(held[1].grad, held[2].grad, "batch")

            graph.replay()   # without the collective: every rank decides for itself here
            torch.cuda.synchronize()
            poll_errors(block=True)
            if not all(torch.isfinite(t.grad.float()).all() for t in held):
                return None
            return replay
        except Exception as exc:  # an eager step is always available
            print(f"bench.py: CUDA-graph capture of the step refused ({exc!r:.200}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
            return None

    for _ in range(args.warmup):
        step_resident()
    run_e2e(args.warmup)
    poll_errors(block=True)
    graph = capture_step()
    if dist is not None:   # all ranks time the same kind of step
        agree = torch.tensor([1 if graph is not None else 0], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0:
            graph = None
    if graph is not None:
        for _ in range(args.warmup):
            graph()
    barrier()
    with ClockSampler(local_rank) as clocks:
        ms_eager = timed(step_resident, args.steps)
        barrier()
        ms = timed(graph, args.steps) if graph is not None else ms_eager
        barrier()
        ms_e2e, _ = run_e2e(args.steps)
        barrier()
    poll_errors(block=True)

    # per-kernel durations, measured with the same inputs through the C ABI
    breakdown = kernel_breakdown(_lib, dev, d_wx, d_R, d_b, d_init, flush, max(3, min(args.steps, 10)))
    if dist is not None:
        breakdown["allreduce_dR_db"] = time_allreduce(dev, dist, GR * N * D * D + 4 * N * D)
    del d_wx, h_wx, dev_sets
    t_ms = torch.tensor([ms, ms_e2e, ms_eager], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_eager = (float(v) for v in t_ms.tolist())
    # side measurements come last, after every figure of the headline line is final
    proj = None if args.no_extras else with_input_projection(dev)
    infer = None if args.no_extras else inference_e2e(dev)
    wide = None if args.no_extras else wide_head_sharded(dev, dist, rank, world)
    try:
        heads = None if args.no_extras else head_sharded_config(dev, dist, rank, world)
    except (ValueError, RuntimeError) as exc:   # reported, never fatal for the headline line
        heads = {"error": repr(exc)[:300]}
    if rank == 0:
        bf16_peak, hbm_peak, peak_kind = _peaks()
        value = world * B * T * args.steps / (ms * 1e-3)
        e2e_value = world * B * T * args.steps / (ms_e2e * 1e-3)
        dom = max(("fwd", "bwd", "wgrad"), key=lambda k: breakdown[k])
        flops = {"fwd": FLOP_FWD, "bwd": FLOP_BWD, "wgrad": FLOP_WGRAD}[dom]
        achieved = flops / (breakdown[dom] * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": "(B*T)/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 operands, f32 state/accumulate", "data": "synthetic",
            "config": config_dict(world),
            "e2e": {"value": e2e_value, "unit": "(B*T)/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": 4,
                    "d2h_note": "training step: only the scalar loss returns to the host; history and gradients stay "
                                "on the device"},
            "launch": (("the step's launches recorded once into a CUDA graph and replayed"
                        + ("; the all-reduce of dR+db follows each replay as an eager NCCL call" if world > 1 else ""))
                       if graph is not None else "eager launches through flashrnn(...)"),
            "eager": {"value": world * B * T * args.steps / (ms_eager * 1e-3), "unit": "(B*T)/s",
                      "ms_per_step": ms_eager / args.steps,
                      "note": "the same step as eager launches through flashrnn(...) + autograd"},
            "gpu_launches": args.steps * 5,
            "kernels_ms": breakdown,
            "roofline": {"bound": "tensor", "kernel": f"frnn_{dom}_kernel", "achieved": achieved, "peak": bf16_peak,
                         "unit": "TFLOP/s", "frac": achieved / bf16_peak, "peak_source": peak_kind,
                         "traffic": NCU_TRAFFIC_BYTES[dom],
                         "traffic_source": f"quoted from the committed ncu summary {NCU_TRAFFIC_PROFILE}, not measured by this run",
                         "note": "step-latency bound: T dependent steps; kernels_ms.*_phase_cycles_per_step is the per-step budget"},
            "clocks": clocks.summary(),
        }
        if shard_check is not None:
            line["sharded_equals_unsharded"] = shard_check
        if proj is not None:
            line["with_input_projection"] = proj
        if infer is not None:
            line["inference_e2e"] = infer
        if wide is not None:
            line["wide_head_row_sharded"] = wide
        if heads is not None:
            line["head_sharded_cfg5b"] = heads
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def check_sharded_equals_unsharded(dev, dist, rank, world):
    """Before anything is timed: on a small shape, this rank's batch shard through flashrnn_sharded must reproduce
    the same rows of the unsharded call run on this GPU (history / dWx bit-identical: batch rows never interact),
    and the all-reduced dR / db must equal the unsharded ones up to summation order. Raises on a mismatch."""
    from flashrnn_b200 import flashrnn
    from flashrnn_b200.sharding import flashrnn_sharded, shard_range
    from flashrnn_b200.workloads import make_inputs

    cell, Bs, Ts, Ns, Ds = "lstm", 8 * world, 24, 2, 128
    wx, R, b, init = (t.to(dev) for t in make_inputs(cell, Bs, Ts, Ns, Ds, 77))
    wx = wx.bfloat16()
    full = [t.detach().requires_grad_(True) for t in (wx, R, b, init)]
    hist_f, _ = flashrnn(*full, function=cell, backend="b200", dtype="bfloat16")
    hist_f[0].sum().backward()
    lo, hi = shard_range(Bs, world, rank)
    mine = [t.detach().requires_grad_(True) for t in (wx[lo:hi].contiguous(), R, b, init[:, lo:hi].contiguous())]
    hist_s, _ = flashrnn_sharded(*mine, function=cell, dtype="bfloat16", axis="batch")
    hist_s[0].sum().backward()
    torch.cuda.synchronize()
    same_rows = bool(torch.equal(hist_s, hist_f[:, lo:hi])) and bool(torch.equal(mine[0].grad, full[0].grad[lo:hi]))
    scale = float(full[1].grad.abs().max())
    err_dR = float((mine[1].grad - full[1].grad).abs().max()) / scale
    err_db = float((mine[2].grad - full[2].grad).abs().max()) / float(full[2].grad.abs().max())
    flags = torch.tensor([float(same_rows), err_dR, err_db], dtype=torch.float64, device=dev)
    worst = flags.clone()
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    ok = bool(flags[0] == 1.0) and float(worst[1]) <= 1e-5 and float(worst[2]) <= 1e-5
    out = {"shape": f"{cell} B{Bs} T{Ts} N{Ns} D{Ds}", "rows_bit_identical_on_every_rank": bool(flags[0] == 1.0),
           "dR_max_err_scaled": float(worst[1]), "db_max_err_scaled": float(worst[2]), "ok": ok}
    if not ok:
        raise RuntimeError(f"sharded run does not reproduce the unsharded one: {out}")
    return out


def time_allreduce(dev, dist, numel, reps=10):
    """Device time (ms, max over ranks) of the one all-reduce of the flat dR+db buffer."""
    buf = torch.zeros(numel, dtype=torch.float32, device=dev)
    for _ in range(3):
        dist.all_reduce(buf)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        dist.all_reduce(buf)
    e1.record()
    e1.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def head_sharded_config(dev, dist, rank, world, steps=3, warmup=2):
    """Extra keys: fwd+bwd step of the head-sharded configuration (LSTM N32 D128 B256 T2048, bf16 Wx) with the 32
    heads split over the ranks, no collective at all. Needs >= 4 GPUs (one GPU's share must fit its memory)."""
    if world < 4 or 32 % world != 0:
        return None
    from flashrnn_b200.sharding import flashrnn_sharded

    cell, Nh, Dh, Bh, Th = "lstm", 32 // world, 128, 256, 2048
    gen = torch.Generator(device=dev).manual_seed(5 + rank)
    wx = torch.randn((Bh, Th, 4, Nh, Dh), generator=gen, device=dev, dtype=torch.bfloat16)
    R = torch.randn((4, Nh, Dh, Dh), generator=gen, device=dev) * Dh ** -0.5
    b = torch.randn((4, Nh, Dh), generator=gen, device=dev) * 0.1
    init = torch.randn((2, Bh, 1, Nh, Dh), generator=gen, device=dev) * 0.5
    times = []
    for i in range(warmup + steps):
        leaves = [t.detach().requires_grad_(True) for t in (wx, R, b, init)]
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        hist, _ = flashrnn_sharded(*leaves, function=cell, dtype="bfloat16", axis="heads")
        hist[0].sum().backward()
        e1.record()
        e1.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
        del hist, leaves
    t = torch.tensor([sum(times) / len(times)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    del wx, R, b, init
    torch.cuda.empty_cache()
    return {"workload": f"lstm bf16 N32 D128 B256 T2048, {Nh} heads per GPU, no collective", "ms_per_step": ms,
            "value": Bh * Th / ms * 1e3, "unit": "(B*T)/s", "steps": steps, "warmup": warmup}


def with_input_projection(dev, steps=5, warmup=2):
    """Extra keys: the headline workload with the input projection in front (the reference benchmark's "-withlinear"
    variant, flashrnn/speed_experiments/kernel_speed_benchmark.py:388-408): x[B,T,N*D] -> Wx by this library's tcgen05
    GEMM -> recurrence, forward + backward with gradients for x, W, R, b and the initial state. Every rank runs it on
    its own data; rank 0's figure is reported."""
    from flashrnn_b200 import flashrnn_projected

    try:
        gen = torch.Generator(device=dev).manual_seed(11)
        I = N * D
        x = torch.randn((B, T, I), generator=gen, device=dev)
        W = torch.randn((4 * N * D, I), generator=gen, device=dev) * I ** -0.5
        R = torch.randn((4, N, D, D), generator=gen, device=dev) * D ** -0.5
        b = torch.randn((4, N, D), generator=gen, device=dev) * 0.1
        init = torch.randn((2, B, 1, N, D), generator=gen, device=dev) * 0.5
        times = []
        for i in range(warmup + steps):
            leaves = [t.detach().requires_grad_(True) for t in (x, W, R, b, init)]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            hist, _ = flashrnn_projected(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], function=CELL)
            hist[0].sum().backward()
            e1.record()
            e1.synchronize()
            if i >= warmup:
                times.append(e0.elapsed_time(e1))
        ms = sum(times) / len(times)
        return {"workload": f"x[B,T,{I}] @ W[{4 * N * D},{I}].T -> {WORKLOAD}, fwd+bwd incl. dx, dW", "ms_per_step": ms,
                "value": B * T / ms * 1e3, "unit": "(B*T)/s", "steps": steps, "warmup": warmup}
    except (ValueError, RuntimeError) as exc:   # reported, never fatal for the headline line
        return {"error": repr(exc)[:300]}


def inference_e2e(dev, steps=5, warmup=2):
    """Extra keys: a forward-only pass of the headline workload from pinned HOST memory back to pinned host memory
    (host->device copy of Wx, the prepared sequence replayed as a CUDA graph, device->host copy of the result, all
    inside the timed region), once per output mode: what the output modes and bf16 snapshots of PreparedSequence
    (flashrnn/flashrnn2/prepared.py:18-192 in the reference) save in state writes and in the copy back."""
    from flashrnn_b200 import PreparedSequence
    from flashrnn_b200.workloads import make_inputs

    try:
        wx, R, b, init = make_inputs(CELL, B, T, N, D, SEED)
        h_wx = wx.to(torch.bfloat16).pin_memory()
        d_wx = torch.empty_like(h_wx, device=dev)
        d_R, d_b, d_init = (t.to(dev) for t in (R, b, init))
        rows = []
        for mode, snap in (("full", torch.float32), ("hidden", torch.float32), ("hidden", torch.bfloat16),
                           ("last", torch.float32)):
            seq = PreparedSequence(d_wx, d_R, d_b, d_init, CELL, output_mode=mode, snapshot_dtype=snap)
            d_wx.copy_(h_wx)
            seq.capture()
            h_out = torch.empty(seq.output.shape, dtype=seq.output.dtype).pin_memory()
            times = []
            for i in range(warmup + steps):
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                d_wx.copy_(h_wx, non_blocking=True)
                seq.run()
                h_out.copy_(seq.output, non_blocking=True)
                e1.record()
                e1.synchronize()
                if i >= warmup:
                    times.append(e0.elapsed_time(e1))
            seq.check()
            seq.close()
            ms = sum(times) / len(times)
            rows.append({"output_mode": mode, "snapshot": str(snap)[6:], "ms_per_pass": ms, "value": B * T / ms * 1e3,
                         "h2d_bytes": h_wx.numel() * 2, "d2h_bytes": h_out.numel() * h_out.element_size()})
            del seq, h_out
        return {"workload": f"{WORKLOAD}, forward only, CUDA-graph replay", "unit": "(B*T)/s", "passes": rows}
    except (ValueError, RuntimeError) as exc:   # reported, never fatal for the headline line
        return {"error": repr(exc)[:300]}


def wide_head_sharded(dev, dist, rank, world):
    """Extra keys: the row-sharded wide head (LSTM, ONE head of D = 4096, B = 32, bf16 Wx) with the rows of R split
    over the ranks and round(h_t) / round(dG_t) exchanged every step by peer stores inside the kernels (no
    collective). T is reduced to 256 steps to keep the run short (the configuration's T is 4096; time is linear
    in T). At one rank the same kernels run with R streamed from HBM / L2 every step (128 MiB does not fit one
    GPU's tensor + shared memory); from 4 ranks on R stays on the SMs, hence the super-linear step."""
    import bench_shapes

    try:
        return bench_shapes.time_wide_head(T=256, steps=2, warmup=1, quiet=True)
    except (ValueError, RuntimeError) as exc:   # reported, never fatal for the headline line
        return {"error": repr(exc)[:300]} if rank == 0 else None


def kernel_breakdown(_lib, dev, d_wx, d_R, d_b, d_init, flush, reps):
    """Average duration (ms) of each of our kernels on the workload, CUDA events on the launch stream."""
    lib = _lib.load()
    plan = _lib.plan(CELL, B, T, N, D)
    S, gw, gb = 2, 4, 4
    f32, bf = torch.float32, torch.bfloat16
    history = torch.empty((S, B, T, N, D), dtype=f32, device=dev)
    carry = torch.empty((S, B, 1, N, D), dtype=f32, device=dev)
    cache = torch.empty(plan.cache_bytes, dtype=torch.uint8, device=dev)
    hbf = torch.empty(plan.hbf_bytes // 2, dtype=bf, device=dev)
    d_history = torch.zeros_like(history)
    d_history[0] = 1.0
    d_carry = torch.zeros_like(carry)
    dwx = torch.empty_like(d_wx)
    dgr = torch.empty(plan.dgr_bytes // 2, dtype=bf, device=dev)
    d_initial = torch.empty_like(carry)
    db_part = torch.empty(plan.dbpart_bytes // 4, dtype=f32, device=dev)
    dR = torch.empty((GR, N, D, D), dtype=f32, device=dev)
    db = torch.empty((gb, N, D), dtype=f32, device=dev)
    work = torch.empty(max(plan.wgrad_work_bytes // 4, 1), dtype=f32, device=dev)
    err = torch.zeros(32, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    cid = _lib.CELLS[CELL]
    d_R = d_R.to(bf).contiguous()

    def fwd():
        _lib.check(lib.frnn_b200_forward(cid, d_wx.data_ptr(), 1, d_R.data_ptr(), d_b.data_ptr(), d_init.data_ptr(),
                                         history.data_ptr(), carry.data_ptr(), cache.data_ptr(), hbf.data_ptr(),
                                         None, B, T, N, D, 0, 0, err.data_ptr(), stream), "forward")

    def bwd():
        _lib.check(lib.frnn_b200_backward(cid, cache.data_ptr(), history.data_ptr(), d_init.data_ptr(),
                                          d_R.data_ptr(), d_history.data_ptr(), d_carry.data_ptr(), dwx.data_ptr(), 1,
                                          dgr.data_ptr(), d_initial.data_ptr(), db_part.data_ptr(), None, B, T, N, D, 0, 0,
                                          err.data_ptr(), stream), "backward")

    def wgrad():
        _lib.check(lib.frnn_b200_wgrad(cid, dgr.data_ptr(), hbf.data_ptr(), db_part.data_ptr(), dR.data_ptr(),
                                       db.data_ptr(), work.data_ptr(), B, T, N, D, err.data_ptr(), stream), "wgrad")

    out = {}
    for name, fn in (("fwd", fwd), ("bwd", bwd), ("wgrad", wgrad)):
        fn()
        total = 0.0
        for _ in range(reps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            total += e0.elapsed_time(e1)
        out[name] = total / reps
    if int(err[0].item()) != 0:
        raise RuntimeError(f"device-side error {err.tolist()}")
    # in-kernel phase timers of CTA 0 (SM cycles per step)
    # err[8..15] are the epilogue warps' phases, err[16..18] the MMA warp's (see the kernels' `prof` blocks)
    names = {
        "fwd": ("wx_stage_wait", "mma_wait", "tmem_read", "epilogue_barrier", "cell", "push_h", "state_stores",
                "commit_to_epilogue"),
        "bwd": ("stage_wait_and_read", "partial_wait_and_sum", "cell", "stores_and_first_tile_wait", "scatter",
                "partial_wait_only", "stage_wait_only", None),
    }
    for name, fn in (("fwd", fwd), ("bwd", bwd)):
        err.zero_()
        err[3] = 1
        fn()
        torch.cuda.synchronize()
        v = err.tolist()
        phases = {k: round(v[8 + i] / T, 1) for i, k in enumerate(names[name]) if k is not None}
        phases.update({"mma_warp_wait": round(v[16] / T, 1), "mma_warp_issue": round(v[17] / T, 1)})
        if name == "fwd":
            phases["push_to_mma_wake"] = round(v[18] / T, 1)
        out[name + "_phase_cycles_per_step"] = phases
    err.zero_()
    return out


if __name__ == "__main__":
    main()
