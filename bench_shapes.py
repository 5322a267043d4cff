"""Per-kernel timing of the recurrence on arbitrary shapes (CUDA events, through the C ABI).

    python bench_shapes.py                 # the benchmark configurations that fit one GPU
    python bench_shapes.py lstm 16 1024 3 256
    torchrun ... bench_shapes.py config5b   # N32 D128 B256 T2048, heads sharded over the ranks
    [torchrun ...] bench_shapes.py wide [T [D [B]]]   # one head of D (4096) units row-sharded over the ranks
    python bench_shapes.py projection      # the input-projection GEMM against torch.matmul (cuBLAS)

The head-dimension sweep mirrors the reference's published one
(flashrnn/speed_experiments/kernel_speed_benchmark.py:104-127: N*D = 768, B = 16, T = 1024).
Prints one markdown table row per shape: forward, backward and dR/db times, fwd+bwd (B*T)/s and the
in-kernel phase timers of CTA 0.
"""

from __future__ import annotations

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

from flashrnn_b200 import _lib  # noqa: E402
from flashrnn_b200.workloads import HEAD_DIM_SWEEP, SIZES, make_inputs  # noqa: E402


def time_shape(cell: str, B: int, T: int, N: int, D: int, reps: int = 5, device: str = "cuda:0") -> dict:
    lib = _lib.load()
    dev = torch.device(device)
    plan = _lib.plan(cell, B, T, N, D)
    if not plan.supported:
        return {"supported": False}
    gr, gw, gb, S = SIZES[cell]
    f32, bf = torch.float32, torch.bfloat16
    wx, R, b, init = make_inputs(cell, B, T, N, D, 3, zero_initial=(cell == "slstm"))
    wx, R = wx.to(dev).to(bf).contiguous(), R.to(dev).to(bf).contiguous()
    b, init = b.to(dev), init.to(dev)
    hist = torch.empty((S, B, T, N, D), dtype=f32, device=dev)
    carry = torch.empty((S, B, 1, N, D), dtype=f32, device=dev)
    cache = torch.empty(max(plan.cache_bytes, 1), dtype=torch.uint8, device=dev)
    hbf = torch.empty(plan.hbf_bytes // 2, dtype=bf, device=dev)
    d_hist = torch.zeros_like(hist)
    d_hist[0] = 1.0
    d_carry = torch.zeros_like(carry)
    dwx = torch.empty_like(wx)
    # bf16 Wx and W-gates == R-gates: one buffer serves as dWx and as the operand of the dR contraction (as functional.py does)
    dgr = dwx if cell != "gru" else torch.empty(plan.dgr_bytes // 2, dtype=bf, device=dev)
    d_init = torch.empty_like(carry)
    db_part = torch.empty(plan.dbpart_bytes // 4, dtype=f32, device=dev)
    dR = torch.empty((gr, N, D, D), dtype=f32, device=dev)
    db = torch.empty((gb, N, D), dtype=f32, device=dev)
    work = torch.empty(max(plan.wgrad_work_bytes // 4, 1), dtype=f32, device=dev)
    xchg = torch.empty(max(plan.xchg_bytes, 1), dtype=torch.uint8, device=dev)
    xchg_ptr = xchg.data_ptr() if plan.xchg_bytes else None
    err = torch.zeros(32, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    cid = _lib.CELLS[cell]
    zero_first = int(cell == "slstm")
    cache_ptr = cache.data_ptr() if plan.cache_bytes else None

    def fwd():
        _lib.check(lib.frnn_b200_forward(cid, wx.data_ptr(), 1, R.data_ptr(), b.data_ptr(), init.data_ptr(),
                                         hist.data_ptr(), carry.data_ptr(), cache_ptr, hbf.data_ptr(), xchg_ptr, B, T, N, D,
                                         zero_first, 0, err.data_ptr(), stream), "forward")

    def bwd():
        _lib.check(lib.frnn_b200_backward(cid, cache_ptr, hist.data_ptr(), init.data_ptr(), R.data_ptr(),
                                          d_hist.data_ptr(), d_carry.data_ptr(), dwx.data_ptr(), 1, dgr.data_ptr(),
                                          d_init.data_ptr(), db_part.data_ptr(), xchg_ptr, B, T, N, D, zero_first, 0,
                                          err.data_ptr(), stream), "backward")

    def wgrad():
        _lib.check(lib.frnn_b200_wgrad(cid, dgr.data_ptr(), hbf.data_ptr(), db_part.data_ptr(), dR.data_ptr(),
                                       db.data_ptr(), work.data_ptr(), B, T, N, D, err.data_ptr(), stream), "wgrad")

    out = {"supported": True, "cluster": plan.cluster, "ctas": plan.grid_ctas}
    for name, fn in (("fwd", fwd), ("bwd", bwd), ("wgrad", wgrad)):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        e1.synchronize()
        out[name] = e0.elapsed_time(e1) / reps
    for name, fn in (("fwd", fwd), ("bwd", bwd)):
        err.zero_()
        err[3] = 1
        fn()
        torch.cuda.synchronize()
        v = err.tolist()
        out[name + "_phases"] = [round(v[8 + i] / T) for i in range(8)] + [round(v[16] / T), round(v[17] / T), 'prologue', v[20]]
        out[name + "_extra"] = [round(v[18] / T), round(v[19] / T), round(v[21] / T)]
    err.zero_()
    if int(err[0].item()) != 0:
        raise RuntimeError(f"device-side error {err.tolist()}")
    return out


def row(cell, B, T, N, D, r, cudnn=None) -> str:
    lib = "" if cudnn is None else f" {N} x {cudnn[1]:.1f} |"
    if not r["supported"]:
        return f"| {cell} | {B} | {T} | {N} | {D} | not supported (R slice exceeds tensor memory) | | | | | |" + lib
    tot = r["fwd"] + r["bwd"] + r["wgrad"]
    return (f"| {cell} | {B} | {T} | {N} | {D} | {r['cluster']} / {r['ctas']} | {r['fwd']:.3f} | {r['bwd']:.3f} | "
            f"{r['wgrad']:.3f} | {B * T / tot * 1e3 / 1e6:.2f} | {r['fwd'] * 1e3 / T:.2f} / {r['bwd'] * 1e3 / T:.2f} |" + lib)


HEADER = ("| cell | B | T | N | D | cluster / CTAs | fwd ms | bwd ms | dR+db ms | fwd+bwd M(B*T)/s | µs/step fwd / bwd |\n"
          "|---|---|---|---|---|---|---|---|---|---|---|")
HEADER_LIB = HEADER.replace("|\n", "| cuDNN layer fwd+bwd ms (heads x one layer) |\n", 1) + "---|"


def time_config5b_sharded(B: int = 256, T: int = 2048, steps: int = 5, warmup: int = 2) -> None:
    """fwd+bwd of N32 D128 B256 T2048 (LSTM, bf16 Wx) with the 32 heads split over the ranks.

    Run under torchrun, one process per GPU (4 or 8 ranks: one GPU's share must fit its memory):
        python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
            bench_shapes.py config5b
    Heads are independent, so the time loop has no collective and the weight gradients stay sharded;
    the reported time is the maximum over the ranks, the rate is B*T of the whole job over that time."""
    import os

    import torch.distributed as dist

    from flashrnn_b200.sharding import flashrnn_sharded, shard_range

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cell, N, D = "lstm", 32, 128
    lo, hi = shard_range(N, world, rank)
    n = hi - lo
    if n * B * T > 8 * 256 * 2048:
        raise SystemExit("config 5b needs at least 4 ranks: more than 8 heads of it do not fit one GPU's memory "
                         "(pass a smaller B and T to try the script on fewer GPUs)")
    gen = torch.Generator(device=dev).manual_seed(5 + rank)
    wx = torch.randn((B, T, 4, n, D), generator=gen, device=dev, dtype=torch.bfloat16)
    R = torch.randn((4, n, D, D), generator=gen, device=dev) * D ** -0.5
    b = torch.randn((4, n, D), generator=gen, device=dev) * 0.1
    init = torch.randn((2, B, 1, n, D), generator=gen, device=dev) * 0.5
    times = []
    for i in range(warmup + steps):
        leaves = [t.detach().requires_grad_(True) for t in (wx, R, b, init)]
        torch.cuda.synchronize()
        if world > 1:
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
    ms = torch.tensor([sum(times) / len(times)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        t_ms = float(ms.item())
        print(f"| config 5b: lstm N{N} D{D} B{B} T{T}, heads over {world} GPUs ({n} per GPU) | "
              f"{t_ms:.2f} ms per fwd+bwd step (max over ranks) | {B * T / t_ms * 1e3 / 1e6:.1f} M (B*T)/s |")
    if world > 1:
        dist.destroy_process_group()


def time_wide_head(T: int = 512, D: int = 4096, B: int = 32, cell: str = "lstm", steps: int = 3, warmup: int = 1,
                   quiet: bool = False):
    """fwd+bwd of ONE head of D units (LSTM, bf16 Wx) row-sharded over the ranks (1 rank: the same kernels on one GPU).

    Under torchrun one process per GPU; the ranks exchange round(h_t) / round(dG_t) by peer stores inside the
    kernels, no collective. CUDA events around the forward call and around backward (loss = sum(h)), maximum over
    the ranks. Returns a dict (rank 0) with ms and the launch plan."""
    import os

    import torch.distributed as dist

    from flashrnn_b200 import poll_errors
    from flashrnn_b200.wide_head import WideHead

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    own_pg = False
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
        own_pg = True
    head = WideHead(cell, B, T, D, wx_dtype=torch.bfloat16) if world > 1 else \
        WideHead(cell, B, T, D, emulate_ranks=1, device=dev, wx_dtype=torch.bfloat16)
    gr, gw, gb, S = SIZES[cell]
    Dl = D // world
    gen = torch.Generator(device=dev).manual_seed(4 + rank)
    wx = torch.randn((B, T, gw, 1, Dl), generator=gen, device=dev, dtype=torch.bfloat16)
    R = torch.randn((gr, 1, Dl, D), generator=gen, device=dev) * D ** -0.5
    b = torch.randn((gb, 1, Dl), generator=gen, device=dev) * 0.1
    init = torch.randn((S, B, 1, 1, Dl), generator=gen, device=dev) * 0.5
    tf, tb = [], []
    for i in range(warmup + steps):
        leaves = [t.detach().requires_grad_(True) for t in (wx, R, b, init)]
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        hist, _ = head(*leaves)
        e1.record()
        hist[0].sum().backward()
        e2.record()
        e2.synchronize()
        poll_errors(block=True)
        if i >= warmup:
            tf.append(e0.elapsed_time(e1))
            tb.append(e1.elapsed_time(e2))
        del hist, leaves
    ms = torch.tensor([sum(tf) / len(tf), sum(tb) / len(tb)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    plan = head.plan
    out = None
    if rank == 0:
        f, bw = (float(v) for v in ms.tolist())
        out = {"workload": f"{cell} bf16 N1 D{D} B{B} T{T}, rows of R over {world} GPU(s)", "fwd_ms": f, "bwd_ms": bw,
               "fwd_us_per_step": f * 1e3 / T, "bwd_us_per_step": bw * 1e3 / T, "value": B * T / (f + bw) * 1e3,
               "unit": "(B*T)/s",
               "fwd_plan": f"{plan.fwd_ctas} CTAs, K split {plan.fwd_ksplit}, {plan.fwd_k_tmem} weight columns in tensor memory + "
                           f"{plan.fwd_ring_chunks} x 64 in {'resident' if plan.fwd_resident else 'streamed'} shared-memory stages ({plan.fwd_ring_stages})",
               "bwd_plan": f"{plan.bwd_ctas} CTAs, K split {plan.bwd_ksplit}, {plan.bwd_k_tmem} + {plan.bwd_ring_chunks} x 64 "
                           f"{'resident' if plan.bwd_resident else 'streamed'} ({plan.bwd_ring_stages})"}
        if not quiet:
            print(f"| {world} | {T} | {f:.2f} | {bw:.2f} | {f * 1e3 / T:.2f} / {bw * 1e3 / T:.2f} | {out['value'] / 1e3:.1f} k | "
                  f"{out['fwd_plan']} | {out['bwd_plan']} |", flush=True)
    if world > 1:
        dist.barrier()
    head.close()
    if own_pg:
        dist.destroy_process_group()
    return out


def time_projection(reps: int = 20) -> None:
    """The input-projection kernel (x[B*T, I] @ W[J, I].T -> bf16 Wx) through the C ABI on preallocated buffers,
    beside torch.matmul on the same operands; CUDA events around `reps` back-to-back launches."""
    lib = _lib.load()
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream(dev).cuda_stream
    print("| B | T | inputs I | outputs J | ours µs | TFLOP/s | torch.matmul µs | TFLOP/s |")
    print("|---|---|---|---|---|---|---|---|")
    for (B, T, I, J) in ((8, 1024, 768, 3072), (16, 1024, 768, 3072), (64, 1024, 768, 3072), (64, 2048, 1024, 4096),
                         (256, 2048, 512, 2048)):
        g = torch.Generator(device="cpu").manual_seed(3)
        x = torch.randn(B * T, I, generator=g).to(dev).bfloat16()
        w = (torch.randn(J, I, generator=g) * I ** -0.5).to(dev).bfloat16()
        out = torch.empty((B * T, J), dtype=torch.bfloat16, device=dev)
        ref = torch.empty_like(out)
        err = torch.zeros(32, dtype=torch.int32, device=dev)

        def ours():
            _lib.check(lib.frnn_b200_input_projection(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 1, B, T, J, I,
                                                      err.data_ptr(), stream), "input_projection")

        def library():
            torch.matmul(x, w.t(), out=ref)

        def timed(fn) -> float:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            e1.synchronize()
            return e0.elapsed_time(e1) / reps * 1e3

        a, b = timed(ours), timed(library)
        if int(err[0]) != 0 or not torch.allclose(out.float(), ref.float(), atol=3e-2, rtol=2e-2):
            raise RuntimeError(f"projection mismatch at B{B} T{T} I{I} J{J} (err {err[:3].tolist()})")
        fl = 2.0 * B * T * I * J
        print(f"| {B} | {T} | {I} | {J} | {a:.1f} | {fl / a / 1e6:.0f} | {b:.1f} | {fl / b / 1e6:.0f} |", flush=True)


def main(argv) -> None:
    if argv and argv[0] == "projection":
        return time_projection()
    if argv and argv[0] == "wide":  # optionally followed by T, D, B
        time_wide_head(*map(int, argv[1:4]))
        return
    if argv and argv[0] == "config5b":  # optionally followed by B and T (defaults: the configuration's 256 and 2048)
        return time_config5b_sharded(*map(int, argv[1:3]))
    if len(argv) == 5:
        cell, B, T, N, D = argv[0], *map(int, argv[1:])
        r = time_shape(cell, B, T, N, D)
        print(HEADER)
        print(row(cell, B, T, N, D, r))
        print(r)
        return
    shapes = [("lstm", 8, 256, 1, 64), ("lstm", 8, 1024, 3, 256), ("slstm", 16, 2048, 4, 128)]
    for cell in ("lstm", "gru", "elman"):
        shapes += [(cell, 16, 1024, n, d) for d, n in HEAD_DIM_SWEEP]
    shapes += [("lstm", 16, 1024, 1, 1024), ("gru", 16, 1024, 1, 1024), ("lstm", 8, 512, 1, 1536)]  # wider than the sweep
    shapes += [("lstm", 256, 2048, 4, 128)]  # one GPU's share of N32 D128 B256 T2048 with the 32 heads split over 8 GPUs
    from flashrnn_b200.cudnn_baseline import time_cudnn

    print(HEADER_LIB)
    for s in shapes:
        cell, B, T, N, D = s
        lib = time_cudnn(cell, B, T, D) if cell in ("lstm", "gru", "elman") else None
        print(row(*s, time_shape(*s), lib), flush=True)


if __name__ == "__main__":
    main(sys.argv[1:])
