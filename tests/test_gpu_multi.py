"""Two-GPU check of the sharded call (needs >= 2 visible GPUs; skipped otherwise).

Each rank (one process per GPU, NCCL) runs its batch or head shard through the CUDA kernels with
``flashrnn_sharded``; together the ranks must reproduce the single-GPU result of the whole call,
including the weight gradients that are all-reduced under batch sharding.
"""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port_no, cell, axis, out):
    import torch.distributed as dist

    from flashrnn_b200 import flashrnn, poll_errors, sharding
    from flashrnn_b200.workloads import make_inputs

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, T, N, D = 12, 24, 4, 64
        wx, R, b, init = (t.to(dev) for t in make_inputs(cell, B, T, N, D, 91, zero_initial=(cell == "slstm")))
        if cell == "slstm":
            init[2, B - 1] = 1.5
        zero = sharding.slstm_zero_normalizer(init) if cell == "slstm" else None
        # single-GPU result of the whole call (every rank computes it for comparison)
        full = [t.clone().requires_grad_(True) for t in (wx, R, b, init)]
        h_full, _ = flashrnn(*full, function=cell, backend="b200", dtype="float32")
        h_full[0].sum().backward()
        swx, sR, sb, sinit, axis = sharding.shard_inputs(wx, R, b, init, world, rank, axis)
        leaves = [t.clone().contiguous().requires_grad_(True) for t in (swx, sR, sb, sinit)]
        h, _ = sharding.flashrnn_sharded(*leaves, function=cell, dtype="float32", axis=axis, zero_normalizer=zero)
        h[0].sum().backward()
        torch.cuda.synchronize()
        poll_errors(block=True)
        if axis == "batch":
            lo, hi = sharding.shard_range(B, world, rank)
            ok = torch.equal(h, h_full[:, lo:hi].detach()) and torch.equal(leaves[0].grad, full[0].grad[lo:hi])
            scale = full[1].grad.abs().max().item()
            ok &= (leaves[1].grad - full[1].grad).abs().max().item() <= 1e-3 * scale     # summation order differs
            ok &= torch.allclose(leaves[2].grad, full[2].grad, rtol=1e-4, atol=1e-3)
        else:
            lo, hi = sharding.shard_range(N, world, rank)
            ok = torch.equal(h, h_full[:, :, :, lo:hi].detach())
            ok &= torch.equal(leaves[1].grad, full[1].grad[:, lo:hi]) and torch.equal(leaves[2].grad, full[2].grad[:, lo:hi])
        out.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cell,axis", [("lstm", "batch"), ("slstm", "batch"), ("gru", "heads")])
def test_two_gpu_shards_reproduce_single_gpu_call(cell, axis):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port_no = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port_no, cell, axis, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(ok for _, ok in results), results
