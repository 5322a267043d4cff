"""World-size-2 check of the multi-GPU host logic on CPU ranks (gloo).

Each rank takes its shard of one logical call, runs the CPU oracle on it as a stand-in for the
kernels, all-reduces dR/db where the sharding axis needs it, and must reproduce the unsharded
result — including the sLSTM first-step predicate, which has to come from the unsharded state.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashrnn_b200 import sharding
from flashrnn_b200.workloads import make_inputs
from oracle import recurrence_port as port


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port_no, cell, axis, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    try:
        B, T, N, D = 6, 5, 2, 8
        wx, R, b, initial = make_inputs(cell, B, T, N, D, 77, zero_initial=(cell == "slstm"))
        if cell == "slstm":
            initial[2, B - 1] = 1.5   # only the LAST batch row has a non-zero normaliser
        S = port.SIZES[cell][3]
        g = torch.Generator().manual_seed(5)
        d_hist = torch.randn((S, B, T, N, D), generator=g)
        d_carry = torch.randn((S, B, 1, N, D), generator=g)
        full_h, full_c, (f_dwx, f_dR, f_db, f_dinit) = port.forward_backward(wx, R, b, initial, cell, d_hist, d_carry)
        zero = sharding.slstm_zero_normalizer(initial) if cell == "slstm" else None
        swx, sR, sb, sinit, axis = sharding.shard_inputs(wx, R, b, initial, world, rank, axis)
        if axis == "heads":
            lo, hi = sharding.shard_range(N, world, rank)
            sdh, sdc = d_hist[:, :, :, lo:hi], d_carry[:, :, :, lo:hi]
        else:
            lo, hi = sharding.shard_range(B, world, rank)
            sdh, sdc = d_hist[:, lo:hi], d_carry[:, lo:hi]
        h, c, (dwx, dR, db, dinit) = port.forward_backward(swx, sR, sb, sinit, cell, sdh, sdc, zero_first=zero)
        sharding.allreduce_weight_grads(dR, db, axis)
        ok = True
        if axis == "heads":
            ok &= torch.allclose(h, full_h[:, :, :, lo:hi], atol=1e-5) and torch.allclose(dwx, f_dwx[:, :, :, lo:hi], atol=1e-5)
            ok &= torch.allclose(dR, f_dR[:, lo:hi], atol=1e-5) and torch.allclose(db, f_db[:, lo:hi], atol=1e-5)
        else:
            ok &= torch.allclose(h, full_h[:, lo:hi], atol=1e-5) and torch.allclose(c, full_c[:, lo:hi], atol=1e-5)
            ok &= torch.allclose(dwx, f_dwx[lo:hi], atol=1e-6) and torch.allclose(dinit, f_dinit[:, lo:hi], atol=1e-6)
            ok &= torch.allclose(dR, f_dR, rtol=1e-2, atol=2e-2) and torch.allclose(db, f_db, rtol=1e-4, atol=1e-4)
        wrong = None
        if cell == "slstm" and axis == "batch" and rank == 0:
            # a shard that evaluates the predicate locally (all its n are zero) gets a different answer
            h_bad, _, _ = port.forward(swx, sR, sb, sinit, cell)
            wrong = bool((h_bad - full_h[:, lo:hi]).abs().max() > 1e-3)
        out.put((rank, bool(ok), wrong))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cell,axis", [("lstm", "batch"), ("lstm", "heads"), ("slstm", "batch"), ("gru", "batch")])
def test_two_rank_shards_reproduce_the_unsharded_call(cell, axis):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port_no = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port_no, cell, axis, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results
    if cell == "slstm":
        assert any(w for _, _, w in results if w is not None), "a local predicate must change the result"


def test_shard_range_and_axis():
    assert [sharding.shard_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sharding.choose_axis(256, 32, 8) == "heads" and sharding.choose_axis(8, 3, 2) == "batch"
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def test_sharded_call_wants_the_axis_and_a_cuda_device():
    import torch

    from flashrnn_b200 import sharding
    from flashrnn_b200.workloads import make_inputs

    wx, R, b, init = make_inputs("lstm", 2, 3, 2, 16, 5)
    with pytest.raises(ValueError, match="axis"):
        sharding.flashrnn_sharded(wx, R, b, init, function="lstm")
    with pytest.raises(ValueError, match="axis"):
        sharding.flashrnn_sharded(wx, R, b, init, function="lstm", axis="time")
    with pytest.raises(RuntimeError, match="CUDA"):     # there is no CPU path behind the sharded call either
        sharding.flashrnn_sharded(wx, R, b, init, function="lstm", axis="heads", dtype="float32")
