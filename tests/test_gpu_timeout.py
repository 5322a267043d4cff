"""Failure path on the GPU: a wait that nothing satisfies runs out, the kernel reports it and the
context stays usable. The stall is requested from the host (err[4] = 1: the CTAs stop publishing
their per-step exchange data); every in-kernel wait is bounded, nothing traps or spins forever."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(_lib, cell, B, T, N, D, dev):
    from flashrnn_b200.workloads import SIZES, make_inputs

    gr, gw, gb, S = SIZES[cell]
    plan = _lib.plan(cell, B, T, N, D)
    wx, R, b, init = make_inputs(cell, B, T, N, D, 9)
    t = dict(wx=wx.to(dev).contiguous(), R=R.to(dev).bfloat16().contiguous(), b=b.to(dev), init=init.to(dev),
             hist=torch.zeros((S, B, T, N, D), device=dev), carry=torch.zeros((S, B, 1, N, D), device=dev),
             cache=torch.zeros(plan.cache_bytes, dtype=torch.uint8, device=dev),
             hbf=torch.zeros(plan.hbf_bytes // 2, dtype=torch.bfloat16, device=dev),
             dwx=torch.zeros((B, T, gw, N, D), device=dev), dgr=torch.zeros(plan.dgr_bytes // 2, dtype=torch.bfloat16, device=dev),
             dinit=torch.zeros((S, B, 1, N, D), device=dev), dbp=torch.zeros(plan.dbpart_bytes // 4, device=dev),
             xchg=torch.zeros(max(plan.xchg_bytes, 16), dtype=torch.uint8, device=dev))
    t["xchg_ptr"] = t["xchg"].data_ptr() if plan.exchange else None
    t["dH"] = torch.ones_like(t["hist"])
    t["dC"] = torch.zeros_like(t["carry"])
    return t


def _forward(lib, _lib, cell, B, T, N, D, t, err, limit_ms):
    return lib.frnn_b200_forward(_lib.CELLS[cell], t["wx"].data_ptr(), 0, t["R"].data_ptr(), t["b"].data_ptr(),
                                 t["init"].data_ptr(), t["hist"].data_ptr(), t["carry"].data_ptr(), t["cache"].data_ptr(),
                                 t["hbf"].data_ptr(), t["xchg_ptr"], B, T, N, D, 0, limit_ms, err.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)


def _backward(lib, _lib, cell, B, T, N, D, t, err, limit_ms):
    return lib.frnn_b200_backward(_lib.CELLS[cell], t["cache"].data_ptr(), t["hist"].data_ptr(), t["init"].data_ptr(),
                                  t["R"].data_ptr(), t["dH"].data_ptr(), t["dC"].data_ptr(), t["dwx"].data_ptr(), 0,
                                  t["dgr"].data_ptr(), t["dinit"].data_ptr(), t["dbp"].data_ptr(), t["xchg_ptr"], B, T, N, D, 0,
                                  limit_ms, err.data_ptr(), torch.cuda.current_stream().cuda_stream)


# one shape that exchanges inside a thread-block cluster, one that exchanges through global memory
@pytest.mark.parametrize("shape", [("lstm", 8, 24, 2, 128), ("lstm", 4, 12, 1, 576), ("lstm", 4, 12, 1, 768),
                                   ("lstm", 64, 12, 1, 768)],
                         ids=["cluster", "global", "global-ksplit", "global-1d"])
def test_stalled_exchange_is_reported_and_context_survives(shape, cuda_device):
    from flashrnn_b200 import _lib

    lib = _lib.load()
    cell, B, T, N, D = shape
    t = _buffers(_lib, cell, B, T, N, D, cuda_device)
    err = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    assert _forward(lib, _lib, cell, B, T, N, D, t, err, 0) == 0
    torch.cuda.synchronize()
    assert err[0].item() == 0
    good = t["hist"].clone()

    # forward: nobody publishes h from step 5 on -> the operand wait of step 6 runs out after 20 ms
    err.zero_()
    err[4], err[5] = 1, 5
    assert _forward(lib, _lib, cell, B, T, N, D, t, err, 20) == 0
    torch.cuda.synchronize()
    code, step = err[0].item(), err[1].item()
    print('forward stall reported', code, step, flush=True)
    assert code == 101 and step == 6, (code, step)

    # the context is intact: the same call without the stall reproduces the first result bit for bit
    err.zero_()
    assert _forward(lib, _lib, cell, B, T, N, D, t, err, 0) == 0
    torch.cuda.synchronize()
    assert err[0].item() == 0 and torch.equal(t["hist"], good)
    print('forward after stall ok', flush=True)

    # backward: no partial dh is scattered from iteration 3 on
    assert _backward(lib, _lib, cell, B, T, N, D, t, err, 0) == 0
    torch.cuda.synchronize()
    assert err[0].item() == 0
    good_dwx = t["dwx"].clone()
    err.zero_()
    err[4], err[5] = 1, 3
    assert _backward(lib, _lib, cell, B, T, N, D, t, err, 20) == 0
    torch.cuda.synchronize()
    print('backward stall reported', err[:3].tolist(), flush=True)
    # the epilogue (106, partial dh) and the MMA warp behind it (107, dg operand) wait with the same limit
    assert err[0].item() in (106, 107), err[:3].tolist()
    err.zero_()
    assert _backward(lib, _lib, cell, B, T, N, D, t, err, 0) == 0
    torch.cuda.synchronize()
    assert err[0].item() == 0 and torch.equal(t["dwx"], good_dwx)


def test_python_layer_raises_on_device_error(cuda_device):
    from flashrnn_b200 import functional

    err = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    err[0], err[1], err[2] = 101, 7, 3
    functional._track(err, "frnn_b200_forward")
    with pytest.raises(RuntimeError, match="code 101.*step 7, CTA 3"):
        functional.poll_errors(block=True)
    functional.poll_errors(block=True)  # the queue is drained
