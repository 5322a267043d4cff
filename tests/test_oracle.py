"""The CPU oracle (oracle/recurrence_port.py) against vectors produced by the reference itself."""

import pytest
import torch

from oracle import recurrence_port as port
from tests import _golden


def _run_port(g):
    meta = g["meta"]
    T, n_chunks = meta["T"], meta["n_chunks"]
    step = T // n_chunks
    wx, R, b, initial = g["wx"], g["R"], g["b"], g["initial"]
    # chunked forward, then chunk-by-chunk backward feeding the carry gradient (what autograd does
    # through the reference's carry, tests/flashrnn2/test_torch_backend.py:94-124)
    tapes, hist, carry = [], [], initial
    zero_first = None
    for c in range(n_chunks):
        h, carry, tape = port.forward(wx[:, c * step:(c + 1) * step], R, b, carry, meta["cell"], True, zero_first)
        tapes.append(tape)
        hist.append(h)
    history = torch.cat(hist, dim=2)
    d_carry = g["d_carry"]
    dwx, dR, db = [], 0, 0
    for c in reversed(range(n_chunks)):
        dwx_c, dR_c, db_c, d_carry = port.backward(tapes[c], g["d_history"][:, :, c * step:(c + 1) * step], d_carry)
        dwx.insert(0, dwx_c)
        dR, db = dR + dR_c, db + db_c
    return history, carry, torch.cat(dwx, dim=1), dR, db, d_carry


@pytest.mark.parametrize("name", _golden.CASES)
def test_port_matches_reference_vectors(name):
    torch.set_num_threads(1)
    g = _golden.load(name)
    s = g["meta"]["time_stride"]
    history, carry, dwx, dR, db, d_initial = _run_port(g)
    got = {"history": history[:, :, ::s], "carry": carry, "dwx": dwx[:, ::s], "dR": dR, "db": db, "d_initial": d_initial}
    for key, val in got.items():
        r = _golden.report(key, val, g[key])
        # fp32 on both sides; only summation order inside einsum's backward and an occasional
        # 1-ulp bf16 rounding flip of the R-path gradient separate the two
        assert r["scaled"] < 2e-4 and r["rel_fro"] < 2e-5, (name, r)
    # forward is the same sequence of torch ops: bit-exact
    assert torch.equal(history[:, :, ::s], g["history"]), name
    assert torch.equal(carry, g["carry"]), name


@pytest.mark.parametrize("cell", ["lstm", "slstm", "gru", "elman"])
def test_port_backward_equals_autograd_in_float64(cell):
    """Without the bf16 rounding the explicit BPTT must equal autograd of the port's own forward
    to 1e-11, which pins every derivative formula (incl. the sLSTM stabiliser path)."""
    from flashrnn_b200.workloads import make_inputs

    wx, R, b, initial = (t.double() for t in make_inputs(cell, 3, 7, 2, 8, 5, False))
    leaves = [t.clone().requires_grad_(True) for t in (wx, R, b, initial)]
    hist, carry, _ = port.forward(*leaves, cell, False)
    g = torch.Generator().manual_seed(3)
    d_history = torch.randn(hist.shape, generator=g, dtype=torch.float64)
    d_carry = torch.randn(carry.shape, generator=g, dtype=torch.float64)
    ((hist * d_history).sum() + (carry * d_carry).sum()).backward()
    _, _, grads = port.forward_backward(wx, R, b, initial, cell, d_history, d_carry, bf16_mma=False)
    for got, leaf in zip(grads, leaves):
        assert torch.allclose(got, leaf.grad, rtol=1e-10, atol=1e-11), cell


@pytest.mark.parametrize("name", ["slstm_v1_zero_init", "slstm_v1_nonzero_init"])
def test_port_v1_slstm_convention_matches_reference_vectors(name):
    """The sLSTM gradient convention of the reference's own kernels (m without gradient, normaliser clamp
    straight-through) against float64 vectors from autograd of the reference's flashrnn2/grad_reference.py."""
    import ast

    import numpy as np

    z = np.load(_golden.GOLDEN / "v1" / f"{name}.npz")
    meta = ast.literal_eval(str(z["meta"]))
    assert meta["convention"] == "v1"
    t = {k: torch.from_numpy(z[k]) for k in z.files if k != "meta"}
    history, carry, (dwx, dR, db, d_initial) = port.forward_backward(
        t["wx"], t["R"], t["b"], t["initial"], "slstm", t["d_history"], t["d_carry"], bf16_mma=False, slstm_v1=True)
    for key, got in (("history", history), ("carry", carry), ("dwx", dwx), ("dR", dR), ("db", db), ("d_initial", d_initial)):
        assert torch.allclose(got, t[key], rtol=1e-10, atol=1e-11), (name, key)
    assert torch.count_nonzero(d_initial[3]) == 0   # d(initial m) = 0 under this convention
