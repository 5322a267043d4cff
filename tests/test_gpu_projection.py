"""The input projection kernel (x @ W.T + bias -> Wx in the recurrence's layout) and the projected recurrence."""

import pytest
import torch

from oracle import recurrence_port as port
from tests import _golden

pytestmark = pytest.mark.gpu


# (B, T, I, J): full tiles, ragged rows, K tail, 128- and 64-column tiles
@pytest.mark.parametrize("shape", [(8, 64, 768, 3072), (3, 37, 200, 768), (2, 5, 72, 192), (1, 1, 8, 64), (16, 129, 512, 1152),
                                   # more tiles than SMs: every CTA walks several tiles through both accumulators
                                   (32, 256, 256, 2048), (61, 131, 64, 192)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
def test_projection_matches_matmul(shape, out_dtype, cuda_device):
    from flashrnn_b200 import input_projection, poll_errors

    B, T, I, J = shape
    g = torch.Generator().manual_seed(B * 100 + T)
    x = torch.randn((B, T, I), generator=g).to(cuda_device)
    w = (torch.randn((J, I), generator=g) * I ** -0.5).to(cuda_device)
    bias = torch.randn((J,), generator=g).to(cuda_device)
    for b in (None, bias):
        out = input_projection(x, w, b, out_dtype)
        torch.cuda.synchronize()
        poll_errors(block=True)
        ref = x.bfloat16().float() @ w.bfloat16().float().t() + (0 if b is None else b)   # same rounded operands, fp32 math
        assert out.dtype == out_dtype and out.shape == (B, T, J)
        tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-4   # bf16 output rounding vs summation order only
        assert (out.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item()), shape


@pytest.mark.parametrize("cell", ["lstm", "gru", "slstm"])
def test_projected_recurrence_matches_oracle(cell, cuda_device):
    """x -> Wx by the projection kernel -> recurrence, forward and all gradients (incl. dx, dW, dbias_w) against
    x @ W.T + the CPU oracle on the same bf16-rounded Wx."""
    from flashrnn_b200 import flashrnn_projected, poll_errors
    from flashrnn_b200.workloads import make_inputs

    B, T, N, D, seed = 6, 14, 2, 64, 410
    gr, gw, gb, S = port.SIZES[cell]
    _, R, b, init = make_inputs(cell, B, T, N, D, seed, zero_initial=(cell == "slstm"))
    g = torch.Generator().manual_seed(seed)
    I = N * D
    x = torch.randn((B, T, I), generator=g)
    W = torch.randn((gw * N * D, I), generator=g) * I ** -0.5
    bw = torch.randn((gw * N * D,), generator=g) * 0.1
    # oracle: library-free fp32 matmul of the bf16-rounded operands, Wx rounded to bf16 as the kernel stores it
    xr, Wr = x.bfloat16().float().requires_grad_(True), W.bfloat16().float().requires_grad_(True)
    bwr = bw.clone().requires_grad_(True)
    wx_ref = (xr @ Wr.t() + bwr).view(B, T, gw, N, D)
    wx_seen = wx_ref.detach().bfloat16().float()
    d_history = torch.zeros((S, B, T, N, D))
    d_history[0] = torch.randn((B, T, N, D), generator=g)
    d_carry = torch.zeros((S, B, 1, N, D))
    ref_h, ref_c, (r_dwx, r_dR, r_db, r_dinit) = port.forward_backward(wx_seen, R, b, init, cell, d_history, d_carry)
    wx_ref.backward(r_dwx)   # chain rule through the projection
    leaves = [t.to(cuda_device).requires_grad_(True) for t in (x, W, R, b, init, bw)]
    h, c = flashrnn_projected(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], bias_w=leaves[5], function=cell)
    (h * d_history.to(cuda_device)).sum().backward()
    torch.cuda.synchronize()
    poll_errors(block=True)
    got = dict(history=h, carry=c, dx=leaves[0].grad, dW=leaves[1].grad, dR=leaves[2].grad, db=leaves[3].grad,
               d_initial=leaves[4].grad, dbias_w=leaves[5].grad)
    want = dict(history=ref_h, carry=ref_c, dx=xr.grad, dW=Wr.grad, dR=r_dR, db=r_db, d_initial=r_dinit, dbias_w=bwr.grad)
    for key in got:
        r = _golden.report(key, got[key].detach().float().cpu(), want[key])
        assert r["max_abs"] <= 2e-2 or r["scaled"] <= 1e-2, (cell, r)
