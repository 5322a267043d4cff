"""On-box GPU library baseline: torch.nn.LSTM / GRU / RNN (cuDNN) for the same recurrence.

Counterpart of the reference's mapper flashrnn/flashrnn2/torch_layer.py:14-77. cuDNN layers own
their input projection and know nothing about block-diagonal heads, so

* ``torch_layer_from`` builds a single-head layer whose input weights are the identity, which makes
  it consume a precomputed ``Wx`` exactly like the recurrence does (used for parity checks), and
* ``time_cudnn`` times an ordinary layer (input size = D, projection included) for one head; a
  model with N heads needs N such layers.

This module is measurement support, not part of the product path.
"""

from __future__ import annotations

import torch

_LAYER = {"lstm": torch.nn.LSTM, "gru": torch.nn.GRU, "elman": torch.nn.RNN}


def torch_layer_from(R: torch.Tensor, b: torch.Tensor, cell: str = "lstm") -> torch.nn.Module:
    """``R[G,1,D,D], b[G,1,D]`` of a single-head lstm / elman -> cuDNN layer fed with ``Wx`` as its input.

    Gate order (i, f, z, o) equals torch's (i, f, g, o). GRU is not mapped: torch applies the reset
    gate after the recurrent bias, the reference before adding its fourth bias (reference.py:84-89).
    """
    if cell not in ("lstm", "elman"):
        raise ValueError("only lstm and elman map onto torch layers one to one")
    G, N, D, _ = R.shape
    if N != 1:
        raise ValueError("cuDNN layers have no block-diagonal heads: pass one head")
    layer = _LAYER[cell](G * D, D, batch_first=True).to(R.device, torch.float32)
    with torch.no_grad():
        layer.weight_ih_l0.copy_(torch.eye(G * D, device=R.device))
        layer.weight_hh_l0.copy_(R[:, 0].reshape(G * D, D))
        layer.bias_ih_l0.copy_(b[:, 0].reshape(G * D))
        layer.bias_hh_l0.zero_()
    layer.flatten_parameters()
    return layer


def time_cudnn(cell: str, B: int, T: int, D: int, reps: int = 5, dtype=torch.bfloat16, device="cuda:0"):
    """(forward ms, forward+backward ms) of one cuDNN layer of hidden size D, loss = sum(h)."""
    layer = _LAYER[cell](D, D, batch_first=True).to(device, dtype)
    layer.flatten_parameters()
    x = torch.randn(B, T, D, device=device, dtype=dtype, requires_grad=True)
    for _ in range(2):
        layer(x)[0].sum().backward()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        layer(x)[0].sum().backward()
    e1.record()
    e1.synchronize()
    fb = e0.elapsed_time(e1) / reps
    with torch.no_grad():
        e0.record()
        for _ in range(reps):
            layer(x)
        e1.record()
        e1.synchronize()
    return e0.elapsed_time(e1) / reps, fb
