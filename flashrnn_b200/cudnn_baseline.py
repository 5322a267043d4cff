"""On-box GPU library baseline: torch.nn.LSTM / GRU / RNN (cuDNN) for the same recurrence.

Counterpart of the reference's mapper flashrnn/flashrnn2/torch_layer.py:14-77. cuDNN layers own
their input projection and know nothing about block-diagonal heads, so

* ``torch_layer_from`` builds a single-head layer whose input weights are the identity, which makes
  it consume a precomputed ``Wx`` exactly like the recurrence does (used for parity checks),
* ``time_cudnn`` times an ordinary layer (input size = D, projection included) for one head; a
  model with N heads needs N such layers, and
* ``paired_times`` / ``compare_with_cudnn`` time two arms in alternating ABBA / BAAB blocks
  (the reference's paired protocol, tools/bw_bench.py:1-17).

This module is measurement support, not part of the product path.
"""

from __future__ import annotations

import torch

_LAYER = {"lstm": torch.nn.LSTM, "gru": torch.nn.GRU, "elman": torch.nn.RNN}


def torch_layer_from(R: torch.Tensor, b: torch.Tensor, cell: str = "lstm") -> torch.nn.Module:
    """``R[GR,1,D,D], b[GB,1,D]`` of a single-head lstm / gru / elman -> cuDNN layer fed with ``Wx`` as its input.

    LSTM / Elman: gate order (i, f, z, o) equals torch's (i, f, g, o); all biases go to ``bias_ih``.
    GRU (the reference maps it the same way, flashrnn/flashrnn2/torch_layer.py:43,50-52): torch orders its gates
    (reset, update, new) and computes ``new = tanh(x_n + b_in + r * (W_hn h + b_hn))``, which is this library's
    ``v = tanh(x_2 + b_3 + r * (R_0 h + b_0))``. So the recurrent blocks go in as (R_1, R_2, R_0), the input-side
    biases as (b_1, b_2, b_3), and b_0 is the recurrent bias of the third block; Wx's gates (reset, update,
    candidate input) already are in torch's order.
    """
    if cell not in _LAYER:
        raise ValueError("lstm, gru and elman map onto torch layers; slstm has no library counterpart")
    GR, N, D, _ = R.shape
    if N != 1:
        raise ValueError("cuDNN layers have no block-diagonal heads: pass one head")
    layer = _LAYER[cell](GR * D, D, batch_first=True).to(R.device, torch.float32)
    with torch.no_grad():
        layer.weight_ih_l0.copy_(torch.eye(GR * D, device=R.device))
        layer.bias_hh_l0.zero_()
        if cell == "gru":
            layer.weight_hh_l0.copy_(torch.cat((R[1, 0], R[2, 0], R[0, 0]), dim=0))
            layer.bias_ih_l0.copy_(torch.cat((b[1, 0], b[2, 0], b[3, 0]), dim=0))
            layer.bias_hh_l0[2 * D:].copy_(b[0, 0])
        else:
            layer.weight_hh_l0.copy_(R[:, 0].reshape(GR * D, D))
            layer.bias_ih_l0.copy_(b[:, 0].reshape(GR * D))
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


def paired_times(step_a, step_b, blocks: int = 10, device="cuda:0"):
    """Paired timing of two step functions in alternating ABBA / BAAB blocks (the reference's protocol for
    comparing two arms, tools/bw_bench.py:1-17): both arms see the same clocks and thermal state, and drift
    cancels inside a block. Each call is bracketed by its own CUDA events on the current stream.

    Returns ``{"a_ms": median, "b_ms": median, "ratio_b_over_a": median of per-block ratios, "blocks": n}``.
    """
    import statistics

    def once(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1)

    with torch.cuda.device(device):
        for fn in (step_a, step_b, step_a, step_b):  # warm-up, both arms
            fn()
        torch.cuda.synchronize()
        a_all, b_all, ratios = [], [], []
        for i in range(blocks):
            order = "ABBA" if i % 2 == 0 else "BAAB"
            t = {"A": [], "B": []}
            for arm in order:
                t[arm].append(once(step_a if arm == "A" else step_b))
            a, b = sum(t["A"]) / 2, sum(t["B"]) / 2
            a_all.append(a)
            b_all.append(b)
            ratios.append(b / a)
    return {"a_ms": statistics.median(a_all), "b_ms": statistics.median(b_all),
            "ratio_b_over_a": statistics.median(ratios), "blocks": blocks}


def compare_with_cudnn(cell: str, B: int, T: int, D: int, blocks: int = 10, device="cuda:0"):
    """Paired fwd+bwd timing of this library (one head, bf16 Wx precomputed) against one cuDNN layer of the same
    hidden size (bf16, input projection of size D included, as the layer cannot be fed a precomputed Wx at
    speed). Loss = sum(h) on both arms."""
    from .functional import flashrnn
    from .workloads import make_inputs

    wx, R, b, init = (t.to(device) for t in make_inputs(cell, B, T, 1, D, 3))
    wx = wx.bfloat16()
    layer = _LAYER[cell](D, D, batch_first=True).to(device, torch.bfloat16)
    layer.flatten_parameters()
    x = torch.randn(B, T, D, device=device, dtype=torch.bfloat16, requires_grad=True)

    def ours():
        leaves = [t.detach().requires_grad_(True) for t in (wx, R, b, init)]
        hist, _ = flashrnn(*leaves, function=cell, backend="b200", dtype="bfloat16")
        hist[0].sum().backward()

    def lib():
        layer.zero_grad(set_to_none=True)
        layer(x)[0].sum().backward()

    out = paired_times(ours, lib, blocks, device)
    out.update(cell=cell, B=B, T=T, D=D, a="flashrnn_b200", b="torch.nn (cuDNN)")
    return out
