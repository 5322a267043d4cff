"""Seeded synthetic inputs for the benchmark configurations.

All tensors are drawn in fp32 on the CPU from ``torch.Generator().manual_seed(seed)`` in the
order Wx, R, b, initial state. Conventions: "N(0, 0.1)" / "N(0, 0.5)" mean standard deviation
0.1 / 0.5; "N(0, 1/D)" means variance 1/D (standard deviation D**-0.5), the reference's own
R / sqrt(D) scaling (flashrnn/tests/utils.py:239-243). The sLSTM forget-gate bias is U(3, 6).
These stand in for the reference's ``torch.randn`` benchmark inputs
(flashrnn/speed_experiments/kernel_speed_benchmark.py:104-127); no dataset is involved.
"""

from __future__ import annotations

import torch

# (recurrent gates, Wx gates, bias gates, states)
SIZES = {"lstm": (4, 4, 4, 2), "slstm": (4, 4, 4, 4), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1)}

# name -> (cell, B, T, N, D, seed, zero_initial)
CONFIGS = {
    "cfg1_lstm_fp32_B8_T256_N1_D64": ("lstm", 8, 256, 1, 64, 0, False),
    "cfg2_lstm_bf16_B8_T1024_N3_D256": ("lstm", 8, 1024, 3, 256, 1, False),
    "cfg3_slstm_bf16_B16_T2048_N4_D128": ("slstm", 16, 2048, 4, 128, 2, True),
}
HEAD_DIM_SWEEP = ((16, 48), (32, 24), (64, 12), (128, 6), (256, 3), (384, 2), (768, 1))  # (D, N), N*D = 768


def make_inputs(cell: str, B: int, T: int, N: int, D: int, seed: int, zero_initial: bool = False):
    """Return fp32 CPU tensors (wx[B,T,GW,N,D], R[GR,N,D,D], b[GB,N,D], initial[S,B,1,N,D])."""
    gr, gw, gb, S = SIZES[cell]
    g = torch.Generator().manual_seed(seed)
    wx = torch.randn((B, T, gw, N, D), generator=g, dtype=torch.float32)
    R = torch.randn((gr, N, D, D), generator=g, dtype=torch.float32) * (D ** -0.5)
    b = torch.randn((gb, N, D), generator=g, dtype=torch.float32) * 0.1
    if cell == "slstm":
        b[1] = torch.rand((N, D), generator=g, dtype=torch.float32) * 3.0 + 3.0
    if zero_initial:
        initial = torch.zeros((S, B, 1, N, D), dtype=torch.float32)
    else:
        initial = torch.randn((S, B, 1, N, D), generator=g, dtype=torch.float32) * 0.5
        if cell == "slstm":
            initial[2] = initial[2].abs() + 1.0  # a normaliser carried over from earlier steps is >= 1
    return wx, R, b, initial


def config_inputs(name: str):
    cell, B, T, N, D, seed, zero = CONFIGS[name]
    return (cell,) + make_inputs(cell, B, T, N, D, seed, zero)
