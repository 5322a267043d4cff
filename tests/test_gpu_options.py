"""The v1 configuration options (forward clip, recurrent-gradient clip, recurrent-gradient cut) and the v1 sLSTM
gradient convention, CUDA path against the CPU oracle run with the same options.

The reference implements the three options only inside its CUDA kernels (flashrnn/flashrnn/fused/lstm_fused_pointwise.cuh:
76-81,116-122, flashrnn_fused_backward_cut.cu), which cannot run in the build container, so the oracle's restatement
of them is not pinned by reference outputs; the v1 sLSTM convention is (tests/golden/v1, from flashrnn2/grad_reference.py).
"""

import pytest
import torch

from oracle import recurrence_port as port
from tests import _golden

gpu = pytest.mark.gpu

KEYS = ("history", "carry", "dwx", "dR", "db", "d_initial")


def _run(cell, B, T, N, D, seed, dev, cfg_kwargs, oracle_kwargs, zero=False, h_only=False):
    from flashrnn_b200 import FlashRNNConfig, flashrnn, poll_errors
    from flashrnn_b200.workloads import make_inputs

    wx, R, b, init = make_inputs(cell, B, T, N, D, seed, zero)
    S = port.SIZES[cell][3]
    gen = torch.Generator().manual_seed(seed + 500)
    d_history = torch.randn((S, B, T, N, D), generator=gen)
    d_carry = torch.randn((S, B, 1, N, D), generator=gen)
    if h_only:
        d_history[1:] = 0
        d_carry[1:] = 0
    ref_h, ref_c, ref_g = port.forward_backward(wx, R, b, init, cell, d_history, d_carry, **oracle_kwargs)
    leaves = [t.to(dev).requires_grad_(True) for t in (wx, R, b, init)]
    cfg = FlashRNNConfig(function=cell, backend="b200", dtype="float32", **cfg_kwargs)
    h, c = flashrnn(*leaves, config=cfg)
    ((h * d_history.to(dev)).sum() + (c * d_carry.to(dev)).sum()).backward()
    torch.cuda.synchronize()
    poll_errors(block=True)
    rows = [_golden.report(k, g.detach().cpu(), r) for k, g, r in zip(KEYS, [h, c] + [t.grad for t in leaves], [ref_h, ref_c] + list(ref_g))]
    for r in rows:
        assert r["max_abs"] <= 2e-2 or r["scaled"] <= 1e-2, (cell, D, cfg_kwargs, r)
    return rows, (ref_h, ref_g)


# cluster path, exchange through global memory (1-D backward), contraction split over clusters (column-owning backward)
SHAPES = [("lstm", 8, 14, 2, 128, 301), ("gru", 5, 9, 1, 64, 302), ("elman", 4, 11, 3, 32, 303), ("slstm", 6, 10, 2, 64, 304),
          ("lstm", 4, 6, 1, 640, 305), ("gru", 3, 5, 1, 768, 306)]


@gpu
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}-B{s[1]}-T{s[2]}-N{s[3]}-D{s[4]}")
def test_clip_and_cut_options_match_the_oracle(shape, cuda_device):
    cell, B, T, N, D, seed = shape
    slstm = cell == "slstm"
    _, (plain_h, plain_g) = _run(cell, B, T, N, D, seed, cuda_device, {}, {}, zero=slstm, h_only=slstm)
    # forward clip: small enough to bite (|h| reaches well beyond 0.2 for every cell)
    _, (clip_h, _) = _run(cell, B, T, N, D, seed, cuda_device, dict(forward_clipval=0.2), dict(forward_clipval=0.2),
                         zero=slstm, h_only=slstm)
    assert clip_h[0].abs().max() <= 0.2 and plain_h[0].abs().max() > 0.25
    # gradient clip on the recurrent path: the carried gradients are O(1), so 0.05 changes the result
    _, (_, gclip_g) = _run(cell, B, T, N, D, seed, cuda_device, dict(gradient_recurrent_clipval=0.05),
                           dict(gradient_recurrent_clipval=0.05), zero=slstm, h_only=slstm)
    assert (gclip_g[0] - plain_g[0]).abs().max() > 1e-3
    _, (_, cut_g) = _run(cell, B, T, N, D, seed, cuda_device, dict(gradient_recurrent_cut=True),
                         dict(gradient_recurrent_cut=True), zero=slstm, h_only=slstm)
    assert (cut_g[0] - plain_g[0]).abs().max() > 1e-3
    # everything at once
    _run(cell, B, T, N, D, seed, cuda_device,
         dict(forward_clipval=0.3, gradient_recurrent_clipval=0.1, gradient_recurrent_cut=False),
         dict(forward_clipval=0.3, gradient_recurrent_clipval=0.1), zero=slstm, h_only=slstm)


@gpu
@pytest.mark.parametrize("zero", [True, False], ids=["zero-start", "carried-state"])
def test_v1_slstm_gradient_convention(zero, cuda_device):
    """slstm_gradient='v1': m carries no gradient (d initial m == 0 exactly), the clamp is straight-through; a gradient fed
    into every state, against the oracle under the same convention."""
    rows, _ = _run("slstm", 6, 12, 2, 64, 310, cuda_device, dict(slstm_gradient="v1"), dict(slstm_v1=True), zero=zero)
    from flashrnn_b200 import FlashRNNConfig, flashrnn
    from flashrnn_b200.workloads import make_inputs

    wx, R, b, init = (t.to(cuda_device) for t in make_inputs("slstm", 6, 12, 2, 64, 310, zero))
    init.requires_grad_(True)
    h, c = flashrnn(wx, R, b, init, config=FlashRNNConfig(function="slstm", dtype="float32", slstm_gradient="v1"))
    (h.sum() + c.sum()).backward()
    assert torch.count_nonzero(init.grad[3]) == 0


def test_option_validation():
    from flashrnn_b200 import FlashRNNConfig

    with pytest.raises(ValueError, match="slstm_gradient"):
        FlashRNNConfig(slstm_gradient="v2").options()
    with pytest.raises(ValueError, match="forward_clipval"):
        FlashRNNConfig(forward_clipval=0.0).options()
    assert FlashRNNConfig().options() == (None, None, False, False)
