"""Parity of the CUDA path (through the C ABI) with the reference vectors and the CPU oracle.

Tolerance (the north star's): max-abs 2e-2 for O(1) tensors; tensors whose magnitude is large
(dR, db, sLSTM c/n) are judged by the error normalised by max|ref| <= 1e-2, the reference's own
convention (tools/bw_qualify.py:12-17).
"""

import pytest
import torch

from oracle import recurrence_port as port
from tests import _golden

pytestmark = pytest.mark.gpu

ATOL, RTOL_SCALED = 2e-2, 1e-2
BF16_MMA = "fp32_state_bf16_mma"  # the only numerical policy of this backend; the reference's default "mathematical" is rejected


def _check(name, key, got, ref, log):
    r = _golden.report(key, got.detach().cpu().float(), ref)
    log.append(r)
    assert r["max_abs"] <= ATOL or r["scaled"] <= RTOL_SCALED, (name, r)
    assert torch.isfinite(got).all(), (name, key)


def _run_gpu(g, dev, dtype=torch.float32):
    from flashrnn_b200 import flashrnn_torch, poll_errors

    meta = g["meta"]
    T, n_chunks = meta["T"], meta["n_chunks"]
    step = T // n_chunks
    leaves = [g[k].to(dev).to(dtype).requires_grad_(True) for k in ("wx", "R", "b", "initial")]
    wx, R, b, carry = leaves
    pieces = []
    for c in range(n_chunks):
        h, carry = flashrnn_torch(wx[:, c * step:(c + 1) * step], R, b, carry, cell=meta["cell"],
                                  numerics="fp32_state_bf16_mma")
        pieces.append(h)
    history = torch.cat(pieces, dim=2)
    loss = (history * g["d_history"].to(dev)).sum() + (carry * g["d_carry"].to(dev)).sum()
    loss.backward()
    torch.cuda.synchronize()
    poll_errors(block=True)
    return history, carry, [t.grad for t in leaves]


@pytest.mark.parametrize("name", _golden.CASES)
def test_cuda_matches_reference_vectors(name, cuda_device):
    g = _golden.load(name)
    s = g["meta"]["time_stride"]
    history, carry, (dwx, dR, db, dinit) = _run_gpu(g, cuda_device)
    log = []
    assert history.dtype == torch.float32 and carry.dtype == torch.float32
    _check(name, "history", history[:, :, ::s], g["history"], log)
    _check(name, "carry", carry, g["carry"], log)
    _check(name, "dwx", dwx[:, ::s], g["dwx"], log)
    _check(name, "dR", dR, g["dR"], log)
    _check(name, "db", db, g["db"], log)
    _check(name, "d_initial", dinit, g["d_initial"], log)
    print(name, [(r["name"], f"{r['max_abs']:.2e}", f"{r['scaled']:.2e}") for r in log])


# (cell, B, T, N, D, seed, zero_initial): shapes that exercise every launch plan
SHAPES = [
    ("lstm", 8, 48, 3, 256, 21, False),    # headline geometry: cluster of 8, batch tile 8
    ("lstm", 16, 20, 2, 128, 22, False),   # two 8-row tiles per head (16-row tiles: tests/test_gpu_full_length.py)
    ("lstm", 20, 12, 1, 64, 23, False),    # two batch tiles, the second ragged (4 rows)
    ("lstm", 3, 17, 2, 48, 24, False),     # unit 16, cluster of 3, ragged batch
    ("lstm", 4, 10, 1, 384, 25, False),    # cluster of 12 (non-portable size)
    ("lstm", 2, 6, 1, 512, 26, False),     # cluster of 16
    ("slstm", 16, 40, 4, 128, 27, True),   # sLSTM geometry of the third config
    ("slstm", 5, 16, 2, 64, 28, False),
    ("gru", 16, 24, 1, 256, 29, False),
    ("gru", 6, 9, 3, 32, 30, False),
    ("elman", 16, 30, 2, 128, 31, False),
    ("elman", 1, 1, 1, 16, 32, False),     # single step, single row
    ("lstm", 16, 12, 1, 768, 35, False),   # 24 CTAs per head: exchange through global memory
    ("gru", 8, 7, 2, 576, 36, False),      # two such groups side by side
    ("slstm", 4, 5, 1, 768, 37, True),
    ("elman", 3, 9, 1, 640, 38, False),
    ("lstm", 8, 10, 1, 1024, 42, False),   # rows of R beyond one CTA's tensor memory: contraction split over two CTAs
    ("gru", 4, 6, 1, 1280, 43, False),
    ("slstm", 3, 5, 1, 1024, 44, True),
    ("elman", 5, 7, 1, 1792, 45, False),
    ("lstm", 24, 5, 1, 1024, 46, False),   # the same with 16-row batch tiles
    ("lstm", 4, 6, 1, 1536, 47, False),    # 96 CTAs per group: 12 unit tiles x 8 K-chunks in the backward
    ("lstm", 6, 7, 1, 608, 48, False),     # not a multiple of 128: split forward, 1-D backward through global memory
    ("lstm", 64, 3, 1, 768, 51, False),    # four 16-row groups: the split forward does not fit, one CTA per 32 units
    ("gru", 33, 3, 1, 960, 52, False),     # three gates: the widest head of the one-CTA-per-32-units kernels (30 CTAs per group)
    ("gru", 9, 5, 1, 736, 49, False),
    ("lstm", 5, 6, 1, 960, 50, False),     # not a multiple of 128: split forward, 1-D backward with 16-unit slices
    ("gru", 3, 4, 1, 1000, 53, False),     # odd wide width: padded to 1024 by the Python layer
    ("lstm", 2, 3, 1, 777, 54, False),     # padded to 832
    ("lstm", 1, 1, 1, 3, 33, False),       # the reference's smallest portable-gate shape
    ("gru", 3, 3, 2, 7, 34, False),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}-B{s[1]}-T{s[2]}-N{s[3]}-D{s[4]}")
def test_cuda_matches_oracle(shape, cuda_device):
    from flashrnn_b200.workloads import make_inputs

    cell, B, T, N, D, seed, zero = shape
    wx, R, b, initial = make_inputs(cell, B, T, N, D, seed, zero)
    gen = torch.Generator().manual_seed(seed + 500)
    S = port.SIZES[cell][3]
    d_history = torch.randn((S, B, T, N, D), generator=gen)
    d_carry = torch.randn((S, B, 1, N, D), generator=gen)
    ref_h, ref_c, (r_dwx, r_dR, r_db, r_dinit) = port.forward_backward(wx, R, b, initial, cell, d_history, d_carry)
    g = dict(meta=dict(cell=cell, T=T, n_chunks=1), wx=wx, R=R, b=b, initial=initial, d_history=d_history, d_carry=d_carry)
    history, carry, (dwx, dR, db, dinit) = _run_gpu(g, cuda_device)
    log = []
    name = str(shape)
    _check(name, "history", history, ref_h, log)
    _check(name, "carry", carry, ref_c, log)
    _check(name, "dwx", dwx, r_dwx, log)
    _check(name, "dR", dR, r_dR, log)
    _check(name, "db", db, r_db, log)
    _check(name, "d_initial", dinit, r_dinit, log)
    print(name, [(r["name"], f"{r['max_abs']:.2e}", f"{r['scaled']:.2e}") for r in log])


def test_carry_continuation_is_exact(cuda_device):
    """Two chunks with the carry passed on reproduce the single call bit for bit (fp32 carry)."""
    from flashrnn_b200 import flashrnn_torch
    from flashrnn_b200.workloads import make_inputs

    for cell in ("lstm", "slstm", "gru", "elman"):
        wx, R, b, initial = (t.to(cuda_device) for t in make_inputs(cell, 8, 32, 2, 64, 40, cell == "slstm"))
        full, full_c = flashrnn_torch(wx, R, b, initial, cell=cell, numerics=BF16_MMA)
        h1, c1 = flashrnn_torch(wx[:, :13], R, b, initial, cell=cell, numerics=BF16_MMA)
        h2, c2 = flashrnn_torch(wx[:, 13:], R, b, c1, cell=cell, numerics=BF16_MMA)
        assert torch.equal(torch.cat((h1, h2), dim=2), full), cell
        assert torch.equal(c2, full_c), cell
        assert torch.equal(full[:, :, -1:], full_c), cell


def test_bf16_inputs_and_flashrnn_entry(cuda_device):
    """flashrnn(..., dtype='bfloat16') == flashrnn_torch on the pre-rounded inputs; states=None is zeros."""
    from flashrnn_b200 import flashrnn, flashrnn_torch
    from flashrnn_b200.workloads import make_inputs

    wx, R, b, initial = (t.to(cuda_device) for t in make_inputs("lstm", 8, 16, 3, 256, 41, True))
    h_a, c_a = flashrnn(wx, R, b, None, function="lstm", backend="b200", dtype="bfloat16")
    h_b, c_b = flashrnn_torch(wx.bfloat16().float(), R, b, initial, cell="lstm", numerics=BF16_MMA)
    assert h_a.shape == (2, 8, 16, 3, 256) and c_a.shape == (2, 8, 1, 3, 256)
    assert torch.equal(h_a, h_b) and torch.equal(c_a, c_b)
    with pytest.raises(ValueError):
        flashrnn(wx, R, b, None, function="lstm", backend="cuda_fused")


@pytest.mark.parametrize("cell", ["lstm", "gru", "elman"])
def test_matches_cudnn_layer(cell, cuda_device):
    """Single head against torch.nn.LSTM / GRU / RNN (cuDNN, fp32) fed with the same precomputed Wx."""
    from flashrnn_b200 import flashrnn_torch
    from flashrnn_b200.cudnn_baseline import torch_layer_from
    from flashrnn_b200.workloads import make_inputs

    B, T, D = 4, 12, 64
    wx, R, b, initial = (t.to(cuda_device) for t in make_inputs(cell, B, T, 1, D, 61))
    hist, carry = flashrnn_torch(wx, R, b, initial, cell=cell, numerics=BF16_MMA)
    layer = torch_layer_from(R, b, cell)
    h0 = initial[0, :, 0, 0].unsqueeze(0).contiguous()
    state = (h0, initial[1, :, 0, 0].unsqueeze(0).contiguous()) if cell == "lstm" else h0
    with torch.backends.cudnn.flags(enabled=True, allow_tf32=False):
        out, _ = layer(wx[:, :, :, 0].reshape(B, T, -1), state)
    assert (hist[0, :, :, 0] - out).abs().max().item() <= 2e-2   # bf16 R / h operands vs fp32 cuDNN


def test_bf16_stream_backward_matches_oracle_on_rounded_inputs(cuda_device):
    """Wx given in bf16 (as config 2 prescribes): all gradients against the oracle run on the same rounded Wx."""
    from flashrnn_b200 import flashrnn
    from flashrnn_b200.workloads import make_inputs

    cell, B, T, N, D = "lstm", 8, 40, 3, 256
    wx, R, b, initial = make_inputs(cell, B, T, N, D, 81)
    wx_r = wx.bfloat16().float()
    d_history = torch.zeros((2, B, T, N, D))
    d_history[0] = 1.0
    ref_h, _, (r_dwx, r_dR, r_db, r_dinit) = port.forward_backward(wx_r, R, b, initial, cell, d_history,
                                                                    torch.zeros((2, B, 1, N, D)))
    leaves = [t.to(cuda_device).requires_grad_(True) for t in (wx.bfloat16(), R, b, initial)]
    hist, _ = flashrnn(*leaves, function=cell, backend="b200", dtype="bfloat16")
    hist[0].sum().backward()
    assert leaves[0].grad.dtype == torch.bfloat16 and leaves[1].grad.dtype == torch.float32
    log = []
    _check("bf16", "history", hist, ref_h, log)
    _check("bf16", "dwx", leaves[0].grad.float(), r_dwx, log)
    _check("bf16", "dR", leaves[1].grad, r_dR, log)
    _check("bf16", "db", leaves[2].grad, r_db, log)
    _check("bf16", "d_initial", leaves[3].grad, r_dinit, log)


def test_repeatable_views_and_read_only_inputs(cuda_device):
    """Same call twice is bit-identical (no atomics anywhere); strided views are accepted; inputs are not written."""
    from flashrnn_b200 import flashrnn_torch
    from flashrnn_b200.workloads import make_inputs

    cell, B, T, N, D = "slstm", 6, 21, 2, 64
    wx, R, b, initial = (t.to(cuda_device) for t in make_inputs(cell, B, T, N, D, 82))
    wx_view = wx.transpose(0, 1).contiguous().transpose(0, 1)          # same values, different strides
    copies = [t.clone() for t in (wx_view, R, b, initial)]
    outs = []
    for _ in range(2):
        leaves = [t.detach().requires_grad_(True) for t in (wx_view, R, b, initial)]
        h, c = flashrnn_torch(*leaves, cell=cell, numerics=BF16_MMA)
        (h.square().sum() + c.sum()).backward()
        outs.append([h.detach(), c.detach()] + [t.grad for t in leaves])
    for a, bb in zip(*outs):
        assert torch.equal(a, bb)
    assert not wx_view.is_contiguous()
    for t, c in zip((wx_view, R, b, initial), copies):
        assert torch.equal(t, c)
    h_ref, _ = flashrnn_torch(wx, R, b, initial, cell=cell, numerics=BF16_MMA)
    assert torch.equal(h_ref, outs[0][0])


def test_random_shapes_with_a_loss_on_the_hidden_state(cuda_device):
    """Thirty seeded random shapes over all cells, widths 16 ... 1536 and ragged batches; the gradient enters through
    h only (what a loss on the hidden state gives; gradients fed into sLSTM's normaliser state meet the clamp's
    discontinuity and are covered by the fixed shapes above)."""
    import random

    from flashrnn_b200 import _lib, flashrnn_torch, poll_errors
    from flashrnn_b200.workloads import make_inputs

    rng = random.Random(20261125)
    widths = [16, 32, 48, 64, 96, 128, 192, 256, 320, 384, 448, 512, 576, 608, 640, 704, 768, 832, 896, 960, 1024, 1152,
              1280, 1408, 1536]
    done = 0
    while done < 30:
        cell = rng.choice(["lstm", "gru", "elman", "slstm"])
        D = rng.choice(widths)
        B = rng.choice([1, 2, 3, 5, 8, 9, 13, 16, 17, 24])
        N = rng.choice([1, 1, 2, 3]) if D <= 512 else 1
        T = rng.choice([1, 2, 3, 5, 8, 11])
        if not _lib.plan(cell, B, T, N, D).supported:
            continue
        done += 1
        zero = cell == "slstm" and rng.random() < 0.5
        wx, R, b, initial = make_inputs(cell, B, T, N, D, 3000 + done, zero)
        S = port.SIZES[cell][3]
        gen = torch.Generator().manual_seed(done)
        d_history = torch.zeros((S, B, T, N, D))
        d_history[0] = torch.randn((B, T, N, D), generator=gen)
        d_carry = torch.zeros((S, B, 1, N, D))
        d_carry[0] = torch.randn((B, 1, N, D), generator=gen)
        ref_h, ref_c, ref_g = port.forward_backward(wx, R, b, initial, cell, d_history, d_carry)
        leaves = [t.to(cuda_device).requires_grad_(True) for t in (wx, R, b, initial)]
        h, c = flashrnn_torch(*leaves, cell=cell, numerics=BF16_MMA)
        ((h * d_history.to(cuda_device)).sum() + (c * d_carry.to(cuda_device)).sum()).backward()
        torch.cuda.synchronize()
        poll_errors(block=True)
        log = []
        name = f"{cell}-B{B}-T{T}-N{N}-D{D}"
        for key, got, ref in zip(("history", "carry", "dwx", "dR", "db", "d_initial"), [h, c] + [t.grad for t in leaves],
                                 [ref_h, ref_c] + list(ref_g)):
            _check(name, key, got, ref, log)


def test_wide_head_batch_larger_than_one_launch(cuda_device):
    """LSTM D=1024 with 40 batch rows: more than the resident CTAs of one launch can take, so the host runs
    two launches; forward and all gradients (dR/db summed over the launches by autograd) against the oracle."""
    from flashrnn_b200 import functional
    from flashrnn_b200.workloads import make_inputs

    cell, B, T, N, D = "lstm", 40, 4, 1, 1024
    assert functional._launch_split(cell, B, T, N, D)[1] < B
    wx, R, b, initial = make_inputs(cell, B, T, N, D, 91)
    gen = torch.Generator().manual_seed(92)
    d_history = torch.randn((2, B, T, N, D), generator=gen)
    d_carry = torch.randn((2, B, 1, N, D), generator=gen)
    ref_h, ref_c, ref_g = port.forward_backward(wx, R, b, initial, cell, d_history, d_carry)
    g = dict(meta=dict(cell=cell, T=T, n_chunks=1), wx=wx, R=R, b=b, initial=initial, d_history=d_history, d_carry=d_carry)
    history, carry, grads = _run_gpu(g, cuda_device)
    log = []
    for key, got, ref in zip(("history", "carry", "dwx", "dR", "db", "d_initial"), [history, carry] + list(grads),
                             [ref_h, ref_c] + list(ref_g)):
        _check("split", key, got, ref, log)



@pytest.mark.parametrize("cell", ["lstm", "gru"])
def test_wide_head_bf16_stream_backward(cell, cuda_device):
    """bf16 Wx on a head that runs the column-owning backward (D = 768): dWx comes back in bf16 through the packet
    path (shared with dgr for the LSTM, separate for the GRU); all gradients against the oracle on the rounded Wx."""
    from flashrnn_b200 import _lib, flashrnn

    from flashrnn_b200.workloads import make_inputs

    B, T, N, D = 5, 6, 1, 768
    assert _lib.plan(cell, B, T, N, D).bwd_ksplit > 0
    wx, R, b, initial = make_inputs(cell, B, T, N, D, 93)
    wx_r = wx.bfloat16().float()
    S = port.SIZES[cell][3]
    d_history = torch.zeros((S, B, T, N, D))
    d_history[0] = torch.randn((B, T, N, D), generator=torch.Generator().manual_seed(94))
    ref_h, _, (r_dwx, r_dR, r_db, r_dinit) = port.forward_backward(wx_r, R, b, initial, cell, d_history,
                                                                    torch.zeros((S, B, 1, N, D)))
    leaves = [t.to(cuda_device).requires_grad_(True) for t in (wx.bfloat16(), R, b, initial)]
    hist, _ = flashrnn(*leaves, function=cell, backend="b200", dtype="bfloat16")
    (hist * d_history.to(cuda_device)).sum().backward()
    assert leaves[0].grad.dtype == torch.bfloat16
    log = []
    _check(cell, "history", hist, ref_h, log)
    _check(cell, "dwx", leaves[0].grad.float(), r_dwx, log)
    _check(cell, "dR", leaves[1].grad, r_dR, log)
    _check(cell, "db", leaves[2].grad, r_db, log)
    _check(cell, "d_initial", leaves[3].grad, r_dinit, log)


def test_several_wide_heads_run_as_one_launch_per_head(cuda_device):
    """GRU with two heads of 1280 units and 17 batch rows: one launch takes one head and 16 rows, so the host runs
    four launches; forward and all gradients against the oracle."""
    from flashrnn_b200 import functional
    from flashrnn_b200.workloads import make_inputs

    cell, B, T, N, D = "gru", 17, 4, 2, 1280
    heads, rows = functional._launch_split(cell, B, T, N, D)
    assert heads < N and rows < B
    wx, R, b, initial = make_inputs(cell, B, T, N, D, 95)
    gen = torch.Generator().manual_seed(96)
    d_history = torch.randn((1, B, T, N, D), generator=gen)
    d_carry = torch.randn((1, B, 1, N, D), generator=gen)
    ref_h, ref_c, ref_g = port.forward_backward(wx, R, b, initial, cell, d_history, d_carry)
    g = dict(meta=dict(cell=cell, T=T, n_chunks=1), wx=wx, R=R, b=b, initial=initial, d_history=d_history, d_carry=d_carry)
    history, carry, grads = _run_gpu(g, cuda_device)
    log = []
    for key, got, ref in zip(("history", "carry", "dwx", "dR", "db", "d_initial"), [history, carry] + list(grads),
                             [ref_h, ref_c] + list(ref_g)):
        _check("heads", key, got, ref, log)

