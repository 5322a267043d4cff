"""CPU restatement of the reference recurrence and of its autograd backward.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this module: it is the checker
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of ``bench.py``.

What it restates (reference = 0z5a/flashrnn):

* ``step_forward`` / ``forward``: one step and the time loop of ``recurrence()``
  (flashrnn/flashrnn2/reference.py:72-114) under the ``fp32_state_bf16_mma`` policy of
  ``flashrnn_torch`` (flashrnn/flashrnn2/torch_backend.py:59-67): state fp32, ``R`` and the
  recurrent hidden operand rounded through bf16, everything else fp32. With
  ``bf16_mma=False`` it is the "mathematical" policy (no rounding; used in float64 to pin the
  formulas to 1e-12).
* ``backward``: explicit reverse-time BPTT that reproduces what torch autograd computes for that
  forward, including the rounding points autograd inherits from the casts
  (torch_backend.py:28-30): the R-path hidden gradient ``dg . R~`` is rounded through bf16, each
  step's ``dR`` contribution is rounded through bf16 before fp32 accumulation, ``dWx = dg`` and
  ``db = sum dg`` stay fp32. The sLSTM stabiliser ``m`` carries a gradient and ``maximum`` splits
  ties 0.5/0.5 exactly as torch does.

Pinned against the reference itself: ``tests/golden/make_golden.py`` runs the reference's
``flashrnn_torch`` + autograd and stores its outputs; ``tests/test_oracle.py`` compares this
module with those vectors.
"""

from __future__ import annotations

import torch

# (recurrent gates, Wx gates, bias gates, states) — reference.py:16-21 / flashrnn.py:46-68
SIZES = {"lstm": (4, 4, 4, 2), "slstm": (4, 4, 4, 4), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1)}


def _bf(x: torch.Tensor, on: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype) if on else x


def forward(wx, R, b, initial, cell="lstm", bf16_mma=True, zero_first=None, forward_clipval=None):
    """Return (history [S,B,T,N,D], carry [S,B,1,N,D], tape). ``tape`` feeds ``backward``.

    ``zero_first`` overrides the sLSTM "all n == 0" predicate of the first step (a shard of a
    larger call must use the predicate of the whole call, state_contract.py:81-97).
    ``forward_clipval`` (v1 option, flashrnn/flashrnn/fused/lstm_fused_pointwise.cuh:76-81): the new hidden state is
    clipped to [-v, v] before it is stored and fed back. The reference implements its v1 options only in its CUDA
    kernels, which cannot run here: this restatement of them is NOT pinned against reference outputs.
    """
    gr, gw, gb, S = SIZES[cell]
    B, T, G, N, D = wx.shape
    assert G == gw and R.shape == (gr, N, D, D) and b.shape == (gb, N, D) and initial.shape == (S, B, 1, N, D)
    Rr = _bf(R, bf16_mma)
    state = [initial[s, :, 0] for s in range(S)]
    hist = [[] for _ in range(S)]
    tape = []
    for t in range(T):
        x = wx[:, t]  # [B,G,N,D]
        h_op = _bf(state[0], bf16_mma)
        ry = torch.einsum("bnp,gnop->bgno", h_op, Rr)
        rec = {"h_op": h_op, "prev": state}
        if cell == "lstm":
            pre = x + ry + b
            si, sf, tz, so = torch.sigmoid(pre[:, 0]), torch.sigmoid(pre[:, 1]), torch.tanh(pre[:, 2]), torch.sigmoid(pre[:, 3])
            c = sf * state[1] + si * tz
            tc = torch.tanh(c)
            new = [so * tc, c]
            rec.update(si=si, sf=sf, tz=tz, so=so, tc=tc)
        elif cell == "slstm":
            pre = x + ry + b
            i, f, z, o = pre[:, 0], pre[:, 1], pre[:, 2], pre[:, 3]
            _, c0, n0, m0 = state
            logf = torch.nn.functional.logsigmoid(f) + m0
            zero = bool(torch.all(n0 == 0)) if (zero_first is None or t > 0) else bool(zero_first)
            m = i if zero else torch.maximum(i, logf)
            ig, fg = torch.exp(i - m), torch.exp(logf - m)
            tz, so = torch.tanh(z), torch.sigmoid(o)
            c = fg * c0 + ig * tz
            pre_n = fg * n0 + ig
            n = torch.maximum(pre_n, torch.ones_like(pre_n))
            new = [so * c / n, c, n, m]
            rec.update(i=i, f=f, logf=logf, ig=ig, fg=fg, tz=tz, so=so, pre_n=pre_n, zero=zero)
        elif cell == "gru":
            cand = ry[:, 0] + b[0]
            r = torch.sigmoid(x[:, 0] + ry[:, 1] + b[1])
            u = torch.sigmoid(x[:, 1] + ry[:, 2] + b[2])
            v = torch.tanh(x[:, 2] + b[3] + r * cand)
            new = [u * state[0] + (1 - u) * v]
            rec.update(cand=cand, r=r, u=u, v=v)
        elif cell == "elman":
            new = [torch.tanh(x[:, 0] + ry[:, 0] + b[0])]
        else:
            raise ValueError(cell)
        if forward_clipval is not None:
            new = [new[0].clamp(-forward_clipval, forward_clipval)] + list(new[1:])
        rec["new"] = new
        tape.append(rec)
        state = new
        for s in range(S):
            hist[s].append(new[s])
    history = torch.stack([torch.stack(hs, dim=1) for hs in hist], dim=0)
    carry = torch.stack(state, dim=0).unsqueeze(2)
    return history, carry, {"steps": tape, "R": Rr, "cell": cell, "bf16_mma": bf16_mma, "shape": (B, T, N, D)}


def _tie_mask(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """d maximum(a, b) / d a as torch defines it: 1 where a > b, 0.5 at a == b, else 0."""
    one, half, zero = torch.ones_like(a), torch.full_like(a, 0.5), torch.zeros_like(a)
    return torch.where(a > b, one, torch.where(a == b, half, zero))


def backward(tape, d_history, d_carry, gradient_recurrent_clipval=None, gradient_recurrent_cut=False, slstm_v1=False):
    """Gradients (dWx, dR, db, d_initial) of sum(history*d_history) + sum(carry*d_carry).

    v1 options (flashrnn/flashrnn/fused/lstm_fused_pointwise.cuh:116-122, flashrnn_fused_backward_cut.cu:90; not pinned,
    see ``forward``): the gradient carried into h_t from step t+1 is clipped before the external one is added; with the
    cut the R path contributes nothing; a forward clip counts as the identity. ``slstm_v1``: the gradient convention of
    the reference's kernels and of flashrnn/flashrnn2/grad_reference.py:1-13 (pinned by a golden vector made from that
    module): m carries no gradient, the normaliser clamp passes its gradient straight through."""
    cell, Rr, on = tape["cell"], tape["R"], tape["bf16_mma"]
    gr, gw, gb, S = SIZES[cell]
    B, T, N, D = tape["shape"]
    dt = Rr.dtype
    dcar = [d_carry[s, :, 0].clone() for s in range(S)]
    dwx = torch.zeros((B, T, gw, N, D), dtype=dt)
    dR = torch.zeros_like(Rr)
    db = torch.zeros((gb, N, D), dtype=dt)
    for t in range(T - 1, -1, -1):
        rec = tape["steps"][t]
        prev, new = rec["prev"], rec["new"]
        carried = dcar
        if gradient_recurrent_clipval is not None and t < T - 1:
            carried = [dcar[0].clamp(-gradient_recurrent_clipval, gradient_recurrent_clipval)] + list(dcar[1:])
        ds = [carried[s] + d_history[s, :, t] for s in range(S)]
        if cell == "lstm":
            si, sf, tz, so, tc = rec["si"], rec["sf"], rec["tz"], rec["so"], rec["tc"]
            dh = ds[0]
            dc = ds[1] + dh * so * (1 - tc * tc)
            d_o = dh * tc * so * (1 - so)
            d_f = dc * prev[1] * sf * (1 - sf)
            d_i = dc * tz * si * (1 - si)
            d_z = dc * si * (1 - tz * tz)
            dg_r = torch.stack((d_i, d_f, d_z, d_o), dim=1)
            dg_w, dg_b = dg_r, dg_r
            dprev = [torch.zeros_like(dh), dc * sf]
        elif cell == "slstm":
            i, f, logf, ig, fg, tz, so = rec["i"], rec["f"], rec["logf"], rec["ig"], rec["fg"], rec["tz"], rec["so"]
            _, c0, n0, _ = prev
            _, c1, n1, _ = new
            dh = ds[0]
            dc = ds[1] + dh * so / n1
            dn = ds[2] - dh * so * c1 / (n1 * n1)
            d_o = dh * (c1 / n1) * so * (1 - so)
            dpre = dn if slstm_v1 else dn * _tie_mask(rec["pre_n"], torch.ones_like(n1))
            d_ig = dc * tz + dpre
            d_fg = dc * c0 + dpre * n0
            d_z = dc * ig * (1 - tz * tz)
            d_i = d_ig * ig
            d_logf = d_fg * fg
            dm = torch.zeros_like(d_i) if slstm_v1 else ds[3] - d_i - d_logf
            if rec["zero"]:
                d_i = d_i + dm
            else:
                wi = _tie_mask(i, logf)
                d_i = d_i + dm * wi
                d_logf = d_logf + dm * (1 - wi)
            d_f = d_logf * (1 - torch.sigmoid(f))
            dg_r = torch.stack((d_i, d_f, d_z, d_o), dim=1)
            dg_w, dg_b = dg_r, dg_r
            dprev = [torch.zeros_like(dh), dc * fg, dpre * fg, torch.zeros_like(dh) if slstm_v1 else d_logf]
        elif cell == "gru":
            cand, r, u, v = rec["cand"], rec["r"], rec["u"], rec["v"]
            dh = ds[0]
            d_u = dh * (prev[0] - v) * u * (1 - u)
            d_v = dh * (1 - u) * (1 - v * v)
            d_r = d_v * cand * r * (1 - r)
            d_cand = d_v * r
            dg_r = torch.stack((d_cand, d_r, d_u), dim=1)
            dg_w = torch.stack((d_r, d_u, d_v), dim=1)
            dg_b = torch.stack((d_cand, d_r, d_u, d_v), dim=1)
            dprev = [dh * u]
        else:
            h1 = new[0]
            d = ds[0] * (1 - h1 * h1)
            dg_r = d.unsqueeze(1)
            dg_w, dg_b = dg_r, dg_r
            dprev = [torch.zeros_like(d)]
        dwx[:, t] = dg_w
        db += dg_b.sum(dim=0)
        dR += _bf(torch.einsum("bgno,bnp->gnop", dg_r, rec["h_op"]), on)
        if not gradient_recurrent_cut:
            dprev[0] = dprev[0] + _bf(torch.einsum("bgno,gnop->bnp", dg_r, Rr), on)
        dcar = dprev
    d_initial = torch.stack(dcar, dim=0).unsqueeze(2)
    return dwx, dR, db, d_initial


def forward_backward(wx, R, b, initial, cell, d_history, d_carry, bf16_mma=True, zero_first=None, forward_clipval=None,
                     gradient_recurrent_clipval=None, gradient_recurrent_cut=False, slstm_v1=False):
    """Convenience: forward + backward, everything detached."""
    with torch.no_grad():
        history, carry, tape = forward(wx, R, b, initial, cell, bf16_mma, zero_first, forward_clipval)
        grads = backward(tape, d_history, d_carry, gradient_recurrent_clipval, gradient_recurrent_cut, slstm_v1)
    return history, carry, grads
