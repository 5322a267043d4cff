"""Generate golden vectors by running the REFERENCE itself (needs the reference checkout).

    python tests/golden/make_golden.py /path/to/reference

For every case the reference's ``flashrnn_torch(..., numerics="fp32_state_bf16_mma")``
(flashrnn/flashrnn2/torch_backend.py:12-67) is run on seeded fp32 inputs, the scalar
``sum(history * d_history) + sum(carry * d_carry)`` is back-propagated with torch autograd, and
inputs, cotangents, outputs and the four gradients are written to ``tests/golden/<case>.npz``.
Large cases store a strided sample of the time axis plus float64 checksums of the inputs, which
the tests regenerate from the seed. The reference is only needed to (re)generate these files;
the test-suite reads the committed ``.npz`` files.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from flashrnn_b200.workloads import SIZES, make_inputs  # noqa: E402

# name -> (cell, B, T, N, D, seed, zero_initial, loss, n_chunks, time_stride)
CASES = {
    "lstm_small": ("lstm", 3, 5, 2, 16, 11, False, "random", 1, 1),
    "lstm_chunked": ("lstm", 2, 8, 2, 16, 12, False, "random", 2, 1),
    "lstm_odd_width": ("lstm", 1, 33, 2, 5, 13, False, "random", 1, 1),
    "slstm_zero_init": ("slstm", 2, 6, 2, 16, 14, True, "random", 1, 1),
    "slstm_nonzero_init": ("slstm", 3, 7, 1, 32, 15, False, "random", 1, 1),
    "slstm_sum_h": ("slstm", 4, 24, 2, 16, 16, True, "sum_h", 1, 1),
    "gru_small": ("gru", 3, 6, 2, 16, 17, False, "random", 1, 1),
    "elman_small": ("elman", 2, 9, 3, 16, 18, False, "random", 1, 1),
    "cfg1_lstm_fp32_B8_T256_N1_D64": ("lstm", 8, 256, 1, 64, 0, False, "sum_h", 1, 16),
    "cfg1_two_chunks_of_128": ("lstm", 8, 256, 1, 64, 0, False, "sum_h", 2, 16),
}


def cotangents(cell, B, T, N, D, seed, loss):
    S = SIZES[cell][3]
    if loss == "sum_h":
        d_history = torch.zeros((S, B, T, N, D))
        d_history[0] = 1.0
        return d_history, torch.zeros((S, B, 1, N, D))
    g = torch.Generator().manual_seed(seed + 1000)
    return torch.randn((S, B, T, N, D), generator=g), torch.randn((S, B, 1, N, D), generator=g)


def run_reference(flashrnn_torch, cell, wx, R, b, initial, d_history, d_carry, n_chunks):
    leaves = [t.clone().requires_grad_(True) for t in (wx, R, b, initial)]
    wx_l, R_l, b_l, init_l = leaves
    T = wx.shape[1]
    step = T // n_chunks
    carry, pieces = init_l, []
    for c in range(n_chunks):
        hist, carry = flashrnn_torch(wx_l[:, c * step:(c + 1) * step], R_l, b_l, carry, cell=cell,
                                     numerics="fp32_state_bf16_mma")
        pieces.append(hist)
    history = torch.cat(pieces, dim=2)
    ((history * d_history).sum() + (carry * d_carry).sum()).backward()
    return history.detach(), carry.detach(), [t.grad for t in leaves]


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from flashrnn import flashrnn_torch  # the reference's own export (flashrnn/__init__.py:2-3)

    torch.set_num_threads(1)
    for name, (cell, B, T, N, D, seed, zero, loss, n_chunks, stride) in CASES.items():
        wx, R, b, initial = make_inputs(cell, B, T, N, D, seed, zero)
        d_history, d_carry = cotangents(cell, B, T, N, D, seed, loss)
        history, carry, (dwx, dR, db, dinit) = run_reference(flashrnn_torch, cell, wx, R, b, initial, d_history,
                                                             d_carry, n_chunks)
        meta = dict(cell=cell, B=B, T=T, N=N, D=D, seed=seed, zero_initial=zero, loss=loss, n_chunks=n_chunks,
                    time_stride=stride)
        out = {"meta": np.array(repr(meta))}
        sl = slice(None, None, stride)
        if stride == 1:
            out.update(wx=wx.numpy(), R=R.numpy(), b=b.numpy(), initial=initial.numpy(),
                       d_history=d_history.numpy(), d_carry=d_carry.numpy())
        else:
            out["input_checksums"] = np.array([t.double().sum().item() for t in (wx, R, b, initial)]
                                              + [t.double().abs().sum().item() for t in (wx, R, b, initial)])
        out.update(history=history[:, :, sl].numpy(), carry=carry.numpy(), dwx=dwx[:, sl].numpy(), dR=dR.numpy(),
                   db=db.numpy(), d_initial=dinit.numpy())
        np.savez_compressed(HERE / f"{name}.npz", **out)
        print(f"{name}: wrote {sum(v.nbytes for v in out.values()) / 1024:.0f} KiB (uncompressed)")


# sLSTM under the gradient convention of the reference's own kernels: float64 autograd of
# flashrnn/flashrnn2/grad_reference.py (m without gradient, normaliser clamp straight-through), "mathematical" forward.
V1_CASES = {"slstm_v1_zero_init": (3, 9, 2, 8, 21, True), "slstm_v1_nonzero_init": (2, 7, 1, 16, 22, False)}


def main_v1(reference_root: str) -> None:
    import importlib.util

    pkg = Path(reference_root) / "flashrnn" / "flashrnn2"   # loaded as a package of its own: the top-level package pulls in CUDA JIT code
    spec = importlib.util.spec_from_file_location("_ref_flashrnn2", pkg / "__init__.py", submodule_search_locations=[str(pkg)])
    module = importlib.util.module_from_spec(spec)
    sys.modules["_ref_flashrnn2"] = module
    spec.loader.exec_module(module)
    from _ref_flashrnn2 import grad_reference

    out_dir = HERE / "v1"
    out_dir.mkdir(exist_ok=True)
    for name, (B, T, N, D, seed, zero) in V1_CASES.items():
        wx, R, b, initial = (t.double() for t in make_inputs("slstm", B, T, N, D, seed, zero))
        leaves = [t.clone().requires_grad_(True) for t in (wx, R, b, initial)]
        history, carry = grad_reference.recurrence(*leaves, cell="slstm")
        g = torch.Generator().manual_seed(seed + 1000)
        d_history = torch.randn(history.shape, generator=g, dtype=torch.float64)
        d_carry = torch.randn(carry.shape, generator=g, dtype=torch.float64)
        ((history * d_history).sum() + (carry * d_carry).sum()).backward()
        meta = dict(cell="slstm", B=B, T=T, N=N, D=D, seed=seed, zero_initial=zero, convention="v1", dtype="float64")
        np.savez_compressed(out_dir / f"{name}.npz", meta=np.array(repr(meta)), wx=wx.numpy(), R=R.numpy(), b=b.numpy(),
                            initial=initial.numpy(), d_history=d_history.numpy(), d_carry=d_carry.numpy(),
                            history=history.detach().numpy(), carry=carry.detach().numpy(), dwx=leaves[0].grad.numpy(),
                            dR=leaves[1].grad.numpy(), db=leaves[2].grad.numpy(), d_initial=leaves[3].grad.numpy())
        print(f"v1/{name}: written")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of a checkout of the reference (0z5a/flashrnn)>")
    main(sys.argv[1])
    main_v1(sys.argv[1])
