"""The input projection in front of the recurrence, fused into this library's data path.

``flashrnn_projected(x, W, R, b, states, ...)`` computes ``Wx = x @ W.T (+ bias_w)`` with a hand-written tcgen05 GEMM
that writes the gate pre-activations directly in the layout and dtype the recurrent kernels stream by TMA
(``[B,T,GW,N,D]``, bf16 by default), then runs the recurrence. The reference leaves this step to the caller
(README.md:16) and benchmarks it as the "-withlinear" variant: a ``torch.nn.Linear(N*D, G*N*D)`` in front of the
kernel (flashrnn/speed_experiments/kernel_speed_benchmark.py:388-408); ``W`` / ``bias_w`` have that layer's layout.

Backward of the projection (``dx = dWx @ W``, ``dW = dWx.T @ x``, ``dbias_w = sum dWx``) uses torch's library GEMMs: they
are plain GEMMs with no recurrence-specific fusion to gain.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .functional import SIZES, FlashRNNConfig, _track, flashrnn, poll_errors


class _Projection(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, out_dtype):
        lib = _lib.load()
        poll_errors()
        B, T, I = x.shape
        J = weight.shape[0]
        dev = x.device
        with torch.cuda.device(dev):
            x16 = x.detach().to(torch.bfloat16).contiguous()
            w16 = weight.detach().to(torch.bfloat16).contiguous()
            b32 = None if bias is None else bias.detach().to(torch.float32).contiguous()
            out = torch.empty((B, T, J), dtype=out_dtype, device=dev)
            err = torch.zeros(32, dtype=torch.int32, device=dev)
            rc = lib.frnn_b200_input_projection(
                x16.data_ptr(), w16.data_ptr(), None if b32 is None else b32.data_ptr(), out.data_ptr(),
                int(out_dtype == torch.bfloat16), B, T, J, I, err.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
            _lib.check(rc, "frnn_b200_input_projection")
            _track(err, "frnn_b200_input_projection")
        ctx.save_for_backward(x16, w16)
        ctx.dtypes = (x.dtype, weight.dtype, None if bias is None else bias.dtype)
        return out

    @staticmethod
    def backward(ctx, d_out):
        x16, w16 = ctx.saved_tensors
        B, T, I = x16.shape
        g = d_out.reshape(B * T, -1).to(torch.bfloat16)
        need = ctx.needs_input_grad
        dx = (g @ w16).reshape(B, T, I).to(ctx.dtypes[0]) if need[0] else None
        dw = (g.t() @ x16.reshape(B * T, I)).to(ctx.dtypes[1]) if need[1] else None
        db = d_out.reshape(B * T, -1).float().sum(0).to(ctx.dtypes[2]) if (need[2] and ctx.dtypes[2] is not None) else None
        return dx, dw, db, None


def input_projection(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``x[B,T,I] @ weight[J,I].T (+ bias[J]) -> [B,T,J]`` on the tensor cores (bf16 operands, fp32 accumulation)."""
    if x.ndim != 3 or weight.ndim != 2 or weight.shape[1] != x.shape[2]:
        raise ValueError("expected x [B,T,I] and weight [J,I]")
    if bias is not None and tuple(bias.shape) != (weight.shape[0],):
        raise ValueError("expected bias [J]")
    if not x.is_cuda:
        raise RuntimeError("flashrnn_b200 runs on CUDA devices only (sm_100a); there is no CPU path")
    if x.shape[2] % 8 or weight.shape[0] % 64:
        raise ValueError("the projection kernel needs I % 8 == 0 and G*N*D % 64 == 0")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out_dtype must be bfloat16 or float32")
    with torch.autocast("cuda", enabled=False):
        return _Projection.apply(x, weight, bias, out_dtype)


def flashrnn_projected(x, W, R, b, states=None, bias_w=None, function: str = "lstm",
                       config: Optional[FlashRNNConfig] = None, dtype: str = "bfloat16"):
    """``x[B,T,I], W[GW*N*D, I], R[G,N,D,D], b[G,N,D], states[S,B,1,N,D]`` -> ``(states[S,B,T,N,D], last[S,B,1,N,D])``.

    The same as ``flashrnn(x @ W.T ... )`` with the projection done by this library; differentiable in x, W, bias_w,
    R, b and states."""
    if config is not None:
        function, dtype = config.function, config.dtype
    if function not in SIZES:
        raise ValueError(f"Unknown function {function}")
    gw = SIZES[function][1]
    N, D = R.shape[1], R.shape[2]
    if W.shape[0] != gw * N * D:
        raise ValueError(f"W must have {gw} * {N} * {D} rows")
    out_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    wx = input_projection(x, W, bias_w, out_dtype).view(x.shape[0], x.shape[1], gw, N, D)
    return flashrnn(wx, R, b, states, function=function, config=config, dtype=dtype)
