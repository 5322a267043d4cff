"""Host side of the B200 recurrence backend: the reference's two public call signatures.

* ``flashrnn(Wx, R, b, states, function, config, backend, dtype)`` mirrors
  flashrnn/flashrnn/flashrnn.py:1117-1138 (same tensor layouts, ``states=None`` means zeros).
* ``flashrnn_torch(wx, recurrent, bias, initial, *, cell, numerics)`` mirrors
  flashrnn/flashrnn2/torch_backend.py:12-67 (same validation and error behaviour).

Both run the hand-written sm_100a kernels through the C ABI; there is no other code path.
State, history, carry and every gradient accumulation are fp32; R and the recurrent hidden
operand are rounded to bf16 for the tensor cores, i.e. the reference's ``fp32_state_bf16_mma``
numerics. The carry returned by one call is a valid ``states`` / ``initial`` of the next one and
stays connected to autograd.
"""

from __future__ import annotations

from dataclasses import dataclass
import time
from typing import Optional

import torch

from . import _lib

# (recurrent gates, Wx gates, bias gates, states); reference.py:16-21, flashrnn.py:46-68
SIZES = {"lstm": (4, 4, 4, 2), "slstm": (4, 4, 4, 4), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1)}
BACKEND = "b200"
_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}

_pending_errors: list = []
_last_poll = 0.0


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _raise_device_error(err: torch.Tensor, what: str) -> None:
    code, step, cta = (int(v) for v in err[:3].tolist())
    if code != 0:
        raise RuntimeError(
            f"{what}: device-side wait ran out (code {code}: {_lib.ERROR_TEXT.get(code, '?')}, step {step}, CTA {cta})"
        )


_captured_errors: list = []   # error words of launches recorded into CUDA graphs: (err, what), newest last


_has_cuda: Optional[bool] = None


def _capturing() -> bool:
    global _has_cuda
    if _has_cuda is None:   # asked once: the availability check costs microseconds on every call otherwise
        _has_cuda = torch.cuda.is_available()
    return _has_cuda and torch.cuda.is_current_stream_capturing()


def _track(err: torch.Tensor, what: str) -> None:
    """Remember an error word; it is read once the kernels that write it have finished.

    While a CUDA graph is being captured no event may be queried: the word (which every replay zeroes and rewrites)
    is then kept for ``poll_errors(block=True)``."""
    if _capturing():
        _captured_errors.append((err, what))
        del _captured_errors[:-256]
        return
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(err.device))
    _pending_errors.append((ev, err, what))


def poll_errors(block: bool = False) -> None:
    """Raise if a finished launch reported a device-side error. ``block=True`` waits for all, including the launches
    of replayed CUDA graphs (their error words are only looked at here). A no-op while a graph is being captured."""
    if _capturing():
        return
    global _last_poll
    if not block:
        # reading an error word back costs a device-to-host copy (tens of microseconds): the non-blocking check at the
        # start of every call looks at most once per 20 ms; the words wait in the queue until then
        now = time.monotonic()
        if now - _last_poll < 0.02:
            return
        _last_poll = now
    keep = []
    while _pending_errors:
        ev, err, what = _pending_errors.pop(0)
        if block:
            ev.synchronize()
        if ev.query():
            _raise_device_error(err, what)
        else:
            keep.append((ev, err, what))
    _pending_errors.extend(keep)
    if block and _captured_errors:
        for device in {err.device for err, _ in _captured_errors}:
            torch.cuda.synchronize(device)
        for err, what in _captured_errors:
            _raise_device_error(err, what + " (in a replayed CUDA graph)")


class _Recurrence(torch.autograd.Function):
    """One fused forward launch; backward = one BPTT launch + the dR/db contraction."""

    @staticmethod
    def forward(ctx, wx, recurrent, bias, initial, cell: str, zero_first: bool, options=None):
        # the C ABI plans for and launches on the current device: make the tensors' device current
        with torch.cuda.device(wx.device):
            return _Recurrence._forward(ctx, wx, recurrent, bias, initial, cell, zero_first, options)

    @staticmethod
    def _forward(ctx, wx, recurrent, bias, initial, cell: str, zero_first: bool, options):
        lib = _lib.load()
        poll_errors()
        B, T, _, N, D = wx.shape
        gr, gw, gb, S = SIZES[cell]
        dev = wx.device
        wx_c = wx.contiguous()
        r_bf = recurrent.detach().to(torch.bfloat16).contiguous()
        b32 = bias.detach().to(torch.float32).contiguous()
        init32 = initial.detach().to(torch.float32).contiguous()
        plan = _lib.plan(cell, B, T, N, D)
        if not plan.supported:
            raise ValueError(
                f"flashrnn_b200: cell={cell} D={D} is outside the sm_100a kernel family "
                f"(the recurrent matrix of a head must fit the tensor memory of the CTAs of one launch: D <= 1792; wider heads "
                f"run through the row-sharded kernels when D is a multiple of 256)"
            )
        history = torch.empty((S, B, T, N, D), dtype=torch.float32, device=dev)
        carry = torch.empty((S, B, 1, N, D), dtype=torch.float32, device=dev)
        train = any(ctx.needs_input_grad[:4])
        cache = hbf = None
        if train:
            if plan.cache_bytes:
                cache = torch.empty(plan.cache_bytes, dtype=torch.uint8, device=dev)
            hbf = torch.empty(plan.hbf_bytes // 2, dtype=torch.bfloat16, device=dev)
        xchg = torch.empty(plan.xchg_bytes, dtype=torch.uint8, device=dev) if plan.xchg_bytes else None
        err = torch.zeros(32, dtype=torch.int32, device=dev)
        rc = lib.frnn_b200_forward_ex(
            _lib.CELLS[cell], wx_c.data_ptr(), int(wx_c.dtype == torch.bfloat16), r_bf.data_ptr(), b32.data_ptr(),
            init32.data_ptr(), history.data_ptr(), carry.data_ptr(), _ptr(cache), _ptr(hbf), _ptr(xchg), B, T, N, D,
            int(zero_first), 0, err.data_ptr(), _stream(dev), _options_struct(options),
        )
        _lib.check(rc, "frnn_b200_forward")
        _track(err, "frnn_b200_forward")
        if train:
            ctx.save_for_backward(r_bf, init32, history, cache if cache is not None else history.new_empty(0), hbf)
            ctx.cell, ctx.zero_first = cell, zero_first
            ctx.shape = (B, T, N, D)
            ctx.dtypes = (wx.dtype, recurrent.dtype, bias.dtype, initial.dtype)
            ctx.plan = plan
            ctx.options = options
        return history, carry

    @staticmethod
    def backward(ctx, d_history, d_carry):
        with torch.cuda.device(ctx.saved_tensors[2].device):
            return _Recurrence._backward(ctx, d_history, d_carry)

    @staticmethod
    def _backward(ctx, d_history, d_carry):
        lib = _lib.load()
        poll_errors()
        r_bf, init32, history, cache, hbf = ctx.saved_tensors
        cell, plan = ctx.cell, ctx.plan
        B, T, N, D = ctx.shape
        gr, gw, gb, S = SIZES[cell]
        dev = history.device
        wx_dtype = ctx.dtypes[0]
        if d_history is None:
            d_history = torch.zeros_like(history)
        if d_carry is None:
            d_carry = torch.zeros((S, B, 1, N, D), dtype=torch.float32, device=dev)
        d_history = d_history.to(torch.float32).contiguous()
        d_carry = d_carry.to(torch.float32).contiguous()
        dwx = torch.empty((B, T, gw, N, D), dtype=wx_dtype, device=dev)
        # bf16 Wx and W-gates == R-gates: dWx doubles as the bf16 operand of the dR contraction (one buffer, one write)
        shared = wx_dtype == torch.bfloat16 and cell != "gru"
        dgr = dwx if shared else torch.empty(plan.dgr_bytes // 2, dtype=torch.bfloat16, device=dev)
        d_initial = torch.empty((S, B, 1, N, D), dtype=torch.float32, device=dev)
        db_part = torch.empty(plan.dbpart_bytes // 4, dtype=torch.float32, device=dev)
        # dR and db are neighbours in one allocation so that a batch-sharded caller sums both with one all-reduce
        wflat = torch.empty(gr * N * D * D + gb * N * D, dtype=torch.float32, device=dev)
        dR = wflat[:gr * N * D * D].view(gr, N, D, D)
        db = wflat[gr * N * D * D:].view(gb, N, D)
        work = None
        if plan.wgrad_work_bytes:
            work = torch.empty(plan.wgrad_work_bytes // 4, dtype=torch.float32, device=dev)
        xchg = torch.empty(plan.xchg_bytes, dtype=torch.uint8, device=dev) if plan.xchg_bytes else None
        err = torch.zeros(32, dtype=torch.int32, device=dev)
        stream = _stream(dev)
        rc = lib.frnn_b200_backward_ex(
            _lib.CELLS[cell], _ptr(cache) if cache.numel() else None, history.data_ptr(), init32.data_ptr(),
            r_bf.data_ptr(), d_history.data_ptr(), d_carry.data_ptr(), dwx.data_ptr(),
            int(wx_dtype == torch.bfloat16), dgr.data_ptr(), d_initial.data_ptr(), db_part.data_ptr(), _ptr(xchg),
            B, T, N, D,
            int(ctx.zero_first), 0, err.data_ptr(), stream, _options_struct(ctx.options),
        )
        _lib.check(rc, "frnn_b200_backward")
        rc = lib.frnn_b200_wgrad(
            _lib.CELLS[cell], dgr.data_ptr(), hbf.data_ptr(), db_part.data_ptr(), dR.data_ptr(), db.data_ptr(),
            _ptr(work), B, T, N, D, err.data_ptr(), stream,
        )
        _lib.check(rc, "frnn_b200_wgrad")
        _track(err, "frnn_b200_backward")
        need = ctx.needs_input_grad
        return (
            dwx if need[0] else None,
            dR.to(ctx.dtypes[1]) if need[1] else None,
            db.to(ctx.dtypes[2]) if need[2] else None,
            d_initial.to(ctx.dtypes[3]) if need[3] else None,
            None,
            None,
            None,
        )


def _options_struct(options):
    """``(forward_clipval, gradient_recurrent_clipval, gradient_recurrent_cut, slstm_v1)`` -> ctypes pointer or None."""
    if options is None or not any(options):
        return None
    import ctypes

    o = _lib.Options()
    o.forward_clipval = float(options[0] or 0.0)
    o.gradient_recurrent_clipval = float(options[1] or 0.0)
    o.gradient_recurrent_cut = int(bool(options[2]))
    o.slstm_v1_gradient = int(bool(options[3]))
    return ctypes.byref(o)


def _pad_width(t: torch.Tensor, pad: int, dims) -> torch.Tensor:
    """Zero-pad the given (negative) dims by ``pad`` at the end."""
    spec = []
    for d in range(-1, -t.ndim - 1, -1):
        spec += [0, pad if d in dims else 0]
    return torch.nn.functional.pad(t, spec)


def _run(wx, recurrent, bias, initial, cell: str, zero_normalizer: Optional[bool] = None, options=None):
    if not wx.is_cuda:
        raise RuntimeError("flashrnn_b200 runs on CUDA devices only (sm_100a); there is no CPU path")
    with torch.cuda.device(wx.device):
        return _run_on_current_device(wx, recurrent, bias, initial, cell, zero_normalizer, options)


_wide_heads: dict = {}   # (cell, B, T, D, device, Wx dtype) -> [WideHead with all of its ranks on this GPU, ...]


def _run_wide(wx, recurrent, bias, initial, cell: str, zero_first: bool):
    """Heads wider than the single-GPU kernel family (1792 < D, D a multiple of 256) on ONE GPU: every head goes through
    the row-sharded kernels with a single rank (their K split inside clusters and weight ring take over), at most 32
    batch rows per launch. The reference covers D <= 2048 on one device with its hybrid kernels
    (flashrnn/flashrnn2/hybrid_fw2d.py:20-23)."""
    from .wide_head import WideHead

    B, T, _, N, D = wx.shape
    dev = wx.device

    def head_for(rows: int) -> "WideHead":
        # A head's exchange buffers double as the saved operands of its backward pass: one that still has a backward
        # pending (`in_use`) is not given out again; pools grow to what one training step needs and are then reused.
        key = (cell, rows, T, D, dev.index, wx.dtype)
        pool = _wide_heads.setdefault(key, [])
        for head in pool:
            if not head.in_use:
                return head
        if sum(len(p) for p in _wide_heads.values()) >= 16:   # other shapes' idle heads make room
            for other in _wide_heads.values():
                for head in [h for h in other if not h.in_use]:
                    other.remove(head)
                    head.close()
        pool.append(WideHead(cell, rows, T, D, emulate_ranks=1, device=dev, wx_dtype=wx.dtype))
        return pool[-1]

    per_head = []
    for n in range(N):
        pieces = []
        for i in range(0, B, 32):
            j = min(B, i + 32)
            pieces.append(head_for(j - i)(wx[i:j, :, :, n:n + 1], recurrent[:, n:n + 1], bias[:, n:n + 1],
                                          initial[:, i:j, :, n:n + 1], zero_normalizer=zero_first))
        per_head.append((torch.cat([h for h, _ in pieces], dim=1), torch.cat([c for _, c in pieces], dim=1))
                        if len(pieces) > 1 else pieces[0])
    if N == 1:
        return per_head[0]
    return torch.cat([h for h, _ in per_head], dim=3), torch.cat([c for _, c in per_head], dim=3)


def _run_on_current_device(wx, recurrent, bias, initial, cell: str, zero_normalizer: Optional[bool], options=None):
    D = wx.shape[-1]
    if cell != "slstm":
        zero_first = False
    elif zero_normalizer is not None:
        zero_first = bool(zero_normalizer)  # predicate of the whole logical call, given by a sharding caller
    else:
        zero_first = bool(torch.all(initial[2] == 0))
    if D > 1792 and D % 256 == 0 and options is None and wx.dtype in (torch.float32, torch.bfloat16):
        return _run_wide(wx, recurrent, bias, initial, cell, zero_first)
    # The kernels tile the head width in multiples of 16 (heads wider than 768: 64, and 128 where only the
    # column-owning backward fits); the smallest such width that a launch supports is used.
    pad = (-D) % 16
    for multiple in (16, 64, 128):
        if _lib.plan(cell, min(wx.shape[0], 8), wx.shape[1], 1, D + (-D) % multiple).supported:
            pad = (-D) % multiple
            break
    if pad:
        # The kernels tile the head width in multiples of 16; zero rows/columns of R, zero
        # inputs and zero initial state keep the padded units at exactly zero.
        wx = _pad_width(wx, pad, (-1,))
        recurrent = _pad_width(recurrent, pad, (-1, -2))
        bias = _pad_width(bias, pad, (-1,))
        initial = _pad_width(initial, pad, (-1,))
    B, T, _, N, Dp = wx.shape
    heads, rows = _launch_split(cell, B, T, N, Dp)
    if heads >= N and rows >= B:
        history, carry = _Recurrence.apply(wx, recurrent, bias, initial, cell, zero_first, options)
    else:
        # Wide heads run with all CTAs of a launch resident at once, which bounds the heads and batch
        # rows one launch can take; more go through several launches (heads and batch rows are
        # independent, and autograd adds up the weight gradients of the batch pieces).
        per_head = []
        for n0 in range(0, N, heads):
            n1 = min(N, n0 + heads)
            wx_h = wx if heads >= N else wx[:, :, :, n0:n1].contiguous()
            pieces = [_Recurrence.apply(wx_h[i:i + rows], recurrent[:, n0:n1], bias[:, n0:n1],
                                        initial[:, i:i + rows, :, n0:n1], cell, zero_first, options)
                      for i in range(0, B, rows)]
            per_head.append((torch.cat([h for h, _ in pieces], dim=1), torch.cat([c for _, c in pieces], dim=1)))
        history = torch.cat([h for h, _ in per_head], dim=3)
        carry = torch.cat([c for _, c in per_head], dim=3)
    if pad:
        history, carry = history[..., :D], carry[..., :D]
    return history, carry


def _launch_split(cell: str, B: int, T: int, N: int, D: int):
    """(heads, batch rows) one launch takes: (N, B) where the shape is supported as a whole; else the most heads
    for which some number of batch rows is supported, with that number of rows (see ``_rows_per_launch``);
    (N, B) again when nothing is (the launch then reports the shape)."""
    for heads in range(N, 0, -1):
        rows = _rows_per_launch(cell, B, T, heads, D)
        if _lib.plan(cell, rows, T, heads, D).supported:
            return heads, rows
    return N, B


def _rows_per_launch(cell: str, B: int, T: int, N: int, D: int) -> int:
    """Batch rows one launch can take: B where the shape is supported as a whole (or not at all, which the
    launch then reports), else the largest multiple of 8 below B for which the plan is supported."""
    if _lib.plan(cell, B, T, N, D).supported:
        return B
    for rows in range((B - 1) // 8 * 8, 0, -8):
        if _lib.plan(cell, rows, T, N, D).supported:
            return rows
    return B


def flashrnn_torch(wx, recurrent, bias, initial, *, cell: str = "lstm", numerics: str = "mathematical",
                   zero_normalizer: Optional[bool] = None):
    """Return full history ``[S,B,T,H,D]`` and carry ``[S,B,1,H,D]`` (both fp32).

    Same signature, defaults and argument checks as flashrnn/flashrnn2/torch_backend.py:12-58. The only
    numerical policy this backend implements is ``fp32_state_bf16_mma`` (tensor cores take bf16 operands);
    the reference's default ``"mathematical"`` (unrounded fp32 contraction) is kept as the default of the
    signature and rejected with a message that names the policy to pass, so that a caller who switches the
    import never gets different arithmetic without asking for it. fp32 inputs follow the reference
    contract exactly, bf16 inputs (Wx, R, b, initial rounded by the caller) are accepted as an extension.
    ``zero_normalizer`` (sLSTM only) overrides the "all initial n == 0" predicate of the first step; a
    batch/head shard passes the predicate of the unsharded call (state_contract.py:81-97).
    """
    if cell not in SIZES:
        raise ValueError(f"unsupported cell: {cell}")
    if numerics != "fp32_state_bf16_mma":
        if numerics == "mathematical":
            raise ValueError("the B200 backend has no unrounded fp32 contraction: pass numerics='fp32_state_bf16_mma' "
                             "(fp32 state, R and the recurrent hidden operand rounded to bf16)")
        raise ValueError(f"unsupported numerical policy: {numerics}")
    tensors = (wx, recurrent, bias, initial)
    if any(t.layout != torch.strided for t in tensors):
        raise ValueError("inputs must have strided tensor layout")
    if tuple(t.ndim for t in tensors) != (5, 4, 3, 5):
        raise ValueError("expected wx/R/b/initial ranks 5/4/3/5")
    if any(size < 1 for size in wx.shape):
        raise ValueError("batch, time, gates, heads and width must be positive")
    if wx.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("fp32_state_bf16_mma requires FP32 inputs (BF16 inputs are accepted as pre-rounded)")
    if any(t.dtype != wx.dtype for t in tensors):
        raise ValueError("all inputs must have the same dtype")
    if any(t.device != wx.device for t in tensors):
        raise ValueError("all inputs must be on the same device")
    batch, steps, gates, heads, width = wx.shape
    gr, gw, gb, S = SIZES[cell]
    if gates != gw:
        raise ValueError("expected nonempty sequence and matching input gate count")
    if recurrent.shape != (gr, heads, width, width):
        raise ValueError("recurrent weights must have layout [G,N,D,P]")
    if bias.shape != (gb, heads, width):
        raise ValueError("bias gate count does not match cell")
    if initial.shape != (S, batch, 1, heads, width):
        raise ValueError("initial state must have layout [S,B,1,N,D]")
    with torch.autocast("cuda", enabled=False):
        return _run(wx, recurrent, bias, initial, cell, zero_normalizer)


@dataclass
class FlashRNNConfig:
    """The fields of the reference's FlashRNNConfig (flashrnn/flashrnn/flashrnn.py:121-170) this backend honours.

    ``gradient_recurrent_cut`` / ``gradient_recurrent_clipval`` / ``forward_clipval`` behave as in the reference's
    fused kernels (flashrnn/flashrnn/fused/lstm_fused_pointwise.cuh:76-81,116-122, flashrnn_fused_backward_cut.cu):
    h_t is clipped before it is stored and fed back (the backward treats the clip as the identity); the gradient
    carried into h_t from step t+1 is clipped before the external gradient of h_t is added; with the cut the R path
    contributes nothing to the hidden-state gradient. ``slstm_gradient="v1"`` selects the gradient convention of the
    reference's own kernels (m without gradient, normaliser clamp straight-through: flashrnn2/grad_reference.py:1-13)
    instead of what autograd gives for the forward formulas (the default, ``"autograd"``)."""

    function: str = "lstm"
    backend: str = BACKEND
    dtype: str = "bfloat16"
    gradient_recurrent_cut: bool = False
    gradient_recurrent_clipval: Optional[float] = None
    forward_clipval: Optional[float] = None
    slstm_gradient: str = "autograd"
    head_dim: int = -1
    num_heads: int = -1
    batch_size: int = -1

    def options(self):
        if self.slstm_gradient not in ("autograd", "v1"):
            raise ValueError("slstm_gradient must be 'autograd' or 'v1'")
        for name in ("gradient_recurrent_clipval", "forward_clipval"):
            v = getattr(self, name)
            if v is not None and not v > 0:
                raise ValueError(f"{name} must be positive or None")
        return (self.forward_clipval, self.gradient_recurrent_clipval, self.gradient_recurrent_cut,
                self.slstm_gradient == "v1")


def flashrnn(Wx, R, b, states=None, function: str = "lstm", config: Optional[FlashRNNConfig] = None,
             backend: str = BACKEND, dtype: str = "bfloat16", zero_normalizer: Optional[bool] = None):
    """``Wx[B,T,G,N,D], R[G,N,D,D], b[G,N,D], states[S,B,1,N,D]`` -> ``(states[S,B,T,N,D], last[S,B,1,N,D])``.

    ``dtype`` is the operand dtype of the streamed input (``Wx`` is cast to it, R always goes to
    the tensor cores in bf16); bias and states keep fp32, and the returned states are fp32.
    """
    options = None
    if config is not None:
        function, backend, dtype = config.function, config.backend, config.dtype
        options = config.options()
    if backend != BACKEND:
        raise ValueError(f"Unknown backend {backend}: this library provides backend='{BACKEND}' only")
    if function not in SIZES:
        raise ValueError(f"Unknown function {function}")
    if dtype not in _DTYPES:
        raise ValueError(f"Unsupported dtype {dtype}: use 'bfloat16' or 'float32'")
    gr, gw, gb, S = SIZES[function]
    B, T, G, N, D = Wx.shape
    if G != gw or R.shape != (gr, N, D, D) or b.shape != (gb, N, D):
        raise ValueError(f"shape mismatch for {function}: Wx {tuple(Wx.shape)}, R {tuple(R.shape)}, b {tuple(b.shape)}")
    if states is None:
        states = torch.zeros((S, B, 1, N, D), dtype=torch.float32, device=Wx.device)
    elif states.shape != (S, B, 1, N, D):
        raise ValueError("states must have layout [S,B,1,N,D]")
    with torch.autocast("cuda", enabled=False):
        return _run(Wx.to(_DTYPES[dtype]), R, b.to(torch.float32), states.to(torch.float32), function,
                    zero_normalizer, options)
