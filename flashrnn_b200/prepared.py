"""Forward-only execution of one fixed sequence shape on preallocated buffers, optionally as a CUDA graph.

The B200 counterpart of the reference's ``PreparedSequence`` (flashrnn/flashrnn2/prepared.py:18-192), with the same
constructor arguments, attributes and methods (``run`` / ``capture`` / ``check`` / ``close``, ``output`` / ``final``):

* inputs, weights and results live at fixed addresses; ``output`` and ``final`` are borrowed — the next ``run()``
  overwrites them; to feed new data, write into the bound tensors in place (``seq.wx.copy_(...)``);
* ``output_mode``: ``"full"`` = every state ``[S,B,T,N,D]``, ``"hidden"`` = h only ``[B,T,N,D]``, ``"last"`` = h of the
  final step ``[B,1,N,D]`` (saves the state writes of an inference pass);
* ``snapshot_dtype``: ``torch.float32`` (default) or ``torch.bfloat16`` for the stored states; carries are always fp32;
* ``chunks``: step counts that add up to T; the sequence then runs as one launch per chunk, every chunk starting from
  the previous chunk's carry (two carry buffers used in turn). ``final`` is the buffer the last chunk writes;
* one instance is used serially, on the stream that is current when ``run()`` is called.

R is rounded to bf16 when the instance is created and again by ``refresh_weights()``. The sLSTM "initial normaliser
is all zero" predicate is evaluated on the device at every run (no host read), so a run can be captured.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib
from .functional import SIZES

_OUTPUT_MODES = ("full", "hidden", "last")


def _require(ok: bool, message: str) -> None:
    if not ok:
        raise ValueError(message)


class PreparedSequence:
    def __init__(self, wx, recurrent, bias, initial, cell: str = "lstm", *, output_mode: str = "full",
                 snapshot_dtype: Optional[torch.dtype] = None, chunks: Optional[Sequence[int]] = None):
        _require(output_mode in _OUTPUT_MODES, "output mode must be full, hidden or last")
        _require(cell in SIZES, f"unknown cell {cell!r}")
        _require(wx.ndim == 5, "expected Wx [B,T,G,N,D]")
        n_r, n_w, n_b, n_states = SIZES[cell]
        B, T, G, N, D = (int(v) for v in wx.shape)
        _require(min(B, T, N, D) >= 1 and G == n_w, "expected nonempty B/T/N/D and the cell's number of input gates")
        _require(tuple(recurrent.shape) == (n_r, N, D, D) and tuple(bias.shape) == (n_b, N, D),
                 "invalid recurrent-weight or bias shape")
        _require(tuple(initial.shape) == (n_states, B, 1, N, D), "invalid initial-state shape")
        bound = (wx, recurrent, bias, initial)
        _require(wx.is_cuda and all(t.device == wx.device and t.is_contiguous() for t in bound),
                 "prepared execution requires contiguous tensors on one CUDA device")
        _require(wx.dtype in (torch.bfloat16, torch.float32) and bias.dtype == torch.float32 and initial.dtype == torch.float32,
                 "Wx must be bf16 or fp32; bias and the initial state fp32")
        _require(not any(t.requires_grad for t in bound), "prepared execution is forward-only")
        snap = torch.float32 if snapshot_dtype is None else snapshot_dtype
        _require(snap in (torch.float32, torch.bfloat16), "snapshot dtype must be FP32 or BF16")
        steps = (T,) if chunks is None else tuple(chunks)
        _require(len(steps) > 0 and all(type(n) is int and n > 0 for n in steps) and sum(steps) == T,
                 "chunk lengths must be positive integers totaling T")
        _require(D % 16 == 0, "prepared execution needs a head width that is a multiple of 16")
        with torch.cuda.device(wx.device):
            plans = [_lib.plan(cell, B, n, N, D) for n in steps]
        _require(all(p.supported for p in plans), f"cell={cell} B={B} N={N} D={D} is outside the sm_100a kernel family")

        self._lib = _lib.load()
        self.wx, self.recurrent, self.bias, self.initial = bound
        self.cell, self.shape, self.chunks = cell, (B, T, N, D), steps
        self.output_mode = _OUTPUT_MODES.index(output_mode)
        self.snapshot_dtype = snap
        dev = wx.device
        out_shape = {"full": (n_states, B, T, N, D), "hidden": (B, T, N, D), "last": (B, 1, N, D)}[output_mode]
        self.output = torch.empty(out_shape, dtype=snap, device=dev)
        self.carries = tuple(torch.empty((n_states, B, 1, N, D), dtype=torch.float32, device=dev) for _ in range(2))
        self.final = self.carries[(len(steps) - 1) % 2]
        self.error_flag = torch.zeros(32, dtype=torch.int32, device=dev)
        self._r_bf16 = torch.empty(recurrent.shape, dtype=torch.bfloat16, device=dev)
        self._zero_word = torch.zeros(1, dtype=torch.int32, device=dev)
        scratch = max(p.xchg_bytes for p in plans)
        self._xchg = torch.empty(scratch, dtype=torch.uint8, device=dev) if scratch else None
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self.refresh_weights()

    def refresh_weights(self) -> None:
        """Round the bound recurrent matrix to bf16 again (after an in-place update of ``recurrent``)."""
        self._r_bf16.copy_(self.recurrent)

    # -- launches ------------------------------------------------------------------------------------------------
    def _enqueue(self) -> None:
        """All launches of one pass over the sequence, on the current stream of the tensors' device."""
        B, T, N, D = self.shape
        if self.cell == "slstm":
            # count the non-zero entries of the initial normaliser; "none" is the predicate the kernel wants
            torch.logical_not(torch.count_nonzero(self.initial[2]).reshape(1), out=self._zero_word)
        stream = torch.cuda.current_stream(self.wx.device).cuda_stream
        state_in, start = self.initial, 0
        for index, steps in enumerate(self.chunks):
            state_out = self.carries[index % 2]
            rc = self._lib.frnn_b200_forward_chunk(
                _lib.CELLS[self.cell], self.wx.data_ptr(), int(self.wx.dtype == torch.bfloat16), self._r_bf16.data_ptr(),
                self.bias.data_ptr(), state_in.data_ptr(), self.output.data_ptr(), int(self.snapshot_dtype == torch.bfloat16),
                state_out.data_ptr(), None if self._xchg is None else self._xchg.data_ptr(), B, T, start, steps, N, D,
                self.output_mode, self._zero_word.data_ptr(), 0, self.error_flag.data_ptr(), stream)
            _lib.check(rc, "frnn_b200_forward_chunk")
            state_in, start = state_out, start + steps

    def run(self):
        """One pass over the bound inputs; returns the borrowed ``(output, final)``."""
        with torch.cuda.device(self.wx.device):
            if self._graph is None:
                self._enqueue()
            else:
                self._graph.replay()
        return self.output, self.final

    def capture(self):
        """Record the launches of ``run()`` in a CUDA graph; later ``run()`` calls replay it."""
        if self._graph is not None:
            raise ValueError("sequence is already captured")
        with torch.cuda.device(self.wx.device):
            self._enqueue()                    # one eager pass first: kernel attributes are set outside the capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):      # records on a capture stream of its own and joins the current one
                self._enqueue()
            self._graph = graph
        return self

    def check(self) -> None:
        """Synchronize and raise if a bounded wait inside a kernel ran out (the outputs are then invalid)."""
        code, step, cta = (int(v) for v in self.error_flag[:3].tolist())
        if code:
            raise RuntimeError(f"prepared sequence: device-side wait ran out (code {code}: "
                               f"{_lib.ERROR_TEXT.get(code, '?')}, step {step}, CTA {cta}); outputs are invalid")

    def close(self) -> None:
        """Drop the captured graph (the buffers stay valid; ``run()`` launches eagerly again)."""
        graph, self._graph = self._graph, None
        if graph is not None:
            torch.cuda.synchronize(self.wx.device)
            del graph
