"""Preallocated forward-only execution of one sequence shape with an explicit output policy.

Mirrors the reference's ``PreparedSequence`` (flashrnn/flashrnn2/prepared.py:18-192): inputs,
weights and outputs have fixed addresses; results are borrowed buffers that the next ``run()``
overwrites; one instance is used serially on one CUDA stream; ``capture()`` records the launch
in a CUDA graph so that ``run()`` becomes a graph replay. Update the bound input tensors in place
(``seq.wx.copy_(...)``) before ``run()``.

Differences: the state history / hidden snapshots are fp32, ``chunks`` other than the whole
sequence are not supported, and Wx may be bf16 or fp32 while R is rounded to bf16 once, when the
instance is created or ``refresh_weights()`` is called.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .functional import SIZES

_MODES = {"full": 0, "hidden": 1, "last": 2}


class PreparedSequence:
    def __init__(self, wx, recurrent, bias, initial, cell: str = "lstm", *, output_mode: str = "full", chunks=None):
        if output_mode not in _MODES:
            raise ValueError("output mode must be full, hidden or last")
        if cell not in SIZES:
            raise ValueError(f"unknown cell {cell!r}")
        if wx.ndim != 5:
            raise ValueError("expected Wx [B,T,G,N,D]")
        gr, gw, gb, states = SIZES[cell]
        batch, steps, gates, heads, width = wx.shape
        if gates != gw or batch < 1 or steps < 1 or heads < 1 or width < 1:
            raise ValueError("expected nonempty B/T/N/D and the cell's number of input gates")
        if recurrent.shape != (gr, heads, width, width) or bias.shape != (gb, heads, width):
            raise ValueError("invalid recurrent-weight or bias shape")
        if initial.shape != (states, batch, 1, heads, width):
            raise ValueError("invalid initial-state shape")
        tensors = (wx, recurrent, bias, initial)
        if not wx.is_cuda or any(x.device != wx.device or not x.is_contiguous() for x in tensors):
            raise ValueError("prepared execution requires contiguous tensors on one CUDA device")
        if wx.dtype not in (torch.bfloat16, torch.float32) or bias.dtype != torch.float32 or initial.dtype != torch.float32:
            raise ValueError("Wx must be bf16 or fp32; bias and the initial state fp32")
        if any(x.requires_grad for x in tensors):
            raise ValueError("prepared execution is forward-only")
        if chunks is not None and tuple(chunks) != (steps,):
            raise ValueError("prepared execution runs the sequence as one chunk")
        if width % 16:
            raise ValueError("prepared execution needs a head width that is a multiple of 16")
        plan = _lib.plan(cell, batch, steps, heads, width)
        if not plan.supported:
            raise ValueError(f"cell={cell} B={batch} N={heads} D={width} is outside the sm_100a kernel family")
        self._lib = _lib.load()
        self.wx, self.recurrent, self.bias, self.initial = tensors
        self.cell, self.shape = cell, (batch, steps, heads, width)
        self.output_mode = _MODES[output_mode]
        dev = wx.device
        shape = (states, batch, steps, heads, width) if output_mode == "full" else (
            batch, 1 if output_mode == "last" else steps, heads, width)
        self.output = torch.empty(shape, dtype=torch.float32, device=dev)
        self.final = torch.empty((states, batch, 1, heads, width), dtype=torch.float32, device=dev)
        self._r_bf16 = torch.empty(recurrent.shape, dtype=torch.bfloat16, device=dev)
        self._zero = torch.zeros((1,), dtype=torch.int32, device=dev)       # sLSTM predicate, refreshed by every run
        self._zero_mask = torch.empty(initial[0].shape, dtype=torch.bool, device=dev)
        self._zero_all = torch.empty((), dtype=torch.bool, device=dev)
        self._xchg = torch.empty(max(plan.xchg_bytes, 16), dtype=torch.uint8, device=dev)
        self._xchg_ptr = self._xchg.data_ptr() if plan.exchange else None
        self.error_flag = torch.zeros(32, dtype=torch.int32, device=dev)
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self.refresh_weights()

    def refresh_weights(self) -> None:
        """Round the bound recurrent matrix to bf16 again (call after updating ``recurrent`` in place)."""
        self._r_bf16.copy_(self.recurrent)

    def _execute(self):
        if self.cell == "slstm":  # "all n == 0", on the device: no host read, so the run can be captured
            torch.eq(self.initial[2], 0, out=self._zero_mask)
            torch.all(self._zero_mask, out=self._zero_all)
            self._zero.copy_(self._zero_all.reshape(1))
        batch, steps, heads, width = self.shape
        rc = self._lib.frnn_b200_forward_prepared(
            _lib.CELLS[self.cell], self.wx.data_ptr(), int(self.wx.dtype == torch.bfloat16), self._r_bf16.data_ptr(),
            self.bias.data_ptr(), self.initial.data_ptr(), self.output.data_ptr(), self.final.data_ptr(), self._xchg_ptr,
            batch, steps, heads, width, self.output_mode, self._zero.data_ptr(), 0, self.error_flag.data_ptr(),
            torch.cuda.current_stream(self.wx.device).cuda_stream,
        )
        _lib.check(rc, "frnn_b200_forward_prepared")
        return self.output, self.final

    def check(self) -> None:
        """Synchronize and raise if a bounded wait inside the kernel ran out (outputs are then invalid)."""
        code, step, cta = (int(v) for v in self.error_flag[:3].tolist())
        if code != 0:
            raise RuntimeError(f"prepared sequence: device-side wait ran out (code {code}: "
                               f"{_lib.ERROR_TEXT.get(code, '?')}, step {step}, CTA {cta}); outputs are invalid")

    def run(self):
        if self._graph is not None:
            self._graph.replay()
            return self.output, self.final
        return self._execute()

    def capture(self):
        if self._graph is not None:
            raise ValueError("sequence is already captured")
        with torch.cuda.device(self.wx.device):
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(3):
                    self._execute()
            torch.cuda.current_stream().wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._execute()
            self._graph = graph
        return self

    def close(self) -> None:
        if self._graph is not None:
            torch.cuda.synchronize(self.wx.device)
            self._graph.reset()
            self._graph = None
