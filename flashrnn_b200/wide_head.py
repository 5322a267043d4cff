"""One WIDE head (D >= 2048, or any multiple of 256) split row-wise over the GPUs of a node.

Rank r of P (one process per GPU) owns the hidden units ``[r*Dl, (r+1)*Dl)``, ``Dl = D/P``: its slices
``Wx[B,T,G,1,Dl]``, the rows ``R[G,1,Dl,D]`` (all input columns of its output units), ``b[G,1,Dl]`` and
``states[S,B,1,1,Dl]`` go in, its slices of the state history, the carry and all gradients come out (``dR`` as the
same row slice: disjoint over the ranks, no reduction). Inside the kernels the ranks exchange ``round_bf16(h_t)``
(forward) and ``round_bf16(dG_t)`` (backward) every step with peer stores over NVLink; NCCL is not used in the time
loop. Counterpart in the reference: flashrnn/flashrnn2/multi_gpu.py:87-297 (forward only, one process driving all
devices) and the ``_mg`` backward flashrnn/flashrnn2/hybrid_bw2d.cu:645-661.

``WideHead`` owns what outlives a call: the exchange buffers (two full-width bf16 histories per rank), a staging
copy of this rank's rows of R that the peers read when they build their column slices for the backward pass, the
ready flags, and the peers' addresses of all of these (CUDA IPC, exchanged once through ``torch.distributed``
before the first launch). ``WideHead(..., emulate_ranks=P)`` runs all P ranks as ONE launch on one GPU over
full-width tensors: the form used to test the multi-rank arithmetic on a single device (kernels that wait on one
another must never be separate launches on one GPU).
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from .functional import SIZES, _track, poll_errors


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class WideHead:
    """Buffers and peer address tables for calls of one shape ``(cell, B <= 32, T, D)``; use serially on one stream."""

    def __init__(self, cell: str, B: int, T: int, D: int, *, group=None, emulate_ranks: Optional[int] = None,
                 device=None, wx_dtype=torch.bfloat16, k_tmem_max: int = 0, ring_stages_max: int = 0,
                 wait_limit_ms: int = 0):
        if cell not in SIZES:
            raise ValueError(f"unknown cell {cell!r}")
        self.lib = _lib.load()
        self.cell, self.B, self.T, self.D = cell, B, T, D
        self.wx_bf16 = int(wx_dtype == torch.bfloat16)
        self.wait_limit_ms = wait_limit_ms
        self.group = group
        self._epoch = 0
        self.profile = False   # True: CTA 0 of the forward adds up its in-kernel phase timers into last_err[8..19]
        self.last_err = None
        self.jitter = 0        # test hook (race verification): seed of pseudo-random stalls inside both kernels, 0 = off
        self.in_use = False    # True from a training forward until its autograd node is gone (backward done or graph dropped)
        self._owned = []      # cudaMalloc'ed slabs of this process
        self._opened = []     # peer mappings
        gr = SIZES[cell][0]
        if emulate_ranks is not None:
            self.P, self.rank, self.here = int(emulate_ranks), 0, int(emulate_ranks)
            self.device = torch.device(device if device is not None else "cuda")
        else:
            import torch.distributed as dist

            if not dist.is_initialized():
                raise RuntimeError("WideHead needs torch.distributed (one process per GPU) or emulate_ranks=P")
            self.P, self.rank, self.here = dist.get_world_size(group), dist.get_rank(group), 1
            self.device = torch.device("cuda", torch.cuda.current_device())
        if self.P < 1 or self.P > 8:
            raise ValueError("a wide head is split over 1 to 8 ranks")
        self.k_tmem_max, self.ring_stages_max = k_tmem_max, ring_stages_max
        with torch.cuda.device(self.device):
            self.plan = self._plan()
            if not self.plan.supported:
                raise ValueError(
                    f"flashrnn_b200: wide head cell={cell} B={B} D={D} over {self.P} rank(s) is not supported "
                    "(needs B <= 32, D a multiple of 256, D/P a multiple of 128, and CTAs that fit the GPU)")
            self.Dl = self.plan.local_width
            self.lw = D if self.here == self.P else self.Dl   # row length of the local tensors
            r_stage_bytes = gr * self.lw * D * 2 if self.here == self.P else gr * self.Dl * D * 2
            # one slab per rank: [ready flags | rows of R (bf16) | h history | dG history], same layout everywhere
            self._off = {"ready": 0, "r": 256}
            self._off["hbf"] = _align(self._off["r"] + r_stage_bytes)
            self._off["dgr"] = _align(self._off["hbf"] + self.plan.hbf_bytes)
            slab_bytes = _align(self._off["dgr"] + self.plan.dgr_bytes)
            if self.here == self.P:
                # all ranks in this process: one staging copy of the full R, P pairs of histories
                self._slabs = []
                for _ in range(self.P):
                    ptr = ctypes.c_void_p()
                    _lib.check(self.lib.frnn_b200_peer_alloc(slab_bytes, ctypes.byref(ptr)), "frnn_b200_peer_alloc")
                    self._owned.append(ptr.value)
                    self._slabs.append(ptr.value)
                self._r_src = [self._slabs[0] + self._off["r"]] * self.P
            else:
                import torch.distributed as dist

                ptr = ctypes.c_void_p()
                _lib.check(self.lib.frnn_b200_peer_alloc(slab_bytes, ctypes.byref(ptr)), "frnn_b200_peer_alloc")
                self._owned.append(ptr.value)
                handle = ctypes.create_string_buffer(64)
                _lib.check(self.lib.frnn_b200_peer_export(ptr, handle), "frnn_b200_peer_export")
                handles = [None] * self.P
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
                self._slabs = []
                for q in range(self.P):
                    if q == self.rank:
                        self._slabs.append(ptr.value)
                        continue
                    peer = ctypes.c_void_p()
                    _lib.check(self.lib.frnn_b200_peer_open(ctypes.create_string_buffer(handles[q], 64), ctypes.byref(peer)),
                               "frnn_b200_peer_open")
                    self._opened.append(peer.value)
                    self._slabs.append(peer.value)
                self._r_src = [s + self._off["r"] for s in self._slabs]
            # the ready flags start at zero (epochs are positive)
            own = self._slabs[self.rank:self.rank + self.here]
            stream = torch.cuda.current_stream(self.device)
            for s in own:
                _zero = _as_tensor(s, 256, torch.uint8, self.device)
                _zero.zero_()
            stream.synchronize()
            if self.here < self.P:
                import torch.distributed as dist

                dist.barrier(group=group)   # every rank's flags are zero before anybody launches
            self.r_stage = _as_tensor(self._slabs[self.rank] + self._off["r"], r_stage_bytes // 2, torch.bfloat16, self.device)

    # ---- helpers ----
    def _shard(self, which: Optional[str], epoch: int) -> _lib.MgShard:
        sh = _lib.MgShard()
        sh.P, sh.rank, sh.ranks_here, sh.epoch = self.P, self.rank, self.here, epoch
        sh.k_tmem_max, sh.ring_stages_max = self.k_tmem_max, self.ring_stages_max
        if which is not None:
            for q in range(self.P):
                sh.buffers[q] = self._slabs[q] + self._off[which]
                sh.ready[q] = self._slabs[q] + self._off["ready"]
        return sh

    def _plan(self) -> _lib.MgPlan:
        sh = _lib.MgShard()
        sh.P, sh.rank, sh.ranks_here = self.P, self.rank, self.here
        sh.k_tmem_max, sh.ring_stages_max = self.k_tmem_max, self.ring_stages_max
        out = _lib.MgPlan()
        rc = self.lib.frnn_b200_mg_plan(_lib.CELLS[self.cell], self.B, self.T, self.D, self.wx_bf16, ctypes.byref(sh),
                                        ctypes.byref(out))
        if rc != 0:
            raise ValueError(f"frnn_b200_mg_plan failed: {_lib.ERROR_TEXT.get(rc, rc)}")
        return out

    def next_epoch(self) -> int:
        self._epoch += 1
        return self._epoch

    def own_buffer(self, which: str, slot: int = 0) -> int:
        return self._slabs[self.rank + slot] + self._off[which]

    def close(self) -> None:
        """Unmap the peers' buffers and free this process's own (call on every rank, after a barrier)."""
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for ptr in self._opened:
                self.lib.frnn_b200_peer_close(ctypes.c_void_p(ptr))
            for ptr in self._owned:
                self.lib.frnn_b200_peer_free(ctypes.c_void_p(ptr))
        self._opened, self._owned = [], []

    # ---- the call ----
    def __call__(self, Wx, R_rows, b, states=None, zero_normalizer: Optional[bool] = None):
        """``Wx[B,T,G,1,lw], R_rows[G,1,lw,D], b[G,1,lw], states[S,B,1,1,lw]`` (lw = D/P; D with emulate_ranks) ->
        ``(states[S,B,T,1,lw], last[S,B,1,1,lw])``, differentiable in all four inputs."""
        gr, gw, gb, S = SIZES[self.cell]
        B, T, D, lw = self.B, self.T, self.D, self.lw
        if tuple(Wx.shape) != (B, T, gw, 1, lw) or tuple(R_rows.shape) != (gr, 1, lw, D) or tuple(b.shape) != (gb, 1, lw):
            raise ValueError(f"wide head: expected Wx {(B, T, gw, 1, lw)}, R rows {(gr, 1, lw, D)}, b {(gb, 1, lw)}")
        if states is None:
            states = torch.zeros((S, B, 1, 1, lw), dtype=torch.float32, device=Wx.device)
        elif tuple(states.shape) != (S, B, 1, 1, lw):
            raise ValueError(f"wide head: expected states {(S, B, 1, 1, lw)}")
        if int(Wx.dtype == torch.bfloat16) != self.wx_bf16:
            raise ValueError("Wx dtype differs from the one this WideHead was planned for")
        zero_first = False
        if self.cell == "slstm":
            if zero_normalizer is not None:
                zero_first = bool(zero_normalizer)
            else:
                flag = torch.all(states[2] == 0).to(torch.int32)
                if self.here < self.P:
                    import torch.distributed as dist

                    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)   # the predicate of the UNSHARDED state
                zero_first = bool(flag.item())
        with torch.autocast("cuda", enabled=False):
            return _WideRecurrence.apply(Wx, R_rows, b.to(torch.float32), states.to(torch.float32), self, zero_first)


class _Lease:
    """Held by the autograd node of a training forward: the head's exchange buffers are the saved operands of its
    backward pass, so the head must not run another forward until the node is gone."""

    def __init__(self, head: WideHead):
        self.head = head
        head.in_use = True

    def __del__(self):
        self.head.in_use = False


def _as_tensor(ptr: int, numel: int, dtype, device) -> torch.Tensor:
    """A torch view of raw device memory owned by the library's peer allocator."""
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Raw:
        pass

    raw = _Raw()
    typestr = {torch.uint8: "|u1", torch.bfloat16: "<u2", torch.int32: "<i4", torch.float32: "<f4"}[dtype]
    raw.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 2}
    t = torch.as_tensor(raw, device=device)
    return t.view(dtype) if dtype == torch.bfloat16 else t


class _WideRecurrence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, wx, r_rows, bias, initial, head: WideHead, zero_first: bool):
        with torch.cuda.device(head.device):
            lib = head.lib
            poll_errors()
            gr, gw, gb, S = SIZES[head.cell]
            B, T, D, lw = head.B, head.T, head.D, head.lw
            dev = wx.device
            wx_c = wx.contiguous()
            b32 = bias.detach().to(torch.float32).contiguous()
            init32 = initial.detach().to(torch.float32).contiguous()
            head.r_stage.copy_(r_rows.detach().reshape(-1))          # fp32 -> bf16 once; the peers read it in backward
            history = torch.empty((S, B, T, 1, lw), dtype=torch.float32, device=dev)
            carry = torch.empty((S, B, 1, 1, lw), dtype=torch.float32, device=dev)
            train = any(ctx.needs_input_grad[:4])
            if train:
                ctx.lease = _Lease(head)
            cache = torch.empty(head.plan.cache_bytes, dtype=torch.uint8, device=dev) if train and head.plan.cache_bytes else None
            err = torch.zeros(32, dtype=torch.int32, device=dev)
            if head.profile:
                err[3] = 1
                head.last_err = err
            if head.jitter:
                err[6] = int(head.jitter)
            sh = head._shard("hbf", head.next_epoch())
            rc = lib.frnn_b200_mg_forward(
                _lib.CELLS[head.cell], wx_c.data_ptr(), head.wx_bf16, head.r_stage.data_ptr(), b32.data_ptr(), init32.data_ptr(),
                history.data_ptr(), carry.data_ptr(), None if cache is None else cache.data_ptr(), ctypes.byref(sh),
                B, T, D, int(zero_first), head.wait_limit_ms, err.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
            _lib.check(rc, "frnn_b200_mg_forward")
            _track(err, "frnn_b200_mg_forward")
            if train:
                ctx.save_for_backward(init32, history, cache if cache is not None else history.new_empty(0))
                ctx.head, ctx.zero_first = head, zero_first
                ctx.dtypes = (wx.dtype, r_rows.dtype, bias.dtype, initial.dtype)
            return history, carry

    @staticmethod
    def backward(ctx, d_history, d_carry):
        head: WideHead = ctx.head
        with torch.cuda.device(head.device):
            lib = head.lib
            poll_errors()
            init32, history, cache = ctx.saved_tensors
            gr, gw, gb, S = SIZES[head.cell]
            B, T, D, lw = head.B, head.T, head.D, head.lw
            dev = history.device
            stream = torch.cuda.current_stream(dev).cuda_stream
            cid = _lib.CELLS[head.cell]
            d_history = (torch.zeros_like(history) if d_history is None else d_history).to(torch.float32).contiguous()
            d_carry = (torch.zeros((S, B, 1, 1, lw), dtype=torch.float32, device=dev) if d_carry is None else d_carry)
            d_carry = d_carry.to(torch.float32).contiguous()
            # this rank's columns of R, from the row slices every rank staged in its forward call
            r_cols = torch.empty(head.plan.r_cols_bytes // 2, dtype=torch.bfloat16, device=dev)
            sh0 = head._shard(None, 0)
            rows = (ctypes.c_void_p * head.P)(*head._r_src)
            _lib.check(lib.frnn_b200_mg_gather_columns(cid, rows, r_cols.data_ptr(), ctypes.byref(sh0), D, stream),
                       "frnn_b200_mg_gather_columns")
            dwx = torch.empty((B, T, gw, 1, lw), dtype=ctx.dtypes[0], device=dev)
            d_initial = torch.empty((S, B, 1, 1, lw), dtype=torch.float32, device=dev)
            db_part = torch.empty(head.plan.dbpart_bytes // 4, dtype=torch.float32, device=dev)
            dR = torch.empty((gr, 1, lw, D), dtype=torch.float32, device=dev)
            db = torch.empty((gb, 1, lw), dtype=torch.float32, device=dev)
            err = torch.zeros(32, dtype=torch.int32, device=dev)
            if head.jitter:
                err[6] = int(head.jitter)
            sh = head._shard("dgr", head.next_epoch())
            rc = lib.frnn_b200_mg_backward(
                cid, cache.data_ptr() if cache.numel() else None, history.data_ptr(), init32.data_ptr(), r_cols.data_ptr(),
                d_history.data_ptr(), d_carry.data_ptr(), dwx.data_ptr(), head.wx_bf16, d_initial.data_ptr(), db_part.data_ptr(),
                ctypes.byref(sh), B, T, D, int(ctx.zero_first), head.wait_limit_ms, err.data_ptr(), stream)
            _lib.check(rc, "frnn_b200_mg_backward")
            rc = lib.frnn_b200_mg_wgrad(cid, head.own_buffer("dgr"), head.own_buffer("hbf"), db_part.data_ptr(), dR.data_ptr(),
                                        db.data_ptr(), ctypes.byref(sh), B, T, D, head.plan.bwd_ksplit, err.data_ptr(), stream)
            _lib.check(rc, "frnn_b200_mg_wgrad")
            _track(err, "frnn_b200_mg_backward")
            need = ctx.needs_input_grad
            return (dwx if need[0] else None, dR.to(ctx.dtypes[1]) if need[1] else None,
                    db.to(ctx.dtypes[2]) if need[2] else None, d_initial.to(ctx.dtypes[3]) if need[3] else None, None, None)
