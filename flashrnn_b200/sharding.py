"""Host-side helpers for running the recurrence on several GPUs (one process per GPU).

Batch rows and heads are independent in the time loop (block-diagonal R, reference.py:83), so a
rank simply runs the kernels on its slice. What has to be shared:

* under batch sharding every rank holds all of R and b, so dR/db are partial sums that are
  all-reduced once per backward, both in one call (the only collective of the path);
* the sLSTM first-step predicate "all of the initial n is zero" is a reduction over the
  UNSHARDED initial state (state_contract.py:52-58, tests/flashrnn2/test_persistent_contract.py:67-133)
  and must be computed before slicing and handed to every rank.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous near-equal split of ``range(total)``; the first ``total % world`` ranks get one more."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("need world >= 1 and 0 <= rank < world")
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def choose_axis(B: int, N: int, world: int) -> str:
    """'heads' when the heads divide evenly (no collective at all), else 'batch'."""
    if world > 1 and N % world == 0:
        return "heads"
    return "batch"


def slstm_zero_normalizer(initial: torch.Tensor) -> bool:
    """The first-step predicate of one logical call, over the whole (unsharded) initial state."""
    return bool(torch.all(initial[2] == 0))


def shard_inputs(Wx, R, b, states, world: int, rank: int, axis: Optional[str] = None):
    """Slice one logical call for ``rank``. Returns (Wx, R, b, states, axis)."""
    B, _, _, N, _ = Wx.shape
    axis = axis or choose_axis(B, N, world)
    if axis == "heads":
        lo, hi = shard_range(N, world, rank)
        return Wx[:, :, :, lo:hi], R[:, lo:hi], b[:, lo:hi], states[:, :, :, lo:hi], axis
    lo, hi = shard_range(B, world, rank)
    return Wx[lo:hi], R, b, states[:, lo:hi], axis


def _flat_view(dR: torch.Tensor, db: torch.Tensor) -> Optional[torch.Tensor]:
    """One 1-D tensor covering dR followed by db when the two are adjacent pieces of one allocation (the backward
    of the recurrence hands them out that way), else None."""
    if (dR.dtype != db.dtype or not dR.is_contiguous() or not db.is_contiguous() or dR.device != db.device
            or dR.untyped_storage().data_ptr() != db.untyped_storage().data_ptr()
            or db.storage_offset() != dR.storage_offset() + dR.numel()):
        return None
    return torch.as_strided(dR, (dR.numel() + db.numel(),), (1,), dR.storage_offset())


def allreduce_weight_grads(dR: torch.Tensor, db: torch.Tensor, axis: str, group=None) -> None:
    """Sum dR/db over the ranks of a batch-sharded call (in place) with ONE all-reduce: the two gradients
    travel as one flat buffer (no copy when they already are neighbours in memory). A no-op for head sharding."""
    import torch.distributed as dist

    if axis != "batch" or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    flat = _flat_view(dR, db)
    if flat is not None:
        dist.all_reduce(flat, group=group)
        return
    flat = torch.cat((dR.reshape(-1), db.reshape(-1).to(dR.dtype)))
    dist.all_reduce(flat, group=group)
    dR.copy_(flat[:dR.numel()].view_as(dR))
    db.copy_(flat[dR.numel():].view_as(db))


class _SumWeightGrads(torch.autograd.Function):
    """Identity on (R, b) in forward; one all-reduce (sum) of both gradients in backward."""

    @staticmethod
    def forward(ctx, R, b, group):
        ctx.group = group
        return R.view_as(R), b.view_as(b)

    @staticmethod
    def backward(ctx, gR, gb):
        if gR is None or gb is None:  # only one of the two is wanted: nothing to fuse
            import torch.distributed as dist

            for g in (gR, gb):
                if g is not None and dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
                    dist.all_reduce(g, group=ctx.group)
            return gR, gb, None
        if not gR.is_contiguous():
            gR = gR.contiguous()
        if not gb.is_contiguous():
            gb = gb.contiguous()
        allreduce_weight_grads(gR, gb, "batch", ctx.group)
        return gR, gb, None


def flashrnn_sharded(Wx, R, b, states=None, function: str = "lstm", dtype: str = "bfloat16", axis: Optional[str] = None,
                     group=None, zero_normalizer: Optional[bool] = None):
    """Run this rank's shard of one logical ``flashrnn`` call (one process per GPU).

    ``Wx`` / ``states`` are this rank's slice along ``axis`` ("batch" or "heads", see ``shard_inputs``).
    Under batch sharding ``R`` and ``b`` are the full replicated weights and their gradients are
    summed over the ranks during backward (ONE NCCL all-reduce of dR and db together, no collective in the time loop);
    under head sharding ``R`` and ``b`` are this rank's head slice and nothing is exchanged.
    For sLSTM pass ``zero_normalizer = slstm_zero_normalizer(unsharded initial state)``.
    Returns this rank's slice of ``(states[S,B,T,N,D], last[S,B,1,N,D])``.
    """
    from .functional import flashrnn

    if axis is None:
        raise ValueError("say along which axis this rank's tensors were sliced: 'batch' or 'heads'")
    if axis == "batch":
        R, b = _SumWeightGrads.apply(R, b, group)
    elif axis != "heads":
        raise ValueError("axis must be 'batch' or 'heads'")
    return flashrnn(Wx, R, b, states, function=function, backend="b200", dtype=dtype, zero_normalizer=zero_normalizer)
