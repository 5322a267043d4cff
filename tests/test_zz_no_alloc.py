"""The allocation-free dR/db entry point against the regular one.

Some callers of the library cannot provide scratch memory (no cudaMalloc allowed while they run,
a fixed memory budget, or only input/output pointers in hand); `frnn_b200_wgrad_noalloc` keeps
its split-K partial tiles in an array built into the library instead. This file checks, through
the C ABI, that it returns what `frnn_b200_wgrad` returns, on two calls in a row with different
inputs (the shared array keeps the first call's contents, which must not leak into the second).
It is named so that pytest collects it last.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _wgrad_both(lib, _lib, cell, B, T, N, D, seed, dev):
    plan = _lib.plan(cell, B, T, N, D)
    assert plan.supported and plan.wgrad_ksplit > 1, "the case must actually use split-K scratch"
    g = torch.Generator().manual_seed(seed)
    gr, gb = plan.gates_r, plan.gates_b
    dgr = torch.randn((B, T, gr, N, D), generator=g).to(dev).bfloat16().contiguous()
    hbf = torch.randn((B, T + 1, N, D), generator=g).to(dev).bfloat16().contiguous()
    db_part = torch.randn((plan.n_btiles, gb, N, D), generator=g).to(dev).contiguous()
    stream = torch.cuda.current_stream(dev).cuda_stream
    outs = []
    for noalloc in (False, True):
        dR = torch.full((gr, N, D, D), float("nan"), device=dev)
        db = torch.full((gb, N, D), float("nan"), device=dev)
        err = torch.zeros(32, dtype=torch.int32, device=dev)
        if noalloc:
            rc = lib.frnn_b200_wgrad_noalloc(_lib.CELLS[cell], dgr.data_ptr(), hbf.data_ptr(), db_part.data_ptr(),
                                             dR.data_ptr(), db.data_ptr(), B, T, N, D, err.data_ptr(), stream)
        else:
            work = torch.empty(plan.wgrad_work_bytes // 4, dtype=torch.float32, device=dev)
            rc = lib.frnn_b200_wgrad(_lib.CELLS[cell], dgr.data_ptr(), hbf.data_ptr(), db_part.data_ptr(),
                                     dR.data_ptr(), db.data_ptr(), work.data_ptr(), B, T, N, D, err.data_ptr(), stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert int(err[0].item()) == 0
        outs.append((dR, db))
    # independent check of the contraction itself
    ref = torch.einsum("btgno,btnp->gnop", dgr.float(), hbf[:, :T].float())
    return outs, ref


def test_noalloc_wgrad_matches_regular_entry_point_twice(cuda_device):
    from flashrnn_b200 import _lib

    lib = _lib.load()
    for call, (cell, B, T, N, D, seed) in enumerate([("lstm", 8, 96, 2, 64, 91), ("gru", 16, 80, 1, 128, 92)]):
        (regular, static), ref = _wgrad_both(lib, _lib, cell, B, T, N, D, seed, cuda_device)
        for a, b in zip(regular, static):
            assert torch.isfinite(b).all(), call
            scale = a.abs().max().item()
            assert (a - b).abs().max().item() <= max(2e-2, 1e-2 * scale), call
        assert (regular[0] - ref).abs().max().item() <= 1e-2 * ref.abs().max().item(), call


def test_noalloc_packed_and_plain_load_kernels_back_to_back(cuda_device):
    """The built-in array also serves the kernel for widths that are not multiples of 64 (plain loads) and the
    narrow-head kernel that packs several heads into one tile. Different shapes and seeds in a row: whatever an
    earlier call left in the array must not show up in a later result. dR against an fp32 einsum of the same bf16
    operands, db against the plain sum of the per-tile partials."""
    from flashrnn_b200 import _lib

    lib = _lib.load()
    cases = [("lstm", 16, 200, 5, 32, 93), ("lstm", 8, 300, 2, 48, 94), ("elman", 16, 128, 6, 32, 95),
             ("lstm", 6, 150, 2, 80, 96), ("gru", 8, 256, 3, 48, 97)]
    for call, (cell, B, T, N, D, seed) in enumerate(cases):
        plan = _lib.plan(cell, B, T, N, D)
        assert plan.supported and plan.wgrad_ksplit > 1
        g = torch.Generator().manual_seed(seed)
        gr, gb = plan.gates_r, plan.gates_b
        dgr = torch.randn((B, T, gr, N, D), generator=g).to(cuda_device).bfloat16().contiguous()
        hbf = torch.randn((B, T + 1, N, D), generator=g).to(cuda_device).bfloat16().contiguous()
        db_part = torch.randn((plan.n_btiles, gb, N, D), generator=g).to(cuda_device).contiguous()
        dR = torch.full((gr, N, D, D), float("nan"), device=cuda_device)
        db = torch.full((gb, N, D), float("nan"), device=cuda_device)
        err = torch.zeros(32, dtype=torch.int32, device=cuda_device)
        rc = lib.frnn_b200_wgrad_noalloc(_lib.CELLS[cell], dgr.data_ptr(), hbf.data_ptr(), db_part.data_ptr(),
                                         dR.data_ptr(), db.data_ptr(), B, T, N, D, err.data_ptr(),
                                         torch.cuda.current_stream(cuda_device).cuda_stream)
        assert rc == 0, (call, rc)
        torch.cuda.synchronize()
        assert int(err[0].item()) == 0
        ref = torch.einsum("btgno,btnp->gnop", dgr.float(), hbf[:, :T].float())
        assert torch.isfinite(dR).all(), call
        assert (dR - ref).abs().max().item() <= 2e-3 * max(ref.abs().max().item(), 1.0), (call, cell, D)
        assert torch.allclose(db, db_part.sum(0), atol=1e-5), call


def test_noalloc_rejects_oversized_problem(cuda_device):
    from flashrnn_b200 import _lib

    lib = _lib.load()
    cell, B, T, N, D = "lstm", 8, 1024, 3, 256   # split-K partials need 18 MiB, more than the built-in 16 MiB
    plan = _lib.plan(cell, B, T, N, D)
    assert plan.wgrad_work_bytes > 16 * 1024 * 1024
    one = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    rc = lib.frnn_b200_wgrad_noalloc(_lib.CELLS[cell], one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                     one.data_ptr(), B, T, N, D, one.data_ptr(), 0)
    assert rc == -6
