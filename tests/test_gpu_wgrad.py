"""dR/db contraction kernels (through the C ABI) against a plain fp32 einsum of the same bf16 operands."""

import pytest
import torch

pytestmark = pytest.mark.gpu

# (cell, B, T, N, D): both the TMA-pipelined kernel (D % 64 == 0) and the plain-load kernel
CASES = [
    ("lstm", 8, 96, 2, 64), ("lstm", 3, 70, 1, 128), ("lstm", 8, 256, 3, 256), ("lstm", 2, 65, 1, 384),
    ("lstm", 2, 33, 1, 512), ("elman", 5, 130, 2, 64), ("gru", 16, 80, 1, 128), ("lstm", 4, 1, 2, 64),
    ("lstm", 3, 40, 2, 48), ("gru", 2, 17, 3, 16), ("slstm", 16, 64, 4, 128),
    ("lstm", 16, 200, 5, 32), ("elman", 3, 70, 7, 16), ("lstm", 16, 128, 48, 16),   # narrow heads packed 2 / 4 to a box
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c[0]}-B{c[1]}-T{c[2]}-N{c[3]}-D{c[4]}")
def test_wgrad_matches_einsum(case, cuda_device):
    from flashrnn_b200 import _lib

    cell, B, T, N, D = case
    lib = _lib.load()
    plan = _lib.plan(cell, B, T, N, D)
    assert plan.supported
    gr, gb = plan.gates_r, plan.gates_b
    g = torch.Generator().manual_seed(B * 1000 + T)
    dgr = torch.randn((B, T, gr, N, D), generator=g).to(cuda_device).bfloat16().contiguous()
    hbf = torch.randn((B, T + 1, N, D), generator=g).to(cuda_device).bfloat16().contiguous()
    db_part = torch.randn((plan.n_btiles, gb, N, D), generator=g).to(cuda_device).contiguous()
    dR = torch.full((gr, N, D, D), float("nan"), device=cuda_device)
    db = torch.full((gb, N, D), float("nan"), device=cuda_device)
    work = torch.empty(max(plan.wgrad_work_bytes // 4, 1), dtype=torch.float32, device=cuda_device)
    err = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    rc = lib.frnn_b200_wgrad(_lib.CELLS[cell], dgr.data_ptr(), hbf.data_ptr(), db_part.data_ptr(), dR.data_ptr(),
                             db.data_ptr(), work.data_ptr(), B, T, N, D, err.data_ptr(),
                             torch.cuda.current_stream(cuda_device).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(err[0].item()) == 0
    ref = torch.einsum("btgno,btnp->gnop", dgr.float(), hbf[:, :T].float())
    assert torch.isfinite(dR).all()
    assert (dR - ref).abs().max().item() <= 2e-3 * max(ref.abs().max().item(), 1.0), case
    assert torch.allclose(db, db_part.sum(0), atol=1e-5), case
