"""Race verification by delay injection: with err[6] = seed the kernels stall, in a quarter of the steps and for up
to 8 us, the epilogue warps or the tensor-core warp of pseudo-randomly chosen CTAs, so that the CTAs of a group (and
the warp roles inside a CTA) drift against each other at every hand-off of the exchange protocols (operand pushes,
partial sums, staged stores, slot reuse). Every result must stay bit-identical to the undisturbed run. The hook is
compiled into the fp32-Wx instantiations of the kernels (the exchange code is the same for both Wx types).

The reference verifies its persistent kernels the same way (tools/race_verify.py: seeded 0-65 us delays plus a content
check of every exchanged operand)."""

import pytest
import torch

from tests.test_gpu_timeout import _backward, _buffers, _forward

pytestmark = pytest.mark.gpu

# every exchange path: thread-block cluster (8- and 16-row tiles, 16-unit slices), global memory with one CTA per
# unit slice, K split inside clusters + global publication (forward and backward), and the 1-D backward over global memory
SHAPES = [
    ("lstm", 8, 40, 3, 256), ("gru", 5, 33, 2, 128), ("slstm", 16, 24, 4, 128), ("elman", 9, 30, 1, 512),
    ("lstm", 200, 16, 4, 128), ("lstm", 24, 20, 2, 48),
    ("lstm", 4, 24, 1, 576), ("gru", 8, 16, 1, 768), ("lstm", 16, 16, 1, 1024), ("lstm", 64, 12, 1, 768),
]
OUTPUTS_FWD = ("hist", "carry", "cache", "hbf")
OUTPUTS_BWD = ("dwx", "dgr", "dinit", "dbp")


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}-B{s[1]}-T{s[2]}-N{s[3]}-D{s[4]}")
def test_results_do_not_depend_on_injected_delays(shape, cuda_device):
    from flashrnn_b200 import _lib

    lib = _lib.load()
    cell, B, T, N, D = shape
    assert _lib.plan(cell, B, T, N, D).supported
    t = _buffers(_lib, cell, B, T, N, D, cuda_device)
    t["dH"] = torch.randn(t["hist"].shape, generator=torch.Generator().manual_seed(3)).to(cuda_device)
    err = torch.zeros(32, dtype=torch.int32, device=cuda_device)

    def run(seed):
        err.zero_()
        err[6] = seed
        assert _forward(lib, _lib, cell, B, T, N, D, t, err, 0) == 0
        torch.cuda.synchronize()
        assert err[0].item() == 0, err[:3].tolist()
        fwd = {k: t[k].clone() for k in OUTPUTS_FWD}
        err.zero_()
        err[6] = seed
        assert _backward(lib, _lib, cell, B, T, N, D, t, err, 0) == 0
        torch.cuda.synchronize()
        assert err[0].item() == 0, err[:3].tolist()
        return {**fwd, **{k: t[k].clone() for k in OUTPUTS_BWD}}

    def same(a, b):   # bit patterns (the gate cache is raw bytes, NaNs cannot occur in the rest)
        return torch.equal(a.view(torch.uint8).flatten(), b.view(torch.uint8).flatten())

    calm = run(0)
    for seed in (1, 77, 4242):
        shaken = run(seed)
        for key, want in calm.items():
            assert same(shaken[key], want), (shape, seed, key)


@pytest.mark.parametrize("case", [("lstm", 8, 20, 1024, 4, 0, 0), ("gru", 5, 16, 512, 2, 0, 0), ("lstm", 6, 12, 2048, 1, 0, 0),
                                  ("lstm", 4, 10, 2048, 2, 128, 3)],
                         ids=lambda c: f"{c[0]}-B{c[1]}-T{c[2]}-D{c[3]}-P{c[4]}-kt{c[5]}")
def test_wide_head_results_do_not_depend_on_injected_delays(case, cuda_device):
    """The row-sharded kernels (all ranks as one launch): write-once history slots, cluster K reduction, staged publication."""
    from flashrnn_b200 import poll_errors
    from flashrnn_b200.wide_head import WideHead
    from tests.test_gpu_wide_head import _inputs

    cell, B, T, D, P, kt, rs = case
    wx, R, b, init, d_history, d_carry = _inputs(cell, B, T, D, 31)
    # fp32 Wx: the hook is compiled into those instantiations (the exchange code does not depend on the Wx type)
    head = WideHead(cell, B, T, D, emulate_ranks=P, device=cuda_device, wx_dtype=torch.float32, k_tmem_max=kt,
                    ring_stages_max=rs, wait_limit_ms=3000)
    try:
        def run(seed):
            head.jitter = seed
            leaves = [x.to(cuda_device).requires_grad_(True) for x in (wx, R, b, init)]
            h, c = head(*leaves)
            ((h * d_history.to(cuda_device)).sum() + (c * d_carry.to(cuda_device)).sum()).backward()
            torch.cuda.synchronize()
            poll_errors(block=True)
            return [h.detach().clone(), c.detach().clone()] + [x.grad.clone() for x in leaves]

        calm = run(0)
        for seed in (5, 909):
            for got, want in zip(run(seed), calm):
                assert torch.equal(got, want), (case, seed)
    finally:
        head.close()
