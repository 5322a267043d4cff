"""A whole training step (forward, loss, backward incl. dR/db) recorded into a CUDA graph and replayed: the launches
of the public call are capturable (cluster launches, cooperative launches with their scratch memset, no host read, no
event query while capturing), the replay reproduces the eager step bit for bit, and the error words of the captured
launches are checked by ``poll_errors(block=True)``."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.filterwarnings("ignore:The AccumulateGrad node")   # the warm-up step runs on a side stream on purpose
@pytest.mark.parametrize("shape", [("lstm", 8, 48, 3, 256), ("gru", 16, 24, 1, 768), ("slstm", 6, 20, 2, 128)],
                         ids=lambda s: f"{s[0]}-B{s[1]}-T{s[2]}-N{s[3]}-D{s[4]}")
def test_training_step_in_a_cuda_graph(shape, cuda_device):
    from flashrnn_b200 import flashrnn, poll_errors
    from flashrnn_b200.workloads import make_inputs

    cell, B, T, N, D = shape
    wx, R, b, init = (t.to(cuda_device) for t in make_inputs(cell, B, T, N, D, 5, zero_initial=(cell == "slstm")))
    wx = wx.bfloat16()
    leaves = [t.clone().requires_grad_(True) for t in (wx, R, b, init)]
    # the sLSTM "initial normaliser is all zero" predicate is passed in: computing it would read the device
    extra = {"zero_normalizer": True} if cell == "slstm" else {}

    def step():
        for t in leaves:
            t.grad = None
        h, c = flashrnn(*leaves, function=cell, backend="b200", dtype="bfloat16", **extra)
        (h[0].sum() + c.sum()).backward()
        return h

    eager_h = step().detach().clone()
    eager_g = [t.grad.clone() for t in leaves]
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):       # warm-up off the default stream, as torch asks for before a capture
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graph_h = step()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    poll_errors(block=True)
    assert torch.equal(graph_h, eager_h)
    for t, want in zip(leaves, eager_g):
        assert torch.equal(t.grad, want)

    # new inputs written in place, replayed: equal to an eager step on the same inputs
    with torch.no_grad():
        leaves[0].mul_(0.5)
    graph.replay()
    torch.cuda.synchronize()
    poll_errors(block=True)
    replay_h, replay_g = graph_h.clone(), [t.grad.clone() for t in leaves]
    assert torch.equal(step().detach(), replay_h)
    for t, want in zip(leaves, replay_g):
        assert torch.equal(t.grad, want)
