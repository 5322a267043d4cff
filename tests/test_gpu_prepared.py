"""Prepared (preallocated, forward-only, replayable) sequences against the CPU oracle and the ordinary forward call.

Follows the reference's tests of PreparedSequence (tests/flashrnn2/test_prepared.py): every output
mode returns the same numbers as the full call, the captured graph replays on updated inputs, and
the sLSTM zero-normaliser predicate is evaluated on the device at every run."""

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16_MMA = "fp32_state_bf16_mma"


def _inputs(cell, B, T, N, D, seed, dev, zero=False, dtype=torch.float32):
    from flashrnn_b200.workloads import make_inputs

    wx, R, b, init = (t.to(dev) for t in make_inputs(cell, B, T, N, D, seed, zero))
    return wx.to(dtype).contiguous(), R.contiguous(), b.contiguous(), init.contiguous()


@pytest.mark.parametrize("shape", [("lstm", 8, 16, 3, 256), ("gru", 5, 9, 2, 48), ("slstm", 16, 12, 4, 128),
                                   ("elman", 3, 7, 1, 64), ("lstm", 4, 6, 1, 768), ("slstm", 3, 5, 1, 1024)],
                         ids=lambda s: f"{s[0]}-B{s[1]}-T{s[2]}-N{s[3]}-D{s[4]}")
def test_output_modes_match_the_full_call(shape, cuda_device):
    from flashrnn_b200 import PreparedSequence, flashrnn_torch

    cell, B, T, N, D = shape
    for zero in ((False, True) if cell == "slstm" else (False,)):
        wx, R, b, init = _inputs(cell, B, T, N, D, 71, cuda_device, zero)
        ref_h, ref_c = flashrnn_torch(wx, R, b, init, cell=cell, numerics=BF16_MMA)
        for mode in ("full", "hidden", "last"):
            seq = PreparedSequence(wx, R, b, init, cell, output_mode=mode)
            out, final = seq.run()
            seq.check()
            want = ref_h if mode == "full" else (ref_h[0] if mode == "hidden" else ref_h[0, :, -1:])
            assert out.shape == want.shape and torch.equal(out, want), (shape, zero, mode)
            assert torch.equal(final, ref_c), (shape, zero, mode)


# a cluster launch and a cooperative launch (wide head, exchange through global memory)
@pytest.mark.parametrize("shape", [("slstm", 8, 24, 2, 128), ("slstm", 4, 10, 1, 768)], ids=["cluster", "global"])
def test_captured_graph_replays_on_updated_inputs(shape, cuda_device):
    from flashrnn_b200 import PreparedSequence, flashrnn_torch

    cell, B, T, N, D = shape
    wx, R, b, init = _inputs(cell, B, T, N, D, 72, cuda_device, zero=True, dtype=torch.bfloat16)
    seq = PreparedSequence(wx, R, b, init, cell, output_mode="hidden").capture()
    out, final = seq.run()
    seq.check()
    ref_h, ref_c = flashrnn_torch(wx.float(), R, b, init, cell=cell, numerics=BF16_MMA)
    assert torch.equal(out, ref_h[0]) and torch.equal(final, ref_c)
    # new inputs and a non-zero normaliser, written into the bound tensors: the replay must pick both up
    wx2, _, _, init2 = _inputs(cell, B, T, N, D, 73, cuda_device, zero=False, dtype=torch.bfloat16)
    seq.wx.copy_(wx2)
    seq.initial.copy_(init2)
    out, final = seq.run()
    seq.check()
    ref_h, ref_c = flashrnn_torch(wx2.float(), R, b, init2, cell=cell, numerics=BF16_MMA)
    assert torch.equal(out, ref_h[0]) and torch.equal(final, ref_c)
    with pytest.raises(ValueError):
        seq.capture()
    seq.close()


def test_prepared_argument_checks(cuda_device):
    from flashrnn_b200 import PreparedSequence

    wx, R, b, init = _inputs("lstm", 2, 3, 1, 32, 74, cuda_device)
    with pytest.raises(ValueError, match="output mode"):
        PreparedSequence(wx, R, b, init, "lstm", output_mode="everything")
    with pytest.raises(ValueError, match="forward-only"):
        PreparedSequence(wx.clone().requires_grad_(True), R, b, init, "lstm")
    with pytest.raises(ValueError, match="totaling T"):
        PreparedSequence(wx, R, b, init, "lstm", chunks=(1, 1))
    with pytest.raises(ValueError, match="totaling T"):
        PreparedSequence(wx, R, b, init, "lstm", chunks=(3, 0))
    with pytest.raises(ValueError, match="snapshot dtype"):
        PreparedSequence(wx, R, b, init, "lstm", snapshot_dtype=torch.float16)
    with pytest.raises(ValueError, match="initial-state"):
        PreparedSequence(wx, R, b, init[:1], "lstm")


# cluster path, exchange through global memory, contraction split over clusters
@pytest.mark.parametrize("shape", [("lstm", 8, 20, 3, 256), ("slstm", 6, 17, 2, 128), ("gru", 5, 12, 1, 768),
                                   ("elman", 3, 9, 1, 1024)], ids=lambda s: f"{s[0]}-B{s[1]}-T{s[2]}-N{s[3]}-D{s[4]}")
def test_every_output_mode_and_chunking_against_the_oracle(shape, cuda_device):
    """Output modes, chunked execution with alternating carries and bf16 snapshots, checked against the CPU oracle
    (tolerance of the parity tests: max-abs 2e-2, or 1e-2 of max|ref| for large tensors) and, bit for bit, against the
    single-launch run: chunking must not change a single value (fp32 carries), bf16 snapshots are the rounded fp32 ones."""
    from flashrnn_b200 import PreparedSequence
    from flashrnn_b200.workloads import make_inputs
    from oracle import recurrence_port as port

    cell, B, T, N, D = shape
    for zero in ((True, False) if cell == "slstm" else (False,)):
        cpu = make_inputs(cell, B, T, N, D, 75, zero)
        ref_h, ref_c, _ = port.forward(*cpu, cell)
        wx, R, b, init = (t.to(cuda_device).contiguous() for t in cpu)

        def close(got, want):
            err = (got.float().cpu() - want).abs().max().item()
            return err <= 2e-2 or err <= 1e-2 * want.abs().max().item()

        whole = {}
        for mode in ("full", "hidden", "last"):
            seq = PreparedSequence(wx, R, b, init, cell, output_mode=mode)
            out, final = seq.run()
            seq.check()
            want = ref_h if mode == "full" else (ref_h[0] if mode == "hidden" else ref_h[0, :, -1:])
            assert out.shape == want.shape and close(out, want), (shape, zero, mode)
            assert close(final, ref_c), (shape, zero, mode)
            whole[mode] = (out.clone(), final.clone())
        chunks = (T // 3, 1, T - T // 3 - 1)
        for mode in ("full", "hidden", "last"):
            seq = PreparedSequence(wx, R, b, init, cell, output_mode=mode, chunks=chunks)
            assert seq.final is seq.carries[(len(chunks) - 1) % 2]
            out, final = seq.run()
            seq.check()
            assert torch.equal(out, whole[mode][0]) and torch.equal(final, whole[mode][1]), (shape, zero, mode, "chunks")
            snap = PreparedSequence(wx, R, b, init, cell, output_mode=mode, chunks=chunks, snapshot_dtype=torch.bfloat16)
            out16, final16 = snap.run()
            snap.check()
            assert out16.dtype == torch.bfloat16 and final16.dtype == torch.float32
            assert torch.equal(out16, whole[mode][0].bfloat16()) and torch.equal(final16, whole[mode][1]), (shape, zero, mode, "bf16")
        # one launch per step (every exchange of the persistent kernel replaced by a kernel boundary) == the persistent run
        steps = PreparedSequence(wx, R, b, init, cell, output_mode="full", chunks=(1,) * T)
        out, final = steps.run()
        steps.check()
        assert torch.equal(out, whole["full"][0]) and torch.equal(final, whole["full"][1]), (shape, zero, "per-step launches")


def test_chunked_sequence_in_a_graph(cuda_device):
    """Three chunk launches (the sLSTM predicate only counts in the first) captured in one graph, replayed on new inputs."""
    from flashrnn_b200 import PreparedSequence, flashrnn_torch

    cell, B, T, N, D = "slstm", 8, 18, 2, 128
    wx, R, b, init = _inputs(cell, B, T, N, D, 76, cuda_device, zero=True, dtype=torch.bfloat16)
    seq = PreparedSequence(wx, R, b, init, cell, output_mode="full", chunks=(5, 6, 7), snapshot_dtype=torch.bfloat16).capture()
    for seed, zero in ((76, True), (77, False)):
        wx2, _, _, init2 = _inputs(cell, B, T, N, D, seed, cuda_device, zero=zero, dtype=torch.bfloat16)
        seq.wx.copy_(wx2)
        seq.initial.copy_(init2)
        out, final = seq.run()
        seq.check()
        ref_h, ref_c = flashrnn_torch(wx2.float(), R, b, init2, cell=cell, numerics=BF16_MMA)
        assert torch.equal(out, ref_h.bfloat16()) and torch.equal(final, ref_c)
    seq.close()
    out, final = seq.run()   # eager again after close()
    assert torch.equal(final, ref_c)
