"""CPU-side checks: the library loads and exports the declared ABI; host argument checks."""

import re
from pathlib import Path

import pytest
import torch

from flashrnn_b200 import _lib, flashrnn, flashrnn_torch
from flashrnn_b200.workloads import make_inputs

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "flashrnn_b200.h").read_text()
    declared = set(re.findall(r"^int\s+(frnn_b200_\w+)\s*\(", header, flags=re.M))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), (declared, set(_lib.SIGNATURES))
    lib = _lib.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.frnn_b200_version() >= 1000


def test_plan_describes_the_headline_workload():
    p = _lib.plan("lstm", 8, 1024, 3, 256)
    assert (p.gates_r, p.gates_w, p.gates_b, p.states) == (4, 4, 4, 2)
    assert (p.unit, p.cluster, p.batch_tile, p.n_btiles, p.grid_ctas, p.supported) == (32, 8, 8, 1, 24, 1)
    assert p.cache_bytes == 8 * 1024 * 4 * 3 * 256 * 2 and p.hbf_bytes == 8 * 1025 * 3 * 256 * 2
    g = _lib.plan("gru", 16, 10, 2, 48)
    assert (g.gates_r, g.gates_b, g.unit, g.cluster, g.batch_tile, g.n_btiles) == (3, 4, 16, 3, 8, 2)
    big = _lib.plan("lstm", 256, 16, 32, 128)                # more groups than SMs: 16-row batch tiles
    assert (big.batch_tile, big.n_btiles, big.cluster) == (16, 16, 4)
    wide = _lib.plan("lstm", 16, 8, 1, 768)                  # wider than a cluster: global-memory exchange
    assert wide.supported and wide.exchange == 1 and wide.xchg_bytes > 0
    assert wide.fwd_ksplit == 2 and wide.fwd_ctas == 2 * 48   # the forward splits the contraction over two CTAs per row tile
    assert wide.bwd_ksplit == 8 and wide.cluster == 6 * 8      # the backward owns columns of R: 6 unit tiles x 8 chunks of the 3072 gate rows
    many = _lib.plan("lstm", 64, 8, 1, 768)                    # four 16-row groups: only the narrower split fits the SMs
    assert many.supported and many.batch_tile == 16 and many.bwd_ksplit == 4 and many.fwd_ctas == 4 * 24
    wider = _lib.plan("lstm", 8, 8, 1, 1024)                   # rows of R beyond one CTA's tensor memory: 16-unit backward slices
    assert wider.supported and wider.exchange == 2 and wider.unit == 16 and wider.cluster == 64
    assert wider.fwd_ksplit == 4 and wider.fwd_ctas == 32 * 4 and wider.fwd_batch_tile == 8   # one 8-row group: the wider forward split fits
    assert wider.bwd_ksplit == 8 and wider.xchg_bytes >= 4 * 16 * 4096 * 2
    odd = _lib.plan("lstm", 8, 8, 1, 960)                      # not a multiple of 128: 1-D backward with 16-unit slices
    assert odd.supported and odd.exchange == 2 and odd.bwd_ksplit == 0 and odd.cluster == 60
    assert not _lib.plan("lstm", 8, 8, 1, 2048).supported     # R no longer fits in the tensor memory of one launch
    assert not _lib.plan("lstm", 64, 8, 1, 1024).supported    # more CTAs than SMs cannot wait on one another
    assert not _lib.plan("lstm", 8, 8, 1, 40).supported       # the ABI wants D % 16 == 0 (Python pads)


def test_argument_checks_mirror_the_reference():
    wx, R, b, init = make_inputs("lstm", 2, 3, 2, 16, 0)
    with pytest.raises(ValueError, match="unsupported cell"):
        flashrnn_torch(wx, R, b, init, cell="rnn", numerics="fp32_state_bf16_mma")
    # the reference's default policy ("mathematical", unrounded fp32) is not implemented: the default call says
    # which policy to pass instead of silently computing something else
    with pytest.raises(ValueError, match="numerics='fp32_state_bf16_mma'"):
        flashrnn_torch(wx, R, b, init)
    with pytest.raises(ValueError, match="numerics='fp32_state_bf16_mma'"):
        flashrnn_torch(wx, R, b, init, numerics="mathematical")
    with pytest.raises(ValueError, match="unsupported numerical policy"):
        flashrnn_torch(wx, R, b, init, numerics="fp16")
    k = dict(numerics="fp32_state_bf16_mma")
    with pytest.raises(ValueError, match="ranks"):
        flashrnn_torch(wx[0], R, b, init, **k)
    with pytest.raises(ValueError, match="same dtype"):
        flashrnn_torch(wx, R.double(), b, init, **k)
    with pytest.raises(ValueError, match="gate count"):
        flashrnn_torch(wx[:, :, :3], R, b, init, **k)
    with pytest.raises(ValueError, match=r"\[G,N,D,P\]"):
        flashrnn_torch(wx, R[:, :1], b, init, **k)
    with pytest.raises(ValueError, match="bias"):
        flashrnn_torch(wx, R, b[:3], init, **k)
    with pytest.raises(ValueError, match=r"\[S,B,1,N,D\]"):
        flashrnn_torch(wx, R, b, init[:1], **k)
    with pytest.raises(ValueError, match="Unknown backend"):
        flashrnn(wx, R, b, backend="cuda_fused")
    with pytest.raises(ValueError, match="Unknown function"):
        flashrnn(wx, R, b, function="mlstm")


def test_there_is_no_cpu_path():
    wx, R, b, init = make_inputs("lstm", 2, 3, 2, 16, 0)
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        flashrnn_torch(wx, R, b, init, numerics="fp32_state_bf16_mma")


def test_wide_head_batches_are_split_over_launches():
    """A launch whose CTAs all wait on one another can only take as many batch rows as fit the SMs; the host
    runs larger batches as several launches (the plan alone decides, no GPU needed)."""
    from flashrnn_b200 import functional

    assert functional._rows_per_launch("lstm", 8, 1024, 3, 256) == 8          # cluster path: never split
    assert functional._rows_per_launch("lstm", 256, 64, 32, 128) == 256
    rows = functional._rows_per_launch("lstm", 64, 8, 1, 1024)                # two 16-row groups of 64 CTAs
    assert rows == 32 and _lib.plan("lstm", rows, 8, 1, 1024).supported
    assert functional._rows_per_launch("lstm", 8, 8, 1, 2048) == 8            # unsupported at any batch: left to the launch to report
    # several wide heads: as many heads per launch as fit, then batch rows
    assert functional._launch_split("lstm", 8, 1024, 3, 256) == (3, 8)
    heads, rows = functional._launch_split("gru", 17, 4, 2, 1280)
    assert heads == 1 and rows == 16 and _lib.plan("gru", rows, 4, heads, 1280).supported
    assert functional._launch_split("lstm", 8, 8, 1, 2048) == (1, 8)



def test_error_polling_on_the_host(monkeypatch):
    """The bookkeeping around the device error words: nothing is queried while a CUDA graph is being captured, the
    non-blocking check is rate-limited, a blocking check also reads the words of captured launches."""
    import torch

    from flashrnn_b200 import functional as F

    class _Done:                       # stands in for a CUDA event that has completed
        def synchronize(self): pass
        def query(self): return True

    monkeypatch.setattr(F, "_pending_errors", [])
    monkeypatch.setattr(F, "_captured_errors", [])
    monkeypatch.setattr(F, "_last_poll", 0.0)
    bad = torch.tensor([101, 7, 3] + [0] * 29, dtype=torch.int32)

    # while capturing: neither recorded as an event nor looked at
    monkeypatch.setattr(F, "_capturing", lambda: True)
    F._track(bad, "captured launch")
    assert F._pending_errors == [] and len(F._captured_errors) == 1
    F.poll_errors(block=True)          # a no-op during capture
    monkeypatch.setattr(F, "_capturing", lambda: False)

    # outside: the non-blocking poll looks at most once per 20 ms ...
    F._pending_errors.append((_Done(), torch.zeros(32, dtype=torch.int32), "fine launch"))
    F.poll_errors()
    assert F._pending_errors == []
    F._pending_errors.append((_Done(), bad, "eager launch"))
    F.poll_errors()                    # within 20 ms of the previous look: the word stays queued
    assert len(F._pending_errors) == 1
    # ... the blocking one always does, and reports code, step and CTA
    with pytest.raises(RuntimeError, match="eager launch.*code 101.*step 7, CTA 3"):
        F.poll_errors(block=True)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: None)
    with pytest.raises(RuntimeError, match="captured launch.*replayed CUDA graph"):
        F.poll_errors(block=True)
