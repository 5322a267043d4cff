"""CPU model of the exchange protocol of the row-sharded wide head (ranks as threads, buffers as numpy arrays).

What the kernels rely on, restated on the host so that it can be exercised without GPUs:
* every rank owns a history buffer with one slot per step, filled with all-ones words by the call before its kernel
  starts; an owner stores its packets of a step into the buffer of EVERY rank, a consumer polls only its OWN buffer and
  takes a packet once none of its words shows the fill pattern (a value that would collide with the pattern is mapped to
  another encoding first);
* every slot is written once per call, so there is no slot reuse inside a call;
* a rank may store into a peer's buffer only after the peer announced (ready flag = epoch of the call) that its buffer
  has been refilled for this call: without that handshake a late peer's refill wipes out early packets and the early rank
  waits forever (modelled below as a bounded wait that runs out).
The threads start with random delays and deliver packets in random order.
"""

import random
import threading
import time

import numpy as np
import pytest

FILL = np.uint32(0xFFFFFFFF)


def _clean(words):
    words = words.copy()
    words[words == FILL] = np.uint32(0x7FFFFFFF)
    return words


def _step_fn(full_prev, rank, width, t):
    """This rank's slice of the next state from the full previous state (any deterministic mixing will do)."""
    acc = (full_prev.astype(np.uint64).sum() + 7 * t) % (1 << 32)
    idx = np.arange(rank * width, (rank + 1) * width, dtype=np.uint64)
    out = ((acc * 2654435761 + idx * 40503 + full_prev[rank * width:(rank + 1) * width]) % (1 << 32)).astype(np.uint32)
    if t == 1:
        out[0] = FILL   # a value that looks like the fill pattern must still get through
    return out


def _reference(P, width, T, init):
    full, hist = init.copy(), [init.copy()]
    for t in range(T):
        nxt = np.concatenate([_clean(_step_fn(full, r, width, t)) for r in range(P)])
        hist.append(nxt)
        full = nxt
    return hist


class _Rank(threading.Thread):
    def __init__(self, rank, world, handshake, limit_s=5.0):
        super().__init__(daemon=True)
        self.rank, self.w, self.handshake, self.limit = rank, world, handshake, limit_s
        self.result, self.error = None, None

    def _wait(self, cond):
        t0 = time.monotonic()
        while not cond():
            if time.monotonic() - t0 > self.limit:
                raise TimeoutError(f"rank {self.rank}: bounded wait ran out")
            time.sleep(0)

    def run(self):
        w, r = self.w, self.rank
        rng = random.Random(1000 * w["epoch"] + r)
        try:
            time.sleep(rng.random() * 0.02 * (3 if r == w["late_rank"] else 1))   # launch skew
            w["buffers"][r][:] = FILL                                              # the call refills its own buffer ...
            if self.handshake:
                for q in range(w["P"]):
                    w["ready"][q][r] = w["epoch"]                                  # ... announces it to everybody ...
                self._wait(lambda: all(w["ready"][r][q] >= w["epoch"] for q in range(w["P"])))  # ... and waits for all
            width, P, T = w["width"], w["P"], w["T"]
            mine = w["init"][r * width:(r + 1) * width]
            seen = []
            for slot in range(T + 1):
                order = [(q, i) for q in range(P) for i in range(0, width, 4)]     # packets of four words
                rng.shuffle(order)
                for q, i in order:
                    w["buffers"][q][slot, r * width + i:r * width + i + 4] = _clean(mine[i:i + 4])
                row = w["buffers"][r][slot]
                self._wait(lambda: not (row == FILL).any())
                full = row.copy()
                seen.append(full)
                if slot < T:
                    mine = _step_fn(full, r, width, slot)
            self.result = seen
        except Exception as exc:  # noqa: BLE001 - reported to the test
            self.error = exc


def _run_call(world, handshake, limit_s=5.0):
    ranks = [_Rank(r, world, handshake, limit_s) for r in range(world["P"])]
    for t in ranks:
        t.start()
    for t in ranks:
        t.join(timeout=30)
    return ranks


@pytest.mark.parametrize("P", [2, 4, 8])
def test_write_once_slots_and_ready_handshake(P):
    width, T = 8, 12
    rng = np.random.default_rng(5)
    world = {"P": P, "width": width, "T": T, "late_rank": P - 1,
             "buffers": [np.zeros((T + 1, P * width), dtype=np.uint32) for _ in range(P)],   # stale contents, not the fill
             "ready": [[0] * P for _ in range(P)]}
    for epoch in (1, 2, 3):   # three calls in a row share buffers and flags
        world["epoch"] = epoch
        world["init"] = rng.integers(0, 1 << 32, size=P * width, dtype=np.uint32)
        world["init"][world["init"] == FILL] = 1
        want = _reference(P, width, T, world["init"])
        ranks = _run_call(world, handshake=True)
        for t in ranks:
            assert t.error is None, t.error
            assert len(t.result) == T + 1
            for got, ref in zip(t.result, want):
                assert np.array_equal(got, ref)


def test_without_the_handshake_a_late_refill_loses_packets():
    """The failure the ready flags exist for: rank 1 refills its buffer after rank 0 already stored into it, so rank 1
    never sees those packets; its bounded wait runs out and is reported instead of hanging."""
    P, width, T = 2, 8, 3
    world = {"P": P, "width": width, "T": T, "late_rank": 1, "epoch": 1,
             "buffers": [np.zeros((T + 1, P * width), dtype=np.uint32) for _ in range(P)],
             "ready": [[0] * P for _ in range(P)], "init": np.arange(1, P * width + 1, dtype=np.uint32)}
    lost = 0
    for attempt in range(20):
        world["epoch"] = attempt + 1
        ranks = _run_call(world, handshake=False, limit_s=0.3)
        lost += any(isinstance(t.error, TimeoutError) for t in ranks)
        if lost:
            break
    assert lost, "the unsynchronised refill never lost a packet in 20 tries (the race is timing dependent)"
