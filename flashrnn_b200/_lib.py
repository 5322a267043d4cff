"""ctypes binding of ``libflashrnn_b200.so`` (the C ABI declared in ``include/flashrnn_b200.h``).

There is no fallback: if the shared library is missing or does not export every entry point the
import of the compute path fails with an explicit error.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_int64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libflashrnn_b200.so"

CELLS = {"lstm": 0, "slstm": 1, "gru": 2, "elman": 3}

ERROR_TEXT = {
    -1: "unknown cell",
    -2: "shape not supported by the sm_100a kernel family (see frnn_b200_plan)",
    -3: "tensor-memory budget exceeded",
    -4: "TMA descriptor could not be built",
    -5: "bad argument",
    -6: "problem too large for the built-in scratch of frnn_b200_wgrad_noalloc",
    101: "recurrent operand of a step never arrived",
    102: "tensor-core completion barrier timed out",
    103: "TMA input stage never filled",
    104: "TMA input stage never released",
    105: "epilogue barrier timed out",
    106: "partial sums of a peer CTA never arrived",
    107: "dg operand barrier timed out",
    108: "a peer rank never announced that its exchange buffer is ready",
    109: "a stage of the streamed weight operand never arrived or was never released",
}


class Plan(ctypes.Structure):
    """Mirror of ``frnn_b200_plan_t``."""

    _fields_ = [
        ("gates_r", c_int), ("gates_w", c_int), ("gates_b", c_int), ("states", c_int), ("cache_gates", c_int),
        ("unit", c_int), ("cluster", c_int), ("batch_tile", c_int), ("n_btiles", c_int), ("grid_ctas", c_int),
        ("supported", c_int),
        ("cache_bytes", c_int64), ("hbf_bytes", c_int64), ("dgr_bytes", c_int64), ("dbpart_bytes", c_int64),
        ("wgrad_work_bytes", c_int64), ("wgrad_ksplit", c_int), ("exchange", c_int), ("xchg_bytes", c_int64),
        ("fwd_ksplit", c_int), ("fwd_ctas", c_int), ("bwd_ksplit", c_int), ("fwd_batch_tile", c_int),
    ]


class Options(ctypes.Structure):
    """Mirror of ``frnn_b200_options_t``."""

    _fields_ = [("forward_clipval", ctypes.c_float), ("gradient_recurrent_clipval", ctypes.c_float),
                ("gradient_recurrent_cut", c_int), ("slstm_v1_gradient", c_int)]


class MgShard(ctypes.Structure):
    """Mirror of ``frnn_b200_mg_shard_t``."""

    _fields_ = [("P", c_int), ("rank", c_int), ("ranks_here", c_int), ("epoch", c_int), ("k_tmem_max", c_int),
                ("ring_stages_max", c_int), ("buffers", c_void_p * 8), ("ready", c_void_p * 8)]


class MgPlan(ctypes.Structure):
    """Mirror of ``frnn_b200_mg_plan_t``."""

    _fields_ = [
        ("supported", c_int), ("local_width", c_int), ("fwd_ksplit", c_int), ("fwd_ctas", c_int),
        ("fwd_k_tmem", c_int), ("fwd_ring_chunks", c_int), ("fwd_ring_stages", c_int), ("fwd_resident", c_int),
        ("bwd_ksplit", c_int), ("bwd_ctas", c_int),
        ("bwd_k_tmem", c_int), ("bwd_ring_chunks", c_int), ("bwd_ring_stages", c_int), ("bwd_resident", c_int),
        ("hbf_bytes", c_int64), ("dgr_bytes", c_int64), ("cache_bytes", c_int64), ("r_cols_bytes", c_int64),
        ("dbpart_bytes", c_int64),
    ]


# name -> (restype, argtypes); must list every function declared in include/flashrnn_b200.h
SIGNATURES = {
    "frnn_b200_version": (c_int, []),
    "frnn_b200_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(Plan)]),
    "frnn_b200_forward": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                  c_void_p]),
    "frnn_b200_forward_prepared": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                           c_void_p]),
    "frnn_b200_forward_ex": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                     c_void_p, POINTER(Options)]),
    "frnn_b200_backward_ex": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_void_p, c_void_p, POINTER(Options)]),
    "frnn_b200_forward_chunk": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                        c_void_p, c_void_p]),
    "frnn_b200_backward": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_void_p, c_void_p]),
    "frnn_b200_wgrad": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                c_int, c_int, c_void_p, c_void_p]),
    "frnn_b200_wgrad_noalloc": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_int, c_void_p, c_void_p]),
    "frnn_b200_input_projection": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p, c_void_p]),
    "frnn_b200_mg_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(MgShard), POINTER(MgPlan)]),
    "frnn_b200_mg_capacity": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "frnn_b200_mg_forward": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     POINTER(MgShard), c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "frnn_b200_mg_gather_columns": (c_int, [c_int, POINTER(c_void_p), c_void_p, POINTER(MgShard), c_int, c_void_p]),
    "frnn_b200_mg_backward": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                      c_void_p, c_void_p, POINTER(MgShard), c_int, c_int, c_int, c_int, c_int, c_void_p,
                                      c_void_p]),
    "frnn_b200_mg_wgrad": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(MgShard), c_int, c_int,
                                   c_int, c_int, c_void_p, c_void_p]),
    "frnn_b200_peer_alloc": (c_int, [ctypes.c_size_t, POINTER(c_void_p)]),
    "frnn_b200_peer_free": (c_int, [c_void_p]),
    "frnn_b200_peer_export": (c_int, [c_void_p, ctypes.c_char_p]),
    "frnn_b200_peer_open": (c_int, [ctypes.c_char_p, POINTER(c_void_p)]),
    "frnn_b200_peer_close": (c_int, [c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once; raise if it is absent or incomplete."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flashrnn_b200.build` "
            "(there is no CPU or PyTorch fallback for the recurrence)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:  # pragma: no cover - build problem
            raise RuntimeError(f"{LIB_PATH} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


_plans: dict = {}


def plan(cell: str, B: int, T: int, N: int, D: int) -> Plan:
    """Launch plan of a shape on the CURRENT CUDA device (the plan depends on its SM count). Remembered per
    (device, shape): the host path asks several times per call."""
    dev = -1
    try:
        import torch

        if torch.cuda.is_available():
            dev = torch.cuda.current_device()
    except ImportError:  # the binding itself does not need torch
        pass
    key = (dev, cell, B, T, N, D)
    hit = _plans.get(key)
    if hit is not None:
        return hit
    out = Plan()
    rc = load().frnn_b200_plan(CELLS[cell], B, T, N, D, ctypes.byref(out))
    if rc != 0:
        raise ValueError(f"frnn_b200_plan failed: {ERROR_TEXT.get(rc, rc)}")
    if len(_plans) > 4096:
        _plans.clear()
    _plans[key] = out
    return out


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}: {ERROR_TEXT.get(rc, 'CUDA error')}")
