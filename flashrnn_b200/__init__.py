"""B200-native (sm_100a) backend for FlashRNN's fused recurrence.

Public surface = the reference's: ``flashrnn``, ``FlashRNNConfig``, ``flashrnn_torch``
(flashrnn/__init__.py:2-5 of the reference), running hand-written CUDA through a C ABI.
"""

from .functional import BACKEND, SIZES, FlashRNNConfig, flashrnn, flashrnn_torch, poll_errors
from .prepared import PreparedSequence
from .projection import flashrnn_projected, input_projection

__all__ = ["BACKEND", "SIZES", "FlashRNNConfig", "PreparedSequence", "flashrnn", "flashrnn_projected", "flashrnn_torch",
           "input_projection", "poll_errors"]
