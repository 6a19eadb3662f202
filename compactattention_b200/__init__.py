"""B200-native (sm_100a) implementation of CompactAttention's chunked-prefill hot path.

The compute lives in ``libcompactattn_b200.so`` (hand-written CUDA behind a C ABI, see
``include/compactattn_b200.h``); this package is the Python host side that mirrors the reference
project's operator interface for the path.
"""
from . import _lib  # noqa: F401

__version__ = "0.1.0"
