"""xlstm_b200 — B200 (sm_100a) engine for the xLSTM training hot path.

The compute lives in libxlstm_b200.so (hand-written CUDA behind a C ABI, declared in
include/xlstm_b200.h). This package is the thin host-side mirror of the reference's
`gpu::ops` functions over that ABI; torch is used only for device memory and streams.
There is no CPU fallback: importing `ops` without the built library raises.

The directory name carries a hyphen, so import it with
`importlib.import_module("neural-networks_b200")`.
"""
from . import _lib  # noqa: F401  (loads the shared library or raises)
from . import ops  # noqa: F401
