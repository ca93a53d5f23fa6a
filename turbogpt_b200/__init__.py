"""turbogpt_b200 — B200-native engine for the dense training step of a byte-level GPT.

The product is the C-ABI library built from ``csrc/`` (see ``include/turbogpt_b200.h``); this
package holds its build recipe and a ctypes mirror of the reference's ``tests/bridge.py``.
There is no CPU path: every compute call needs the CUDA library and a B200.
"""
from .bridge import Config, ConfigEx, Native, OneCycle, StepRates, library_path, load_library  # noqa: F401
