"""rexsc_b200 -- B200 (sm_100a) implementation of the REX-SC stochastic-computing arithmetic hot path.

``rexsc_b200.ops`` mirrors the reference's extension ops; ``rexsc_b200.dropin`` holds modules named like the
reference's extensions (``sc_extension_cuda``, ``fixed_extension_cuda``, ...) -- put that directory on
``sys.path`` (``rexsc_b200.install_dropin()``) and the unchanged reference front end imports them.
"""
from __future__ import annotations

import os
import sys

__version__ = "0.1.0"

DROPIN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dropin")


def install_dropin() -> str:
    """Make ``import sc_extension_cuda`` / ``fixed_extension_cuda`` / ``sc_extension`` / ``fixed_extension``
    resolve to this library (the names utils_functional.py:17-20 of the reference imports)."""
    if DROPIN_DIR not in sys.path:
        sys.path.insert(0, DROPIN_DIR)
    return DROPIN_DIR
