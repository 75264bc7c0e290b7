"""Importable name of the package whose sources live in ``skyrl-tx-rocm_b200/``.

The source directory carries the project's hyphenated name, which Python cannot
import directly; this shim points the package search path at it.
"""

import os as _os

__path__.append(_os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "skyrl-tx-rocm_b200"))

from .ops import *  # noqa: E402,F401,F403
from . import ops as _ops  # noqa: E402

__all__ = _ops.__all__
