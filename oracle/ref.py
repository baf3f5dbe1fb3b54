"""Loader for the reference's own CUDA build (``oracle/_ref``). Test infrastructure only.

The module is loaded from its file path under a private spec, so it never shadows (and is
never shadowed by) the drop-in ``flash_gaussian_splatting`` package of this repository.
"""
from __future__ import annotations

import importlib.util
import os

from . import build as _build

_mod = None


def available() -> bool:
    return os.path.exists(_build.REF_SO)


def load():
    """Returns the reference extension module (its ``ops`` submodule holds the operators), or None."""
    global _mod
    if _mod is None and available():
        import torch  # noqa: F401  (the extension links against libtorch)
        spec = importlib.util.spec_from_file_location("flash_gaussian_splatting", _build.REF_SO)
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        _mod = m
    return _mod
