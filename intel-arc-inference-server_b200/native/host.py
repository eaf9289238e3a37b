"""Loader of the native host library (``b200host``): builds it on first use when a compiler is there."""
from __future__ import annotations

import importlib.util
import os

from . import build as _build

_mod = None
_err = None


def module():
    global _mod, _err
    if _mod is None and _err is None:
        try:
            path = _build.LIB
            if not _build.is_current():
                try:
                    path = _build.build()
                except Exception:
                    if not os.path.exists(_build.LIB):
                        raise
            spec = importlib.util.spec_from_file_location("b200host", path)
            _mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(_mod)
        except Exception as e:  # noqa: BLE001
            _err = e
    if _mod is None:
        raise ImportError(f"native host library unavailable: {_err}")
    return _mod


def available() -> bool:
    try:
        module()
        return True
    except ImportError:
        return False


def __getattr__(name):
    return getattr(module(), name)
