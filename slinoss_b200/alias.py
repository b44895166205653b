"""Optional literal drop-in: make ``import slinoss`` resolve to this package.

``slinoss_b200`` keeps the reference's module tree (``ops.v2x2ssd``, ``ops.scanprep``, ``ops.mixer``,
``layers``, ``blocks``) under another top-level name so that both can be imported side by side (the
reference uses absolute ``from slinoss...`` imports).  Code written against the reference runs unchanged
after ``slinoss_b200.alias.install()`` when the reference itself is not importable; with the reference on
``sys.path`` the call refuses unless ``force=True``.
"""

from __future__ import annotations

import importlib
import importlib.util
import sys

SUBMODULES = ("ops", "ops.v2x2ssd", "ops.scanprep", "ops.mixer", "ops.block", "layers", "blocks")


def install(force: bool = False) -> None:
    """Register ``slinoss`` and its sub-modules as aliases of ``slinoss_b200`` in ``sys.modules``."""
    if "slinoss" in sys.modules and getattr(sys.modules["slinoss"], "__name__", "") == "slinoss_b200":
        return
    if not force and ("slinoss" in sys.modules or importlib.util.find_spec("slinoss") is not None):
        raise ImportError("a package named 'slinoss' is already importable; pass force=True to shadow it")
    pkg = importlib.import_module("slinoss_b200")
    sys.modules["slinoss"] = pkg
    for name in SUBMODULES:
        sys.modules[f"slinoss.{name}"] = importlib.import_module(f"slinoss_b200.{name}")


def uninstall() -> None:
    for key in [k for k in sys.modules if k == "slinoss" or k.startswith("slinoss.")]:
        if getattr(sys.modules[key], "__name__", "").startswith("slinoss_b200"):
            del sys.modules[key]


__all__ = ["install", "uninstall"]
