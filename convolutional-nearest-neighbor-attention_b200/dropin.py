"""Make the reference's own ``vit.py`` / ``main.py`` construct the CUDA-backed layers.

``vit.py`` binds the layer classes with ``from layers import ...`` (reference vit.py:10-18),
so the names must be rebound both in the reference's ``layers`` module and, when it was
imported already, in ``vit``.  Nothing else of the reference is touched.
"""
from __future__ import annotations

import sys

from . import layers as _ours

_NAMES = ("MultiHeadConvNNAttention", "MultiHeadBranchingAttention", "MultiHeadBranchingConv")


def install(reference_layers=None, reference_vit=None) -> list:
    """Rebind the three hot-path classes; returns the modules that were patched."""
    patched = []
    for mod in (reference_layers or sys.modules.get("layers"), reference_vit or sys.modules.get("vit")):
        if mod is None:
            continue
        for n in _NAMES:
            if hasattr(mod, n):
                if not hasattr(mod, "_convnn_b200_saved"):
                    mod._convnn_b200_saved = {}
                mod._convnn_b200_saved.setdefault(n, getattr(mod, n))
                setattr(mod, n, getattr(_ours, n))
        patched.append(mod)
    return patched


def uninstall() -> None:
    for mod in (sys.modules.get("layers"), sys.modules.get("vit")):
        saved = getattr(mod, "_convnn_b200_saved", None) if mod is not None else None
        if saved:
            for n, cls in saved.items():
                setattr(mod, n, cls)
            mod._convnn_b200_saved = {}
