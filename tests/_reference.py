"""Locates an installed copy of the reference project for the drop-in tests.

The reference is never part of this repository.  `__graft_entry__.build()` installs it, unmodified,
under `baseline/_ref/` (git-ignored) on machines that have the checkout; tests that need it skip
when it is absent.  Here the reference is the CALLER of this library (its model and its autograd
Function run on these kernels), never the checker.
"""
import importlib
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def available() -> bool:
    return os.path.isdir(os.path.join(REF_DIR, "flash_win_attn_v2"))


def forget():
    """Drop every module of the reference package (and the substitution) from sys.modules."""
    for name in [m for m in sys.modules if m == "flash_win_attn_v2" or m.startswith("flash_win_attn_v2.")]:
        del sys.modules[name]


def import_reference():
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module("flash_win_attn_v2")
