"""Swap the reference project's Triton kernels for this library, leaving the rest of it untouched.

The reference's autograd Function imports two names from `flash_win_attn_v2.kernels`
(flash_win_attn_v2/flash_window_attention_v2.py:3) and looks them up as module globals at call
time (:22, :40).  `install()` therefore either

* registers this package's `kernels` module as `flash_win_attn_v2.kernels` before the reference
  is imported (its Triton files are then never imported), or
* if the reference is already imported, rebinds the two names inside
  `flash_win_attn_v2.flash_window_attention_v2`.

After that `flash_win_attn_v2.flash_win_attn_v2_func`, `WindowAttention` and `SwinTransformerV2`
(with `is_flash=True`) run on the sm_100a kernels.
"""
from __future__ import annotations

import sys

from . import kernels


def install() -> None:
    mod = sys.modules.get("flash_win_attn_v2.flash_window_attention_v2")
    if mod is not None:
        mod._flash_attn_forward = kernels._flash_attn_forward
        mod._flash_attn_backward = kernels._flash_attn_backward
    sys.modules["flash_win_attn_v2.kernels"] = kernels
    pkg = sys.modules.get("flash_win_attn_v2")
    if pkg is not None:
        pkg.kernels = kernels


def uninstall() -> None:
    """Forget the substitution (the reference must be re-imported to get its own kernels back)."""
    if sys.modules.get("flash_win_attn_v2.kernels") is kernels:
        del sys.modules["flash_win_attn_v2.kernels"]
