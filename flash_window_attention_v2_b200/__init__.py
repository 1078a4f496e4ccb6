"""Swin-V2 scaled-cosine window attention, forward and backward, on hand-written sm_100a kernels.

Public surface (same call signatures as the reference project):

* `flash_win_attn_v2_func(q, k, v, logit_scale=None, bias=None, mask=None)`
* `FlashWindowAttentionV2` (the autograd Function behind it)
* `kernels._flash_attn_forward` / `kernels._flash_attn_backward` (the replaced boundary)
* `install()` to route an installed copy of the reference project through these kernels
* `sharded` for window-sharded multi-GPU use
* `host_io.HostBatchPipeline` for batches that live in pinned host memory (copies and kernels of
  consecutive batches overlapped)
"""
from .flash_window_attention_v2 import FlashWindowAttentionV2, flash_win_attn_v2_func  # noqa: F401
from .install import install, uninstall  # noqa: F401
