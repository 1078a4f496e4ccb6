"""Drop-in replacement for the reference package `flash_win_attn_v2.kernels`.

Exports the same two names with the same signatures, argument meaning and
assertion behaviour (flash_win_attn_v2/kernels/__init__.py:1-2):

* `_flash_attn_forward`  (attn_kernel_forward.py:261-345)
* `_flash_attn_backward` (attn_kernel_backward.py:567-711)

Both marshal raw device pointers into the C ABI of libfwa2_b200.so (hand-written
sm_100a kernels).  PyTorch is used only for device memory and the current
stream.  There is no Triton, no alternative backend and no CPU path: without
the compiled library, or on a failure inside it, these functions raise.
"""
from __future__ import annotations

import ctypes as C
import math
import threading

import torch

from .. import _lib

__all__ = ["_flash_attn_forward", "_flash_attn_backward", "check_device_status", "poll_device_status",
           "DeviceTimeoutError", "finalize_grads"]

_DTYPES = {torch.float16: _lib.FWA2_F16, torch.bfloat16: _lib.FWA2_BF16}
# Per device: (status block in device memory, its mirror in pinned host memory).  A kernel whose
# bounded wait ran out writes the device block; every backward call ends with an asynchronous
# 16-byte copy into the mirror, and every boundary call starts by looking at the mirror, so a
# device-side timeout surfaces as an exception one or two calls later without any host
# synchronisation on the normal path.
_status_words: dict[int, tuple] = {}


class DeviceTimeoutError(RuntimeError):
    """A bounded wait inside a kernel ran out; the outputs of that call are incomplete."""


def _status_entry(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ent = _status_words.get(idx)
    if ent is None:
        dev_block = torch.zeros(4, dtype=torch.int32, device=device)
        host_block = torch.zeros(4, dtype=torch.int32).pin_memory()
        ent = (dev_block, host_block)
        _status_words[idx] = ent
    return ent


def _status(device: torch.device) -> torch.Tensor:
    return _status_entry(device)[0]


def _describe(st) -> str:
    return (f"fwa2 device status: a bounded wait ran out at site {st[0] >> 8} (kind {st[0] & 255}), "
            f"block {st[1]}, detail {st[2]}; outputs of the affected call are incomplete")


def poll_device_status(device=None) -> None:
    """Raise if an earlier call on `device` reported a device-side timeout.  Reads the pinned host
    mirror only: no synchronisation, safe to call anywhere (also while a stream is capturing)."""
    if not _status_words:
        return
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ent = _status_words.get(idx)
    if ent is None:
        return
    st = ent[1].tolist()
    if st[0] != 0:
        ent[1].zero_()
        if ent[0].is_cuda and not torch.cuda.is_current_stream_capturing():
            ent[0].zero_()     # (while capturing, the block is cleared by the next synchronous check)
        raise DeviceTimeoutError(_describe(st))


def _mirror_status(device: torch.device) -> None:
    """Enqueue the 16-byte copy of the status block into its pinned mirror on the current stream."""
    dev_block, host_block = _status_entry(device)
    host_block.copy_(dev_block, non_blocking=True)


def check_device_status(device=None) -> None:
    """Synchronise and raise if a kernel recorded a device-side timeout."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    torch.cuda.synchronize(device)
    dev_block, host_block = _status_entry(device)
    st = dev_block.cpu().tolist()
    if st[0] != 0:
        dev_block.zero_()
        host_block.zero_()
        raise DeviceTimeoutError(_describe(st))


def _t4(dst: _lib.Tensor4, x: torch.Tensor) -> None:
    """Fill a tensor descriptor of an argument block in place."""
    st = x.stride()
    dst.ptr, dst.stride_bw, dst.stride_h, dst.stride_n = x.data_ptr(), st[0], st[1], st[2]


# One argument block per thread and direction, reused from call to call (the forward runs on the
# caller's thread, the backward on an autograd engine thread; the library reads the block during
# the call only).
_tls = threading.local()


def _fwd_block() -> _lib.FwdArgs:
    a = getattr(_tls, "fwd", None)
    if a is None:
        a = _tls.fwd = _lib.FwdArgs()
        a.struct_size = C.sizeof(_lib.FwdArgs)
        a.abi_version = _lib.FWA2_ABI_VERSION
    return a


def _bwd_block() -> _lib.BwdArgs:
    a = getattr(_tls, "bwd", None)
    if a is None:
        a = _tls.bwd = _lib.BwdArgs()
        a.struct_size = C.sizeof(_lib.BwdArgs)
        a.abi_version = _lib.FWA2_ABI_VERSION
    return a


def _tma_ok(x: torch.Tensor) -> bool:
    """Inner stride 1, every other stride a multiple of 8 elements, 16-byte aligned base."""
    if x.data_ptr() % 16 != 0:
        return False
    if x.is_contiguous():          # the common case, one call: rows of 32 elements, so every
        return x.shape[-1] % 8 == 0   # outer stride is a multiple of 8 as well
    if x.stride(-1) != 1:
        return False
    return all(x.shape[i] == 1 or (x.stride(i) > 0 and x.stride(i) % 8 == 0) for i in range(3))


class _on_device:
    """`with torch.cuda.device(dev)` only when `dev` is not already current (the context manager
    costs several microseconds of a call whose kernels take a few tens)."""
    __slots__ = ("ctx",)

    def __init__(self, device: torch.device):
        idx = device.index
        self.ctx = None if (idx is None or idx == torch.cuda.current_device()) else torch.cuda.device(device)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)
        return False


def _rows(x: torch.Tensor) -> torch.Tensor:
    return x if _tma_ok(x) else x.contiguous()


def _table(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A (planes, N, N) table with a row pitch TMA can address (multiple of 8 elements)."""
    if t.dtype != dtype:
        t = t.to(dtype)
    n = t.shape[-1]
    if n % 8 != 0:
        t = torch.nn.functional.pad(t, (0, 8 - n % 8))
    elif not t.is_contiguous():
        t = t.contiguous()
    return t


def _stream(device) -> C.c_void_p:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return C.c_void_p(torch._C._cuda_getCurrentRawStream(idx))


def _flash_attn_forward(q, k, v, logit_scale, bias=None, mask=None, scale_type="scalar",
                        _variant: int = 0, _max_ctas: int = 0, _trace=None):
    poll_device_status(q.device)      # a timeout reported by an earlier call must not stay silent
    batch_window_size, n_heads, seqlen_q, d = q.shape
    _, _, seqlen_k, _ = k.shape
    assert k.shape == (batch_window_size, n_heads, seqlen_k, d)
    assert v.shape == (batch_window_size, n_heads, seqlen_k, d)
    assert d <= 128, "FlashAttention only support head dimensions up to 128"
    assert d == 32, "this library is built for head dimension 32 (every Swin-V2 configuration uses it)"
    assert q.dtype == k.dtype == v.dtype, "All tensors must have the same type"
    assert q.dtype in [torch.float16, torch.bfloat16], "Only support fp16 and bf16"
    assert q.is_cuda and k.is_cuda and v.is_cuda and logit_scale.is_cuda
    assert seqlen_q == seqlen_k, "window attention is self-attention: seqlen_q must equal seqlen_k"
    if scale_type == "tensor":
        assert logit_scale.shape == (n_heads, 1, 1)
        assert logit_scale.dtype == q.dtype
        if not logit_scale.is_contiguous():
            logit_scale = logit_scale.contiguous()
    else:
        assert logit_scale.dtype == torch.float32 and logit_scale.numel() == 1
    if bias is not None:
        assert bias.dtype == q.dtype
        assert bias.is_cuda
        assert bias.shape == (n_heads, seqlen_q, seqlen_k)
    n_windows = 0
    if mask is not None:
        assert mask.dtype in [q.dtype, torch.float]
        assert mask.is_cuda
        assert mask.shape[1:] == (seqlen_q, seqlen_k)
        n_windows = mask.shape[0]
        assert batch_window_size % n_windows == 0

    seqlen_q_rounded = math.ceil(seqlen_q / 64) * 64
    lse = torch.empty((batch_window_size, n_heads, seqlen_q_rounded), device=q.device, dtype=torch.float32)
    o = torch.empty_like(q)
    if not _tma_ok(o):
        o = torch.empty(q.shape, device=q.device, dtype=q.dtype)

    qc, kc, vc = _rows(q), _rows(k), _rows(v)
    bias_t = _table(bias, q.dtype) if bias is not None else None
    mask_t = _table(mask, q.dtype) if mask is not None else None

    a = _fwd_block()
    a.dtype = _DTYPES[q.dtype]
    a.bw, a.heads, a.n, a.head_dim = batch_window_size, n_heads, seqlen_q, d
    a.n_windows = n_windows
    _t4(a.q, qc), _t4(a.k, kc), _t4(a.v, vc), _t4(a.o, o)
    a.lse = lse.data_ptr()
    a.lse_stride_bw, a.lse_stride_h = lse.stride(0), lse.stride(1)
    a.logit_scale = logit_scale.data_ptr()
    a.scale_is_tensor = 1 if scale_type == "tensor" else 0
    a.bias = bias_t.data_ptr() if bias_t is not None else None
    a.mask = mask_t.data_ptr() if mask_t is not None else None
    a.bias_row_stride = bias_t.stride(1) if bias_t is not None else 0
    a.mask_row_stride = mask_t.stride(1) if mask_t is not None else 0
    # Scratch for the combined fp32 table (bias + mask); the library asks for it only where it pays:
    # windows of 129 to 256 tokens with both tables and enough images per window type.
    workspace, ws_bytes = None, 0
    if bias_t is not None and mask_t is not None and 128 < seqlen_q <= 256:
        ws_bytes = _lib.lib().fwa2_fwd_workspace_bytes(batch_window_size, n_heads, seqlen_q, n_windows, 1, 1, _variant)
        if ws_bytes:
            workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    a.workspace = workspace.data_ptr() if workspace is not None else None
    a.workspace_bytes = ws_bytes
    a.status = _status(q.device).data_ptr()
    a.variant = _variant
    a.max_ctas = _max_ctas
    a.developer0, a.developer1 = (_trace.data_ptr(), _trace.numel() // 4) if _trace is not None else (None, 0)
    with _on_device(q.device):
        _lib.check(_lib.lib().fwa2_forward(C.byref(a), _stream(q.device)), "fwa2_forward")
    return o, lse, logit_scale


def _flash_attn_backward(do, q, k, v, logit_scale, o, lse, dq, dk, dv, dscale, db,
                         bias=None, mask=None, scale_type="scalar", _partial_out=None,
                         _variant: int = 0, _max_ctas: int = 0, _workspace=None, _trace=None):
    """Fills dq, dk, dv (and dscale, db when given) in place; returns None.

    `_partial_out` (fp32, H*N*N + H elements) is an extension used by the window-sharded
    multi-GPU path: when given, the window-summed dBias / dLogitScale are left there in fp32
    (before the clamp gate and the cast) and `db` / `dscale` are not written.
    """
    poll_device_status(q.device)
    if do.stride(-1) != 1:
        do = do.contiguous()
    batch_window_size, n_heads, seqlen_q, d = q.shape
    _, _, seqlen_k, _ = k.shape
    assert d <= 128
    assert d == 32, "this library is built for head dimension 32 (every Swin-V2 configuration uses it)"
    assert seqlen_q == seqlen_k
    seqlen_q_rounded = math.ceil(seqlen_q / 64) * 64
    assert lse.shape == (batch_window_size, n_heads, seqlen_q_rounded)
    assert q.stride(-1) == k.stride(-1) == v.stride(-1) == o.stride(-1) == 1
    assert dq.stride(-1) == dk.stride(-1) == dv.stride(-1) == 1
    assert q.dtype in _DTYPES and q.dtype == k.dtype == v.dtype == o.dtype == do.dtype
    has_bias = bias is not None
    if has_bias:
        assert bias.dtype in [q.dtype, torch.float]
        assert bias.is_cuda
        assert bias.shape == (n_heads, seqlen_q, seqlen_k)
        assert db is not None or _partial_out is not None
    n_windows = 0
    if mask is not None:
        assert mask.dtype in [q.dtype, torch.float]
        assert mask.is_cuda
        n_windows = mask.shape[0]
    if scale_type == "tensor":
        assert dscale is not None or _partial_out is not None
        if not logit_scale.is_contiguous():
            logit_scale = logit_scale.contiguous()

    qc, kc, vc, oc, doc = _rows(q), _rows(k), _rows(v), _rows(o), _rows(do)
    outs = []
    for g in (dq, dk, dv):
        outs.append(g if _tma_ok(g) else torch.empty(g.shape, device=g.device, dtype=g.dtype))
    bias_t = _table(bias, q.dtype) if has_bias else None
    mask_t = _table(mask, q.dtype) if mask is not None else None
    db_c = db if (db is None or db.is_contiguous()) else torch.empty(db.shape, device=db.device, dtype=db.dtype)
    ds_c = dscale if (dscale is None or dscale.is_contiguous()) else torch.empty(
        dscale.shape, device=dscale.device, dtype=dscale.dtype)

    L = _lib.lib()
    with _on_device(q.device):
        ws_bytes = L.fwa2_bwd_workspace_bytes(batch_window_size, n_heads, seqlen_q, n_windows,
                                              1 if has_bias else 0, 1 if mask is not None else 0)
        assert ws_bytes > 0
        if _workspace is not None:
            assert _workspace.numel() * _workspace.element_size() >= ws_bytes
            workspace = _workspace
        else:
            workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)

        a = _bwd_block()
        a.dtype = _DTYPES[q.dtype]
        a.bw, a.heads, a.n, a.head_dim = batch_window_size, n_heads, seqlen_q, d
        a.n_windows = n_windows
        _t4(a.q, qc), _t4(a.k, kc), _t4(a.v, vc), _t4(a.o, oc), _t4(a.dout, doc)
        _t4(a.dq, outs[0]), _t4(a.dk, outs[1]), _t4(a.dv, outs[2])
        a.lse = lse.data_ptr()
        a.lse_stride_bw, a.lse_stride_h = lse.stride(0), lse.stride(1)
        a.logit_scale = logit_scale.data_ptr()
        a.scale_is_tensor = 1 if scale_type == "tensor" else 0
        a.bias = bias_t.data_ptr() if bias_t is not None else None
        a.mask = mask_t.data_ptr() if mask_t is not None else None
        a.bias_row_stride = bias_t.stride(1) if bias_t is not None else 0
        a.mask_row_stride = mask_t.stride(1) if mask_t is not None else 0
        a.dbias = db_c.data_ptr() if (db_c is not None and has_bias) else None
        a.dscale = ds_c.data_ptr() if (ds_c is not None and scale_type == "tensor") else None
        a.partial_out = _partial_out.data_ptr() if _partial_out is not None else None
        a.workspace = workspace.data_ptr()
        a.workspace_bytes = ws_bytes
        a.status = _status(q.device).data_ptr()
        a.variant = _variant
        a.max_ctas = _max_ctas
        a.developer0, a.developer1 = (_trace.data_ptr(), _trace.numel() // 4) if _trace is not None else (None, 0)
        _lib.check(L.fwa2_backward(C.byref(a), _stream(q.device)), "fwa2_backward")
        _mirror_status(q.device)

    for dst, src in zip((dq, dk, dv), outs):
        if dst is not src:
            dst.copy_(src)
    if db is not None and db_c is not db:
        db.copy_(db_c)
    if dscale is not None and ds_c is not dscale:
        dscale.copy_(ds_c)
    return None


def finalize_grads(partial, logit_scale, db, dscale):
    """Cast an fp32 [H*N*N dBias | H dLogitScale] buffer (possibly summed over GPUs) into
    `db` / `dscale`, applying 1[g <= ln 100] to dLogitScale."""
    h = db.shape[0] if db is not None else dscale.shape[0]
    n = db.shape[-1] if db is not None else int(round(math.sqrt((partial.numel() - h) / h)))
    ref = db if db is not None else dscale
    assert partial.dtype == torch.float32 and partial.is_contiguous()
    assert db is None or db.is_contiguous()
    with torch.cuda.device(partial.device):
        _lib.check(_lib.lib().fwa2_finalize_grads(
            partial.data_ptr(), _DTYPES[ref.dtype], h, n,
            logit_scale.data_ptr() if dscale is not None else None,
            db.data_ptr() if db is not None else None,
            dscale.data_ptr() if dscale is not None else None,
            _stream(partial.device)), "fwa2_finalize_grads")
