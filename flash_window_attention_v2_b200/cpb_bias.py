"""The step in front of the operator in a Swin-V2 block, fused with it.

`swin_transformer_v2.py:283-287` builds the relative-position bias as
`16 * sigmoid(table[index].view(N, N, H).permute(2, 0, 1))` with `table = cpb_mlp(coords)` of shape
(R, H) and `index` the (N, N) relative-position index.  `cpb_bias(table, index)` is that step as
one kernel; `flash_win_attn_v2_cpb_func(q, k, v, logit_scale, table, index, mask)` is the attention
operator fed by it, whose backward hands the gradient of `table` straight from the fp32
window-summed dBias of the attention backward -- the (H, N, N) gradient never exists in 16 bits.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from . import kernels as _kernels

_inverse_cache: dict = {}


def _index32(index: torch.Tensor) -> torch.Tensor:
    return index.reshape(-1).to(torch.int32).contiguous()


def inverse_index(index: torch.Tensor, rows: int):
    """CSR inverse of the (N, N) index: (row_offsets int32 (rows + 1), positions int32 (N * N)),
    positions of a row ascending.  Cached per index tensor (it is a module buffer)."""
    key = (index.data_ptr(), tuple(index.shape), index.device, rows, index._version)
    hit = _inverse_cache.get(key)
    if hit is not None:
        return hit
    flat = index.reshape(-1).to(torch.int64)
    order = torch.sort(flat, stable=True).indices.to(torch.int32).contiguous()
    counts = torch.bincount(flat, minlength=rows)
    offsets = torch.zeros(rows + 1, dtype=torch.int32, device=index.device)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    # one entry per index buffer (every Swin block has its own), oldest dropped beyond 64
    if len(_inverse_cache) >= 64:
        _inverse_cache.pop(next(iter(_inverse_cache)))
    _inverse_cache[key] = (offsets, order)
    return offsets, order


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def cpb_bias_forward(table: torch.Tensor, index: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """bias (H, N, N) of `dtype` = 16 * sigmoid(table[index]) (no autograd)."""
    assert table.is_cuda and table.dim() == 2 and table.is_contiguous()
    assert table.dtype in (torch.float32, dtype) and dtype in _kernels._DTYPES
    rows, heads = table.shape
    n = index.shape[0]
    assert index.shape == (n, n)
    bias = torch.empty(heads, n, n, dtype=dtype, device=table.device)
    with torch.cuda.device(table.device):
        _lib.check(_lib.lib().fwa2_cpb_bias_forward(
            table.data_ptr(), 1 if table.dtype == torch.float32 else 0, _index32(index).data_ptr(),
            _kernels._DTYPES[dtype], n, heads, rows, bias.data_ptr(), _stream(table.device)), "fwa2_cpb_bias_forward")
    return bias


def cpb_bias_backward(dbias_f32: torch.Tensor, table: torch.Tensor, index: torch.Tensor, dtype: torch.dtype):
    """dtable (R, H) fp32 from the fp32 dBias (H * N * N values, e.g. the head of `partial_out`)."""
    rows, heads = table.shape
    n = index.shape[0]
    assert dbias_f32.dtype == torch.float32 and dbias_f32.is_contiguous() and dbias_f32.numel() >= heads * n * n
    offsets, positions = inverse_index(index, rows)
    dtable = torch.empty(rows, heads, dtype=torch.float32, device=table.device)
    with torch.cuda.device(table.device):
        _lib.check(_lib.lib().fwa2_cpb_bias_backward(
            dbias_f32.data_ptr(), table.data_ptr(), 1 if table.dtype == torch.float32 else 0,
            _kernels._DTYPES[dtype], offsets.data_ptr(), positions.data_ptr(), n, heads, rows,
            dtable.data_ptr(), _stream(table.device)), "fwa2_cpb_bias_backward")
    return dtable


class _CpbBias(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, index, dtype):
        ctx.save_for_backward(table, index)
        ctx.out_dtype = dtype
        return cpb_bias_forward(table.contiguous(), index, dtype)

    @staticmethod
    def backward(ctx, dbias):
        table, index = ctx.saved_tensors
        dt = cpb_bias_backward(dbias.float().contiguous(), table.contiguous(), index, ctx.out_dtype)
        return dt.to(table.dtype), None, None


def cpb_bias(table: torch.Tensor, index: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
    """Differentiable 16 * sigmoid(table[index]) -> (H, N, N); `dtype` defaults to the table's."""
    return _CpbBias.apply(table, index, dtype if dtype is not None else table.dtype)


class FlashWindowAttentionV2Cpb(torch.autograd.Function):
    """flash_win_attn_v2_func with the bias given as (table, index); same outputs, and the gradient
    of `table` instead of the gradient of the bias."""

    @staticmethod
    def forward(ctx, q, k, v, logit_scale, table, index, mask=None):
        if logit_scale is not None:
            scale_type = "tensor"
            ls = logit_scale if logit_scale.stride(-1) == 1 else logit_scale.contiguous()
        else:
            scale_type = "scalar"
            ls = torch.tensor(1.0 / math.sqrt(q.shape[-1]), device=q.device)
        q, k, v = [x if x.stride(-1) == 1 else x.contiguous() for x in (q, k, v)]
        table_c = table.contiguous()
        bias = cpb_bias_forward(table_c, index, q.dtype)
        o, lse, ls = _kernels._flash_attn_forward(q, k, v, ls, bias=bias, mask=mask, scale_type=scale_type)
        ctx.save_for_backward(q, k, v, o, lse, ls, bias, mask, table_c, index)
        ctx.scale_type = scale_type
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, ls, bias, mask, table, index = ctx.saved_tensors
        h, n = q.shape[1], q.shape[2]
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        partial = torch.empty(h * n * n + h, dtype=torch.float32, device=q.device)
        _kernels._flash_attn_backward(do, q, k, v, ls, o, lse, dq, dk, dv, None, None, bias=bias, mask=mask,
                                      scale_type=ctx.scale_type, _partial_out=partial)
        dscale = None
        if ctx.scale_type == "tensor":
            dscale = torch.empty_like(ls)
            _kernels.finalize_grads(partial, ls, None, dscale)
        dtable = cpb_bias_backward(partial, table, index, q.dtype).to(table.dtype)
        return dq, dk, dv, dscale, dtable, None, None


def flash_win_attn_v2_cpb_func(q, k, v, logit_scale, table, index, mask=None):
    return FlashWindowAttentionV2Cpb.apply(q, k, v, logit_scale, table, index, mask)
