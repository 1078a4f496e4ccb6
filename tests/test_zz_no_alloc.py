"""The allocation-free backward entry point (fwa2_backward_static_scratch).

It serves callers that may not allocate device memory at the point of the call (inside a host
framework that owns the allocator, in a warmed-up serving loop that bans allocator calls).  The test
goes through the C ABI directly: everything the call touches is allocated beforehand, the entry
point gets no workspace, and its results must equal those of the regular entry point (the
kernels are deterministic, so the comparison is exact) on two calls in a row, the second of
which finds the first one's leftovers in the shared scratch array.
"""
import ctypes as C
import math

import pytest
import torch

from flash_window_attention_v2_b200 import _lib
from flash_window_attention_v2_b200 import kernels as K
from flash_window_attention_v2_b200.workloads import Workload, make_inputs

pytestmark = pytest.mark.gpu


def _bwd_args(t, o, lse, outs, workspace):
    q = t["q"]
    a = _lib.BwdArgs()
    a.struct_size = C.sizeof(_lib.BwdArgs)
    a.abi_version = _lib.FWA2_ABI_VERSION
    a.dtype = _lib.FWA2_BF16 if q.dtype == torch.bfloat16 else _lib.FWA2_F16
    a.bw, a.heads, a.n, a.head_dim = q.shape
    a.n_windows = t["mask"].shape[0]
    t4 = lambda x: _lib.Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2))
    a.q, a.k, a.v, a.o, a.dout = t4(q), t4(t["k"]), t4(t["v"]), t4(o), t4(t["do"])
    a.dq, a.dk, a.dv = t4(outs["dq"]), t4(outs["dk"]), t4(outs["dv"])
    a.lse, a.lse_stride_bw, a.lse_stride_h = lse.data_ptr(), lse.stride(0), lse.stride(1)
    a.logit_scale, a.scale_is_tensor = t["logit_scale"].data_ptr(), 1
    a.bias, a.mask = t["bias"].data_ptr(), t["mask"].data_ptr()
    a.bias_row_stride, a.mask_row_stride = t["bias"].stride(1), t["mask"].stride(1)
    a.dbias, a.dscale = outs["db"].data_ptr(), outs["dscale"].data_ptr()
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return a


@pytest.mark.parametrize("w", [Workload("na64", batch=4, nw=4, heads=3, window=8, dtype="fp16"),
                               Workload("na256", batch=2, nw=4, heads=2, window=16, dtype="bf16")],
                         ids=lambda w: w.name)
def test_static_scratch_backward_matches_workspace_backward(w):
    dev = torch.device("cuda:0")
    L = _lib.lib()
    t = make_inputs(w, seed=0, device=dev)
    o, lse, _ = K._flash_attn_forward(t["q"], t["k"], t["v"], t["logit_scale"], bias=t["bias"], mask=t["mask"],
                                      scale_type="tensor")
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def fresh():
        return dict(dq=torch.full_like(t["q"], float("nan")), dk=torch.full_like(t["k"], float("nan")),
                    dv=torch.full_like(t["v"], float("nan")), db=torch.full_like(t["bias"], float("nan")),
                    dscale=torch.full_like(t["logit_scale"], float("nan")))

    need = L.fwa2_bwd_workspace_bytes(t["q"].shape[0], w.heads, w.n, w.nw, 1, 1)
    assert 0 < need <= 48 << 20
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    ref = fresh()
    _lib.check(L.fwa2_backward(C.byref(_bwd_args(t, o, lse, ref, ws)), stream), "fwa2_backward")

    for call in range(2):
        got = fresh()
        _lib.check(L.fwa2_backward_static_scratch(C.byref(_bwd_args(t, o, lse, got, None)), stream),
                   "fwa2_backward_static_scratch")
        K.check_device_status(dev)
        for key in ref:
            assert torch.equal(got[key], ref[key]), (call, key)


def test_static_scratch_refuses_oversized_problems():
    L = _lib.lib()
    a = _lib.BwdArgs()
    a.struct_size = C.sizeof(_lib.BwdArgs)
    a.abi_version = _lib.FWA2_ABI_VERSION
    a.dtype, a.bw, a.heads, a.n, a.head_dim, a.n_windows = 1, 4096, 16, 576, 32, 64
    a.bias = 256          # never dereferenced: the size check comes first
    assert L.fwa2_bwd_workspace_bytes(4096, 16, 576, 64, 1, 0) > 48 << 20
    assert L.fwa2_backward_static_scratch(C.byref(a), None) == -12
    assert b"scratch" in L.fwa2_strerror(-12)
