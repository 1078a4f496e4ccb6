"""The reference's own `WindowAttention` module (flash_win_attn_v2/swin_transformer_v2.py:188-298)
with `is_flash=True`, routed through these kernels by `install()`, against the same module with
`is_flash=False` (its classic PyTorch path) evaluated in fp32 on the same parameters and inputs.
Forward output and every parameter / input gradient are compared, shifted and unshifted."""
import copy

import pytest
import torch

from flash_window_attention_v2_b200 import install, kernels, uninstall
from flash_window_attention_v2_b200.workloads import shift_mask
from tests import _reference as ref

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref.available(), reason="reference not installed under baseline/_ref")]


@pytest.fixture()
def reference_on_these_kernels():
    ref.forget()
    install()
    pkg = ref.import_reference()
    yield pkg
    uninstall()
    ref.forget()


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))


@pytest.mark.parametrize("window,heads,shifted,dtype", [
    (16, 4, True, torch.bfloat16), (16, 4, False, torch.bfloat16), (8, 3, True, torch.float16),
    (12, 2, True, torch.float16),
])
def test_window_attention_module(reference_on_these_kernels, window, heads, shifted, dtype):
    pkg = reference_on_these_kernels
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    dim, n = heads * 32, window * window
    images, nw = 3, 4
    flash = pkg.WindowAttention(dim, (window, window), heads, is_flash=True).to(dev)
    with torch.no_grad():      # make bias, scale and the qkv biases non-trivial
        flash.q_bias.normal_(0, 0.5)
        flash.v_bias.normal_(0, 0.5)
        flash.logit_scale.add_(torch.randn_like(flash.logit_scale) * 0.3)
    classic = copy.deepcopy(flash)
    classic.is_flash = False
    flash = flash.to(dtype)
    # the classic twin sees the parameters the 16-bit module sees, in fp32
    classic.load_state_dict({k: v.float() for k, v in flash.state_dict().items()})
    x = torch.randn(images * nw, n, dim, device=dev).to(dtype)
    g = torch.randn(images * nw, n, dim, device=dev).to(dtype)
    mask = shift_mask(2 * window, window, window // 2).to(dev) if shifted else None

    xf = x.clone().requires_grad_(True)
    yf = flash(xf, mask.to(dtype) if mask is not None else None)
    yf.backward(g)
    xc = x.float().requires_grad_(True)
    yc = classic(xc, mask)
    yc.backward(g.float())
    kernels.check_device_status(dev)

    tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
    assert rel(yf, yc) < tol
    assert rel(xf.grad, xc.grad) < tol
    got = dict(flash.named_parameters())
    for name, pc in classic.named_parameters():
        if pc.grad is None:
            continue
        e = rel(got[name].grad, pc.grad)
        # logit_scale sums largely cancelling terms; the 16-bit module also rounds its gradient
        lim = 5 * tol if name == "logit_scale" else 2 * tol
        assert e < lim, (name, e)
