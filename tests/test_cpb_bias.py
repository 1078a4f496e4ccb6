"""The bias-preparation step in front of the operator (16 * sigmoid of a gathered table) and the
attention function fed by it: the numpy oracle is pinned against torch autograd of the reference's
own expression (swin_transformer_v2.py:283-287) on the CPU; the CUDA kernels are held to the oracle."""
import math

import numpy as np
import pytest
import torch

from oracle import window_attention_oracle as orc


def _reference_expression(table, index):
    n = index.shape[0]
    b = table[index.view(-1)].view(n, n, -1).permute(2, 0, 1).contiguous()
    return 16 * torch.sigmoid(b)


@pytest.mark.parametrize("wh,ww,heads", [(8, 8, 3), (7, 7, 4), (16, 16, 2), (4, 6, 5)])
def test_oracle_matches_the_reference_expression_and_its_autograd(wh, ww, heads):
    g = torch.Generator().manual_seed(wh * 100 + ww)
    rows = (2 * wh - 1) * (2 * ww - 1)
    index = torch.from_numpy(orc.relative_position_index(wh, ww))
    assert index.min() == 0 and index.max() == rows - 1
    table = torch.randn(rows, heads, generator=g, dtype=torch.float64, requires_grad=True)
    bias = _reference_expression(table, index)
    dbias = torch.randn(bias.shape, generator=g, dtype=torch.float64)
    (dtable,) = torch.autograd.grad(bias, table, dbias)
    np.testing.assert_allclose(orc.cpb_bias(table.detach().numpy(), index.numpy()), bias.detach().numpy(), rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(orc.cpb_bias_backward(dbias.numpy(), table.detach().numpy(), index.numpy()),
                               dtable.numpy(), rtol=1e-11, atol=1e-11)


@pytest.mark.gpu
@pytest.mark.parametrize("wh,heads,dtype,table_f32", [(8, 3, torch.float16, False), (8, 3, torch.bfloat16, True),
                                                       (7, 4, torch.bfloat16, False), (16, 6, torch.float16, False)])
def test_cuda_bias_step_matches_the_oracle(wh, heads, dtype, table_f32):
    from flash_window_attention_v2_b200.cpb_bias import cpb_bias_backward, cpb_bias_forward
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(wh)
    rows, n = (2 * wh - 1) ** 2, wh * wh
    index = torch.from_numpy(orc.relative_position_index(wh, wh)).to(dev)
    table = (2.0 * torch.randn(rows, heads, generator=g)).to(torch.float32 if table_f32 else dtype).to(dev)
    bias = cpb_bias_forward(table, index, dtype)
    want = orc.cpb_bias(table.float().cpu().numpy(), index.cpu().numpy())
    # one unit in the last place of the 16-bit result (the sigmoid is rounded before the exact * 16)
    ulp = 16.0 * (2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7)
    assert np.abs(bias.float().cpu().numpy() - want).max() <= ulp
    dbias = torch.randn(heads, n, n, generator=g).to(dev)
    got = cpb_bias_backward(dbias, table, index, dtype).cpu().numpy()
    ref = orc.cpb_bias_backward(dbias.cpu().numpy(), table.float().cpu().numpy(), index.cpu().numpy())
    assert orc.rel_err(got, ref) < 2e-6
    again = cpb_bias_backward(dbias, table, index, dtype).cpu().numpy()
    assert np.array_equal(got, again)           # fixed summation order


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_attention_fed_by_the_bias_step(dtype):
    """flash_win_attn_v2_cpb_func == flash_win_attn_v2_func(bias = 16 sigmoid(table[index])) in the
    outputs and in dq, dk, dv, dscale; its table gradient follows the oracle chain (attention
    backward in fp64, then the bias step's backward), with no 16-bit dBias in between."""
    from flash_window_attention_v2_b200 import flash_win_attn_v2_func
    from flash_window_attention_v2_b200.cpb_bias import cpb_bias_forward, flash_win_attn_v2_cpb_func
    from flash_window_attention_v2_b200.workloads import Workload, make_inputs
    dev = torch.device("cuda:0")
    w = Workload("n64", batch=4, nw=4, heads=3, window=8, dtype="fp16" if dtype == torch.float16 else "bf16")
    t = make_inputs(w, seed=3, device=dev)
    rows = (2 * 8 - 1) ** 2
    index = torch.from_numpy(orc.relative_position_index(8, 8)).to(dev)
    table = torch.randn(rows, 3, generator=torch.Generator().manual_seed(5)).to(dtype).to(dev)

    def leaves():
        return [t[x].detach().requires_grad_(True) for x in ("q", "k", "v")] + [t["logit_scale"].detach().requires_grad_(True)]

    q, k, v, ls = leaves()
    tb = table.detach().requires_grad_(True)
    o = flash_win_attn_v2_cpb_func(q, k, v, ls, tb, index, t["mask"])
    dq, dk, dv, dls, dtable = torch.autograd.grad(o, (q, k, v, ls, tb), t["do"])

    q2, k2, v2, ls2 = leaves()
    bias = cpb_bias_forward(table, index, dtype).requires_grad_(True)
    o2 = flash_win_attn_v2_func(q2, k2, v2, ls2, bias, t["mask"])
    dq2, dk2, dv2, dls2, _ = torch.autograd.grad(o2, (q2, k2, v2, ls2, bias), t["do"])
    for a, b in ((o, o2), (dq, dq2), (dk, dk2), (dv, dv2), (dls, dls2)):
        assert torch.equal(a, b)

    f = lambda x: x.float().cpu().numpy()
    ref = orc.forward_backward(f(t["q"]), f(t["k"]), f(t["v"]), f(t["do"]), f(t["logit_scale"]), f(bias.detach()), f(t["mask"]),
                               dtype=np.float64)
    want = orc.cpb_bias_backward(ref["dbias"], f(table), f(index).astype(np.int64))
    assert orc.rel_err(f(dtable), want) < (2e-3 if dtype == torch.float16 else 1e-2)
