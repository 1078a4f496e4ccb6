"""The CPU oracle against golden vectors produced by the reference itself."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import CASES, build_inputs  # noqa: E402

from oracle import window_attention_oracle as orc  # noqa: E402


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_golden(name, golden_dir):
    gold = np.load(os.path.join(golden_dir, name + ".npz"))
    w, t = build_inputs(name)
    np_in = {k: (v.double().numpy() if v is not None else None) for k, v in t.items()}
    res = orc.forward_backward(np_in["q"], np_in["k"], np_in["v"], np_in["do"],
                               np_in["logit_scale"], np_in["bias"], np_in["mask"], dtype=np.float64)
    for key in ("o", "dq", "dk", "dv", "dbias", "dscale"):
        if key not in gold.files:
            assert res[key] is None
            continue
        # golden tensors are stored as float32: agreement is limited by that rounding
        assert orc.rel_err(res[key], gold[key]) < 2e-7, key
        # float64 norms are stored exactly
        assert abs(np.linalg.norm(res[key].ravel()) - float(gold[key + "_norm64"])) \
            <= 1e-10 * max(1.0, float(gold[key + "_norm64"])), key


def test_oracle_fp32_close_to_fp64():
    w, t = build_inputs("cfg1")
    np_in = {k: (v.numpy() if v is not None else None) for k, v in t.items()}
    r32 = orc.forward_backward(np_in["q"], np_in["k"], np_in["v"], np_in["do"],
                               np_in["logit_scale"], np_in["bias"], np_in["mask"], dtype=np.float32)
    r64 = orc.forward_backward(np_in["q"], np_in["k"], np_in["v"], np_in["do"],
                               np_in["logit_scale"], np_in["bias"], np_in["mask"], dtype=np.float64)
    for key in ("o", "dq", "dk", "dv", "dbias", "dscale"):
        assert orc.rel_err(r32[key], r64[key]) < 5e-6, key


def test_lse_rows_sum_to_one():
    w, t = build_inputs("n144_ragged")
    o, lse = orc.forward(t["q"].numpy(), t["k"].numpy(), t["v"].numpy(), t["logit_scale"].numpy(),
                         t["bias"].numpy(), t["mask"].numpy())
    a, *_ = orc._scores(t["q"].double().numpy(), t["k"].double().numpy(), t["logit_scale"].numpy(),
                        t["bias"].numpy(), t["mask"].numpy(), np.float64)
    assert np.allclose(np.exp(a - lse[..., None]).sum(-1), 1.0, atol=1e-12)


def test_shift_mask_matches_workload_builder():
    from flash_window_attention_v2_b200.workloads import shift_mask
    m = orc.swin_shift_mask(16, 16, 8, 4)
    assert m.shape == (4, 64, 64)
    assert np.array_equal(m, shift_mask(16, 8, 4).numpy())
    assert 0.5 < (m == 0).mean() < 0.6
