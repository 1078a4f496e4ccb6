"""`install()` is what lets the reference's own files run unchanged on these kernels
(flash_win_attn_v2/flash_window_attention_v2.py:3 imports the two names, :22 and :40 look them up
as module globals).  Both orders are checked: install before the reference is imported, and after.
Needs the reference installed under baseline/_ref (skipped otherwise); no GPU."""
import sys

import pytest

from flash_window_attention_v2_b200 import install, kernels, uninstall
from tests import _reference as ref

pytestmark = pytest.mark.skipif(not ref.available(), reason="reference not installed under baseline/_ref")


@pytest.fixture(autouse=True)
def clean_modules():
    ref.forget()
    yield
    uninstall()
    ref.forget()


def test_install_before_import_never_loads_the_triton_files():
    install()
    pkg = ref.import_reference()
    fw = sys.modules["flash_win_attn_v2.flash_window_attention_v2"]
    assert fw._flash_attn_forward is kernels._flash_attn_forward
    assert fw._flash_attn_backward is kernels._flash_attn_backward
    assert sys.modules["flash_win_attn_v2.kernels"] is kernels
    assert "flash_win_attn_v2.kernels.attn_kernel_forward" not in sys.modules
    assert "flash_win_attn_v2.kernels.attn_kernel_backward" not in sys.modules
    # the public function of the reference is its own autograd Function, now on these kernels
    assert pkg.flash_win_attn_v2_func.__self__ is fw.FlashWindowAttentionV2


def test_install_after_import_rebinds_the_two_names():
    pkg = ref.import_reference()
    fw = sys.modules["flash_win_attn_v2.flash_window_attention_v2"]
    assert fw._flash_attn_forward is not kernels._flash_attn_forward      # the Triton wrappers
    install()
    assert fw._flash_attn_forward is kernels._flash_attn_forward
    assert fw._flash_attn_backward is kernels._flash_attn_backward
    assert pkg.kernels is kernels
