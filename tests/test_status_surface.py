"""A device-side timeout must not stay silent: the boundary functions look at a pinned host mirror
of the status block at the start of every call and raise.  Host-level test: the mirror is filled by
hand (no kernel is made to time out, no GPU is needed)."""
import pytest
import torch

from flash_window_attention_v2_b200 import kernels as K


def _fake_entry(idx=0):
    dev_block = torch.zeros(4, dtype=torch.int32)      # stands in for the device block
    host_block = torch.zeros(4, dtype=torch.int32)     # stands in for the pinned mirror
    K._status_words[idx] = (dev_block, host_block)
    return dev_block, host_block


def test_poll_is_silent_when_clean(monkeypatch):
    monkeypatch.setattr(K, "_status_words", {})
    _fake_entry(0)
    K.poll_device_status(torch.device("cuda", 0))       # nothing recorded: no exception


def test_poll_raises_once_and_clears(monkeypatch):
    monkeypatch.setattr(K, "_status_words", {})
    _, host_block = _fake_entry(0)
    host_block[0] = (52 << 8) | 1      # site 52, kind 1 (timeout)
    host_block[1] = 7                  # block
    with pytest.raises(K.DeviceTimeoutError) as ei:
        K.poll_device_status(torch.device("cuda", 0))
    assert "site 52" in str(ei.value) and "block 7" in str(ei.value)
    K.poll_device_status(torch.device("cuda", 0))       # cleared: the next call is clean again


def test_boundary_functions_check_first(monkeypatch):
    """Both boundary functions raise on a stale timeout before they look at their arguments."""
    monkeypatch.setattr(K, "_status_words", {})
    _, host_block = _fake_entry(0)
    q = torch.zeros(4, 2, 64, 32, dtype=torch.bfloat16)        # CPU tensors: never reached
    monkeypatch.setattr(K, "poll_device_status", lambda device=None: (_ for _ in ()).throw(K.DeviceTimeoutError("x")))
    with pytest.raises(K.DeviceTimeoutError):
        K._flash_attn_forward(q, q, q, torch.zeros(2, 1, 1), scale_type="tensor")
    with pytest.raises(K.DeviceTimeoutError):
        K._flash_attn_backward(q, q, q, q, None, q, None, q, q, q, None, None)
