"""CPU-only checks of the C-ABI library: it loads without a GPU, exports every symbol that
include/fwa2.h declares, and rejects bad arguments before touching the device."""
import ctypes as C
import os
import re

import pytest

from flash_window_attention_v2_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.lib()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "fwa2.h")).read()
    declared = set(re.findall(r"\b(fwa2_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_variant_bits_match_the_header():
    """The variant bits the Python binding names are the ones include/fwa2.h defines, and no two
    of them share a bit."""
    header = open(os.path.join(ROOT, "include", "fwa2.h")).read()
    defined = {name: int(value) for name, value in re.findall(r"#define\s+(FWA2_(?:FWD|BWD)_[A-Z_]+)\s+(\d+)", header)}
    assert defined, "no variant bits found in the header"
    for name, value in defined.items():
        assert getattr(_lib, name) == value, name
        assert value & (value - 1) == 0, name          # a single bit
    assert len(set(defined.values())) == len(defined)


def test_struct_sizes_match_header_layout():
    # plain-C layout: 4 + 4 + 4 + 4*4 + 4 = 32 bytes of scalars, then 8-byte aligned members
    assert C.sizeof(_lib.Tensor4) == 32
    assert C.sizeof(_lib.FwdArgs) % 8 == 0 and C.sizeof(_lib.BwdArgs) % 8 == 0
    assert _lib.FwdArgs.q.offset == 32 and _lib.BwdArgs.q.offset == 32


def test_abi_version_and_strerror(lib):
    assert lib.fwa2_abi_version() == _lib.FWA2_ABI_VERSION
    assert lib.fwa2_strerror(0) == b"ok"
    assert b"head dimension" in lib.fwa2_strerror(-3)


def test_forward_workspace_size_needs_no_device(lib):
    """The forward asks for scratch (one fp32 table bias + mask per window type and head) only for
    windows of 129 to 256 tokens with both tables, and then only when told to or when every table
    serves enough images to pay for the pass that builds it."""
    f = lib.fwa2_fwd_workspace_bytes
    table = 64 * 3 * 256 * 256 * 4
    assert f(64 * 64, 3, 256, 64, 1, 1, 0) == table             # 64 images per window type
    assert f(8 * 64, 3, 256, 64, 1, 1, 0) == 0                  # 8 images: separate tables
    assert f(8 * 64, 3, 256, 64, 1, 1, _lib.FWA2_FWD_COMBINE_TABLES) == table
    assert f(64 * 64, 3, 256, 64, 1, 1, _lib.FWA2_FWD_SEPARATE_TABLES) == 0
    assert f(64 * 64, 3, 256, 64, 1, 1, _lib.FWA2_FWD_GENERAL_KERNEL) == 0
    assert f(64 * 64, 3, 256, 64, 0, 1, 0) == 0 and f(64 * 64, 3, 256, 64, 1, 0, 0) == 0
    assert f(64 * 64, 3, 64, 64, 1, 1, 64) == 0 and f(64 * 64, 3, 128, 64, 1, 1, 64) == 0
    assert f(64 * 64, 3, 257, 64, 1, 1, 64) == 0
    assert f(40 * 4, 2, 144, 4, 1, 1, 0) == 4 * 2 * 144 * 160 * 4    # rows of 144 padded to 160 floats
    assert f(4097, 3, 256, 64, 1, 1, 64) == 0                   # BW no multiple of the window types
    assert f(0, 3, 256, 64, 1, 1, 64) == 0


def _fwd_args(**kw):
    a = _lib.FwdArgs()
    a.struct_size = C.sizeof(_lib.FwdArgs)
    a.abi_version = _lib.FWA2_ABI_VERSION
    a.dtype, a.bw, a.heads, a.n, a.head_dim = 1, 4, 2, 64, 32
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_forward_rejects_bad_arguments_without_a_device(lib):
    assert lib.fwa2_forward(None, None) == -1
    assert lib.fwa2_forward(C.byref(_fwd_args(struct_size=8)), None) == -10
    assert lib.fwa2_forward(C.byref(_fwd_args(dtype=7)), None) == -2
    assert lib.fwa2_forward(C.byref(_fwd_args(head_dim=64)), None) == -3
    assert lib.fwa2_forward(C.byref(_fwd_args(n=0)), None) == -4
    assert lib.fwa2_forward(C.byref(_fwd_args(n=641)), None) == -4
    # valid sizes but null tensors
    assert lib.fwa2_forward(C.byref(_fwd_args()), None) == -1


def test_backward_rejects_bad_arguments_without_a_device(lib):
    a = _lib.BwdArgs()
    a.struct_size = C.sizeof(_lib.BwdArgs)
    a.abi_version = _lib.FWA2_ABI_VERSION
    a.dtype, a.bw, a.heads, a.n, a.head_dim = 0, 4, 2, 64, 16
    assert lib.fwa2_backward(C.byref(a), None) == -3
    a.head_dim = 32
    assert lib.fwa2_backward(C.byref(a), None) == -1


def test_workspace_size_formula(lib):
    # no device here: the library assumes 148 SMs
    assert lib.fwa2_bwd_workspace_bytes(0, 3, 64, 4, 1, 1) == 0
    small = lib.fwa2_bwd_workspace_bytes(8, 3, 64, 4, 1, 1)
    big = lib.fwa2_bwd_workspace_bytes(4096, 3, 256, 64, 1, 1)
    nobias = lib.fwa2_bwd_workspace_bytes(4096, 3, 256, 64, 0, 1)
    assert 0 < small < big and nobias < big
    # 147 partial buffers of 256 x 256 fp32 dominate
    assert big >= 147 * 256 * 256 * 4


def test_entry_points_reject_null_buffers_on_the_host(lib):
    """A null pointer must come back as an error code, never reach a kernel."""
    assert lib.fwa2_selftest_mma(0, 1, None, None, None, None, None) == -1
    assert lib.fwa2_finalize_grads(None, 1, 3, 64, None, None, None, None) == -1
    arr = (C.c_void_p * 2)(None, None)
    assert lib.fwa2_peer_reduce_finalize(arr, arr, 0, 2, 1, 1, 3, 64, None, None, None, None, None) == -1
    assert lib.fwa2_peer_reduce_finalize(arr, arr, 0, 9, 1, 1, 3, 64, None, None, None, None, None) == -4
