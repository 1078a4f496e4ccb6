"""ctypes binding of libfwa2_b200.so (the C ABI declared in include/fwa2.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.  `build()` compiles the library in-tree with nvcc for
sm_100a.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libfwa2_b200.so")
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["fwa2_api.cu", "fwa2_fwd.cu", "fwa2_fwd_duo.cu", "fwa2_bwd.cu", "fwa2_bwd_quad.cu", "fwa2_reduce.cu", "fwa2_selftest.cu",
           "fwa2_static_scratch.cu", "fwa2_cpb_bias.cu", "fwa2_peer_reduce.cu"]

FWA2_ABI_VERSION = 2
FWA2_F16, FWA2_BF16 = 0, 1
# bits of fwd / bwd args.variant (include/fwa2.h)
FWA2_FWD_P_IN_SMEM = 1
FWA2_BWD_SKIP_TABLES = 2
FWA2_BWD_SKIP_REDUCE = 4
FWA2_BWD_GENERAL_KERNEL = 16
FWA2_FWD_GENERAL_KERNEL = 32
FWA2_FWD_COMBINE_TABLES = 64
FWA2_FWD_SEPARATE_TABLES = 128


class Tensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_bw", C.c_int64), ("stride_h", C.c_int64),
                ("stride_n", C.c_int64)]


class FwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("abi_version", C.c_uint32), ("dtype", C.c_int32),
        ("bw", C.c_int32), ("heads", C.c_int32), ("n", C.c_int32), ("head_dim", C.c_int32),
        ("n_windows", C.c_int32),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4),
        ("lse", C.c_void_p), ("lse_stride_bw", C.c_int64), ("lse_stride_h", C.c_int64),
        ("logit_scale", C.c_void_p), ("scale_is_tensor", C.c_int32),
        ("bias", C.c_void_p), ("mask", C.c_void_p),
        ("bias_row_stride", C.c_int64), ("mask_row_stride", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p), ("variant", C.c_int32), ("max_ctas", C.c_int32),
        ("developer0", C.c_void_p), ("developer1", C.c_int32), ("reserved0", C.c_int32),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("abi_version", C.c_uint32), ("dtype", C.c_int32),
        ("bw", C.c_int32), ("heads", C.c_int32), ("n", C.c_int32), ("head_dim", C.c_int32),
        ("n_windows", C.c_int32),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4), ("dout", Tensor4),
        ("dq", Tensor4), ("dk", Tensor4), ("dv", Tensor4),
        ("lse", C.c_void_p), ("lse_stride_bw", C.c_int64), ("lse_stride_h", C.c_int64),
        ("logit_scale", C.c_void_p), ("scale_is_tensor", C.c_int32),
        ("bias", C.c_void_p), ("mask", C.c_void_p),
        ("bias_row_stride", C.c_int64), ("mask_row_stride", C.c_int64),
        ("dbias", C.c_void_p), ("dscale", C.c_void_p), ("partial_out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p), ("variant", C.c_int32), ("max_ctas", C.c_int32),
        ("developer0", C.c_void_p), ("developer1", C.c_int32), ("reserved0", C.c_int32),
    ]


EXPORTS = ("fwa2_abi_version", "fwa2_strerror", "fwa2_last_cuda_error", "fwa2_forward",
           "fwa2_fwd_workspace_bytes", "fwa2_bwd_workspace_bytes", "fwa2_backward", "fwa2_finalize_grads",
           "fwa2_selftest_mma", "fwa2_backward_static_scratch",
           "fwa2_cpb_bias_forward", "fwa2_cpb_bias_backward", "fwa2_peer_reduce_finalize")


def nvcc_command(out_path: str = LIB_PATH, verbose: bool = False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xcompiler", "-fPIC", "-shared", "-o", out_path]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    return cmd + [os.path.join(CSRC, s) for s in SOURCES]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources into libfwa2_b200.so next to this file (cross-compiles for
    sm_100a; no GPU needed).  Skipped when the library is newer than every source."""
    srcs = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "fwa2.h")]
    if not force and os.path.exists(LIB_PATH):
        if os.path.getmtime(LIB_PATH) >= max(os.path.getmtime(s) for s in srcs):
            return LIB_PATH
    res = subprocess.run(nvcc_command(verbose=verbose), capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with "
                "`python -c 'import __graft_entry__ as g; g.build()'` (needs nvcc). "
                "There is no fallback implementation.")
        L = C.CDLL(LIB_PATH)
        L.fwa2_abi_version.restype = C.c_int
        L.fwa2_strerror.restype = C.c_char_p
        L.fwa2_strerror.argtypes = [C.c_int]
        L.fwa2_last_cuda_error.restype = C.c_int
        L.fwa2_forward.restype = C.c_int
        L.fwa2_forward.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
        L.fwa2_fwd_workspace_bytes.restype = C.c_size_t
        L.fwa2_fwd_workspace_bytes.argtypes = [C.c_int32] * 7
        L.fwa2_bwd_workspace_bytes.restype = C.c_size_t
        L.fwa2_bwd_workspace_bytes.argtypes = [C.c_int32] * 6
        L.fwa2_backward.restype = C.c_int
        L.fwa2_backward.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
        L.fwa2_finalize_grads.restype = C.c_int
        L.fwa2_finalize_grads.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p]
        L.fwa2_selftest_mma.restype = C.c_int
        L.fwa2_selftest_mma.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p]
        L.fwa2_backward_static_scratch.restype = C.c_int
        L.fwa2_backward_static_scratch.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
        L.fwa2_cpb_bias_forward.restype = C.c_int
        L.fwa2_cpb_bias_forward.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                            C.c_int32, C.c_void_p, C.c_void_p]
        L.fwa2_cpb_bias_backward.restype = C.c_int
        L.fwa2_cpb_bias_backward.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                             C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
        L.fwa2_peer_reduce_finalize.restype = C.c_int
        L.fwa2_peer_reduce_finalize.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int32, C.c_int32,
                                                C.c_uint32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                                C.c_void_p, C.c_void_p, C.c_void_p]
        if L.fwa2_abi_version() != FWA2_ABI_VERSION:
            raise RuntimeError("libfwa2_b200.so ABI version mismatch; rebuild it")
        _lib = L
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        L = lib()
        raise RuntimeError(f"{what} failed: {L.fwa2_strerror(code).decode()} "
                           f"(code {code}, cuda error {L.fwa2_last_cuda_error()})")
