"""ctypes binding of the C ABI declared in include/monarch_attention_b200.h.

The shared library is the product: if it is missing this module raises - there is
no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

ABI_VERSION = 1
F32, BF16, F16 = 0, 1, 2
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_TCGEN05, KERNEL_TCGEN05_STAGED, KERNEL_WARP_MMA, KERNEL_HEAD_FUSED = 0, 1, 2, 3, 5, 6
KERNEL_NAMES = {KERNEL_AUTO: "auto", KERNEL_GENERIC: "generic", KERNEL_TCGEN05: "tcgen05-fused",
                KERNEL_TCGEN05_STAGED: "tcgen05-staged",
                KERNEL_WARP_MMA: "warp-mma", KERNEL_HEAD_FUSED: "head-fused"}
OK, INVALID_ARGUMENT, UNSUPPORTED, CUDA_ERROR, DEVICE_WAIT_EXPIRED, WORKSPACE_TOO_SMALL = range(6)

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libmonarch_attention_b200.so")

EXPORTS = (
    "ma_b200_workspace_bytes", "ma_b200_workspace_layout_of", "ma_b200_forward", "ma_b200_forward_timed",
    "ma_b200_device_status", "ma_b200_status_string", "ma_b200_last_error", "ma_b200_abi_version",
    "ma_b200_forward_static_scratch", "ma_b200_static_scratch_bytes", "ma_b200_static_scratch_last_error",
    "ma_b200_host_scratch_bytes", "ma_b200_forward_host", "ma_b200_forward_host_streamed", "ma_b200_host_last_error",
    "ma_b200_poll_device_status", "ma_b200_selftest_wait_expiry", "ma_b200_selftest_generic_general_form",
)


class Tensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_e", C.c_int64), ("stride_h", C.c_int64), ("stride_n", C.c_int64)]


class Problem(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32),
        ("E", C.c_int32), ("H", C.c_int32), ("N", C.c_int32), ("D", C.c_int32), ("Dv", C.c_int32),
        ("block_size", C.c_int32), ("num_steps", C.c_int32), ("pre_pad", C.c_int32),
        ("qk_dtype", C.c_int32), ("v_dtype", C.c_int32), ("kernel", C.c_int32),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("out", Tensor4),
        ("mask", C.c_void_p), ("mask_stride_e", C.c_int64),
    ]


class WorkspaceLayout(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("status", "counters", "ar", "cr", "al", "cl", "y", "total")] + \
               [("M", C.c_int32), ("kernel", C.c_int32)]


_lib = None


def load() -> C.CDLL:
    """Load the shared library (once).  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} not found: build it with `python -m monarch_attention_b200.build` "
            "(needs nvcc with sm_100a support). There is no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    pp = C.POINTER(Problem)
    lib.ma_b200_workspace_bytes.argtypes = [pp]
    lib.ma_b200_workspace_bytes.restype = C.c_size_t
    lib.ma_b200_workspace_layout_of.argtypes = [pp, C.POINTER(WorkspaceLayout)]
    lib.ma_b200_workspace_layout_of.restype = C.c_int
    lib.ma_b200_forward.argtypes = [pp, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.ma_b200_forward.restype = C.c_int
    lib.ma_b200_forward_timed.argtypes = [pp, C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(C.c_float), C.c_int32]
    lib.ma_b200_forward_timed.restype = C.c_int
    lib.ma_b200_device_status.argtypes = [C.c_void_p, C.c_void_p]
    lib.ma_b200_device_status.restype = C.c_int
    lib.ma_b200_poll_device_status.argtypes = [C.c_int]
    lib.ma_b200_poll_device_status.restype = C.c_int
    lib.ma_b200_selftest_wait_expiry.argtypes = [pp, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.ma_b200_selftest_wait_expiry.restype = C.c_int
    lib.ma_b200_selftest_generic_general_form.argtypes = [C.c_int]
    lib.ma_b200_selftest_generic_general_form.restype = None
    lib.ma_b200_status_string.argtypes = [C.c_int]
    lib.ma_b200_status_string.restype = C.c_char_p
    lib.ma_b200_last_error.argtypes = []
    lib.ma_b200_last_error.restype = C.c_char_p
    lib.ma_b200_abi_version.argtypes = []
    lib.ma_b200_abi_version.restype = C.c_int32
    lib.ma_b200_forward_static_scratch.argtypes = [pp, C.c_void_p]
    lib.ma_b200_forward_static_scratch.restype = C.c_int
    lib.ma_b200_static_scratch_bytes.argtypes = []
    lib.ma_b200_static_scratch_bytes.restype = C.c_size_t
    lib.ma_b200_static_scratch_last_error.argtypes = []
    lib.ma_b200_static_scratch_last_error.restype = C.c_char_p
    lib.ma_b200_host_scratch_bytes.argtypes = [pp, C.c_int]
    lib.ma_b200_host_scratch_bytes.restype = C.c_size_t
    lib.ma_b200_forward_host.argtypes = [pp, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.ma_b200_forward_host.restype = C.c_int
    lib.ma_b200_forward_host_streamed.argtypes = [pp, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.ma_b200_forward_host_streamed.restype = C.c_int
    lib.ma_b200_host_last_error.argtypes = []
    lib.ma_b200_host_last_error.restype = C.c_char_p
    if lib.ma_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libmonarch_attention_b200.so was built for a different ABI version; rebuild it")
    _lib = lib
    return lib


def raise_for_status(code: int, detail: str | None = None) -> None:
    """Map a return code to the Python exception the module API documents."""
    if code == OK:
        return
    lib = load()
    text = lib.ma_b200_status_string(code).decode()
    if detail is None:
        detail = lib.ma_b200_last_error().decode()
    msg = f"monarch_attention_b200: {text}: {detail}"
    if code in (INVALID_ARGUMENT, UNSUPPORTED, WORKSPACE_TOO_SMALL):
        raise ValueError(msg)
    raise RuntimeError(msg)
