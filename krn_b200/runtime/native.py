"""ctypes prototypes over `libkrn_b200.so` (declared in include/krn_b200.h) and status → exception mapping.

The reference binds each compiled C program the same way: load through `Libraries`, `getattr` the entry,
set `argtypes` explicitly (src/krn/runtime/cpu.py:168-175). A non-zero status raises `CUDAError` with the
library's own text, as the reference does for a failed driver call (src/krn/runtime/cuda_backend.py:97-105);
refusals of a shape or type raise `TargetError`, whose message has the reference's four parts.
"""

from __future__ import annotations

import ctypes
from functools import cache

from krn_b200.errors import CUDAError, TargetError
from krn_b200.hw.libraries import KERNEL_LIBRARY, Libraries

ABI_VERSION = 2
OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE_TIMEOUT, ERR_DEVICE_INDEX = range(7)
F32, F16, BF16, E4M3, E5M2 = range(5)

_i64, _int, _ptr, _f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_float

PROTOTYPES: dict[str, tuple[type, list[type]]] = {
    "krn_b200_version": (_int, []),
    "krn_b200_last_error": (ctypes.c_size_t, [ctypes.c_char_p, ctypes.c_size_t]),
    "krn_b200_device_status": (_int, [ctypes.POINTER(_int), ctypes.POINTER(_int), ctypes.POINTER(ctypes.c_uint)]),
    "krn_b200_gemm_tn": (_int, [_int, _int, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "krn_b200_gemm_fp8": (_int, [_int, _int, _int, _int, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "krn_b200_copy_2d": (_int, [_ptr, _i64, _ptr, _i64, _i64, _i64, _ptr]),
    "krn_b200_matmul": (_int, [_int, _int, _int, _int, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "krn_b200_gemm_nn": (_int, [_int, _int, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "krn_b200_gemm_tn_gather": (_int, [_int, _int, _ptr, _ptr, ctypes.POINTER(_ptr), _int, _int, _i64, _i64, _i64, _i64,
                                       _i64, _i64, ctypes.POINTER(_ptr), ctypes.c_uint32, _ptr]),
    "krn_b200_gemm_fp8_blockscaled_tn": (
        _int, [_int, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "krn_b200_gemm_mxfp8_tn": (
        _int, [_int, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "krn_b200_gemm_mxfp4_tn": (
        _int, [_int, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "krn_b200_gemm_nvfp4_tn": (
        _int, [_int, _ptr, _ptr, _ptr, _ptr, _f32, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _ptr]),
    "krn_b200_gemm_fp8_blockscaled_tn_gather": (
        _int, [_int, _ptr, _ptr, _ptr, _ptr, ctypes.POINTER(_ptr), _int, _int, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
               _i64, ctypes.POINTER(_ptr), ctypes.c_uint32, _ptr]),
    "krn_b200_attn_fwd": (
        _int, [_int, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _int,
               ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64), _ptr]),
    "krn_b200_attn_decode_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64]),
    "krn_b200_attn_decode_fp8_paged": (
        _int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f32,
               _ptr, _i64, _ptr]),
    "krn_b200_attn_decode_fp8_paged_noalloc": (
        _int, [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f32,
               _ptr]),
    "krn_b200_scatter_columns": (_int, [_ptr, _ptr, _i64, _i64, _i64, _i64, _int, _ptr]),
}


@cache
def library() -> ctypes.CDLL:
    """The kernel library with every prototype bound. Raises `LibraryNotFound` if it is not built: there is
    no fallback path."""
    handle = Libraries.load(KERNEL_LIBRARY).handle
    for name, (restype, argtypes) in PROTOTYPES.items():
        entry = getattr(handle, name)
        entry.restype, entry.argtypes = restype, argtypes
    version = handle.krn_b200_version()
    if version != ABI_VERSION:
        raise CUDAError(f"KRN_B200_ABI: kernel library has ABI {version}, this host expects {ABI_VERSION}")
    return handle


def last_error() -> str:
    buffer = ctypes.create_string_buffer(512)
    library().krn_b200_last_error(buffer, 512)
    return buffer.value.decode(errors="replace")


def check(status: int, feature: str) -> None:
    """Raise for a non-zero status of an entry point."""
    if status == OK:
        return
    message = last_error()
    if status == ERR_UNSUPPORTED:
        reason, _, instead = message.partition(" Instead: ")
        raise TargetError(feature, "sm_100a", reason.rstrip(". "), instead.rstrip(". ") or "use a supported shape and type")
    name = {ERR_INVALID_ARGUMENT: "KRN_B200_ERR_INVALID_ARGUMENT", ERR_CUDA: "KRN_B200_ERR_CUDA",
            ERR_WORKSPACE: "KRN_B200_ERR_WORKSPACE", ERR_DEVICE_TIMEOUT: "KRN_B200_ERR_DEVICE_TIMEOUT",
            ERR_DEVICE_INDEX: "KRN_B200_ERR_DEVICE_INDEX"}.get(status, str(status))
    raise CUDAError(f"{name}: {message}")


def device_status() -> tuple[int, int, int]:
    """(code, site, block) of the current device's status word; clears it. Call after a synchronisation."""
    code, site, block = _int(0), _int(0), ctypes.c_uint(0)
    check(library().krn_b200_device_status(ctypes.byref(code), ctypes.byref(site), ctypes.byref(block)), "status word")
    return code.value, site.value, block.value


def raise_device_status() -> None:
    code, site, block = device_status()
    if code == ERR_DEVICE_INDEX:
        raise CUDAError(f"KRN_B200_ERR_DEVICE_INDEX: a kernel met an index outside its tensor at site {site} in block "
                        f"{block}; the access was skipped")
    if code != OK:
        name = "KRN_B200_ERR_DEVICE_TIMEOUT" if code == ERR_DEVICE_TIMEOUT else str(code)
        raise CUDAError(f"{name}: a bounded device-side wait expired at site {site} in block {block}")
