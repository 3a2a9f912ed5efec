"""GPU memory management for the GEMM path.

Same function names and meaning as the reference's gradtuity/cuda_mem.py:30-153
(`cuda_malloc`, `cuda_free`, `cuda_memset`, `cuda_memcpy_htod/dtoh/dtod`,
`cuda_device_synchronize`), but routed through libgt_b200.so: allocation comes from a
stream-ordered pool instead of one cudaMalloc/cudaFree per tensor, all work is ordered on
the library's compute stream, and every call checks its status.
"""

from __future__ import annotations

import ctypes
from ctypes import byref, c_void_p

from . import _lib


def cuda_malloc(nbytes: int) -> int:
    ptr = c_void_p()
    _lib.check(_lib.load_library().gt_malloc(_lib.context(), nbytes, byref(ptr)), "gt_malloc")
    return ptr.value


def cuda_free(ptr: int) -> None:
    if ptr and _lib._ctx is not None:
        _lib.load_library().gt_free(_lib._ctx, c_void_p(ptr))


def cuda_memset(ptr: int, value: int, nbytes: int) -> None:
    _lib.check(_lib.load_library().gt_memset(_lib.context(), c_void_p(ptr), value, nbytes), "gt_memset")


def cuda_memcpy_htod(dst_ptr: int, host_data) -> None:
    """Copy host bytes (bytes, bytearray, memoryview or a C-contiguous numpy array) to the GPU."""
    if isinstance(host_data, (bytes, bytearray)):
        n = len(host_data)
        src = (ctypes.c_char * n).from_buffer_copy(host_data) if isinstance(host_data, bytes) else (ctypes.c_char * n).from_buffer(host_data)
        addr = ctypes.addressof(src)
    else:  # numpy array or anything exposing the buffer protocol contiguously
        mv = memoryview(host_data)
        if not mv.c_contiguous:
            raise ValueError("host buffer must be C-contiguous")
        n = mv.nbytes
        src = host_data
        addr = host_data.ctypes.data if hasattr(host_data, "ctypes") else ctypes.addressof(ctypes.c_char.from_buffer(mv))
    _lib.check(_lib.load_library().gt_memcpy_h2d(_lib.context(), c_void_p(dst_ptr), c_void_p(addr), n), "gt_memcpy_h2d")
    del src


def cuda_memcpy_dtoh(src_ptr: int, nbytes: int) -> bytes:
    buf = ctypes.create_string_buffer(nbytes)
    _lib.check(_lib.load_library().gt_memcpy_d2h(_lib.context(), ctypes.cast(buf, c_void_p), c_void_p(src_ptr), nbytes), "gt_memcpy_d2h")
    return buf.raw


def cuda_memcpy_dtoh_into(src_ptr: int, array) -> None:
    """Copy device memory straight into a C-contiguous numpy array."""
    _lib.check(_lib.load_library().gt_memcpy_d2h(_lib.context(), c_void_p(array.ctypes.data), c_void_p(src_ptr), array.nbytes), "gt_memcpy_d2h")


def cuda_memcpy_dtod(dst_ptr: int, src_ptr: int, nbytes: int) -> None:
    _lib.check(_lib.load_library().gt_memcpy_d2d(_lib.context(), c_void_p(dst_ptr), c_void_p(src_ptr), nbytes), "gt_memcpy_d2d")


def cuda_device_synchronize() -> None:
    _lib.check(_lib.load_library().gt_sync(_lib.context()), "gt_sync")
