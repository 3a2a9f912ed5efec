"""ctypes binding of libgt_b200.so, the C-ABI library that holds the sm_100a GEMM kernels.

The library is loaded the way the reference loads libcudart / libcuda / libnccl
(gradtuity/cuda_mem.py:13-22, gradtuity/dist/nccl.py:27-37): `ctypes.CDLL` on a path taken
from an environment variable, here ``GRADTUITY_GEMM_LIBRARY``; when the variable is unset the
copy built next to this file is used.  Every symbol gets explicit ``argtypes``/``restype``
(as gradtuity/dist/nccl.py:67-68,83-89 does) and every non-zero status becomes a
``RuntimeError`` carrying the decoded text (gradtuity/cuda_driver.py:98-104).

There is no fallback: a missing library or a missing GPU raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIBRARY = os.path.join(_HERE, "libgt_b200.so")

# enums of include/gt_b200.h
LAYOUT_NN, LAYOUT_NT, LAYOUT_TN = 0, 1, 2
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_BIAS_GELU, EPI_CAUSAL, EPI_BIAS_ADD, EPI_GELU_GRAD = 0, 1, 2, 3, 4, 5, 6
PREC_TF32, PREC_TF32X3, PREC_FP32 = 0, 1, 2
CAUSAL_MASK_VALUE = -1.0e9
GEMM_A_LOWER, GEMM_AT_LOWER, GEMM_CAUSAL_SKIP_MASKED, GEMM_BIAS_PER_BATCH = 1, 2, 4, 8

GT_OK = 0
GT_ERR_INVALID_ARG = -1
GT_ERR_CUDA = -2
GT_ERR_UNSUPPORTED = -3
GT_ERR_TIMEOUT = -4
GT_ERR_NOMEM = -5
GT_ERR_NCCL = -6
GT_ERR_TOO_LARGE = -7
GT_ERR_NOT_INIT = -8

_F = POINTER(c_float)

# name -> (restype, argtypes); mirrors include/gt_b200.h declaration by declaration
SIGNATURES = {
    "gt_init": (c_int, [c_int, POINTER(c_void_p)]),
    "gt_destroy": (c_int, [c_void_p]),
    "gt_strerror": (c_char_p, [c_int]),
    "gt_last_error": (c_char_p, [c_void_p]),
    "gt_ctx_stream": (c_void_p, [c_void_p]),
    "gt_sm_count": (c_int, [c_void_p]),
    "gt_device_status": (c_int, [c_void_p, POINTER(c_int)]),
    "gt_malloc": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "gt_free": (c_int, [c_void_p, c_void_p]),
    "gt_memset": (c_int, [c_void_p, c_void_p, c_int, c_size_t]),
    "gt_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "gt_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "gt_memcpy_d2d": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "gt_sync": (c_int, [c_void_p]),
    "gt_host_alloc": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "gt_host_free": (c_int, [c_void_p, c_void_p]),
    "gt_memcpy_h2d_async": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "gt_memcpy_d2h_async": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "gt_event_create": (c_int, [c_void_p, POINTER(c_void_p)]),
    "gt_event_destroy": (c_int, [c_void_p, c_void_p]),
    "gt_event_record": (c_int, [c_void_p, c_void_p]),
    "gt_event_elapsed_ms": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(c_float)]),
    "gt_gemm": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64,
                        c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                        c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p]),
    "gt_gemm_gelu_grad_colsum": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64,
                                         c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                         c_void_p, c_void_p, c_float, c_int]),
    "gt_gemm_batched": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64,
                                c_void_p, c_int64, c_int64, c_int64,
                                c_void_p, c_int64, c_int64, c_int64,
                                c_void_p, c_int64, c_int64, c_int64,
                                c_int64, c_int64,
                                c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p]),
    "gt_gemm_batched_ex": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64,
                                   c_void_p, c_int64, c_int64, c_int64,
                                   c_void_p, c_int64, c_int64, c_int64,
                                   c_void_p, c_int64, c_int64, c_int64,
                                   c_int64, c_int64,
                                   c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p]),
    "gt_gemm_3xtf32_noalloc": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64,
                                       c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                       c_void_p, c_float, c_int, c_int, c_void_p]),
    "gt_gemm_path": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64,
                             c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                             c_int, POINTER(c_int)]),
    "gt_selftest_bounded_wait": (c_int, [c_void_p, c_int64]),
    "gt_gemm_host": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                             c_void_p, c_float, c_int, c_int, c_int]),
    "gt_attention_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int64, c_int64, c_int64, c_int64, c_float, c_void_p]),
    "gt_attention_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int, c_int,
                                      c_void_p]),
    "gt_attention_backward_bias": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int,
                                           c_int, c_void_p]),
    "gt_launch_count": (c_int, [c_void_p, POINTER(c_int64)]),
    "gt_fill": (c_int, [c_void_p, c_void_p, c_float, c_int64]),
    "gt_add": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "gt_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "gt_scale": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int]),
    "gt_relu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64]),
    "gt_relu_mask_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "gt_gelu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64]),
    "gt_gelu_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "gt_add_scalar": (c_int, [c_void_p, c_void_p, c_void_p, c_int64]),
    "gt_add_bias": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64]),
    "gt_sum_all": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "gt_colsum_acc": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "gt_colsum_acc_beside": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "gt_colsum_acc_batched_beside": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64]),
    "gt_join_beside": (c_int, [c_void_p]),
    "gt_beside_begin": (c_int, [c_void_p]),
    "gt_beside_end": (c_int, [c_void_p]),
    "gt_beside_touches": (c_int, [c_void_p, c_void_p, c_size_t]),
    "gt_repack_rows": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64]),
    "gt_maxpool2d": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p] + [c_int64] * 8),
    "gt_maxpool2d_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "gt_im2col": (c_int, [c_void_p, c_void_p, c_int64, c_void_p] + [c_int64] * 8),
    "gt_col2im": (c_int, [c_void_p, c_void_p, c_void_p, c_int64] + [c_int64] * 8 + [c_int]),
    "gt_softmax": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int]),
    "gt_softmax_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_float]),
    "gt_layernorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float]),
    "gt_layernorm_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int64, c_int64, c_int]),
    "gt_layernorm_backward_colsum": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int64, c_int64, c_int]),
    "gt_embedding": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "gt_embedding_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "gt_embedding_backward_scaled": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float]),
    "gt_cross_entropy": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int]),
    "gt_cross_entropy_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                       c_int64, c_int64, c_int, c_float]),
    "gt_cross_entropy_backward": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_float,
                                          c_int64, c_int64, c_int]),
    "gt_adamw": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_float, c_float, c_float,
                         c_float, c_float, c_float, c_void_p]),
    "gt_sumsq": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int]),
    "gt_clip_scale": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float]),
    "gt_scale_by_device_scalar": (c_int, [c_void_p, c_void_p, c_void_p, c_int64]),
    "gt_dist_get_unique_id": (c_int, [c_void_p, c_char_p]),
    "gt_dist_init": (c_int, [c_void_p, c_int, c_int, c_char_p]),
    "gt_dist_destroy": (c_int, [c_void_p]),
    "gt_dist_allreduce": (c_int, [c_void_p, c_void_p, c_int64, c_int]),
    "gt_dist_broadcast": (c_int, [c_void_p, c_void_p, c_int64, c_int]),
    "gt_dist_allgather": (c_int, [c_void_p, c_void_p, c_void_p, c_int64]),
    "gt_dist_wait": (c_int, [c_void_p, c_int]),
    "gt_dist_info": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int)]),
    "gt_dist_timeline": (c_int, [c_void_p, POINTER(c_float), c_int, POINTER(c_int)]),
    "gt_adamw_multi": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_float, c_float, c_float, c_float,
                               c_float, c_float, c_void_p]),
    "gt_sumsq_multi": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64]),
    "gt_transpose12": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int]),
}

_lib = None
_ctx = None
_ctx_device = None


def library_path() -> str:
    return os.environ.get("GRADTUITY_GEMM_LIBRARY") or DEFAULT_LIBRARY


def load_library() -> ctypes.CDLL:
    """Load libgt_b200.so and type every exported function. Raises if the file is missing."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"libgt_b200.so not found at {path!r}. Build it with "
            "`make -C gradtuity_b200/csrc` (or `python -c 'import __graft_entry__ as g; g.build()'`) "
            "or point GRADTUITY_GEMM_LIBRARY at it. There is no CPU fallback."
        )
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    """Raise RuntimeError for a non-zero status, with the library's own description."""
    if status == GT_OK:
        return
    lib = load_library()
    text = lib.gt_strerror(status).decode()
    detail = ""
    if _ctx is not None:
        d = lib.gt_last_error(_ctx)
        if d:
            detail = ": " + d.decode()
    raise RuntimeError(f"{what} failed with status {status} ({text}){detail}")


def context() -> c_void_p:
    """The process-wide library context, bound to device LOCAL_RANK (default 0)."""
    global _ctx, _ctx_device
    if _ctx is not None:
        return _ctx
    lib = load_library()
    device = int(os.environ.get("GRADTUITY_DEVICE", os.environ.get("LOCAL_RANK", "0")))
    handle = c_void_p()
    status = lib.gt_init(device, byref(handle))
    if status != GT_OK:
        raise RuntimeError(
            f"gt_init(device={device}) failed with status {status} "
            f"({lib.gt_strerror(status).decode()}); a B200 (sm_100) GPU is required"
        )
    _ctx = handle
    _ctx_device = device
    return _ctx


def device_status() -> int:
    """Synchronise and return (then clear) the device status word; raises on GT_ERR_TIMEOUT."""
    lib = load_library()
    st = c_int(0)
    check(lib.gt_device_status(context(), byref(st)), "gt_device_status")
    if st.value != 0:
        raise RuntimeError(f"device status {st.value} ({lib.gt_strerror(st.value).decode()})")
    return st.value


def launch_count() -> int:
    lib = load_library()
    n = c_int64(0)
    check(lib.gt_launch_count(context(), byref(n)), "gt_launch_count")
    return n.value
