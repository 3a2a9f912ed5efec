"""Raw-pointer GEMM calls: the Python face of gt_gemm / gt_gemm_batched.

These take device addresses as ints, the way the reference's kernel launches do
(`matmul_kernel[grid](a_ptr, b_ptr, c_ptr, M, N, K, strides...)`, gradtuity/tensor.py:576-593),
but one call covers what there takes a kernel choice, a grid and six strides.
"""

from __future__ import annotations

import os
from ctypes import c_void_p

from . import _lib
from ._lib import (EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RELU, EPI_CAUSAL, EPI_NONE, LAYOUT_NN, LAYOUT_NT,
                   LAYOUT_TN, PREC_FP32, PREC_TF32, PREC_TF32X3)

_PRECISIONS = {"tf32": PREC_TF32, "3xtf32": PREC_TF32X3, "fp32": PREC_FP32}


def default_precision() -> int:
    """Precision selected by GRADTUITY_GEMM_PRECISION (tf32 | 3xtf32 | fp32); tf32 by default."""
    name = os.environ.get("GRADTUITY_GEMM_PRECISION", "tf32").lower()
    if name not in _PRECISIONS:
        raise ValueError(f"GRADTUITY_GEMM_PRECISION must be one of {sorted(_PRECISIONS)}, got {name!r}")
    return _PRECISIONS[name]


def _p(x):
    return c_void_p(x) if x else None


def gemm(layout: int, M: int, N: int, K: int, a_ptr: int, lda: int, b_ptr: int, ldb: int,
         c_ptr: int, ldc: int, *, bias_ptr: int = 0, aux_ptr: int = 0, alpha: float = 1.0,
         accumulate: bool = False, epilogue: int = EPI_NONE, precision: int | None = None) -> None:
    lib = _lib.load_library()
    if precision is None:
        precision = default_precision()
    _lib.check(lib.gt_gemm(_lib.context(), layout, M, N, K, _p(a_ptr), lda, _p(b_ptr), ldb, _p(c_ptr), ldc,
                           _p(bias_ptr), _p(aux_ptr), alpha, 1 if accumulate else 0, epilogue, precision, None),
               "gt_gemm")


def gemm_gelu_grad_colsum(layout: int, M: int, N: int, K: int, a_ptr: int, lda: int, b_ptr: int, ldb: int,
                          c_ptr: int, ldc: int, pre_ptr: int, colsum_ptr: int, *, alpha: float = 1.0,
                          precision: int | None = None) -> None:
    """C = alpha * op(A) op(B) * gelu'(pre) and colsum[n] += sum_m C[m, n] in one launch: dX of the second layer
    of a GELU MLP with the bias gradient of the first taken from the output tiles on their way out."""
    lib = _lib.load_library()
    if precision is None:
        precision = default_precision()
    _lib.check(lib.gt_gemm_gelu_grad_colsum(_lib.context(), layout, M, N, K, _p(a_ptr), lda, _p(b_ptr), ldb, _p(c_ptr), ldc,
                                            _p(pre_ptr), _p(colsum_ptr), alpha, precision),
               "gt_gemm_gelu_grad_colsum")


def gemm_batched(layout: int, M: int, N: int, K: int,
                 a_ptr: int, lda: int, sa0: int, sa1: int,
                 b_ptr: int, ldb: int, sb0: int, sb1: int,
                 c_ptr: int, ldc: int, sc0: int, sc1: int,
                 batch0: int, batch1: int = 1, *, bias_ptr: int = 0, aux_ptr: int = 0, alpha: float = 1.0,
                 accumulate: bool = False, epilogue: int = EPI_NONE, precision: int | None = None, flags: int = 0) -> None:
    lib = _lib.load_library()
    if precision is None:
        precision = default_precision()
    _lib.check(lib.gt_gemm_batched_ex(_lib.context(), layout, M, N, K, _p(a_ptr), lda, sa0, sa1, _p(b_ptr), ldb, sb0, sb1,
                                      _p(c_ptr), ldc, sc0, sc1, batch0, batch1, _p(bias_ptr), _p(aux_ptr), alpha,
                                      1 if accumulate else 0, epilogue, precision, flags, None),
               "gt_gemm_batched_ex")


def gemm_3xtf32_noalloc(layout: int, M: int, N: int, K: int, a_ptr: int, lda: int, b_ptr: int, ldb: int,
                        c_ptr: int, ldc: int, *, bias_ptr: int = 0, alpha: float = 1.0,
                        accumulate: bool = False, epilogue: int = EPI_NONE) -> None:
    """3xTF32 GEMM that never allocates device memory: for callers that have handed the whole
    GPU to their own memory pool or cannot afford an allocation's synchronisation mid-step.
    The operand split uses a fixed 32 MiB array inside the library, so A and B together are
    limited (about 4 Mi elements); beyond that the call raises with "exceeds the fixed maximum".
    Calls share that array: do not let two of them overlap on the GPU."""
    lib = _lib.load_library()
    _lib.check(lib.gt_gemm_3xtf32_noalloc(_lib.context(), layout, M, N, K, _p(a_ptr), lda, _p(b_ptr), ldb, _p(c_ptr), ldc,
                                          _p(bias_ptr), alpha, 1 if accumulate else 0, epilogue, None),
               "gt_gemm_3xtf32_noalloc")


def matmul_host(a, b, out=None, *, layout: int = LAYOUT_NN, bias=None, alpha: float = 1.0, epilogue: int = EPI_NONE,
                precision: int | None = None, chunks: int = 8):
    """op(a) @ op(b) for numpy float32 arrays in HOST memory, result in `out` (host): the copies over PCIe are
    overlapped with the product block by block (`gt_gemm_host`).  a, b are the stored-layout 2-D arrays of the
    layout (NN: (M, K), (K, N); NT: (M, K), (N, K); TN: (K, M), (K, N)).  Pinned arrays make the overlap real;
    pageable ones work, with serialised copies."""
    import numpy as np

    for name, arr in (("a", a), ("b", b)):
        if arr.dtype != np.float32 or arr.ndim != 2 or arr.strides[1] != 4:
            raise ValueError(f"matmul_host: {name} must be a 2-D float32 array with contiguous rows")
    M = a.shape[1] if layout == LAYOUT_TN else a.shape[0]
    K = a.shape[0] if layout == LAYOUT_TN else a.shape[1]
    N = b.shape[0] if layout == LAYOUT_NT else b.shape[1]
    kb = b.shape[1] if layout == LAYOUT_NT else b.shape[0]
    if kb != K:
        raise ValueError(f"matmul_host shape mismatch: inner dimensions {K} vs {kb}")
    if out is None:
        out = np.empty((M, N), dtype=np.float32)
    elif out.dtype != np.float32 or out.shape != (M, N) or out.strides[1] != 4:
        raise ValueError("matmul_host: out must be a float32 (M, N) array with contiguous rows")
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        if bias.shape != (N,):
            raise ValueError(f"matmul_host: bias must have shape ({N},)")
    if precision is None:
        precision = default_precision()
    lib = _lib.load_library()
    _lib.check(lib.gt_gemm_host(_lib.context(), layout, M, N, K, c_void_p(a.ctypes.data), a.strides[0] // 4,
                                c_void_p(b.ctypes.data), b.strides[0] // 4, c_void_p(out.ctypes.data), out.strides[0] // 4,
                                c_void_p(bias.ctypes.data) if bias is not None else None, alpha, epilogue, precision, chunks),
               "gt_gemm_host")
    return out
