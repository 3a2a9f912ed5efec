"""Tensor factories and parameter helpers with the reference's names and meaning
(gradtuity/functional.py:18-257): zeros, ones, full, randn, zero_grad.

`randn` draws with numpy's Generator instead of one `random.gauss` call per element (the
reference spends minutes there for a 124 M-parameter model, gradtuity/functional.py:110); the
distribution and the signature are the same, the stream of values is not.
"""
from __future__ import annotations

from ctypes import c_void_p

import numpy as np

from . import _lib
from .cuda_mem import cuda_memset
from .tensor import Tensor, empty_tensor

_rng = np.random.default_rng()


def zeros(shape, requires_grad: bool = False) -> Tensor:
    return Tensor._zeros(tuple(shape), requires_grad=requires_grad)


def zeros_like(t: Tensor, requires_grad: bool = False) -> Tensor:
    return Tensor._zeros_like(t, requires_grad=requires_grad)


def ones(shape, requires_grad: bool = False) -> Tensor:
    return Tensor._ones(tuple(shape), requires_grad=requires_grad)


def ones_like(t: Tensor, requires_grad: bool = False) -> Tensor:
    return Tensor._ones_like(t, requires_grad=requires_grad)


def full(shape, fill_value: float, requires_grad: bool = False) -> Tensor:
    t = empty_tensor(tuple(shape), requires_grad=requires_grad)
    _lib.check(_lib.load_library().gt_fill(_lib.context(), c_void_p(t.ptr), float(fill_value), t.numel), "gt_fill")
    return t


def full_like(t: Tensor, fill_value: float, requires_grad: bool = False) -> Tensor:
    return full(t.shape, fill_value, requires_grad=requires_grad)


def randn(shape, requires_grad: bool = False, seed: int | None = None, std: float = 1.0) -> Tensor:
    global _rng
    if len(shape) not in (1, 2, 3, 4):
        raise ValueError(f"Only rank 1, 2, 3, or 4 tensors supported, got rank {len(shape)}")
    if seed is not None:
        _rng = np.random.default_rng(seed)
    a = _rng.standard_normal(tuple(shape), dtype=np.float32)
    if std != 1.0:
        a *= np.float32(std)
    return Tensor.from_numpy(a, requires_grad=requires_grad)


def zero_grad(params: list[Tensor]) -> None:
    """Zero every parameter's gradient, allocating it if absent (gradtuity/functional.py:206-229)."""
    # Parameters that sit side by side in memory (the packed q / k / v weights of CausalSelfAttention) get
    # their fresh gradients side by side too, so that a batched backward can address them as one batch.
    i, n = 0, len(params)
    while i < n:
        p = params[i]
        if not p.requires_grad:
            i += 1
            continue
        if p.grad is not None:
            cuda_memset(p.grad.ptr, 0, p.grad.nbytes)
            i += 1
            continue
        j = i + 1
        while (j < n and params[j].requires_grad and params[j].grad is None
               and params[j].ptr == params[j - 1].ptr + params[j - 1].numel * 4):
            j += 1
        if j - i == 1:
            p.grad = zeros(p.shape)
        else:
            from .tensor import Storage, alloc_storage
            total = sum(q.numel for q in params[i:j]) * 4
            block = alloc_storage(total, zero=True)
            off = 0
            for q in params[i:j]:
                q.grad = Tensor._from_ptr(block.ptr + off, q.shape, owns_memory=False, base=block)
                off += q.numel * 4
        i = j
