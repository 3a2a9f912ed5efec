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


GRAD_ALIGN = 256          # bytes; every gradient inside a block of gradients starts on this boundary


def zero_grad(params: list[Tensor]) -> None:
    """Zero every parameter's gradient, allocating it if absent (gradtuity/functional.py:206-229).

    Gradients that do not exist yet are carved out of ONE zero-filled block, in the order of `params` (so the
    gradients of parameters that sit side by side in memory, the packed q / k / v weights of CausalSelfAttention,
    sit side by side too and a batched backward can address them as one batch).  Existing gradients that are
    neighbours inside such a block (or inside the data-parallel gradient arena) are cleared by one memset per run of
    neighbours instead of one per parameter: one memset for a whole model after the first step."""
    from .tensor import Storage, alloc_storage, join_side_stream

    join_side_stream()          # an optimizer step still running on the side stream reads the gradients
    fresh = [p for p in params if p.requires_grad and p.grad is None]
    if fresh:
        offsets, total = [], 0
        for p in fresh:
            offsets.append(total)
            total += -(-p.numel * 4 // GRAD_ALIGN) * GRAD_ALIGN
        block = alloc_storage(total, zero=True)
        block.grads_only = True
        for p, off in zip(fresh, offsets):
            p.grad = Tensor._from_ptr(block.ptr + off, p.shape, owns_memory=False, base=block)
        fresh_ids = {id(p) for p in fresh}
    else:
        fresh_ids = set()
    runs: dict[int, list[tuple[int, int]]] = {}
    for p in params:
        if not p.requires_grad or id(p) in fresh_ids:
            continue
        base = p.grad._st.base
        if base is not None and getattr(base, "grads_only", False):
            runs.setdefault(id(base), []).append((p.grad._st.ptr, p.grad.nbytes))
        else:
            cuda_memset(p.grad.ptr, 0, p.grad.nbytes)
    for spans in runs.values():
        spans.sort()
        start, end = spans[0][0], spans[0][0] + spans[0][1]
        for ptr, nbytes in spans[1:]:
            # a gap shorter than the alignment in front of an aligned start is padding: nothing else can live there
            if ptr - end < GRAD_ALIGN and (ptr % GRAD_ALIGN == 0 or ptr == end) and ptr >= end:
                end = ptr + nbytes
            else:
                cuda_memset(start, 0, end - start)
                start, end = ptr, ptr + nbytes
        cuda_memset(start, 0, end - start)
