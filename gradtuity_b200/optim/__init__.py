"""Optimizers for the training step: `AdamW`, `SGD`, `clip_grad_norm_` with the reference's
signatures and update rules (gradtuity/optim/__init__.py:99-159, gradtuity/optim/utils.py:15-52).

The update arithmetic is the reference's `adamw_step_kernel` (gradtuity/kernels_cuda/optim_kernels.py:23-46).
`clip_grad_norm_` keeps the norm and the clip factor on the device: one reduction chain instead of a
multiply, a sum and a device-to-host `.item()` per parameter; the returned norm costs one read.
"""
from __future__ import annotations

import math
import os
from ctypes import c_void_p

from .. import _lib
from .. import tensor as _tensor
from ..tensor import Tensor, empty_tensor


def _call(name, *args):
    _lib.check(getattr(_lib.load_library(), name)(_lib.context(), *args), name)


class _TensorTable:
    """Device-side list {p, g, m, v, n} of a parameter set plus the block -> (tensor, offset) map
    that the multi-tensor kernels read.  Rebuilt only when one of the pointers changes."""

    CHUNK_MIN = 65536

    def __init__(self) -> None:
        self.key = None
        self.tensors_ptr = 0
        self.chunks_ptr = 0
        self.n_chunks = 0
        self.chunk_elems = 0

    def update(self, entries: list[tuple[int, int, int, int, int]], max_chunks: int | None = None) -> None:
        key = tuple(entries)
        if key == self.key:
            return
        import numpy as np

        from ..cuda_mem import cuda_free, cuda_malloc, cuda_memcpy_htod

        total = sum(e[4] for e in entries)
        chunk = self.CHUNK_MIN
        if max_chunks is not None:
            while sum((e[4] + chunk - 1) // chunk for e in entries) > max_chunks:
                chunk *= 2
        tens = np.zeros((len(entries), 5), dtype=np.int64)
        for i, e in enumerate(entries):
            tens[i] = e
        rows = []
        for i, e in enumerate(entries):
            for start in range(0, e[4], chunk):
                rows.append((i, start))
        ch = np.zeros(len(rows), dtype=np.dtype([("tensor", "<i4"), ("pad", "<i4"), ("start", "<i8")]))
        ch["tensor"] = [r[0] for r in rows]
        ch["start"] = [r[1] for r in rows]
        for old in (self.tensors_ptr, self.chunks_ptr):
            if old:
                cuda_free(old)
        self.tensors_ptr = cuda_malloc(tens.nbytes)
        self.chunks_ptr = cuda_malloc(ch.nbytes)
        cuda_memcpy_htod(self.tensors_ptr, tens)
        cuda_memcpy_htod(self.chunks_ptr, ch)
        self.n_chunks, self.chunk_elems, self.key = len(rows), chunk, key
        _ = total


class Optimizer:
    def __init__(self, params: list[Tensor]) -> None:
        self.params = list(params)

    def zero_grad(self) -> None:
        from ..functional import zero_grad

        zero_grad(self.params)

    def step(self) -> None:
        raise NotImplementedError


class SGD(Optimizer):
    def __init__(self, params: list[Tensor], lr: float = 1e-2) -> None:
        super().__init__(params)
        self.lr = lr

    def step(self) -> None:
        for p in self.params:
            if p.grad is None:
                continue
            _call("gt_scale", c_void_p(p.ptr), c_void_p(p.grad.ptr), -float(self.lr), p.numel, 1)


class AdamW(Optimizer):
    """Decoupled weight decay Adam; state m, v on the GPU, step count on the host."""

    BESIDE_MIN_ELEMS = 16 << 20          # below 64 MB of parameters the update is not worth splitting over two streams
    _next_join_id = 0

    def __init__(self, params: list[Tensor], lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01) -> None:
        super().__init__(params)
        self.lr = lr
        self.beta1, self.beta2 = betas[0], betas[1]
        self.eps = eps
        self.weight_decay = weight_decay
        n = len(self.params)
        self.m: list[Tensor | None] = [None] * n
        self.v: list[Tensor | None] = [None] * n
        self.step_count = 0
        self._table = _TensorTable()
        self._table_late = _TensorTable()
        self._keep = None                # what the part of the last step that runs on the side stream still reads

    def _validate_hyperparams(self) -> None:
        if self.lr <= 0:
            raise ValueError(f"lr must be > 0, got {self.lr}")
        if not (0 <= self.beta1 < 1):
            raise ValueError(f"beta1 must be in [0, 1), got {self.beta1}")
        if not (0 <= self.beta2 < 1):
            raise ValueError(f"beta2 must be in [0, 1), got {self.beta2}")
        if self.eps <= 0:
            raise ValueError(f"eps must be > 0, got {self.eps}")
        if self.weight_decay < 0:
            raise ValueError(f"weight_decay must be >= 0, got {self.weight_decay}")

    def step(self, grad_scale: Tensor | None = None) -> None:
        """One update.  grad_scale: optional (1,) device tensor multiplied into every gradient
        inside the update kernel (the clip factor of `clip_grad_norm_(..., defer=True)`)."""
        self._validate_hyperparams()
        self.step_count += 1
        t = self.step_count
        bc1 = 1.0 / (1.0 - self.beta1 ** t)
        bc2 = 1.0 / (1.0 - self.beta2 ** t)
        gs = c_void_p(grad_scale.ptr) if grad_scale is not None else None
        entries = []
        for i, p in enumerate(self.params):
            if p.grad is None:
                continue
            if p.grad.shape != p.shape:
                raise ValueError(f"param[{i}] grad shape {p.grad.shape} does not match param shape {p.shape}")
            if self.m[i] is None:
                self.m[i] = Tensor._zeros_like(p)
                self.v[i] = Tensor._zeros_like(p)
            entries.append((p.ptr, p.grad.ptr, self.m[i].ptr, self.v[i].ptr, p.numel))
        if not entries:
            return
        hyper = (float(self.lr), float(self.beta1), float(self.beta2), float(self.eps), float(self.weight_decay), float(bc1), float(bc2), gs)

        def launch(table: _TensorTable) -> None:       # one launch for a whole list (the reference launches once per tensor)
            _call("gt_adamw_multi", c_void_p(table.tensors_ptr), c_void_p(table.chunks_ptr), table.n_chunks, table.chunk_elems, *hyper)

        # A large model's update is 0.6 ms of pure memory traffic.  The parameters the next forward pass needs first (the
        # first ones of the list, up to a little over half of the bytes) are updated on the compute stream; the rest goes
        # to the side stream, where it runs beside the compute-bound first layers of that forward pass, and the first
        # access to one of those parameters (`Tensor.ptr`) joins the two streams.
        total = sum(e[4] for e in entries)
        late_from = len(entries)
        if total >= self.BESIDE_MIN_ELEMS and os.environ.get("GRADTUITY_ADAMW_BESIDE", "1") != "0":
            seen = 0
            for k, e in enumerate(entries):
                seen += e[4]
                if seen >= 0.55 * total:
                    late_from = k + 1
                    break
        if late_from >= len(entries):
            self._table.update(entries)
            launch(self._table)
            return
        self._table.update(entries[:late_from])
        self._table_late.update(entries[late_from:])
        launch(self._table)
        _call("gt_beside_begin")
        try:
            launch(self._table_late)
        finally:
            _call("gt_beside_end")
        self._keep = grad_scale                  # read by the kernel on the side stream: must outlive it
        join_id = _tensor._pending_join[0] = AdamW._next_join_id = AdamW._next_join_id + 1
        late_ptrs = {e[0] for e in entries[late_from:]}
        for p in self.params:
            if p.grad is not None and p._st.ptr in late_ptrs:
                p._join_id = join_id


_clip_table = _TensorTable()


def clip_grad_norm_(params, max_norm: float, eps: float = 1e-6, defer: bool = False):
    """Scale all gradients so that their global L2 norm is at most max_norm
    (gradtuity/optim/utils.py:15-52).  Returns the pre-clip norm as a float.

    defer=True skips the in-place scaling and the host read and returns `(norm_tensor,
    scale_tensor)` device tensors instead, for `AdamW.step(grad_scale=scale_tensor)`."""
    params = [p for p in params if p.grad is not None]
    if not params:
        return 0.0 if not defer else (None, None)
    sumsq = empty_tensor((1,))
    _clip_table.update([(0, p.grad.ptr, 0, 0, p.grad.numel) for p in params], max_chunks=4096)
    _call("gt_sumsq_multi", c_void_p(sumsq.ptr), c_void_p(_clip_table.tensors_ptr), c_void_p(_clip_table.chunks_ptr),
          _clip_table.n_chunks, _clip_table.chunk_elems)
    scale = empty_tensor((1,))
    norm = empty_tensor((1,))
    _call("gt_clip_scale", c_void_p(scale.ptr), c_void_p(norm.ptr), c_void_p(sumsq.ptr), float(max_norm), float(eps))
    if defer:
        return norm, scale
    for p in params:
        _call("gt_scale_by_device_scalar", c_void_p(p.grad.ptr), c_void_p(scale.ptr), p.grad.numel)
    return norm.item()


__all__ = ["Optimizer", "SGD", "AdamW", "clip_grad_norm_"]
