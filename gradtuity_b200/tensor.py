"""Tensor with GPU storage and autograd: the host-side mirror of gradtuity/tensor.py for the
GEMM path.

Public surface and behaviour follow the reference (`Tensor(data, shape=None, requires_grad=False,
name="")`, `.shape/.ptr/.numel/.nbytes/.ndim`, `.backward()`, `.grad`, `.view`, `.detach`,
`.to_list`, `.item`, and the op methods `matmul`, `bmm`, `linear`, `linear_tied`, `linear_relu`,
`add`, `relu`, `gelu`, `sum`, `add_bias`, `mul`, `scale` …; gradtuity/tensor.py:164-2734): CUDA
only, float32 only, contiguous row-major only, rank 1-4, same `ValueError` texts for shape
mistakes, gradients accumulated into `.grad` buffers that are created zeroed on first use.

What differs is below the method signatures.  Every GEMM is one call into libgt_b200.so
(`gt_gemm` / `gt_gemm_batched`, tcgen05 + TMA on sm_100a) instead of a `kernel[grid](...)`
launch of a 32x32x32 Triton/NVRTC kernel; NT and TN operands are read in place; `bmm` is a
single strided-batched launch instead of a Python loop over slices; bias, ReLU and GELU are
fused into the producing GEMM's epilogue; memory comes from a stream-ordered pool.  There is
no Triton, no backend switch and no CPU path.
"""

from __future__ import annotations

import math
import os
import struct
from contextlib import contextmanager
from ctypes import c_void_p
from typing import Callable, Optional

from . import _lib
from . import gemm as _gemm
from ._lib import (EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RELU, EPI_NONE, LAYOUT_NN, LAYOUT_NT, LAYOUT_TN)
from .cuda_mem import (cuda_device_synchronize, cuda_free, cuda_malloc, cuda_memcpy_dtod, cuda_memcpy_dtoh,
                       cuda_memcpy_dtoh_into, cuda_memcpy_htod, cuda_memset)

F32 = 4

# Object told about the progress of backward(): begin(topo), node_done(parents), end().
# The data-parallel gradient exchange installs one to send finished gradient buckets while the
# rest of backward still runs (gradtuity_b200/dist/ddp.py).
_backward_observer = None


def set_backward_observer(observer) -> None:
    global _backward_observer
    _backward_observer = observer


def _call(name: str, *args) -> None:
    lib = _lib.load_library()
    _lib.check(getattr(lib, name)(_lib.context(), *args), name)


# The id of the side-stream work that has not been joined yet (0: none), in a list so that other modules can set it.
_pending_join = [0]


def join_side_stream() -> None:
    """Order the compute stream behind whatever runs on the library's side stream (no-op when nothing does)."""
    _pending_join[0] = 0
    _call("gt_join_beside")


def _vp(ptr: int):
    return c_void_p(ptr) if ptr else None


class Storage:
    """GPU memory buffer: ptr, nbytes, and ownership (gradtuity/tensor.py:87-101)."""

    __slots__ = ("ptr", "nbytes", "owns", "base", "grads_only")

    def __init__(self, ptr: int, nbytes: int, owns: bool = True, base: "Storage | None" = None) -> None:
        self.ptr = ptr
        self.nbytes = nbytes
        self.owns = owns
        # A non-owning view keeps its owner alive; with a pooled, stream-ordered allocator a
        # freed block can be handed out again at once, so a view must never outlive its owner.
        self.base = base
        # True for a block that holds nothing but parameter gradients, each starting on a 256-byte boundary
        # (functional.zero_grad, the data-parallel arena): neighbours in it may be cleared with one memset.
        self.grads_only = False

    def free(self) -> None:
        if self.owns and self.ptr:
            cuda_free(self.ptr)
            self.ptr = 0

    def __del__(self) -> None:
        try:
            self.free()
        except Exception:
            pass


def _validate_shape(shape: tuple[int, ...]) -> None:
    if len(shape) not in (1, 2, 3, 4):
        raise ValueError(f"Only rank 1, 2, 3, or 4 tensors supported, got rank {len(shape)}")
    for i, dim in enumerate(shape):
        if dim <= 0:
            raise ValueError(f"Dimension {i} must be positive, got {dim}")


def prod(shape: tuple[int, ...]) -> int:
    return math.prod(shape)


def alloc_storage(nbytes: int, zero: bool = False) -> Storage:
    ptr = cuda_malloc(nbytes)
    if zero:
        cuda_memset(ptr, 0, nbytes)
    return Storage(ptr, nbytes, owns=True)


@contextmanager
def temp_storage(nbytes: int, zero: bool = False):
    st = alloc_storage(nbytes, zero=zero)
    try:
        yield st
    finally:
        st.free()


def empty_tensor(shape: tuple[int, ...], *, requires_grad: bool = False, zero: bool = False, name: str = "") -> "Tensor":
    """Allocate a tensor (optionally zero-filled)."""
    _validate_shape(shape)
    st = alloc_storage(prod(shape) * F32, zero=zero)
    return Tensor._wrap(st, shape, requires_grad=requires_grad, name=name)


class _GradGroup:
    """One buffer for the gradients of several tensors that a single backward wants to read as one batch
    (the q, k, v outputs of `linear_qkv`): member i's gradient is slice i.  The buffer is allocated when the
    first member's gradient is asked for; a slice nobody wrote is zeroed before the group's owner reads it."""

    def __init__(self, members: int, numel_each: int) -> None:
        self.members = members
        self.numel_each = numel_each
        self.storage: Storage | None = None
        self.written = [False] * members
        self.colsum_done = [False] * members        # the kernel that wrote slice i has added its column sums to the bias gradient

    def slice_tensor(self, index: int, shape: tuple[int, ...], zero: bool) -> "Tensor":
        if self.storage is None:
            self.storage = alloc_storage(self.members * self.numel_each * F32)
        ptr = self.storage.ptr + index * self.numel_each * F32
        if zero:
            cuda_memset(ptr, 0, self.numel_each * F32)
        self.written[index] = True
        return Tensor._from_ptr(ptr, shape, owns_memory=False, base=self.storage)


def ensure_grad(t: "Tensor") -> None:
    """Allocate a zero grad tensor if t.grad is None (gradtuity/tensor.py:152-155)."""
    if t.grad is None:
        if t._grad_slot is not None:
            group, index = t._grad_slot
            t.grad = group.slice_tensor(index, t.shape, zero=True)
        else:
            t.grad = empty_tensor(t.shape, zero=True, requires_grad=False)


def accum_grad(t: "Tensor", g: "Tensor") -> None:
    """t.grad += g (gradtuity/tensor.py:158-161)."""
    ensure_grad(t)
    _call("gt_scale", _vp(t.grad.ptr), _vp(g.ptr), 1.0, t.numel, 1)


def pass_grad(t: "Tensor", g: "Tensor") -> None:
    """t.grad (+)= g.  An interior node that has no gradient yet takes over g's buffer instead of
    receiving a copy: g is the finished gradient of the node whose backward is running, nothing
    reads it afterwards, and each backward hands its g to at most one parent this way.  Leaves
    (parameters) always get their own buffer."""
    if t.grad is None and t._backward is not None and g.numel == t.numel and t._grad_slot is None:
        if g._pitch is not None and t.shape[-1] == g.shape[-1]:
            # a padded-row gradient keeps its pitch on the way up (the view between the LM head and the loss)
            t.grad = Tensor._wrap(Storage(g._st.ptr, g._st.nbytes, owns=False, base=g._st), t.shape)
            t.grad._pitch = g._pitch
        else:
            t.grad = Tensor._from_ptr(g.ptr, t.shape, owns_memory=False, base=g._st)
    else:
        accum_grad(t, g)


def empty_padded_tensor(shape: tuple[int, ...], pitch: int) -> "Tensor":
    """A tensor whose rows (last dimension) sit `pitch` floats apart in memory.  Only the ops that
    say so read such a tensor in place (linear_tied, cross_entropy, view with the last dimension
    kept); any other access goes through `.ptr`, which first packs the rows."""
    _validate_shape(shape)
    rows = prod(shape) // shape[-1]
    t = Tensor._wrap(alloc_storage(rows * pitch * F32), shape)
    if pitch != shape[-1]:
        t._pitch = pitch
    return t


def grad_target(t: "Tensor") -> tuple[int, bool]:
    """Where a backward GEMM should put its contribution to t.grad: (pointer, accumulate).
    A gradient that does not exist yet is allocated WITHOUT zero-filling and the GEMM writes it
    (C = ...); an existing one is accumulated into (C += ...), which is the reference's contract
    (gradtuity/tensor.py:152-155 zero-fills and always accumulates)."""
    if t.grad is None:
        if t._grad_slot is not None:
            group, index = t._grad_slot
            t.grad = group.slice_tensor(index, t.shape, zero=False)
        else:
            t.grad = empty_tensor(t.shape, requires_grad=False)
        return t.grad.ptr, False
    return t.grad.ptr, True


class Tensor:
    """A float32, contiguous, row-major tensor on the GPU with autograd support."""

    # Row pitch in floats when the rows of the last dimension are padded in memory (None: packed).
    _pitch = None
    # (group, index) when this tensor's gradient must live in a slice of a shared buffer (see _GradGroup).
    _grad_slot = None
    # The embedding table this tensor was gathered from (set by `embedding`).
    _embedding_of = None
    # The bias of the Linear layer that produced this tensor, when the column sums of this tensor's finished gradient
    # are that bias's gradient (linear_add, mlp_gelu): the op that writes the last contribution may compute them.
    _grad_colsum_bias = None
    # Children of this node whose backward has not run yet (valid during backward()).
    _n_pending = 0
    # On a gradient tensor: its column sums have already been added to the producer's bias gradient.
    _colsum_done = False
    # Non-zero while work on the side stream (the second half of an optimizer step) may still be writing this tensor:
    # the first access to its memory orders the compute stream behind that work (see `ptr`).
    _join_id = 0

    def __init__(self, data, shape: tuple[int, ...] | None = None, requires_grad: bool = False, name: str = "") -> None:
        if shape is None:
            shape, flat = self._infer_shape_and_flatten(data)
        else:
            flat = self._flatten(data)
            expected = 1
            for s in shape:
                expected *= s
            if len(flat) != expected:
                raise ValueError(f"Data has {len(flat)} elements but shape {shape} requires {expected} elements")
        if len(shape) not in (1, 2, 3, 4):
            raise ValueError(f"Only rank 1, 2, 3, or 4 tensors supported, got rank {len(shape)}")
        _validate_shape(tuple(shape))
        self._shape = tuple(shape)
        n = len(flat)
        st = alloc_storage(n * F32)
        cuda_memcpy_htod(st.ptr, struct.pack(f"{n}f", *flat))
        self._st = st
        self.requires_grad = requires_grad
        self.grad = None
        self.name = name
        self._parents = ()
        self._backward = None
        self._ctx = None

    # ---- construction helpers -----------------------------------------------------------

    @classmethod
    def _wrap(cls, st: Storage, shape: tuple[int, ...], requires_grad: bool = False, name: str = "") -> "Tensor":
        _validate_shape(shape)
        t = object.__new__(cls)
        t._st = st
        t._shape = tuple(shape)
        t.requires_grad = requires_grad
        t.grad = None
        t.name = name
        t._parents = ()
        t._backward = None
        t._ctx = None
        return t

    @classmethod
    def _from_ptr(cls, ptr: int, shape: tuple[int, ...], owns_memory: bool = True, requires_grad: bool = False,
                  name: str = "", base: Storage | None = None) -> "Tensor":
        st = Storage(ptr, prod(shape) * F32, owns=owns_memory, base=base)
        return cls._wrap(st, shape, requires_grad=requires_grad, name=name)

    @classmethod
    def from_numpy(cls, array, requires_grad: bool = False, name: str = "") -> "Tensor":
        """Upload a numpy array (converted to contiguous float32) in one host-to-device copy.

        Not in the reference, whose constructor walks nested Python lists
        (gradtuity/tensor.py:192-220); needed to load seeded benchmark inputs of 10^8 elements.
        """
        import numpy as np

        a = np.ascontiguousarray(array, dtype=np.float32)
        t = empty_tensor(tuple(a.shape), requires_grad=requires_grad, name=name)
        cuda_memcpy_htod(t.ptr, a)
        return t

    def numpy(self, out=None):
        """Download into a numpy float32 array of this tensor's shape (a new one, or `out`,
        which may live in pinned host memory)."""
        import numpy as np

        if out is None:
            out = np.empty(self._shape, dtype=np.float32)
        elif out.dtype != np.float32 or out.size != self.numel or not out.flags.c_contiguous:
            raise ValueError("out must be a C-contiguous float32 array with this tensor's number of elements")
        cuda_memcpy_dtoh_into(self.ptr, out)
        return out

    @classmethod
    def _zeros(cls, shape, requires_grad: bool = False) -> "Tensor":
        return empty_tensor(tuple(shape), zero=True, requires_grad=requires_grad)

    @classmethod
    def _zeros_like(cls, t: "Tensor", requires_grad: bool = False) -> "Tensor":
        return empty_tensor(t.shape, zero=True, requires_grad=requires_grad)

    @classmethod
    def _ones(cls, shape, requires_grad: bool = False) -> "Tensor":
        t = empty_tensor(tuple(shape), requires_grad=requires_grad)
        _call("gt_fill", _vp(t.ptr), 1.0, t.numel)
        return t

    @classmethod
    def _ones_like(cls, t: "Tensor", requires_grad: bool = False) -> "Tensor":
        return cls._ones(t.shape, requires_grad=requires_grad)

    # ---- properties ---------------------------------------------------------------------

    def data_ptr(self) -> int:
        return self.ptr

    @property
    def ptr(self) -> int:
        if self._join_id and self._join_id == _pending_join[0]:
            join_side_stream()
        if self._pitch is not None:
            self._pack_rows()
        return self._st.ptr

    def _pack_rows(self) -> None:
        """Replace a padded-row buffer by a packed copy (for every op that expects contiguous data)."""
        cols = self._shape[-1]
        rows = self.numel // cols
        packed = alloc_storage(rows * cols * F32)
        _call("gt_repack_rows", _vp(packed.ptr), cols, _vp(self._st.ptr), self._pitch, rows, cols)
        self._st = packed
        self._pitch = None

    def _rows(self) -> tuple[int, int]:
        """(pointer, row pitch in floats) without packing."""
        if self._join_id and self._join_id == _pending_join[0]:
            join_side_stream()
        return self._st.ptr, (self._pitch if self._pitch is not None else self._shape[-1])

    @property
    def shape(self) -> tuple[int, ...]:
        return self._shape

    @property
    def numel(self) -> int:
        return prod(self._shape)

    @property
    def nbytes(self) -> int:
        return self._st.nbytes

    @property
    def ndim(self) -> int:
        return len(self._shape)

    @property
    def owns_memory(self) -> bool:
        storage = getattr(self, "_st", None)
        if storage is None:
            raise AttributeError("Tensor has no _st (storage)")
        return storage.owns

    # ---- autograd -----------------------------------------------------------------------

    def backward(self) -> None:
        """Back-propagate from this scalar (gradtuity/tensor.py:355-413).

        Same contract as the reference: seeds grad with 1.0, walks the graph in reverse
        topological order, releases interior nodes as it goes.  The order is built with an
        explicit stack, so graph depth is not limited by Python's recursion limit.
        """
        if self.numel != 1:
            raise ValueError(f"backward() only works on scalar tensors (numel=1), got numel={self.numel}")
        if not self.requires_grad:
            raise RuntimeError(
                "backward() called on a tensor that doesn't require grad. Set requires_grad=True on leaf tensors."
            )
        self.grad = Tensor._ones_like(self)
        self.grad._unit_seed = True          # ops that prepared their gradient for an upstream of exactly 1 check this

        visited: set[int] = set()
        topo: list[Tensor] = []
        stack: list[tuple[Tensor, int]] = [(self, 0)]
        visited.add(id(self))
        while stack:
            node, i = stack.pop()
            parents = node._parents
            if i < len(parents):
                stack.append((node, i + 1))
                p = parents[i]
                if id(p) not in visited:
                    visited.add(id(p))
                    stack.append((p, 0))
            else:
                topo.append(node)

        for node in topo:
            node._n_pending = 0
        for node in topo:
            for p in node._parents:
                p._n_pending += 1
        obs = _backward_observer
        if obs is not None:
            obs.begin(topo)
        for i in range(len(topo) - 1, -1, -1):
            node = topo[i]
            parents = node._parents
            if node._backward is not None and node.grad is not None:
                node._backward(node.grad)
            for p in parents:
                p._n_pending -= 1
            if parents:
                node._parents = ()
                node._backward = None
                node._ctx = None
                if obs is not None:
                    obs.node_done(parents)
            topo[i] = None
        if obs is not None:
            obs.end()

    def _set_graph(self, parents: tuple["Tensor", ...], backward_fn: Callable[["Tensor"], None], ctx: Optional[dict] = None) -> None:
        """Attach graph fields only if some parent requires grad (gradtuity/tensor.py:415-445)."""
        self.requires_grad = any(p.requires_grad for p in parents)
        if self.requires_grad:
            self._parents = parents
            self._backward = backward_fn
            self._ctx = ctx

    def detach(self) -> "Tensor":
        if self._join_id and self._join_id == _pending_join[0]:
            join_side_stream()               # the alias carries no mark of its own
        shared = Storage(self._st.ptr, self._st.nbytes, owns=False, base=self._st)
        out = Tensor._wrap(shared, self._shape, requires_grad=False, name=f"{self.name}_detached" if self.name else "")
        out._pitch = self._pitch
        return out

    def view(self, new_shape) -> "Tensor":
        """Same storage, different shape; one dimension may be -1/None (gradtuity/tensor.py:465-524)."""
        if self._join_id and self._join_id == _pending_join[0]:
            join_side_stream()               # the alias carries no mark of its own
        dims = list(new_shape)
        infer = None
        product = 1
        for i, d in enumerate(dims):
            if d is None or d == -1:
                if infer is not None:
                    raise ValueError("view() allows only one dimension to be -1")
                infer = i
            else:
                if d <= 0:
                    raise ValueError(f"view() dimension {i} must be positive, got {d}")
                product *= d
        if infer is not None:
            inferred = self.numel // product
            if inferred * product != self.numel:
                raise ValueError(f"view() shape {tuple(new_shape)} is incompatible with numel {self.numel}")
            dims[infer] = inferred
        elif product != self.numel:
            raise ValueError(f"view() shape {tuple(new_shape)} has {product} elements, but tensor has {self.numel} elements")
        if self._pitch is not None and dims[-1] == self._shape[-1]:
            out = Tensor._wrap(Storage(self._st.ptr, self._st.nbytes, owns=False, base=self._st), tuple(dims))
            out._pitch = self._pitch
        else:
            out = Tensor._from_ptr(self.ptr, tuple(dims), owns_memory=False, requires_grad=False, base=self._st)
        src = self

        def _backward(out_grad: "Tensor") -> None:
            if src.requires_grad:
                pass_grad(src, out_grad)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    # ---- the GEMM family ----------------------------------------------------------------

    def matmul(self, other: "Tensor") -> "Tensor":
        """C[M,N] = A[M,K] @ B[K,N]; backward dA += dC·Bᵀ (NT), dB += Aᵀ·dC (TN), both read in
        place and accumulated by the GEMM epilogue (gradtuity/tensor.py:530-657)."""
        if self.ndim != 2:
            raise ValueError(f"matmul requires 2D tensors, got self.shape={self._shape}")
        if other.ndim != 2:
            raise ValueError(f"matmul requires 2D tensors, got other.shape={other._shape}")
        if self._shape[1] != other._shape[0]:
            raise ValueError(
                f"matmul shape mismatch: {self._shape} @ {other._shape} "
                f"(inner dimensions {self._shape[1]} vs {other._shape[0]})"
            )
        M, K = self._shape
        _, N = other._shape
        out = empty_tensor((M, N))
        _gemm.gemm(LAYOUT_NN, M, N, K, self.ptr, K, other.ptr, N, out.ptr, N)
        a, b = self, other

        def _backward(g: "Tensor") -> None:
            if a.requires_grad:
                ptr, acc = grad_target(a)
                _gemm.gemm(LAYOUT_NT, M, K, N, g.ptr, N, b.ptr, N, ptr, K, accumulate=acc)
            if b.requires_grad:
                ptr, acc = grad_target(b)
                _gemm.gemm(LAYOUT_TN, K, N, M, a.ptr, K, g.ptr, N, ptr, N, accumulate=acc)

        out._set_graph(parents=(self, other), backward_fn=_backward)
        return out

    def bmm(self, other: "Tensor") -> "Tensor":
        """Batched matmul, rank 3 (B,M,K)@(B,K,N) or rank 4 (B,H,M,K)@(B,H,K,N), as ONE
        strided-batched launch forward and two backward (the reference loops over slices in
        Python: gradtuity/tensor.py:760-896)."""
        ndim = self.ndim
        if ndim not in (3, 4):
            raise ValueError(f"bmm requires ndim 3 or 4, got self.ndim={ndim}")
        if other.ndim != ndim:
            raise ValueError(f"bmm requires same ndim for both tensors, got {ndim} vs {other.ndim}")
        if ndim == 3:
            Bf, M, K = self.shape
            B2, K2, N = other.shape
            if B2 != Bf:
                raise ValueError(f"bmm batch dim mismatch: {self.shape} vs {other.shape}")
            if K2 != K:
                raise ValueError(f"bmm inner dim mismatch: a.shape[2]={K} vs b.shape[1]={K2}")
            out = empty_tensor((Bf, M, N))
        else:
            B, H, M, K = self.shape
            B2, H2, K2, N = other.shape
            if B2 != B or H2 != H:
                raise ValueError(f"bmm batch/head dim mismatch: {self.shape} vs {other.shape}")
            if K2 != K:
                raise ValueError(f"bmm inner dim mismatch: a.shape[3]={K} vs b.shape[2]={K2}")
            Bf = B * H
            out = empty_tensor((B, H, M, N))
        _gemm.gemm_batched(LAYOUT_NN, M, N, K, self.ptr, K, M * K, 0, other.ptr, N, K * N, 0,
                           out.ptr, N, M * N, 0, Bf)
        a, b = self, other

        def _backward(g: "Tensor") -> None:
            if a.requires_grad:
                ptr, acc = grad_target(a)
                _gemm.gemm_batched(LAYOUT_NT, M, K, N, g.ptr, N, M * N, 0, b.ptr, N, K * N, 0,
                                   ptr, K, M * K, 0, Bf, accumulate=acc)
            if b.requires_grad:
                ptr, acc = grad_target(b)
                _gemm.gemm_batched(LAYOUT_TN, K, N, M, a.ptr, K, M * K, 0, g.ptr, N, M * N, 0,
                                   ptr, N, K * N, 0, Bf, accumulate=acc)

        out._set_graph(parents=(self, other), backward_fn=_backward)
        return out

    def _linear_checks(self, weight: "Tensor", bias: "Tensor", opname: str) -> None:
        if self.ndim != 2:
            raise ValueError(f"{opname} requires 2D input, got shape {self._shape}")
        if weight.ndim != 2:
            raise ValueError(f"weight must be 2D, got shape {weight._shape}")
        if bias.ndim != 1:
            raise ValueError(f"bias must be 1D, got shape {bias._shape}")
        if self._shape[1] != weight._shape[0]:
            raise ValueError(f"{opname} shape mismatch: input {self._shape} @ weight {weight._shape}")
        if weight._shape[1] != bias._shape[0]:
            raise ValueError(f"bias size {bias._shape[0]} doesn't match weight out_features {weight._shape[1]}")

    def _linear_backward(self, x: "Tensor", weight: "Tensor", bias: "Tensor", dz_ptr: int, M: int, K: int, N: int,
                         bias_done: bool = False) -> None:
        """dX += dZ·Wᵀ (NT), dW += Xᵀ·dZ (TN), db += column sums of dZ (gradtuity/tensor.py:1628-1679).
        `bias_done`: the kernel that wrote dZ has already added its column sums to the bias gradient."""
        if bias.requires_grad and not bias_done:
            # the column sums are memory-bound and read what the two GEMMs read: they run beside them, on the side stream
            ensure_grad(bias)
            _call("gt_colsum_acc_beside", _vp(bias.grad.ptr), _vp(dz_ptr), M, N, N)
        if x.requires_grad:
            ptr, acc = grad_target(x)
            _gemm.gemm(LAYOUT_NT, M, K, N, dz_ptr, N, weight.ptr, N, ptr, K, accumulate=acc)
        if weight.requires_grad:
            ptr, acc = grad_target(weight)
            _gemm.gemm(LAYOUT_TN, K, N, M, x.ptr, K, dz_ptr, N, ptr, N, accumulate=acc)
        if bias.requires_grad and not bias_done:
            _call("gt_join_beside")          # before dZ can be freed and the bias gradient read

    def linear(self, weight: "Tensor", bias: "Tensor") -> "Tensor":
        """Y = X @ W + b with W stored (in_features, out_features); bias fused into the GEMM
        epilogue (gradtuity/tensor.py:1561-1682)."""
        self._linear_checks(weight, bias, "linear")
        M, K = self._shape
        _, N = weight._shape
        out = empty_tensor((M, N))
        _gemm.gemm(LAYOUT_NN, M, N, K, self.ptr, K, weight.ptr, N, out.ptr, N, bias_ptr=bias.ptr, epilogue=EPI_BIAS)
        x = self

        def _backward(g: "Tensor") -> None:
            self._linear_backward(x, weight, bias, g.ptr, M, K, N)

        out._set_graph(parents=(self, weight, bias), backward_fn=_backward)
        return out

    def linear_qkv(self, wq: "Tensor", wk: "Tensor", wv: "Tensor", bq: "Tensor", bk: "Tensor", bv: "Tensor"):
        """(x @ Wq + bq, x @ Wk + bk, x @ Wv + bv) for x of shape (..., E): the three projections of
        CausalSelfAttention (gradtuity/nn.py:534-536 calls `linear` three times).  When the three weights sit
        at a uniform distance in memory and the three biases are adjacent (nn.CausalSelfAttention allocates
        them that way), forward and backward are batched launches: one NN GEMM with a shared A and a bias row
        per batch entry; dX as one NT launch whose three batch entries add into the same buffer; dW as one TN
        launch with a shared A.  Otherwise this is three `linear` calls.  Results are the same either way."""
        x = self
        lead = x._shape[:-1]
        K = x._shape[-1]
        M = x.numel // K
        for w, b in ((wq, bq), (wk, bk), (wv, bv)):
            if w.ndim != 2 or b.ndim != 1 or w._shape[0] != K or w._shape != wq._shape or b._shape[0] != w._shape[1]:
                raise ValueError(f"linear_qkv shape mismatch: input {x._shape}, weight {w._shape}, bias {b._shape}")
        N = wq._shape[1]
        out_shape = lead + (N,)
        sw = wk.ptr - wq.ptr
        batched = (x.ndim >= 2 and sw > 0 and wv.ptr - wk.ptr == sw and sw % 16 == 0 and bk.ptr - bq.ptr == N * F32
                   and bv.ptr - bk.ptr == N * F32 and N % 4 == 0 and K % 4 == 0 and wq.ptr % 16 == 0 and x.ptr % 16 == 0
                   and bq.ptr % 16 == 0 and _gemm.default_precision() != _lib.PREC_FP32
                   and "GRADTUITY_GEMM_DETERMINISTIC" not in os.environ)      # the shared-dX launch adds in no fixed order
        if not batched:
            x2 = x.view((M, K))
            return tuple(x2.linear(w, b).view(out_shape) for w, b in ((wq, bq), (wk, bk), (wv, bv)))
        from ._lib import GEMM_BIAS_PER_BATCH
        sw //= F32
        y3 = alloc_storage(3 * M * N * F32)
        _gemm.gemm_batched(LAYOUT_NN, M, N, K, x.ptr, K, 0, 0, wq.ptr, N, sw, 0, y3.ptr, N, M * N, 0, 3, 1,
                           bias_ptr=bq.ptr, epilogue=EPI_BIAS, flags=GEMM_BIAS_PER_BATCH)
        outs = [Tensor._from_ptr(y3.ptr + i * M * N * F32, out_shape, owns_memory=False, base=y3) for i in range(3)]
        ws, bs = (wq, wk, wv), (bq, bk, bv)
        if not (x.requires_grad or any(w.requires_grad for w in ws) or any(b.requires_grad for b in bs)):
            return tuple(outs)
        # Graph: a hidden node holds the batched backward; q, k, v are its children and their gradients are
        # the three slices of one buffer, so the backward reads them as one batch without copying.
        hub = Tensor._from_ptr(y3.ptr, (3, M, N), owns_memory=False, base=y3)
        group = _GradGroup(3, M * N)

        def _hub_backward(_g: "Tensor") -> None:
            for i in range(3):
                if not group.written[i]:
                    group.slice_tensor(i, (M, N), zero=True)
            dy = group.storage.ptr
            # the three bias gradients: nothing to do when the attention backward has added them already; else one launch
            # when they sit N floats apart (they do when zero_grad made them), beside the GEMMs
            if all(group.colsum_done[i] or not b.requires_grad for i, b in enumerate(bs)):
                pass
            elif all(b.requires_grad for b in bs) and not any(group.colsum_done):
                for b in bs:
                    ensure_grad(b)
                gp = [b.grad.ptr for b in bs]
                if gp[1] - gp[0] == gp[2] - gp[1] and (gp[1] - gp[0]) % F32 == 0:
                    _call("gt_colsum_acc_batched_beside", _vp(gp[0]), (gp[1] - gp[0]) // F32, _vp(dy), M * N, M, N, N, 3)
                else:
                    for i, b in enumerate(bs):
                        _call("gt_colsum_acc_beside", _vp(b.grad.ptr), _vp(dy + i * M * N * F32), M, N, N)
            else:
                for i, b in enumerate(bs):
                    if b.requires_grad and not group.colsum_done[i]:
                        ensure_grad(b)
                        _call("gt_colsum_acc_beside", _vp(b.grad.ptr), _vp(dy + i * M * N * F32), M, N, N)
            if x.requires_grad:
                ptr, acc = grad_target(x)
                if not acc:
                    cuda_memset(ptr, 0, M * K * F32)
                _gemm.gemm_batched(LAYOUT_NT, M, K, N, dy, N, M * N, 0, wq.ptr, N, sw, 0, ptr, K, 0, 0, 3, 1, accumulate=True)
            if any(w.requires_grad for w in ws):
                if all(w.requires_grad and w.grad is None for w in ws):
                    blk = alloc_storage(3 * K * N * F32)
                    for i, w in enumerate(ws):
                        w.grad = Tensor._from_ptr(blk.ptr + i * K * N * F32, w.shape, owns_memory=False, base=blk)
                    g0, sg, acc = blk.ptr, K * N, False
                else:
                    for w in ws:
                        if w.requires_grad:
                            ensure_grad(w)
                    ptrs = [w.grad.ptr if w.requires_grad else 0 for w in ws]
                    sg = ptrs[1] - ptrs[0]
                    uniform = all(w.requires_grad for w in ws) and sg > 0 and ptrs[2] - ptrs[1] == sg and sg % 16 == 0
                    g0, sg, acc = (ptrs[0], sg // F32, True) if uniform else (0, 0, True)
                if g0:
                    _gemm.gemm_batched(LAYOUT_TN, K, N, M, x.ptr, K, 0, 0, dy, N, M * N, 0, g0, N, sg, 0, 3, 1, accumulate=acc)
                else:
                    for i, w in enumerate(ws):
                        if w.requires_grad:
                            _gemm.gemm(LAYOUT_TN, K, N, M, x.ptr, K, dy + i * M * N * F32, N, w.grad.ptr, N, accumulate=True)
            _call("gt_join_beside")

        hub._set_graph(parents=(x,) + ws + bs, backward_fn=_hub_backward)

        def _child_backward(_g: "Tensor") -> None:
            if hub.grad is None:                       # the slices already hold the gradients: only wake the hub
                hub.grad = Tensor._from_ptr(group.storage.ptr, (3, M, N), owns_memory=False, base=group.storage)

        for i, o in enumerate(outs):
            o._grad_slot = (group, i)
            o._set_graph(parents=(hub,), backward_fn=_child_backward)
            if bs[i].requires_grad:
                o._grad_colsum_bias = bs[i]
        return tuple(outs)

    @staticmethod
    def _aux_epilogue_ok(ptrs, dims) -> bool:
        """The aux-reading GEMM epilogues need the tensor-core path: tf32 / 3xtf32, 16-byte aligned buffers,
        leading dimensions that are multiples of 4."""
        if _gemm.default_precision() == _lib.PREC_FP32:
            return False
        return all(p % 16 == 0 for p in ptrs) and all(d % 4 == 0 for d in dims)

    def linear_add(self, weight: "Tensor", bias: "Tensor", residual: "Tensor") -> "Tensor":
        """residual + X @ W + b.  A Linear layer and the residual add that follows it in a transformer block
        (gpt2/model.py:64-71: `x = x + attn(...)`, `x = x + mlp(...)`) as one GEMM whose epilogue reads the
        residual; otherwise `residual.add(x.linear(w, b))`.  `residual` may have any shape with M * N elements;
        the result has its shape."""
        self._linear_checks(weight, bias, "linear_add")
        M, K = self._shape
        _, N = weight._shape
        if residual.numel != M * N:
            raise ValueError(f"linear_add: residual shape {residual._shape} does not hold {M} x {N} elements")
        if not self._aux_epilogue_ok((self.ptr, weight.ptr, bias.ptr, residual.ptr), (K, N)):
            return residual.add(self.linear(weight, bias).view(residual._shape))
        from ._lib import EPI_BIAS_ADD
        out = empty_tensor(residual._shape)
        _gemm.gemm(LAYOUT_NN, M, N, K, self.ptr, K, weight.ptr, N, out.ptr, N, bias_ptr=bias.ptr, aux_ptr=residual.ptr,
                   epilogue=EPI_BIAS_ADD)
        x = self

        def _backward(g: "Tensor") -> None:
            self._linear_backward(x, weight, bias, g.ptr, M, K, N, bias_done=g._colsum_done)
            if residual.requires_grad:
                pass_grad(residual, g)

        out._set_graph(parents=(self, weight, bias, residual), backward_fn=_backward)
        if bias.requires_grad:
            out._grad_colsum_bias = bias
        return out

    def mlp_gelu(self, w1: "Tensor", b1: "Tensor", w2: "Tensor", b2: "Tensor", residual: "Tensor | None" = None) -> "Tensor":
        """(residual +) gelu(X @ W1 + b1) @ W2 + b2: the MLP of a GPT-2 block (gpt2/model.py:68-71).  Forward: the
        first GEMM stores the pre-activation beside the activation, the second adds the residual in its epilogue.
        Backward: the dX GEMM of the second layer multiplies by gelu'(pre-activation) in its epilogue, so the
        separate GELU-backward pass over the (M, inner) tensor and its temporary disappear."""
        self._linear_checks(w1, b1, "mlp_gelu")
        M, K = self._shape
        _, I = w1._shape
        if w2.ndim != 2 or b2.ndim != 1 or w2._shape[0] != I or b2._shape[0] != w2._shape[1]:
            raise ValueError(f"mlp_gelu shape mismatch: hidden {I}, second weight {w2._shape}, second bias {b2._shape}")
        N = w2._shape[1]
        if residual is not None and residual.numel != M * N:
            raise ValueError(f"mlp_gelu: residual shape {residual._shape} does not hold {M} x {N} elements")
        ptrs = [self.ptr, w1.ptr, b1.ptr, w2.ptr, b2.ptr] + ([residual.ptr] if residual is not None else [])
        if not self._aux_epilogue_ok(ptrs, (K, I, N)):
            y = self.linear_gelu(w1, b1).linear(w2, b2)
            return y if residual is None else residual.add(y.view(residual._shape))
        from ._lib import EPI_BIAS_ADD, EPI_GELU_GRAD
        h = alloc_storage(M * I * F32)
        pre = alloc_storage(M * I * F32)
        _gemm.gemm(LAYOUT_NN, M, I, K, self.ptr, K, w1.ptr, I, h.ptr, I, bias_ptr=b1.ptr, aux_ptr=pre.ptr, epilogue=EPI_BIAS_GELU)
        out = empty_tensor(residual._shape if residual is not None else (M, N))
        if residual is not None:
            _gemm.gemm(LAYOUT_NN, M, N, I, h.ptr, I, w2.ptr, N, out.ptr, N, bias_ptr=b2.ptr, aux_ptr=residual.ptr, epilogue=EPI_BIAS_ADD)
        else:
            _gemm.gemm(LAYOUT_NN, M, N, I, h.ptr, I, w2.ptr, N, out.ptr, N, bias_ptr=b2.ptr, epilogue=EPI_BIAS)
        x = self
        if not (x.requires_grad or w1.requires_grad or b1.requires_grad or w2.requires_grad or b2.requires_grad
                or (residual is not None and residual.requires_grad)):
            h.free(); pre.free()

        def _backward(g: "Tensor") -> None:
            if b2.requires_grad and not g._colsum_done:             # beside the GEMMs that follow
                ensure_grad(b2)
                _call("gt_colsum_acc_beside", _vp(b2.grad.ptr), _vp(g.ptr), M, N, N)
            if w2.requires_grad:
                ptr, acc = grad_target(w2)
                _gemm.gemm(LAYOUT_TN, I, N, M, h.ptr, I, g.ptr, N, ptr, N, accumulate=acc)
            h.free()
            if x.requires_grad or w1.requires_grad or b1.requires_grad:
                with temp_storage(M * I * F32) as dpre:
                    # d(pre-activation) = (dY @ W2^T) * gelu'(pre), the product in the GEMM's epilogue
                    # with the first layer's bias gradient (the column sums of dpre) taken from the output tiles
                    fused_db1 = b1.requires_grad and os.environ.get("GRADTUITY_NO_GEMM_COLSUM") is None
                    if fused_db1:
                        ensure_grad(b1)
                        _gemm.gemm_gelu_grad_colsum(LAYOUT_NT, M, I, N, g.ptr, N, w2.ptr, N, dpre.ptr, I, pre.ptr, b1.grad.ptr)
                    else:
                        _gemm.gemm(LAYOUT_NT, M, I, N, g.ptr, N, w2.ptr, N, dpre.ptr, I, aux_ptr=pre.ptr, epilogue=EPI_GELU_GRAD)
                    pre.free()
                    self._linear_backward(x, w1, b1, dpre.ptr, M, K, I, bias_done=fused_db1)
            else:
                pre.free()
            _call("gt_join_beside")
            if residual is not None and residual.requires_grad:
                pass_grad(residual, g)

        out._set_graph(parents=(self, w1, b1, w2, b2) + ((residual,) if residual is not None else ()), backward_fn=_backward)
        if b2.requires_grad and out._shape[-1] == N:
            out._grad_colsum_bias = b2
        return out

    def linear_relu(self, weight: "Tensor", bias: "Tensor") -> "Tensor":
        """Y = relu(X @ W + b), one kernel; backward masks dY by [Y > 0] into a temporary and
        proceeds as `linear` (gradtuity/tensor.py:1781-1904)."""
        self._linear_checks(weight, bias, "linear_relu")
        M, K = self._shape
        _, N = weight._shape
        out = empty_tensor((M, N))
        _gemm.gemm(LAYOUT_NN, M, N, K, self.ptr, K, weight.ptr, N, out.ptr, N, bias_ptr=bias.ptr, epilogue=EPI_BIAS_RELU)
        x = self
        y = out

        def _backward(g: "Tensor") -> None:
            with temp_storage(M * N * F32) as st:
                _call("gt_relu_mask_mul", _vp(st.ptr), _vp(g.ptr), _vp(y.ptr), M * N, 0)
                self._linear_backward(x, weight, bias, st.ptr, M, K, N)

        out._set_graph(parents=(self, weight, bias), backward_fn=_backward)
        return out

    def linear_gelu(self, weight: "Tensor", bias: "Tensor") -> "Tensor":
        """Y = gelu_tanh(X @ W + b) in one kernel that also stores the pre-activation Z, which the
        backward needs.  Equals the reference's `x.linear(w, b).gelu()` (gpt2/model.py:70,
        gradtuity/tensor.py:954-984) without the separate 100 MB element-wise passes."""
        self._linear_checks(weight, bias, "linear_gelu")
        M, K = self._shape
        _, N = weight._shape
        out = empty_tensor((M, N))
        pre = empty_tensor((M, N))
        _gemm.gemm(LAYOUT_NN, M, N, K, self.ptr, K, weight.ptr, N, out.ptr, N, bias_ptr=bias.ptr,
                   aux_ptr=pre.ptr, epilogue=EPI_BIAS_GELU)
        x = self

        def _backward(g: "Tensor") -> None:
            with temp_storage(M * N * F32) as st:
                _call("gt_gelu_backward", _vp(st.ptr), _vp(g.ptr), _vp(pre.ptr), M * N, 0)
                self._linear_backward(x, weight, bias, st.ptr, M, K, N)

        out._set_graph(parents=(self, weight, bias), backward_fn=_backward)
        return out

    def linear_tied(self, weight: "Tensor") -> "Tensor":
        """Y = X @ Wᵀ with W stored (V, E) (the tied LM head); backward dX += dY·W (NN),
        dW += dYᵀ·X (TN) (gradtuity/tensor.py:1684-1779)."""
        if self.ndim != 2:
            raise ValueError(f"linear_tied requires 2D input, got shape {self._shape}")
        if weight.ndim != 2:
            raise ValueError(f"weight must be 2D, got shape {weight._shape}")
        if self._shape[1] != weight._shape[1]:
            raise ValueError(
                f"linear_tied shape mismatch: input last dim {self._shape[1]} != weight last dim {weight._shape[1]}"
            )
        M, E = self._shape
        V, _ = weight._shape
        if V % 4 != 0 and M * V >= (1 << 22):
            # Large logits with an odd vocabulary (50257): rows padded to a 128-byte multiple, so the
            # GEMM stores them through TMA, the loss kernels use vector loads and the two backward GEMMs
            # read dlogits through TMA.  cross_entropy and view() keep the padding; anything else packs.
            out = empty_padded_tensor((M, V), (V + 31) // 32 * 32)
        else:
            out = empty_tensor((M, V))
        out_ptr, out_ld = out._rows()
        _gemm.gemm(LAYOUT_NT, M, V, E, self.ptr, E, weight.ptr, E, out_ptr, out_ld)
        x = self

        def _backward(g: "Tensor") -> None:
            g_ptr, g_ld = g._rows()
            tmp = None
            if g_ld % 4 != 0 and M * V >= (1 << 22) and (x.requires_grad and weight.requires_grad):
                # dL is read by two large GEMMs and its rows are not 16-byte aligned (odd vocabulary):
                # one copy to a padded pitch lets both take the TMA path instead of 4-byte copies.
                g_ld = (V + 3) // 4 * 4
                tmp = alloc_storage(M * g_ld * F32)
                _call("gt_repack_rows", _vp(tmp.ptr), g_ld, _vp(g.ptr), V, M, V)
                g_ptr = tmp.ptr
            if x.requires_grad:
                ptr, acc = grad_target(x)
                _gemm.gemm(LAYOUT_NN, M, E, V, g_ptr, g_ld, weight.ptr, E, ptr, E, accumulate=acc)
            if weight.requires_grad:
                ptr, acc = grad_target(weight)
                _gemm.gemm(LAYOUT_TN, V, E, M, g_ptr, g_ld, x.ptr, E, ptr, E, accumulate=acc)
            if tmp is not None:
                tmp.free()

        out._set_graph(parents=(self, weight), backward_fn=_backward)
        return out

    # ---- attention: the batched per-head products ---------------------------------------------

    def causal_attention(self, k: "Tensor", v: "Tensor", num_heads: int) -> "Tensor":
        """Causal multi-head attention on projection outputs: self = Q, k, v, all (B, S, E).

        Computes exactly what the reference's CausalSelfAttention computes between its
        projections (gradtuity/nn.py:534-549): S = Q Kᵀ / sqrt(d) per head, P = causal softmax,
        O = P V, heads merged back to (B, S, E).  The per-head slices of the (B, S, H, d) buffers are
        addressed in place, so none of transpose4d_12 / transpose4d_last2 / scale_inplace runs and no
        (B, H, S, d) copy exists.  Two forms (see GRADTUITY_ATTENTION below): fused forward and backward
        kernels that keep only each row's log-sum-exp (head dimension 64, S a multiple of 128, tf32),
        or, for every other shape, the three batched products and their four backward products as single
        strided-batched GEMM launches, with the 1/sqrt(d) scale and the causal mask in the score GEMM's
        epilogue (tiles wholly above the diagonal are not computed) and P (B, H, S, S) kept for the
        backward, as in the reference.
        """
        q = self
        if q.ndim != 3 or k.shape != q.shape or v.shape != q.shape:
            raise ValueError(f"causal_attention requires q, k, v of the same (B, S, E) shape, got {q.shape}, {k.shape}, {v.shape}")
        B, S, E = q.shape
        H = num_heads
        if H <= 0 or E % H != 0:
            raise ValueError(f"embed_dim ({E}) must be divisible by num_heads ({H})")
        D = E // H
        scale = 1.0 / (D ** 0.5)
        from ._lib import EPI_CAUSAL, GEMM_A_LOWER, GEMM_AT_LOWER, GEMM_CAUSAL_SKIP_MASKED, PREC_FP32
        # P and dS are zero above the diagonal.  When every operand can take the tensor-core path
        # the GEMMs are told so: score tiles wholly above the diagonal are neither computed nor
        # written, the softmax kernels write zeros only up to the end of each row's 128-wide
        # diagonal block, and the products that read P / dS contract only over the k-blocks that can
        # be non-zero.  That removes about 45 % of the (B, H, S, S) traffic; the values used are the same.
        trimmed = (S % 4 == 0 and D % 4 == 0 and _gemm.default_precision() != PREC_FP32)
        f_skip = GEMM_CAUSAL_SKIP_MASKED if trimmed else 0
        f_lower = GEMM_A_LOWER if trimmed else 0
        f_upper = GEMM_AT_LOWER if trimmed else 0
        sm_mode = 2 if trimmed else 1
        out = empty_tensor((B, S, E))
        # GRADTUITY_ATTENTION selects the form when the head dimension is 64, S a multiple of 128 and the
        # GEMM precision tf32:
        #   flash (default)   fused forward and backward kernels; no (B, H, S, S) tensor exists, only each
        #                     row's log-sum-exp is kept and P is recomputed in the backward;
        #   fused_forward     fused forward that also writes P, backward as four batched GEMMs + softmax backward;
        #   materialized      S, then P, then O as three launches (the reference's structure), as for every
        #                     other shape.
        from ._lib import PREC_TF32
        mode = os.environ.get("GRADTUITY_ATTENTION", "flash")
        if mode not in ("flash", "fused_forward", "materialized"):
            raise ValueError(f"GRADTUITY_ATTENTION must be flash, fused_forward or materialized, got {mode!r}")
        fusable = trimmed and D == 64 and S % 128 == 0 and _gemm.default_precision() == PREC_TF32
        if fusable and mode == "flash":
            lse = empty_tensor((B, H, S))
            _call("gt_attention_forward", _vp(out.ptr), None, _vp(lse.ptr), _vp(q.ptr), _vp(k.ptr), _vp(v.ptr),
                  B, S, H, D, scale, None)
            o_st = out._st          # the closure keeps the buffer, not the tensor (no reference cycle)

            def _backward_flash(g: "Tensor") -> None:
                if not (q.requires_grad or k.requires_grad or v.requires_grad):
                    return
                targets, scratch = [], []
                for t in (q, k, v):
                    if t.requires_grad:
                        targets.append(grad_target(t))
                    else:
                        st = alloc_storage(B * S * E * F32)
                        scratch.append(st)
                        targets.append((st.ptr, False))
                # A projection bias whose gradient is the column sums of dQ / dK / dV (linear_qkv marks its outputs): the
                # kernels add them when this call writes the whole of that gradient (nothing accumulated, no other consumer left).
                dbias = [0, 0, 0]
                if os.environ.get("GRADTUITY_NO_ATTN_COLSUM") is None:
                    for n, t in enumerate((q, k, v)):
                        cb = t._grad_colsum_bias
                        if (cb is not None and t.requires_grad and not targets[n][1] and t._n_pending == 1 and t._grad_slot is not None
                                and cb.numel == E):
                            ensure_grad(cb)
                            dbias[n] = cb.grad.ptr
                            t._grad_slot[0].colsum_done[t._grad_slot[1]] = True
                delta = alloc_storage(B * H * S * F32)
                _call("gt_attention_backward_bias", _vp(targets[0][0]), _vp(targets[1][0]), _vp(targets[2][0]), _vp(dbias[0]), _vp(dbias[1]),
                      _vp(dbias[2]), _vp(g.ptr), _vp(q.ptr), _vp(k.ptr), _vp(v.ptr), _vp(o_st.ptr), _vp(lse.ptr), _vp(delta.ptr), B, S, H, D,
                      scale, int(targets[0][1]), int(targets[1][1]), int(targets[2][1]), None)
                delta.free()
                for st in scratch:
                    st.free()

            out._set_graph(parents=(q, k, v), backward_fn=_backward_flash)
            return out
        p = empty_tensor((B, H, S, S))
        fused = fusable and mode == "fused_forward"
        if fused:
            lse = empty_tensor((B, H, S))
            _call("gt_attention_forward", _vp(out.ptr), _vp(p.ptr), _vp(lse.ptr), _vp(q.ptr), _vp(k.ptr), _vp(v.ptr),
                  B, S, H, D, scale, None)
        else:
            # scores[b, h] = scale * Q[b, :, h, :] K[b, :, h, :]^T, masked: NT, in-place heads
            _gemm.gemm_batched(LAYOUT_NT, S, S, D, q.ptr, E, D, S * E, k.ptr, E, D, S * E,
                               p.ptr, S, S * S, H * S * S, H, B, alpha=scale, epilogue=EPI_CAUSAL, flags=f_skip)
            _call("gt_softmax", _vp(p.ptr), _vp(p.ptr), B * H * S, S, sm_mode)
            # O[b, :, h, :] = P[b, h] V[b, :, h, :]: NN, output written straight into (B, S, H, d)
            _gemm.gemm_batched(LAYOUT_NN, S, D, S, p.ptr, S, S * S, H * S * S, v.ptr, E, D, S * E,
                               out.ptr, E, D, S * E, H, B, flags=f_lower)

        def _backward(g: "Tensor") -> None:
            need_qk = q.requires_grad or k.requires_grad
            if v.requires_grad:
                ptr, acc = grad_target(v)
                # dV[b, :, h, :] += P[b, h]^T dO[b, :, h, :]   (TN)
                _gemm.gemm_batched(LAYOUT_TN, S, D, S, p.ptr, S, S * S, H * S * S, g.ptr, E, D, S * E,
                                   ptr, E, D, S * E, H, B, accumulate=acc, flags=f_upper)
            if need_qk:
                with temp_storage(B * H * S * S * F32) as st:
                    # dP[b, h] = dO[b, :, h, :] V[b, :, h, :]^T   (NT); only the lower triangle is needed
                    _gemm.gemm_batched(LAYOUT_NT, S, S, D, g.ptr, E, D, S * E, v.ptr, E, D, S * E,
                                       st.ptr, S, S * S, H * S * S, H, B, epilogue=EPI_CAUSAL, flags=f_skip)
                    # dS = scale * P * (dP - sum P dP), zero above the diagonal, in place
                    _call("gt_softmax_backward", _vp(st.ptr), _vp(p.ptr), _vp(st.ptr), B * H * S, S, sm_mode, scale)
                    if q.requires_grad:
                        ptr, acc = grad_target(q)
                        # dQ[b, :, h, :] += dS[b, h] K[b, :, h, :]   (NN)
                        _gemm.gemm_batched(LAYOUT_NN, S, D, S, st.ptr, S, S * S, H * S * S, k.ptr, E, D, S * E,
                                           ptr, E, D, S * E, H, B, accumulate=acc, flags=f_lower)
                    if k.requires_grad:
                        ptr, acc = grad_target(k)
                        # dK[b, :, h, :] += dS[b, h]^T Q[b, :, h, :]   (TN)
                        _gemm.gemm_batched(LAYOUT_TN, S, D, S, st.ptr, S, S * S, H * S * S, q.ptr, E, D, S * E,
                                           ptr, E, D, S * E, H, B, accumulate=acc, flags=f_upper)

        out._set_graph(parents=(q, k, v), backward_fn=_backward)
        return out

    # ---- the other ops of the GPT-2 step --------------------------------------------------------

    def softmax(self, dim: int = -1) -> "Tensor":
        if dim != -1 and dim != self.ndim - 1:
            raise ValueError(f"softmax v1 only supports dim=-1, got dim={dim}")
        cols = self._shape[-1]
        rows = self.numel // cols
        out = empty_tensor(self.shape)
        _call("gt_softmax", _vp(out.ptr), _vp(self.ptr), rows, cols, 0)
        x = self

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                with temp_storage(x.numel * F32) as st:
                    _call("gt_softmax_backward", _vp(st.ptr), _vp(out.ptr), _vp(g.ptr), rows, cols, 0, 1.0)
                    ensure_grad(x)
                    _call("gt_scale", _vp(x.grad.ptr), _vp(st.ptr), 1.0, x.numel, 1)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def softmax_with_causal_mask(self) -> "Tensor":
        """Row softmax of a (B, H, S, S) score tensor under the causal mask; masked probabilities
        are exactly 0 (gradtuity/tensor.py:1035-1084)."""
        if self.ndim != 4:
            raise ValueError(f"softmax_with_causal_mask requires ndim=4, got ndim={self.ndim}")
        if self._shape[2] != self._shape[3]:
            raise ValueError(f"softmax_with_causal_mask requires square last two dims, got {self._shape}")
        cols = self._shape[-1]
        rows = self.numel // cols
        out = empty_tensor(self.shape)
        _call("gt_softmax", _vp(out.ptr), _vp(self.ptr), rows, cols, 1)
        x = self

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                with temp_storage(x.numel * F32) as st:
                    _call("gt_softmax_backward", _vp(st.ptr), _vp(out.ptr), _vp(g.ptr), rows, cols, 1, 1.0)
                    ensure_grad(x)
                    _call("gt_scale", _vp(x.grad.ptr), _vp(st.ptr), 1.0, x.numel, 1)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def layer_norm(self, gamma: "Tensor", beta: "Tensor", eps: float = 1e-5) -> "Tensor":
        """LayerNorm over the last dimension (gradtuity/tensor.py:1086-1188)."""
        if self.ndim not in (2, 3, 4):
            raise ValueError(f"layer_norm v1 requires ndim in (2, 3, 4), got ndim={self.ndim}")
        if gamma.ndim != 1 or beta.ndim != 1:
            raise ValueError(f"layer_norm requires 1D gamma and beta, got gamma.ndim={gamma.ndim}, beta.ndim={beta.ndim}")
        Hd = self.shape[-1]
        if gamma.shape[0] != Hd or beta.shape[0] != Hd:
            raise ValueError(f"layer_norm gamma/beta must have shape (H,) with H={Hd}, got gamma={gamma.shape}, beta={beta.shape}")
        Nr = self.numel // Hd
        out = empty_tensor(self.shape)
        mean = empty_tensor((Nr,))
        rstd = empty_tensor((Nr,))
        _call("gt_layernorm", _vp(out.ptr), _vp(mean.ptr), _vp(rstd.ptr), _vp(self.ptr), _vp(gamma.ptr), _vp(beta.ptr), Nr, Hd, float(eps))
        x = self

        def _backward(g: "Tensor") -> None:
            dx_ptr, dx_acc = 0, True
            if x.requires_grad:
                dx_ptr, dx_acc = grad_target(x)
            dg_ptr = db_ptr = 0
            if gamma.requires_grad:
                ensure_grad(gamma)
                dg_ptr = gamma.grad.ptr
            if beta.requires_grad:
                ensure_grad(beta)
                db_ptr = beta.grad.ptr
            cs_ptr = 0
            cb = x._grad_colsum_bias
            if (cb is not None and dx_ptr and x._n_pending == 1 and cb.numel == Hd and not x.grad._colsum_done
                    and os.environ.get("GRADTUITY_NO_LN_COLSUM") is None):
                # This is the last contribution to x.grad (every other consumer of x has run): the kernel adds the
                # column sums of the finished gradient to the bias gradient of the layer that produced x.
                ensure_grad(cb)
                cs_ptr = cb.grad.ptr
                x.grad._colsum_done = True
            _call("gt_layernorm_backward_colsum", _vp(dx_ptr), _vp(dg_ptr), _vp(db_ptr), _vp(cs_ptr), _vp(g.ptr), _vp(x.ptr), _vp(mean.ptr),
                  _vp(rstd.ptr), _vp(gamma.ptr), Nr, Hd, 1 if dx_acc else 0)

        out._set_graph(parents=(self, gamma, beta), backward_fn=_backward)
        return out

    def embedding(self, indices) -> "Tensor":
        """Row gather out = self[indices], self = (V, D) weight; indices 1-D or 2-D list / tuple /
        Tensor of float-encoded ids (gradtuity/tensor.py:659-758).  Index range is checked on the
        device (status word) rather than by a host loop over a device-to-host copy."""
        if self.ndim != 2:
            raise ValueError(f"embedding requires 2D weight, got shape {self._shape}")
        idx = indices if isinstance(indices, Tensor) else Tensor(indices)
        if idx.ndim not in (1, 2):
            raise ValueError(f"embedding indices must be 1D or 2D, got shape {idx.shape}")
        V, D = self._shape
        n = idx.numel
        out = empty_tensor(idx.shape + (D,))
        _call("gt_embedding", _vp(out.ptr), _vp(self.ptr), _vp(idx.ptr), n, D, V)
        w = self

        def _backward(g: "Tensor") -> None:
            if w.requires_grad:
                obs = _backward_observer
                # a data-parallel plan may keep the rows aside and exchange them instead of reducing the whole table again
                if obs is not None and obs.take_embedding_rows(w, idx, g, n, D, V):
                    return
                ensure_grad(w)
                _call("gt_embedding_backward", _vp(w.grad.ptr), _vp(g.ptr), _vp(idx.ptr), n, D, V)

        out._set_graph(parents=(self,), backward_fn=_backward)
        out._embedding_of = w
        return out

    def cross_entropy(self, targets: "Tensor", reduction: str = "mean") -> "Tensor":
        """Softmax cross-entropy of (B, C) logits against float-encoded class ids
        (gradtuity/tensor.py:1452-1525).  The upstream gradient is read on the device, so the
        backward needs no device-to-host copy."""
        if self.ndim != 2:
            raise ValueError(f"cross_entropy expects 2D logits, got ndim={self.ndim}")
        if targets.ndim != 1:
            raise ValueError(f"cross_entropy expects 1D targets, got ndim={targets.ndim}")
        Bn, C = self.shape
        if targets.shape[0] != Bn:
            raise ValueError(f"cross_entropy batch size mismatch: logits {Bn} vs targets {targets.shape[0]}")
        if reduction not in ("mean", "sum"):
            raise ValueError(f"cross_entropy reduction must be 'mean' or 'sum', got {reduction!r}")
        out = empty_tensor((1,))
        row_loss = empty_tensor((Bn,))
        row_lse = empty_tensor((Bn,))
        x_ptr, x_ld = self._rows()
        grad_scale = (1.0 / Bn) if reduction == "mean" else 1.0
        # When the logits will need a gradient and have none yet, the loss kernel writes it in the same launch (the row
        # is read from HBM once instead of twice), for an upstream gradient of 1: what backward() seeds when this loss
        # is where it starts.  Any other upstream value rescales the stored gradient in the backward.
        early = None
        if self.requires_grad and self.grad is None and Bn * C >= (1 << 20) and os.environ.get("GRADTUITY_CE_UNFUSED") is None:
            early = empty_padded_tensor(self.shape, x_ld)
            e_ptr, e_ld = early._rows()
            _call("gt_cross_entropy_fused", _vp(out.ptr), _vp(row_loss.ptr), _vp(row_lse.ptr), _vp(e_ptr), e_ld, _vp(x_ptr), x_ld,
                  _vp(targets.ptr), Bn, C, 1 if reduction == "mean" else 0, grad_scale)
        else:
            _call("gt_cross_entropy", _vp(out.ptr), _vp(row_loss.ptr), _vp(row_lse.ptr), _vp(x_ptr), x_ld, _vp(targets.ptr), Bn, C,
                  1 if reduction == "mean" else 0)
        logits = self

        def _backward(g: "Tensor") -> None:
            nonlocal early
            if logits.requires_grad and early is not None and logits.grad is None:
                if not getattr(g, "_unit_seed", False):
                    e_ptr, e_ld = early._rows()
                    _call("gt_scale_by_device_scalar", _vp(e_ptr), _vp(g.ptr), Bn * e_ld)
                logits.grad, early = early, None
                return
            early = None
            if logits.requires_grad:
                fresh = logits.grad is None
                if fresh:
                    # written, not accumulated: no memset; padded like the logits so the LM-head GEMMs read it by TMA
                    logits.grad = empty_padded_tensor(logits.shape, logits._rows()[1])
                d_ptr, d_ld = logits.grad._rows()
                lx_ptr, lx_ld = logits._rows()
                _call("gt_cross_entropy_backward", _vp(d_ptr), d_ld, _vp(lx_ptr), lx_ld, _vp(targets.ptr), _vp(row_lse.ptr),
                      _vp(g.ptr), (1.0 / Bn) if reduction == "mean" else 1.0, Bn, C, 0 if fresh else 1)

        out._set_graph(parents=(self, targets), backward_fn=_backward)
        return out

    def conv2d(self, weight: "Tensor", bias: "Tensor", stride: int = 1, padding: int = 0) -> "Tensor":
        """2D convolution as im2col + GEMM: input (N, C_in, H, W), weight (C_out, C_in, kH, kW), bias
        (C_out,) -> (N, C_out, H_out, W_out), H_out = (H + 2*padding - kH) // stride + 1
        (gradtuity/tensor.py:1906-2167; same argument checks and messages).

        Forward: col = im2col(x), Y = col @ W_flat^T + b as one NT GEMM with the bias in the
        epilogue, then (N, H_out*W_out, C_out) -> (N, C_out, H_out*W_out).  Backward: db = column sums
        of dY, dW += dY^T @ col (TN, written straight in the weight's (C_out, C_in*kH*kW) layout),
        dcol = dY @ W_flat (NN), dx += col2im(dcol).  Two things differ from the reference on purpose:
        its forward passes the strides of W_flat where those of W_flat^T belong (reads past the
        weight, noted in gradtuity/tests/test_nn.py:316-322), and it returns the (N*H_out*W_out, C_out)
        product re-viewed as (N, C_out, H_out, W_out) without transposing; this is the NCHW convolution."""
        x = self
        if x.ndim != 4:
            raise ValueError(f"conv2d requires 4D input, got shape {x._shape}")
        if weight.ndim != 4:
            raise ValueError(f"conv2d weight must be 4D, got shape {weight._shape}")
        if bias.ndim != 1:
            raise ValueError(f"conv2d bias must be 1D, got shape {bias._shape}")
        N, C_in, H, W = x._shape
        C_out, C_in_w, kH, kW = weight._shape
        if C_in != C_in_w:
            raise ValueError(f"conv2d input channels {C_in} != weight channels {C_in_w}")
        if bias._shape[0] != C_out:
            raise ValueError(f"conv2d bias size {bias._shape[0]} != out_channels {C_out}")
        H_out = (H + 2 * padding - kH) // stride + 1
        W_out = (W + 2 * padding - kW) // stride + 1
        if H_out <= 0 or W_out <= 0:
            raise ValueError(f"conv2d output spatial size invalid: H_out={H_out}, W_out={W_out}")
        from ._lib import EPI_BIAS
        rows, ncols, hw = N * H_out * W_out, C_in * kH * kW, H_out * W_out
        ld_col = (ncols + 3) // 4 * 4                     # 16-byte aligned rows for the GEMMs that read col
        col = alloc_storage(rows * ld_col * F32, zero=ld_col != ncols)
        _call("gt_im2col", _vp(col.ptr), ld_col, _vp(x.ptr), N, C_in, H, W, kH, kW, stride, padding)
        y_flat = alloc_storage(rows * C_out * F32)
        _gemm.gemm(LAYOUT_NT, rows, C_out, ncols, col.ptr, ld_col, weight.ptr, ncols, y_flat.ptr, C_out,
                   bias_ptr=bias.ptr, epilogue=EPI_BIAS)
        out = empty_tensor((N, C_out, H_out, W_out))
        _call("gt_transpose12", _vp(out.ptr), _vp(y_flat.ptr), N, hw, C_out, 1, 0)
        y_flat.free()
        if not (x.requires_grad or weight.requires_grad):
            col.free()
            col = None

        def _backward(g: "Tensor") -> None:
            nonlocal col
            with temp_storage(rows * C_out * F32) as dy:
                _call("gt_transpose12", _vp(dy.ptr), _vp(g.ptr), N, C_out, hw, 1, 0)      # (N, C_out, HW) -> (N*HW, C_out)
                if bias.requires_grad:
                    ensure_grad(bias)
                    _call("gt_colsum_acc", _vp(bias.grad.ptr), _vp(dy.ptr), rows, C_out, C_out)
                if weight.requires_grad:
                    if col is None:
                        col = alloc_storage(rows * ld_col * F32, zero=ld_col != ncols)
                        _call("gt_im2col", _vp(col.ptr), ld_col, _vp(x.ptr), N, C_in, H, W, kH, kW, stride, padding)
                    ptr, acc = grad_target(weight)
                    _gemm.gemm(LAYOUT_TN, C_out, ncols, rows, dy.ptr, C_out, col.ptr, ld_col, ptr, ncols, accumulate=acc)
                if col is not None:
                    col.free()
                    col = None
                if x.requires_grad:
                    with temp_storage(rows * ld_col * F32) as dcol:
                        _gemm.gemm(LAYOUT_NN, rows, ncols, C_out, dy.ptr, C_out, weight.ptr, ncols, dcol.ptr, ld_col)
                        fresh = x.grad is None
                        if fresh:
                            x.grad = empty_tensor(x.shape)
                        _call("gt_col2im", _vp(x.grad.ptr), _vp(dcol.ptr), ld_col, N, C_in, H, W, kH, kW, stride, padding,
                              0 if fresh else 1)

        out._set_graph(parents=(self, weight, bias), backward_fn=_backward)
        return out

    def maxpool2d(self, kernel_size=2, stride=None) -> "Tensor":
        """2D max pooling (N, C, H, W) -> (N, C, H_out, W_out); the stride defaults to the kernel size
        (gradtuity/tensor.py:2169-2260)."""
        x = self
        if x.ndim != 4:
            raise ValueError(f"maxpool2d requires 4D input, got shape {x._shape}")
        kH, kW = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        if stride is None:
            sh = sw = kH
        elif isinstance(stride, int):
            sh = sw = stride
        else:
            sh, sw = stride
        N, C, H, W = x._shape
        H_out = (H - kH) // sh + 1
        W_out = (W - kW) // sw + 1
        if H_out <= 0 or W_out <= 0:
            raise ValueError(f"maxpool2d output size invalid: H_out={H_out}, W_out={W_out}")
        out = empty_tensor((N, C, H_out, W_out))
        idx = alloc_storage(out.numel * F32)
        _call("gt_maxpool2d", _vp(out.ptr), _vp(idx.ptr), _vp(x.ptr), N, C, H, W, kH, kW, sh, sw)

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                ensure_grad(x)
                _call("gt_maxpool2d_backward", _vp(x.grad.ptr), _vp(g.ptr), _vp(idx.ptr), N * C, H * W, H_out * W_out)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def transpose4d_12(self) -> "Tensor":
        """(B, d1, d2, D) -> (B, d2, d1, D), materialised (gradtuity/tensor.py:1227-1260)."""
        if self.ndim != 4:
            raise ValueError(f"transpose4d_12 requires ndim=4, got ndim={self.ndim}")
        Bn, d1, d2, D = self._shape
        out = empty_tensor((Bn, d2, d1, D))
        _call("gt_transpose12", _vp(out.ptr), _vp(self.ptr), Bn, d1, d2, D, 0)
        x = self

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                ensure_grad(x)
                _call("gt_transpose12", _vp(x.grad.ptr), _vp(g.ptr), Bn, d2, d1, D, 1)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def transpose4d_last2(self) -> "Tensor":
        """(B, H, M, N) -> (B, H, N, M), materialised (gradtuity/tensor.py:1190-1225)."""
        if self.ndim != 4:
            raise ValueError(f"transpose4d_last2 requires ndim=4, got ndim={self.ndim}")
        Bn, Hn, Mr, Nc = self._shape
        out = empty_tensor((Bn, Hn, Nc, Mr))
        # rows of one element: (B*H, M, N, 1) -> (B*H, N, M, 1)
        _call("gt_transpose12", _vp(out.ptr), _vp(self.ptr), Bn * Hn, Mr, Nc, 1, 0)
        x = self

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                ensure_grad(x)
                _call("gt_transpose12", _vp(x.grad.ptr), _vp(g.ptr), Bn * Hn, Nc, Mr, 1, 1)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def scale_inplace(self, scalar: float) -> "Tensor":
        """x *= scalar in the same buffer, as a graph node (gradtuity/tensor.py:2395-2427)."""
        _call("gt_scale", _vp(self.ptr), _vp(self.ptr), float(scalar), self.numel, 0)
        out = Tensor._from_ptr(self.ptr, self._shape, owns_memory=False, base=self._st)
        x = self
        s = float(scalar)

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                ensure_grad(x)
                _call("gt_scale", _vp(x.grad.ptr), _vp(g.ptr), s, x.numel, 1)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def mse_loss(self, target: "Tensor") -> "Tensor":
        """mean((self - target)^2) as a (1,) tensor (gradtuity/tensor.py:1390-1450)."""
        if self.shape != target.shape:
            raise ValueError(f"mse_loss shape mismatch: {self.shape} vs {target.shape}")
        diff = self.add(target.scale(-1.0))
        return diff.mul(diff).sum().scale(1.0 / self.numel)

    # ---- element-wise ops beside the GEMMs ------------------------------------------------

    def add(self, other: "Tensor") -> "Tensor":
        if self.shape != other.shape:
            raise ValueError(f"Shape mismatch for add: {self.shape} vs {other.shape}")
        out = empty_tensor(self.shape)
        _call("gt_add", _vp(out.ptr), _vp(self.ptr), _vp(other.ptr), self.numel, 0)
        a, b = self, other

        def _backward(g: "Tensor") -> None:
            if a.requires_grad:
                pass_grad(a, g)          # may take over g's buffer
            if b.requires_grad:
                accum_grad(b, g)         # always a copy / accumulate

        out._set_graph(parents=(self, other), backward_fn=_backward)
        return out

    def relu(self) -> "Tensor":
        out = empty_tensor(self.shape)
        _call("gt_relu", _vp(out.ptr), _vp(self.ptr), self.numel)
        x = self

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                ensure_grad(x)
                _call("gt_relu_mask_mul", _vp(x.grad.ptr), _vp(g.ptr), _vp(x.ptr), x.numel, 1)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def gelu(self, approx: str = "tanh") -> "Tensor":
        if approx != "tanh":
            raise ValueError(f'gelu approx must be "tanh" in v1, got {approx!r}')
        out = empty_tensor(self.shape)
        _call("gt_gelu", _vp(out.ptr), _vp(self.ptr), self.numel)
        x = self

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                ensure_grad(x)
                _call("gt_gelu_backward", _vp(x.grad.ptr), _vp(g.ptr), _vp(x.ptr), x.numel, 1)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def sum(self) -> "Tensor":
        """Sum of all elements as a (1,) tensor (gradtuity/tensor.py:1368-1388)."""
        out = empty_tensor((1,))
        _call("gt_sum_all", _vp(out.ptr), _vp(self.ptr), self.numel, 0)
        src = self

        def _backward(g: "Tensor") -> None:
            if src.requires_grad:
                ensure_grad(src)
                _call("gt_add_scalar", _vp(src.grad.ptr), _vp(g.ptr), src.numel)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def add_bias(self, bias: "Tensor") -> "Tensor":
        if self.ndim != 2:
            raise ValueError(f"add_bias requires 2D input, got shape {self._shape}")
        if bias.ndim != 1:
            raise ValueError(f"bias must be 1D, got shape {bias._shape}")
        if self._shape[1] != bias._shape[0]:
            raise ValueError(f"Bias size {bias._shape[0]} doesn't match input features {self._shape[1]}")
        rows, cols = self._shape
        out = empty_tensor(self.shape)
        _call("gt_add_bias", _vp(out.ptr), _vp(self.ptr), _vp(bias.ptr), rows, cols)
        x = self

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                accum_grad(x, g)
            if bias.requires_grad:
                ensure_grad(bias)
                _call("gt_colsum_acc", _vp(bias.grad.ptr), _vp(g.ptr), rows, cols, cols)

        out._set_graph(parents=(self, bias), backward_fn=_backward)
        return out

    def mul(self, other: "Tensor") -> "Tensor":
        if self.shape != other.shape:
            raise ValueError(f"Shape mismatch for mul: {self.shape} vs {other.shape}")
        out = empty_tensor(self.shape)
        _call("gt_mul", _vp(out.ptr), _vp(self.ptr), _vp(other.ptr), self.numel, 0)
        a, b = self, other

        def _backward(g: "Tensor") -> None:
            if a.requires_grad:
                ensure_grad(a)
                _call("gt_mul", _vp(a.grad.ptr), _vp(g.ptr), _vp(b.ptr), a.numel, 1)
            if b.requires_grad:
                ensure_grad(b)
                _call("gt_mul", _vp(b.grad.ptr), _vp(g.ptr), _vp(a.ptr), b.numel, 1)

        out._set_graph(parents=(self, other), backward_fn=_backward)
        return out

    def scale(self, scalar: float) -> "Tensor":
        out = empty_tensor(self.shape)
        _call("gt_scale", _vp(out.ptr), _vp(self.ptr), float(scalar), self.numel, 0)
        x = self
        s = float(scalar)

        def _backward(g: "Tensor") -> None:
            if x.requires_grad:
                ensure_grad(x)
                _call("gt_scale", _vp(x.grad.ptr), _vp(g.ptr), s, x.numel, 1)

        out._set_graph(parents=(self,), backward_fn=_backward)
        return out

    def mul_scalar_inplace_(self, scalar: float) -> None:
        _call("gt_scale", _vp(self.ptr), _vp(self.ptr), float(scalar), self.numel, 0)

    def __add__(self, other: "Tensor") -> "Tensor":
        return self.add(other)

    def __radd__(self, other: "Tensor") -> "Tensor":
        return other.add(self)

    def __mul__(self, other):
        if isinstance(other, Tensor):
            return self.mul(other)
        return self.scale(float(other))

    def __rmul__(self, other):
        return self.__mul__(other)

    def __neg__(self) -> "Tensor":
        return self.scale(-1.0)

    def __sub__(self, other: "Tensor") -> "Tensor":
        return self.add(other.scale(-1.0))

    def __rsub__(self, other: "Tensor") -> "Tensor":
        return other.add(self.scale(-1.0))

    # ---- host access --------------------------------------------------------------------

    def to_list(self) -> list:
        host = cuda_memcpy_dtoh(self.ptr, self.numel * F32)
        flat = list(struct.unpack(f"{self.numel}f", host))
        return self._unflatten(flat, self._shape)

    def item(self) -> float:
        if self.numel != 1:
            raise ValueError(f"item() only works for single-element tensors, got {self.numel} elements")
        return struct.unpack("f", cuda_memcpy_dtoh(self.ptr, F32))[0]

    def __repr__(self) -> str:
        g = ", requires_grad=True" if self.requires_grad else ""
        n = f", name={self.name!r}" if self.name else ""
        return f"Tensor(shape={self._shape}{g}{n})"

    # ---- nested-list plumbing -----------------------------------------------------------

    @staticmethod
    def _infer_shape_and_flatten(data) -> tuple[tuple[int, ...], list[float]]:
        shape: list[int] = []
        probe = data
        while isinstance(probe, (list, tuple)):
            shape.append(len(probe))
            if len(probe) == 0:
                break
            probe = probe[0]
        flat: list[float] = []

        def walk(x, depth: int) -> None:
            if depth == len(shape):
                if isinstance(x, (list, tuple)):
                    raise ValueError("Inconsistent nesting depth in tensor data")
                flat.append(float(x))
                return
            if not isinstance(x, (list, tuple)) or len(x) != shape[depth]:
                raise ValueError(f"Inconsistent shape at depth {depth}: expected length {shape[depth]}")
            for y in x:
                walk(y, depth + 1)

        walk(data, 0)
        return tuple(shape), flat

    @staticmethod
    def _flatten(data) -> list[float]:
        if not isinstance(data, (list, tuple)):
            return [float(data)]
        out: list[float] = []
        stack = [iter(data)]
        while stack:
            try:
                x = next(stack[-1])
            except StopIteration:
                stack.pop()
                continue
            if isinstance(x, (list, tuple)):
                stack.append(iter(x))
            else:
                out.append(float(x))
        return out

    @staticmethod
    def _unflatten(flat: list[float], shape: tuple[int, ...]) -> list:
        if len(shape) == 1:
            return list(flat)
        step = prod(shape[1:])
        return [Tensor._unflatten(flat[i * step:(i + 1) * step], shape[1:]) for i in range(shape[0])]
