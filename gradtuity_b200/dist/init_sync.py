"""One-time broadcast of the initial parameters from one rank, with the strict signature check
of gradtuity/dist/init_sync.py:38-104: (num_tensors, total_numel) travel first as 16 raw bytes
and every rank compares them with its own before any parameter is overwritten.  Unlike the
reference, the verdict is then shared (one all-reduced flag), so a mismatch raises on every rank
instead of leaving the matching ranks blocked in the parameter broadcasts.

The parameters then travel in ONE broadcast: they are first moved into a single flat arena (each parameter
keeps its Tensor object, name, shape and values; only its storage becomes a slice of the arena), where the
reference issues one ncclBroadcast per tensor (196 for GPT-2-small, gradtuity/dist/init_sync.py:88-104)."""
from __future__ import annotations

import os
import struct

from . import comm
from . import env as dist_env


def _extract_params_and_buffers(model_or_params, sync_buffers: bool) -> tuple[list, list]:
    if isinstance(model_or_params, (list, tuple)):
        return list(model_or_params), []
    params = list(model_or_params.parameters())
    buffers = list(model_or_params.buffers()) if sync_buffers and hasattr(model_or_params, "buffers") else []
    return params, buffers


ARENA_ALIGN_ELEMS = 64          # every parameter starts on a 256-byte boundary


def arena_layout(params: list) -> tuple[list[int], list[int], int]:
    """(order, offsets, total) for the flat parameter arena.  `order` lists indices into `params`: the list order,
    except that parameters which already share one allocation (the packed q / k / v weights of an attention layer)
    are placed together, in address order, at the position of the first of them, so that their adjacency
    survives the move.  `offsets[i]` is the element offset of params[order[i]]."""
    def owner(t):
        st = t._st
        return id(st.base) if getattr(st, "base", None) is not None else id(st)

    groups: dict[int, list[int]] = {}
    for i, t in enumerate(params):
        groups.setdefault(owner(t), []).append(i)
    order, seen = [], set()
    for i, t in enumerate(params):
        if i in seen:
            continue
        members = sorted(groups[owner(t)], key=lambda j: params[j]._st.ptr)
        for j in members:
            if j not in seen:
                seen.add(j)
                order.append(j)
    offsets, pos = [], 0
    for j in order:
        offsets.append(pos)
        n = params[j].numel
        pos += (n + ARENA_ALIGN_ELEMS - 1) // ARENA_ALIGN_ELEMS * ARENA_ALIGN_ELEMS
    return order, offsets, pos


class DeviceArenaOps:
    """How flatten_parameters touches memory (tests substitute host arrays)."""

    def alloc(self, numel: int):
        from ..tensor import Tensor

        return Tensor._zeros((numel,))

    def copy(self, dst_ptr: int, src_ptr: int, nbytes: int) -> None:
        from ..cuda_mem import cuda_memcpy_dtod

        cuda_memcpy_dtod(dst_ptr, src_ptr, nbytes)

    def whole(self, base, numel: int):
        from ..tensor import Tensor

        return Tensor._from_ptr(base.ptr, (numel,), owns_memory=False, base=base)

    def rebind(self, t, arena, offset_elems: int) -> None:
        from ..tensor import Storage

        t._st = Storage(arena.ptr + 4 * offset_elems, 4 * t.numel, owns=False, base=arena._st)


def flatten_parameters(params: list, mem=None):
    """Move every parameter into one allocation and return it (a 1-D tensor; the parameters keep it alive).
    Tensor objects are kept, so optimizers, state dicts and the tied LM head see no change.  A parameter list
    that already is one arena laid out this way is left alone and its arena returned."""
    mem = mem or DeviceArenaOps()
    params = [t for i, t in enumerate(params) if all(t is not u for u in params[:i])]      # a tied tensor once
    order, offsets, total = arena_layout(params)
    base = getattr(params[order[0]]._st, "base", None)
    if base is not None and base.nbytes == 4 * max(total, 1) and all(
            getattr(params[j]._st, "base", None) is base and params[j]._st.ptr == base.ptr + 4 * off for j, off in zip(order, offsets)):
        return mem.whole(base, max(total, 1))         # already one arena with this layout
    for t in params:
        if getattr(t, "_pitch", None) is not None:
            t.ptr                                     # pack padded rows first
    arena = mem.alloc(max(total, 1))
    for j, off in zip(order, offsets):
        t = params[j]
        mem.copy(arena.ptr + 4 * off, t._st.ptr, 4 * t.numel)
    for j, off in zip(order, offsets):
        mem.rebind(params[j], arena, off)
    return arena


_arena_ops = None               # tests may install host memory ops


def init_sync(model_or_params, *, src: int = 0, sync_buffers: bool = True, bucket_mb: float = 25.0, strict: bool = True) -> None:
    _ = bucket_mb
    world = dist_env.get_world_size()
    if world == 1:
        return
    rank = dist_env.get_rank()
    if not (0 <= src < world):
        raise ValueError(f"init_sync src must be in [0, {world}), got {src}")
    params, buffers = _extract_params_and_buffers(model_or_params, sync_buffers)
    tensors = params + buffers
    num_tensors = len(tensors)
    total_numel = sum(t.numel for t in tensors)
    if os.environ.get("GRADTUITY_DIST_DEBUG_INIT_SYNC") == "1" and rank == 0:
        print(f"init_sync: broadcasting {num_tensors} params (total numel {total_numel})")
    backend = comm._require()
    if strict:
        from ..cuda_mem import cuda_memcpy_dtoh, cuda_memcpy_htod
        from ..tensor import Tensor

        sig = Tensor._zeros((4,))                       # 16 bytes: two int64, moved as raw bits
        if rank == src:
            cuda_memcpy_htod(sig.ptr, struct.pack("qq", num_tensors, total_numel))
        backend.broadcast(sig.ptr, 4, src)
        backend.wait(host_sync=True)
        root_tensors, root_numel = struct.unpack("qq", cuda_memcpy_dtoh(sig.ptr, 16))
        mismatch = num_tensors != root_tensors or total_numel != root_numel
        # Every rank learns whether ANY rank disagrees before a single parameter is sent, so that
        # all of them stop here together and none is left waiting inside a collective.
        flag = Tensor.from_numpy([1.0 if mismatch else 0.0])
        backend.allreduce_async(flag.ptr, 1, average=False)
        backend.wait(host_sync=True)
        if flag.item() > 0:
            raise RuntimeError(
                f"init_sync strict check failed: rank {rank} has num_tensors={num_tensors} total_numel={total_numel}, "
                f"root has num_tensors={root_tensors} total_numel={root_numel}. Ensure same model architecture and "
                "parameter order on all ranks."
            )
    if params:
        arena = flatten_parameters(params, mem=_arena_ops)
        backend.broadcast(arena.ptr, arena.numel, src)            # one collective for every parameter
    for t in buffers:
        backend.broadcast(t.ptr, t.numel, src)
    backend.wait(host_sync=True)
