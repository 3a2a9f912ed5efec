"""One-time broadcast of the initial parameters from one rank, with the strict signature check
of gradtuity/dist/init_sync.py:38-104: (num_tensors, total_numel) travel first as 16 raw bytes
and every rank compares them with its own before any parameter is overwritten.  Unlike the
reference, the verdict is then shared (one all-reduced flag), so a mismatch raises on every rank
instead of leaving the matching ranks blocked in the parameter broadcasts."""
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
    for t in tensors:
        backend.broadcast(t.ptr, t.numel, src)
    backend.wait(host_sync=True)
