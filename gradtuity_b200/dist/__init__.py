"""Single-node data parallelism over NCCL, with the reference's entry points
(gradtuity/dist/__init__.py): init, destroy_process_group, sync_grads, init_sync, barrier,
get_rank / get_world_size / get_local_rank / get_master_addr / get_master_port / get_env_ranks,
distributed_indices, shard_size, print_rank."""
from __future__ import annotations

from . import comm, ddp, sampler
from . import env as _env
from . import init_sync as _init_sync

get_rank = _env.get_rank
get_world_size = _env.get_world_size
get_local_rank = _env.get_local_rank
get_master_addr = _env.get_master_addr
get_master_port = _env.get_master_port
get_env_ranks = _env.get_env_ranks


def init() -> None:
    comm.init_process_group()


def destroy_process_group() -> None:
    ddp.reset()
    comm.destroy_process_group()


def barrier() -> None:
    comm.barrier()


def sync_grads(params: list, bucket_mb: float = ddp.DEFAULT_BUCKET_MB) -> None:
    ddp.sync_grads(params, bucket_mb=bucket_mb)


def init_sync(model_or_params, *, src: int = 0, sync_buffers: bool = True, bucket_mb: float = 25.0, strict: bool = True) -> None:
    _init_sync.init_sync(model_or_params, src=src, sync_buffers=sync_buffers, bucket_mb=bucket_mb, strict=strict)


def print_rank(message: str = "", ranks: list[int] = [0], **kwargs) -> None:
    if get_rank() in ranks:
        print(message, **kwargs)


no_sync = ddp.no_sync            # added: backward calls inside it send no gradient buckets
distributed_indices = sampler.distributed_indices
shard_size = sampler.shard_size

__all__ = ["init", "destroy_process_group", "sync_grads", "init_sync", "get_rank", "get_world_size", "get_local_rank",
           "get_master_addr", "get_master_port", "get_env_ranks", "barrier", "distributed_indices", "shard_size", "print_rank", "no_sync"]
