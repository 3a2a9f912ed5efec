"""Index sharding across ranks (gradtuity/dist/sampler.py:13-41): rank r takes r, r + W, r + 2W, ..."""
from __future__ import annotations

from . import env as dist_env


def distributed_indices(num_samples: int) -> range:
    return range(dist_env.get_rank(), num_samples, dist_env.get_world_size())


def shard_size(num_samples: int) -> int:
    return len(distributed_indices(num_samples))
