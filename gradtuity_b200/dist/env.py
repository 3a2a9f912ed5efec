"""Rank / world-size discovery from the environment, as gradtuity/dist/env.py:14-110:
RANK / WORLD_SIZE / LOCAL_RANK (or the SLURM equivalents) and MASTER_ADDR / MASTER_PORT."""
from __future__ import annotations

import os


def _first(names: tuple[str, ...], what: str) -> str:
    for n in names:
        v = os.environ.get(n)
        if v is not None:
            return v
    raise RuntimeError(f"{what} not set. Set {' or '.join(names)}.")


def get_rank() -> int:
    return int(_first(("RANK", "SLURM_PROCID"), "Distributed rank"))


def get_world_size() -> int:
    return int(_first(("WORLD_SIZE", "SLURM_NTASKS"), "World size"))


def get_local_rank() -> int:
    return int(_first(("LOCAL_RANK", "SLURM_LOCALID"), "Local rank"))


def get_master_addr() -> str:
    return _first(("MASTER_ADDR",), "Master address")


def get_master_port() -> str:
    return _first(("MASTER_PORT",), "Master port")


def get_env_ranks() -> tuple[int, int, int, str, str]:
    return (get_rank(), get_world_size(), get_local_rank(), get_master_addr(), get_master_port())
