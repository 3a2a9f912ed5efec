"""Process group: device selection, unique-id rendezvous, communicator, collectives.

Same functions and behaviour as gradtuity/dist/comm.py:23-170 (`init_process_group`,
`destroy_process_group`, `allreduce_inplace`, `broadcast`, `barrier`, file-based exchange of the
128-byte NCCL unique id with a 60 s timeout and the same diagnostics), but the collectives go
through libgt_b200.so's `gt_dist_*` entry points: they run on a communication stream ordered by
events, not between device-wide synchronisations on the NULL stream.

`Backend` is the seam the gradient exchange talks to.  `NcclBackend` is the product;
tests substitute a host backend to exercise the bucketing and overlap logic without GPUs.
"""
from __future__ import annotations

import os
import time
from ctypes import c_void_p, create_string_buffer

from . import env as dist_env

NCCL_UNIQUE_ID_BYTES = 128
RENDEZVOUS_TIMEOUT_S = 60.0


class Backend:
    """What sync_grads needs from a communicator."""

    world_size = 1

    def allreduce_async(self, ptr: int, numel: int, average: bool) -> None:
        raise NotImplementedError

    def broadcast(self, ptr: int, numel: int, src: int) -> None:
        raise NotImplementedError

    def allgather_async(self, dst_ptr: int, src_ptr: int, numel: int) -> None:
        """dst (world_size x numel floats) = every rank's numel floats at src, in rank order."""
        raise NotImplementedError

    def wait(self, host_sync: bool = False) -> None:
        raise NotImplementedError


class NcclBackend(Backend):
    def __init__(self, rank: int, world_size: int, uid: bytes) -> None:
        from .. import _lib

        self._lib = _lib
        self.rank, self.world_size = rank, world_size
        lib = _lib.load_library()
        _lib.check(lib.gt_dist_init(_lib.context(), rank, world_size, uid), "gt_dist_init")

    def allreduce_async(self, ptr: int, numel: int, average: bool) -> None:
        lib = self._lib.load_library()
        self._lib.check(lib.gt_dist_allreduce(self._lib.context(), c_void_p(ptr), numel, 1 if average else 0), "gt_dist_allreduce")

    def broadcast(self, ptr: int, numel: int, src: int) -> None:
        lib = self._lib.load_library()
        self._lib.check(lib.gt_dist_broadcast(self._lib.context(), c_void_p(ptr), numel, src), "gt_dist_broadcast")

    def allgather_async(self, dst_ptr: int, src_ptr: int, numel: int) -> None:
        lib = self._lib.load_library()
        self._lib.check(lib.gt_dist_allgather(self._lib.context(), c_void_p(dst_ptr), c_void_p(src_ptr), numel), "gt_dist_allgather")

    def wait(self, host_sync: bool = False) -> None:
        lib = self._lib.load_library()
        self._lib.check(lib.gt_dist_wait(self._lib.context(), 1 if host_sync else 0), "gt_dist_wait")

    def timeline(self) -> list[tuple[int, float, float, float]]:
        """Collectives between the last two waits as (elements, enqueue ms, start ms, end ms), then a row
        (0, compute-stream resume ms, 0, 0); empty unless GRADTUITY_DIST_TIMELINE=1 was set before init()."""
        from ctypes import byref, c_float, c_int

        buf = (c_float * (4 * 80))()
        n = c_int(0)
        self._lib.check(self._lib.load_library().gt_dist_timeline(self._lib.context(), buf, 80, byref(n)), "gt_dist_timeline")
        return [(int(buf[4 * i]), buf[4 * i + 1], buf[4 * i + 2], buf[4 * i + 3]) for i in range(n.value)]

    def destroy(self) -> None:
        self._lib.load_library().gt_dist_destroy(self._lib.context())


_backend: Backend | None = None


def _unique_id_file() -> str:
    """Path of the unique-id file (gradtuity/dist/comm.py:23-34)."""
    path = os.environ.get("GRADTUITY_NCCL_UID_FILE")
    if path is not None:
        return path
    job = os.environ.get("SLURM_JOB_ID")
    if job is not None:
        return f"/tmp/gradtuity_nccl_{job}.bin"
    # Launcher-less single-node runs: every rank derives the same name from the rendezvous address.
    addr, port = os.environ.get("MASTER_ADDR"), os.environ.get("MASTER_PORT")
    if addr is not None and port is not None:
        return f"/tmp/gradtuity_nccl_{addr}_{port}.bin"
    return f"/tmp/gradtuity_nccl_{os.getpid()}_{int(time.time())}.bin"


def exchange_unique_id(rank: int, make_id, uid_file: str, timeout: float = RENDEZVOUS_TIMEOUT_S,
                       not_before: float | None = None) -> bytes:
    """Rank 0 writes the id produced by make_id() to uid_file; the others poll for it.
    not_before: files last modified before this time (a leftover of an earlier job that used the
    same path) are ignored."""
    if rank == 0:
        uid = make_id()
        if len(uid) != NCCL_UNIQUE_ID_BYTES:
            raise RuntimeError(f"unique id has {len(uid)} bytes, expected {NCCL_UNIQUE_ID_BYTES}")
        tmp = uid_file + ".tmp"
        with open(tmp, "wb") as f:
            f.write(uid)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, uid_file)
        return uid
    start = time.monotonic()
    def ready() -> bool:
        try:
            st = os.stat(uid_file)
        except OSError:
            return False
        return st.st_size == NCCL_UNIQUE_ID_BYTES and (not_before is None or st.st_mtime >= not_before)

    while not ready():
        if time.monotonic() - start > timeout:
            exists = os.path.isfile(uid_file)
            raise RuntimeError(
                f"Rank {rank}: UniqueId file {uid_file!r} did not reach {NCCL_UNIQUE_ID_BYTES} bytes within {timeout}s "
                f"(file exists={exists}, size={os.path.getsize(uid_file) if exists else 0}). "
                "Ensure rank 0 is running and GRADTUITY_NCCL_UID_FILE is the same on all ranks."
            )
        time.sleep(0.01)
    with open(uid_file, "rb") as f:
        uid = f.read()
    if len(uid) != NCCL_UNIQUE_ID_BYTES:
        raise RuntimeError(f"Rank {rank}: read {len(uid)} bytes from {uid_file!r}, expected {NCCL_UNIQUE_ID_BYTES}.")
    return uid


def _make_nccl_id() -> bytes:
    from .. import _lib

    buf = create_string_buffer(NCCL_UNIQUE_ID_BYTES)
    _lib.check(_lib.load_library().gt_dist_get_unique_id(_lib.context(), buf), "gt_dist_get_unique_id")
    return buf.raw


def init_process_group() -> None:
    """Bind this process to GPU LOCAL_RANK and create the communicator (no-op group at world size 1)."""
    global _backend
    if _backend is not None:
        return
    rank, world, local = dist_env.get_rank(), dist_env.get_world_size(), dist_env.get_local_rank()
    os.environ.setdefault("GRADTUITY_DEVICE", str(local))
    if world == 1:
        return
    uid_file = _unique_id_file()
    # Under the launcher the file name is unique to the job; otherwise guard against a leftover.
    fresh = None if os.environ.get("GRADTUITY_LAUNCHER") == "1" else time.time() - 120.0
    uid = exchange_unique_id(rank, _make_nccl_id, uid_file, not_before=fresh)
    _backend = NcclBackend(rank, world, uid)
    barrier()
    if rank == 0:
        try:
            os.remove(uid_file)
        except OSError:
            pass


def set_backend(backend: Backend | None) -> None:
    """Install a communicator object directly (tests)."""
    global _backend
    _backend = backend


def get_backend() -> Backend | None:
    return _backend


def destroy_process_group() -> None:
    global _backend
    if _backend is not None and hasattr(_backend, "destroy"):
        _backend.destroy()
    _backend = None


def _require() -> Backend:
    if _backend is None:
        raise RuntimeError("Process group not initialized; call init() first")
    return _backend


def allreduce_inplace(ptr: int, numel: int) -> None:
    """In-place sum of numel floats at ptr over all ranks; complete when this returns to the
    compute stream's point of view."""
    if _backend is None and dist_env.get_world_size() == 1:
        return
    b = _require()
    b.allreduce_async(ptr, numel, average=False)
    b.wait()


def broadcast(ptr: int, numel: int, src: int = 0) -> None:
    if dist_env.get_world_size() == 1:
        return
    b = _require()
    b.broadcast(ptr, numel, src)
    b.wait()


def barrier() -> None:
    """All ranks meet (all-reduce of one float, then a host wait), gradtuity/dist/comm.py:155-170."""
    if dist_env.get_world_size() == 1:
        return
    b = _require()
    if isinstance(b, NcclBackend):
        from ..tensor import Tensor

        t = Tensor._zeros((1,))
        b.allreduce_async(t.ptr, 1, average=False)
        b.wait(host_sync=True)
    else:
        b.wait(host_sync=True)
