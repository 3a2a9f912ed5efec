"""Host stand-ins for the pieces of the gradient exchange that touch the GPU, so that the
bucketing, arena and overlap logic of gradtuity_b200.dist.ddp can run in CPU processes:
numpy-backed tensors, numpy memory ops, and a communicator over torch.distributed's gloo."""
import ctypes

import numpy as np


class FakeTensor:
    def __init__(self, array, requires_grad=False):
        self.array = np.ascontiguousarray(array, dtype=np.float32)
        self.requires_grad = requires_grad
        self.grad = None
        self._parents = ()
        self._st = self

    @property
    def ptr(self):
        return self.array.ctypes.data

    @property
    def numel(self):
        return self.array.size

    @property
    def shape(self):
        return self.array.shape


def as_array(ptr, numel):
    return np.ctypeslib.as_array((ctypes.c_float * numel).from_address(ptr))


class HostMemoryOps:
    def alloc_zeroed(self, numel):
        return FakeTensor(np.zeros(numel, np.float32))

    def ensure_grad(self, p):
        if p.grad is None:
            p.grad = FakeTensor(np.zeros(p.shape, np.float32))

    def copy(self, dst_ptr, src_ptr, nbytes):
        ctypes.memmove(dst_ptr, src_ptr, nbytes)

    def alloc(self, numel):
        return FakeTensor(np.zeros(numel, np.float32))

    def scatter_rows(self, dw_ptr, rows_ptr, idx_ptr, n, d, v, alpha):
        dw = as_array(dw_ptr, v * d).reshape(v, d)
        rows = as_array(rows_ptr, n * d).reshape(n, d)
        idx = as_array(idx_ptr, n).astype(np.int64)
        np.add.at(dw, idx, alpha * rows)

    def view(self, arena, offset_elems, shape):
        n = int(np.prod(shape))
        v = FakeTensor.__new__(FakeTensor)
        v.array = arena.array[offset_elems:offset_elems + n].reshape(shape)     # shares the arena's memory
        v.requires_grad = False
        v.grad = None
        v._parents = ()
        v._st = arena
        return v


class RecordingBackend:
    """Single-process communicator that records calls; 'all-reduce' multiplies by a constant so
    that a test can see which ranges were touched and how often."""

    def __init__(self, world_size=2):
        self.world_size = world_size
        self.calls = []
        self.waits = 0

    def allreduce_async(self, ptr, numel, average):
        self.calls.append((ptr, numel, average))
        as_array(ptr, numel)[:] *= 10.0

    def broadcast(self, ptr, numel, src):
        self.calls.append(("bcast", ptr, numel, src))

    def allgather_async(self, dst_ptr, src_ptr, numel):
        self.calls.append(("gather", dst_ptr, src_ptr, numel))
        for r in range(self.world_size):                       # every "rank" holds this process's values
            as_array(dst_ptr, self.world_size * numel)[r * numel:(r + 1) * numel] = as_array(src_ptr, numel)

    def wait(self, host_sync=False):
        self.waits += 1


class GlooBackend:
    """All-reduce over torch.distributed (gloo) on host memory addressed by raw pointers."""

    def __init__(self):
        import torch.distributed as dist

        self.dist = dist
        self.world_size = dist.get_world_size()

    def allreduce_async(self, ptr, numel, average):
        import torch

        t = torch.from_numpy(as_array(ptr, numel))
        self.dist.all_reduce(t)
        if average:
            t /= self.world_size

    def broadcast(self, ptr, numel, src):
        import torch

        self.dist.broadcast(torch.from_numpy(as_array(ptr, numel)), src)

    def allgather_async(self, dst_ptr, src_ptr, numel):
        import torch

        out = torch.from_numpy(as_array(dst_ptr, self.world_size * numel))
        self.dist.all_gather(list(out.chunk(self.world_size)), torch.from_numpy(as_array(src_ptr, numel).copy()))

    def wait(self, host_sync=False):
        pass


class HostArenaOps:
    """Host stand-in for gradtuity_b200.dist.init_sync.DeviceArenaOps: parameters are FakeTensors whose
    `_st` is a small storage record (ptr, nbytes, base), the arena a numpy array."""

    class St:
        def __init__(self, array, base=None):
            self.array = array
            self.ptr = array.ctypes.data
            self.nbytes = array.nbytes
            self.base = base
            self.owns = base is None

    def alloc(self, numel):
        t = FakeTensor(np.zeros(numel, np.float32))
        t._st = HostArenaOps.St(t.array)
        return t

    def copy(self, dst_ptr, src_ptr, nbytes):
        ctypes.memmove(dst_ptr, src_ptr, nbytes)

    def whole(self, base, numel):
        t = FakeTensor.__new__(FakeTensor)
        t.array = base.array[:numel]
        t.requires_grad, t.grad, t._parents, t._st = False, None, (), base
        return t

    def rebind(self, t, arena, offset_elems):
        n = t.numel
        shape = t.shape
        t.array = arena.array[offset_elems:offset_elems + n].reshape(shape)
        t._st = HostArenaOps.St(t.array, base=arena._st)


def host_param(array, base=None):
    """A FakeTensor parameter with a storage record, optionally a view into `base` (another host_param's storage)."""
    t = FakeTensor(array, requires_grad=True)
    t._st = HostArenaOps.St(t.array, base=base)
    return t
