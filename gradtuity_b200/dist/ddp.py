"""Gradient synchronisation for data parallelism: `sync_grads(params, bucket_mb=100)`.

Same call, same meaning and the same bucket rule as gradtuity/dist/ddp.py:24-106 (consecutive
parameters are grouped until adding the next one would exceed `bucket_mb`; GRADTUITY_BUCKET_MB
overrides it; the result is the mean over ranks; the default size is 100 MB instead of 25, which
changes no result).  What differs is how the buckets travel:

* the gradients of all parameters live in ONE flat arena (each `p.grad` becomes a view into it the
  first time `sync_grads` sees the list), so a bucket is a contiguous range that is all-reduced in
  place: no per-bucket cudaMalloc, no device-to-device pack and unpack, no separate scale kernel
  (the division by the world size is the collective's ncclAvg);
* from the second step on, `Tensor.backward()` reports every graph node it has finished; when the
  last consumer of the last parameter of a bucket has run, that bucket's all-reduce is enqueued on
  the communication stream at once, so it overlaps the rest of backward.  `sync_grads` then only
  enqueues what is left (parameters that were not in the graph) and makes the compute stream wait.

The API does not change: `sync_grads` is still called after `backward()` (gpt2/train.py:127-128).

Several backward calls per sync (gradient accumulation, two losses).  Only the FIRST backward after a
`sync_grads` sends buckets early; any further backward before the next `sync_grads` first makes the
compute stream wait for the collectives already in flight (its `grad +=` kernels write the same arena),
sends nothing itself, and `sync_grads` then reduces every bucket again.  Averaging is linear, so a bucket
that was averaged after the first backward and then received local additions still ends as the mean over
ranks of the summed gradients.  A backward that is never followed by `sync_grads` (a "no sync" micro-step,
where the reference does not communicate at all) must run inside `no_sync()`, which keeps it from sending.
"""
from __future__ import annotations

import os

from . import comm
from . import env as dist_env

F32 = 4
ARENA_ALIGN_ELEMS = 64          # 256-byte alignment of every gradient inside the arena
# The reference's default is 25 MB (gradtuity/dist/ddp.py:24).  Bucket boundaries do not change any result; on NVLink a
# GPT-2-small step has 16 all-reduces of 0.1-0.2 ms at 25 MB and 6 at 100 MB, and loses 0.35 ms less to them (2 GPUs).
DEFAULT_BUCKET_MB = 100
SPARSE_MIN_BYTES = 32 << 20     # embedding tables smaller than this are not worth a separate exchange of rows
# GRADTUITY_BUCKET_RAMP=3: the buckets at the front of the parameter list (the last ones backward completes) hold 1/8, 1/4,
# 1/2 of the bucket size, so that less is left to reduce when backward ends.  Measured on 2 GPUs: the wait behind the last
# node drops from 0.65 to 0.49 ms, the step time by no more than the run-to-run spread (17.6-17.7 ms either way): off.
BUCKET_RAMP = 0


def bucketize(nbytes_list: list[int], bucket_max_bytes: int, ramp: int = 0) -> list[list[int]]:
    """Indices of consecutive entries per bucket: a bucket is closed when the next entry would
    push it past bucket_max_bytes and it is not empty (gradtuity/dist/ddp.py:59-71).
    ramp > 0 (not in the reference): the first buckets of the list are smaller, bucket_max_bytes / 2^ramp, then twice
    that, and so on up to bucket_max_bytes (a bucket that is one oversized entry does not count).  The front of the
    parameter list is what backward finishes last, so these are the buckets whose all-reduce has little or nothing
    left to hide behind: the less they hold, the shorter the wait at the end of backward."""
    buckets: list[list[int]] = []
    cur: list[int] = []
    cur_bytes = 0
    level = max(int(ramp), 0)
    for i, n in enumerate(nbytes_list):
        limit = max(bucket_max_bytes >> level, 1)
        if cur_bytes + n > limit and cur:
            buckets.append(cur)
            if cur_bytes <= limit and level > 0:
                level -= 1
            cur, cur_bytes = [], 0
        cur.append(i)
        cur_bytes += n
    if cur:
        buckets.append(cur)
    return buckets


def arena_offsets(numels: list[int], align: int = ARENA_ALIGN_ELEMS) -> tuple[list[int], int]:
    """Element offset of every gradient in the flat arena, each aligned; and the arena size."""
    offs, pos = [], 0
    for n in numels:
        offs.append(pos)
        pos += (n + align - 1) // align * align
    return offs, pos


class DeviceMemoryOps:
    """How the plan touches memory; the product version works on GPU tensors."""

    def alloc_zeroed(self, numel: int):
        from ..tensor import Tensor

        return Tensor._zeros((numel,))

    def ensure_grad(self, p) -> None:
        from ..tensor import ensure_grad

        ensure_grad(p)

    def copy(self, dst_ptr: int, src_ptr: int, nbytes: int) -> None:
        from ..cuda_mem import cuda_memcpy_dtod

        cuda_memcpy_dtod(dst_ptr, src_ptr, nbytes)

    def view(self, arena, offset_elems: int, shape):
        from ..tensor import Tensor

        return Tensor._from_ptr(arena.ptr + offset_elems * F32, tuple(shape), owns_memory=False, base=arena._st)

    def alloc(self, numel: int):
        from ..tensor import empty_tensor

        return empty_tensor((numel,))

    def scatter_rows(self, dw_ptr: int, rows_ptr: int, idx_ptr: int, n: int, d: int, v: int, alpha: float) -> None:
        from ctypes import c_void_p

        from .. import _lib

        _lib.check(_lib.load_library().gt_embedding_backward_scaled(_lib.context(), c_void_p(dw_ptr), c_void_p(rows_ptr), c_void_p(idx_ptr),
                                                                  n, d, v, float(alpha)), "gt_embedding_backward_scaled")


class GradPlan:
    """Arena, views and buckets for one parameter list, plus the per-step readiness counters."""

    def __init__(self, params: list, bucket_max_bytes: int, mem=None) -> None:
        self.mem = mem or DeviceMemoryOps()
        self.params = list(params)
        self.index = {id(p): i for i, p in enumerate(self.params)}
        numels = [p.numel for p in self.params]
        self.offsets, total = arena_offsets(numels)
        self.arena = self.mem.alloc_zeroed(max(total, 1))
        if hasattr(self.arena, "_st"):
            self.arena._st.grads_only = True          # zero_grad may clear neighbouring gradients with one memset
        for p, off in zip(self.params, self.offsets):
            self.mem.ensure_grad(p)
            self.mem.copy(self.arena.ptr + off * F32, p.grad.ptr, p.numel * F32)
            p.grad = self.mem.view(self.arena, off, p.shape)
        self.views = [p.grad for p in self.params]
        self.buckets = bucketize([n * F32 for n in numels], bucket_max_bytes, int(os.environ.get("GRADTUITY_BUCKET_RAMP", BUCKET_RAMP)))
        self.bucket_of = {}
        self.ranges = []                                   # (ptr, numel) per bucket, padding included
        for b, idxs in enumerate(self.buckets):
            for i in idxs:
                self.bucket_of[i] = b
            start = self.offsets[idxs[0]]
            end = self.offsets[idxs[-1]] + numels[idxs[-1]]
            self.ranges.append((self.arena.ptr + start * F32, end - start))
        # per-step state
        self.armed = False          # set by finish(): the next backward (and only that one) may send early
        self.active = False
        self.launched: set[int] = set()
        self.launch_order: list[int] = []
        self._consumers: dict[int, int] = {}
        self._bucket_left: list[int] = []
        # Embedding tables whose gradient also has a dense part (the tied LM head): in an early-sending backward the
        # rows that the embedding backward would scatter into the table's gradient, the last node of the graph, are
        # kept aside instead, so that the table's bucket is final, and goes out, right after the dense part; finish()
        # gathers every rank's rows and adds them (divided by the world size) to the reduced gradient.
        self._defer: set[int] = set()                  # parameter indices whose embedding rows are kept aside in this backward
        self.deferred: list[tuple] = []                # (parameter index, indices tensor, rows tensor, n, D, V)

    def intact(self) -> bool:
        """True while every parameter's grad is still the arena view this plan installed."""
        return all(p.grad is v for p, v in zip(self.params, self.views))

    # ---- called by Tensor.backward() ------------------------------------------------------------
    def begin(self, topo: list) -> None:
        cons = {}
        for node in topo:
            for par in node._parents:
                i = self.index.get(id(par))
                if i is not None:
                    cons[i] = cons.get(i, 0) + 1
        if not cons:
            # a graph that touches none of this plan's parameters (another model, a metric): not our backward
            self.active = False
            return
        if self.launched:
            # a backward since the last sync_grads sent these buckets: this backward adds into the same
            # arena, so it must run behind them; finish() will reduce every bucket again
            comm._require().wait()
        self.launched.clear()
        self.launch_order.clear()
        self.active = self.armed and not _no_sync_depth and self.intact()
        self.armed = False
        if not self.active:
            return
        self._defer = set()
        self.deferred = []
        if os.environ.get("GRADTUITY_SPARSE_EMBED_SYNC", "0") == "1":          # measured neutral on 2 GPUs: opt-in
            for node in topo:
                w = getattr(node, "_embedding_of", None)
                i = self.index.get(id(w)) if w is not None else None
                # worth it for a table of at least 32 MB that has another (dense) consumer in the graph, when the rows of
                # all ranks together are less data than the table (8192 tokens x 768 of a 50257 x 768 table: up to 6 ranks)
                if (i is not None and cons.get(i, 0) >= 2 and i not in self._defer and self.params[i].numel * F32 >= SPARSE_MIN_BYTES
                        and dist_env.get_world_size() * node.numel <= self.params[i].numel):
                    self._defer.add(i)
                    cons[i] -= 1
        self._consumers = cons
        self._bucket_left = [sum(1 for i in idxs if i in cons) for idxs in self.buckets]
        self._in_graph = [any(i in cons for i in idxs) for idxs in self.buckets]
        self._all_in_graph = [all(i in cons for i in idxs) for idxs in self.buckets]

    def node_done(self, parents: tuple) -> None:
        if not self.active:
            return
        for par in parents:
            i = self.index.get(id(par))
            if i is None:
                continue
            left = self._consumers.get(i)
            if left is None or left <= 0:         # <= 0: the node whose rows were kept aside reports after the bucket went out
                continue
            left -= 1
            self._consumers[i] = left
            if left == 0:
                b = self.bucket_of[i]
                self._bucket_left[b] -= 1
                # a bucket goes out early only if ALL its parameters took part in this graph
                if self._bucket_left[b] == 0 and self._all_in_graph[b]:
                    self._launch(b)

    def end(self) -> None:
        pass

    def take_embedding_rows(self, w, idx, rows, n: int, d: int, v: int) -> bool:
        """Called by the embedding backward: True if the plan keeps the rows (the caller then leaves w.grad alone)."""
        if not self.active:
            return False
        i = self.index.get(id(w))
        if i is None or i not in self._defer:
            return False
        self.deferred.append((i, idx, rows, n, d, v))
        return True

    # ---- collectives ---------------------------------------------------------------------------
    def _launch(self, b: int) -> None:
        if b in self.launched:
            return
        ptr, numel = self.ranges[b]
        comm._require().allreduce_async(ptr, numel, average=True)
        self.launched.add(b)
        self.launch_order.append(b)

    def finish(self) -> None:
        """Enqueue every bucket not sent during backward, then order the compute stream behind all."""
        for b in range(len(self.buckets)):
            self._launch(b)
        backend = comm._require()
        gathered = []
        for (i, idx, rows, n, d, v) in self.deferred:
            world = backend.world_size
            all_idx, all_rows = self.mem.alloc(world * n), self.mem.alloc(world * n * d)
            backend.allgather_async(all_idx.ptr, idx.ptr, n)
            backend.allgather_async(all_rows.ptr, rows.ptr, n * d)
            gathered.append((i, all_idx, all_rows, world * n, d, v, 1.0 / world))
        backend.wait()
        for (i, all_idx, all_rows, n_all, d, v, alpha) in gathered:
            self.mem.scatter_rows(self.views[i].ptr, all_rows.ptr, all_idx.ptr, n_all, d, v, alpha)
        self.deferred = []
        self._defer = set()
        self.active = False
        self.armed = True
        self.launched = set()


_plans: dict[tuple, GradPlan] = {}
_mem_ops = None            # tests may install host memory ops
_no_sync_depth = 0


class no_sync:
    """Context manager: backward calls inside it send no gradient buckets (for micro-steps that are not
    followed by `sync_grads`).  Not in the reference, whose backward never communicates."""

    def __enter__(self):
        global _no_sync_depth
        _no_sync_depth += 1
        return self

    def __exit__(self, *exc):
        global _no_sync_depth
        _no_sync_depth -= 1
        return False


def _observer_install(plan: GradPlan | None) -> None:
    from .. import tensor as _tensor

    _tensor.set_backward_observer(plan)


def sync_grads(params: list, bucket_mb: float = DEFAULT_BUCKET_MB) -> None:
    """Average gradients over ranks. Every parameter gets a grad (zeros if missing); parameter
    order must be the same on all ranks."""
    world = dist_env.get_world_size()
    if world == 1:
        return
    comm._require()
    env_mb = os.environ.get("GRADTUITY_BUCKET_MB")
    if env_mb is not None:
        bucket_mb = float(env_mb)
    key = (tuple(id(p) for p in params), float(bucket_mb))
    plan = _plans.get(key)
    if plan is None or not plan.intact():
        plan = GradPlan(params, int(bucket_mb * 1024 * 1024), mem=_mem_ops)
        _plans.clear()                       # one live parameter list at a time; drops stale arenas
        _plans[key] = plan
        _observer_install(plan)
    plan.finish()


def reset() -> None:
    """Forget plans and stop observing backward (tests, process-group teardown)."""
    _plans.clear()
    try:
        _observer_install(None)
    except Exception:
        pass
