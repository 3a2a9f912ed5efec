"""CPU: host logic of the data-parallel path: environment parsing, the bucket rule, the gradient
arena, the backward-overlap bookkeeping, the unique-id rendezvous, the launcher, and a
world_size-2 run over gloo."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest

from gradtuity_b200.dist import comm, ddp
from gradtuity_b200.dist import env as dist_env
from tests._dist_host import FakeTensor, HostMemoryOps, RecordingBackend

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "dist_worker.py")


@pytest.fixture(autouse=True)
def _clean():
    yield
    ddp.reset()
    ddp._mem_ops = None
    comm.set_backend(None)


def test_env_parsing(monkeypatch):
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID", "MASTER_ADDR", "MASTER_PORT"):
        monkeypatch.delenv(k, raising=False)
    with pytest.raises(RuntimeError, match="RANK"):
        dist_env.get_rank()
    with pytest.raises(RuntimeError, match="WORLD_SIZE"):
        dist_env.get_world_size()
    monkeypatch.setenv("SLURM_PROCID", "3"); monkeypatch.setenv("SLURM_NTASKS", "8"); monkeypatch.setenv("SLURM_LOCALID", "1")
    assert (dist_env.get_rank(), dist_env.get_world_size(), dist_env.get_local_rank()) == (3, 8, 1)
    monkeypatch.setenv("RANK", "5"); monkeypatch.setenv("WORLD_SIZE", "6"); monkeypatch.setenv("LOCAL_RANK", "2")
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1"); monkeypatch.setenv("MASTER_PORT", "1234")
    assert dist_env.get_env_ranks() == (5, 6, 2, "127.0.0.1", "1234")


@pytest.fixture(autouse=True)
def _reference_bucket_rule(monkeypatch):
    """The tests below pin bucket layouts that follow the reference's rule; the front-of-list ramp has its own test."""
    monkeypatch.setattr(ddp, "BUCKET_RAMP", 0)
    monkeypatch.setenv("GRADTUITY_BUCKET_RAMP", "0")          # inherited by the spawned workers


def test_world_size_one_is_a_no_op(monkeypatch):
    monkeypatch.setenv("RANK", "0"); monkeypatch.setenv("WORLD_SIZE", "1"); monkeypatch.setenv("LOCAL_RANK", "0")
    p = FakeTensor(np.ones(4), requires_grad=True)
    ddp.sync_grads([p])                    # no backend installed: must not be needed
    assert p.grad is None
    comm.allreduce_inplace(0, 4)
    comm.broadcast(0, 4)
    comm.barrier()


def test_bucket_rule_matches_the_reference():
    # a bucket closes when the next entry would exceed the limit and the bucket is not empty
    assert ddp.bucketize([10, 10, 30, 5, 5], 20) == [[0, 1], [2], [3, 4]]
    assert ddp.bucketize([100], 20) == [[0]]
    assert ddp.bucketize([], 20) == []
    assert ddp.bucketize([20, 1], 20) == [[0], [1]]
    # GPT-2-small: the 154 MB embedding gradient ends up alone, about 21 buckets in all
    sizes = [50257 * 768, 1024 * 768]
    for _ in range(12):
        sizes += [768, 768] + [768 * 768] * 4 + [768] * 4 + [768, 768, 768 * 3072, 3072, 3072 * 768, 768]
    sizes += [768, 768]
    assert sum(sizes) == 124439808
    b = ddp.bucketize([4 * s for s in sizes], 25 * 1024 * 1024)
    assert b[0] == [0] and 15 <= len(b) <= 25


def test_bucket_ramp_makes_the_front_of_the_list_small():
    """ramp = 3: the first regular buckets hold at most 1/8, 1/4, 1/2 of the limit (they are what backward completes
    last, so their all-reduce hides behind nothing); an oversized single entry does not use up a step of the ramp;
    every index appears once, in order, whatever the ramp."""
    sizes = [50257 * 768, 1024 * 768]
    for _ in range(12):
        sizes += [768, 768] + [768 * 768] * 4 + [768] * 4 + [768, 768, 768 * 3072, 3072, 3072 * 768, 768]
    sizes += [768, 768]
    nbytes = [4 * s for s in sizes]
    limit = 100 << 20
    b = ddp.bucketize(nbytes, limit, 3)
    assert [i for idx in b for i in idx] == list(range(len(sizes)))
    held = [sum(nbytes[i] for i in idx) for idx in b]
    assert b[0] == [0] and held[0] > limit
    assert held[1] <= limit // 8 and held[2] <= limit // 4 and held[3] <= limit // 2
    assert all(h <= limit for h in held[1:]) and max(held[4:]) > limit // 2
    assert ddp.bucketize([10, 10, 30, 5, 5], 20, 0) == ddp.bucketize([10, 10, 30, 5, 5], 20)
    assert ddp.bucketize([4, 4, 4, 4, 4, 4, 4, 4], 16, 2) == [[0], [1, 2], [3, 4, 5, 6], [7]]


def test_arena_offsets_are_aligned():
    offs, total = ddp.arena_offsets([3, 64, 65, 1])
    assert offs == [0, 64, 128, 256] and total == 320


def _plan(monkeypatch, shapes, bucket_bytes):
    monkeypatch.setenv("RANK", "0"); monkeypatch.setenv("WORLD_SIZE", "2"); monkeypatch.setenv("LOCAL_RANK", "0")
    monkeypatch.setenv("GRADTUITY_BUCKET_MB", str(bucket_bytes / (1024 * 1024)))
    be = RecordingBackend()
    comm.set_backend(be)
    ddp._mem_ops = HostMemoryOps()
    params = [FakeTensor(np.zeros(s), requires_grad=True) for s in shapes]
    for i, p in enumerate(params):
        p.grad = FakeTensor(np.full(p.shape, float(i + 1)))
    return params, be


def test_first_sync_moves_grads_into_one_arena_and_reduces_every_bucket_once(monkeypatch):
    params, be = _plan(monkeypatch, [(4,), (100,), (8,), (8,)], 300)
    ddp.sync_grads(params)
    plan = next(iter(ddp._plans.values()))
    assert plan.buckets == [[0], [1], [2, 3]]
    assert [c[1] for c in be.calls] == [4, 100, 64 + 8]          # ranges include alignment padding
    assert all(c[2] is True for c in be.calls) and be.waits == 1
    for i, p in enumerate(params):                                 # values survived the move, touched exactly once
        assert p.grad is plan.views[i]
        np.testing.assert_allclose(p.grad.array, 10.0 * (i + 1))
    base = plan.arena.ptr
    assert [p.grad.ptr - base for p in params] == [0, 256, 768, 1024]


def test_backward_observer_sends_buckets_as_soon_as_their_last_consumer_ran(monkeypatch):
    from gradtuity_b200 import tensor as tmod

    params, be = _plan(monkeypatch, [(4,), (4,), (4,), (4,)], 40)       # two params per bucket
    ddp.sync_grads(params)
    plan = next(iter(ddp._plans.values()))
    assert tmod._backward_observer is plan and plan.buckets == [[0, 1], [2, 3]]
    be.calls.clear()
    # graph: n3 uses p3 and p2; n2 uses p2; n1 uses p1; p0 unused this step.  Reverse walk: n3, n2, n1.
    def node(*parents):
        n = FakeTensor(np.zeros(1)); n._parents = parents; return n
    n1, n2, n3 = node(params[1]), node(params[2]), node(params[3], params[2])
    topo = [params[1], n1, params[2], n2, params[3], n3]
    plan.begin(topo)
    plan.node_done(n3._parents)
    assert be.calls == []                       # p2 still has a consumer
    plan.node_done(n2._parents)
    assert len(be.calls) == 1 and be.calls[0][0] == plan.ranges[1][0]      # bucket 1 went out during backward
    plan.node_done(n1._parents)
    assert len(be.calls) == 1                   # bucket 0 holds p0, which was not in the graph: it waits
    plan.end()
    ddp.sync_grads(params)
    assert [c[0] for c in be.calls] == [plan.ranges[1][0], plan.ranges[0][0]]   # every bucket exactly once
    # a replaced grad tensor invalidates the plan: the next sync rebuilds it
    params[0].grad = FakeTensor(np.ones(4))
    ddp.sync_grads(params)
    assert next(iter(ddp._plans.values())) is not plan


def test_embedding_rows_of_a_tied_table_are_exchanged_instead_of_a_late_reduce(monkeypatch):
    """A large table with a dense consumer (the tied LM head) and an embedding consumer: in an early-sending backward the
    table's bucket goes out as soon as the dense consumer has run, the embedding backward hands its rows to the plan, and
    sync_grads gathers the rows of all ranks and adds them divided by the world size."""
    monkeypatch.setattr(ddp, "SPARSE_MIN_BYTES", 64)
    monkeypatch.setenv("GRADTUITY_SPARSE_EMBED_SYNC", "1")
    V, D, n = 6, 4, 5
    params, be = _plan(monkeypatch, [(V, D), (8,)], 40)
    table = params[0]
    ddp.sync_grads(params)
    plan = next(iter(ddp._plans.values()))
    be.calls.clear()
    for p in params:
        p.grad.array[...] = 0

    def node(*parents):
        t = FakeTensor(np.zeros(1)); t._parents = parents; return t
    emb, head, other = node(table), node(table), node(params[1])
    emb._embedding_of = table
    topo = [table, emb, params[1], other, head]
    plan.begin(topo)
    assert plan._defer == {0}
    table.grad.array[...] += 1.0                    # the dense consumer (runs first in the reverse walk)
    plan.node_done(head._parents)
    assert [c[0] for c in be.calls] == [plan.ranges[0][0]]          # the table's bucket is out although the embedding has not run
    plan.node_done(other._parents)
    idx = FakeTensor(np.array([0, 2, 2, 5, 1], np.float32))
    rows = FakeTensor(np.arange(n * D, dtype=np.float32).reshape(n, D))
    assert plan.take_embedding_rows(table, idx, rows, n, D, V) is True
    plan.node_done(emb._parents)                    # must not count the table a second time
    plan.end()
    ddp.sync_grads(params)
    gathers = [c for c in be.calls if c[0] == "gather"]
    assert [c[3] for c in gathers] == [n, n * D]
    want = np.full((V, D), 10.0, np.float32)        # the recording all-reduce multiplied the dense part by 10
    np.add.at(want, idx.array.astype(int), rows.array)             # world 2, both "ranks" hold the same rows: 2 * rows / 2
    np.testing.assert_allclose(table.grad.array, want)
    # a backward that does not send early keeps the rows local: the plan refuses them
    plan.armed = False
    plan.begin(topo)
    assert plan.take_embedding_rows(table, idx, rows, n, D, V) is False


def test_only_the_first_backward_after_a_sync_sends_buckets(monkeypatch):
    """backward(); backward(); sync_grads(): the second backward waits for the first one's collectives,
    sends nothing, and sync_grads reduces every bucket again; inside no_sync() nothing is sent at all."""
    params, be = _plan(monkeypatch, [(4,), (4,)], 16)                    # one parameter per bucket
    ddp.sync_grads(params)
    plan = next(iter(ddp._plans.values()))

    def node(*parents):
        n = FakeTensor(np.zeros(1)); n._parents = parents; return n

    def backward():
        n0, n1 = node(params[0]), node(params[1])
        plan.begin([params[0], n0, params[1], n1])
        plan.node_done(n1._parents)
        plan.node_done(n0._parents)
        plan.end()

    be.calls.clear(); waits = be.waits
    other = FakeTensor(np.zeros(3), requires_grad=True)      # a backward through another model's graph in between
    plan.begin([other, node(other)])
    plan.node_done((other,))
    plan.end()
    assert be.calls == [] and plan.armed                     # ... is not this plan's backward and leaves it armed
    backward()
    assert len(be.calls) == 2 and be.waits == waits          # first backward after a sync: both buckets early
    backward()
    assert len(be.calls) == 2 and be.waits == waits + 1      # second: nothing sent, compute ordered behind the comm stream
    ddp.sync_grads(params)
    assert len(be.calls) == 4                                # every bucket reduced again
    be.calls.clear()
    with ddp.no_sync():
        backward()
    assert be.calls == []
    backward()                                               # the arming was used up by the no_sync backward
    assert be.calls == []
    ddp.sync_grads(params)
    assert len(be.calls) == 2


def test_two_ranks_accumulate_two_backwards_then_sync_over_gloo():
    r = _launch("accumulate")
    assert r.returncode == 0, r.stderr[-3000:]


def test_two_ranks_exchange_embedding_rows_over_gloo():
    r = _launch("embedding")
    assert r.returncode == 0, r.stderr[-3000:]


def test_parameters_move_into_one_arena_and_travel_in_one_broadcast(monkeypatch):
    """init_sync: strict signature check, then ONE broadcast over a flat arena that holds every parameter;
    tensors that shared an allocation before (packed q/k/v weights) stay adjacent; a second call reuses the arena."""
    import importlib

    from tests._dist_host import HostArenaOps, host_param

    isync = importlib.import_module("gradtuity_b200.dist.init_sync")      # the package re-exports the function under this name

    monkeypatch.setenv("RANK", "0"); monkeypatch.setenv("WORLD_SIZE", "2"); monkeypatch.setenv("LOCAL_RANK", "0")
    rng = np.random.default_rng(0)
    block = host_param(rng.standard_normal(3 * 64))                      # one allocation holding q, k, v
    q, k, v = (host_param(block.array[i * 64:(i + 1) * 64], base=block._st) for i in range(3))
    a, o, b = host_param(rng.standard_normal((5, 3))), host_param(rng.standard_normal(70)), host_param(rng.standard_normal(2))
    params = [a, k, o, q, v, b]                                          # sorted-name order separates q, k, v
    before = [p.array.copy() for p in params]
    order, offsets, total = isync.arena_layout(params)
    assert [params[j] for j in order] == [a, q, k, v, o, b]
    assert offsets == [0, 64, 128, 192, 256, 384] and total == 448
    arena = isync.flatten_parameters(params, mem=HostArenaOps())
    for p, want in zip(params, before):
        np.testing.assert_array_equal(p.array, want)                     # values and shapes survive the move
        assert p._st.base is arena._st
    assert k.ptr - q.ptr == 64 * 4 and v.ptr - k.ptr == 64 * 4          # still side by side
    again = isync.flatten_parameters(params, mem=HostArenaOps())
    assert again.ptr == arena.ptr and again.numel == total                # recognised, not copied again

    class Bcast(RecordingBackend):
        def broadcast(self, ptr, numel, src):
            self.calls.append(("bcast", ptr, numel, src))

    be = Bcast()
    comm.set_backend(be)
    monkeypatch.setattr(isync, "_arena_ops", HostArenaOps())
    isync.init_sync(params, strict=False)
    assert be.calls == [("bcast", arena.ptr, total, 0)]                   # one collective for all six tensors


def test_rendezvous_times_out_with_a_diagnostic(tmp_path):
    with pytest.raises(RuntimeError, match="did not reach 128 bytes"):
        comm.exchange_unique_id(1, None, str(tmp_path / "never.bin"), timeout=0.2)
    with pytest.raises(RuntimeError, match="unique id has"):
        comm.exchange_unique_id(0, lambda: b"short", str(tmp_path / "x.bin"))


def test_collectives_without_a_group_raise(monkeypatch):
    monkeypatch.setenv("RANK", "0"); monkeypatch.setenv("WORLD_SIZE", "2"); monkeypatch.setenv("LOCAL_RANK", "0")
    with pytest.raises(RuntimeError, match="not initialized"):
        comm.allreduce_inplace(0, 1)
    with pytest.raises(RuntimeError, match="not initialized"):
        ddp.sync_grads([FakeTensor(np.zeros(2), requires_grad=True)])


def _launch(mode, nproc=2, timeout=120):
    cmd = [sys.executable, "-m", "gradtuity_b200.launch", "--nproc", str(nproc), "--master-addr", "127.0.0.1", WORKER, mode]
    return subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=timeout)


def test_two_ranks_rendezvous_through_the_uid_file():
    r = _launch("rendezvous")
    assert r.returncode == 0, r.stderr[-2000:]


def test_two_ranks_sync_grads_over_gloo():
    r = _launch("allreduce")
    assert r.returncode == 0, r.stderr[-3000:]


def test_two_ranks_sync_grads_over_gloo_with_the_bucket_ramp(monkeypatch):
    """Smaller buckets at the front of the parameter list move boundaries, not values: the same means come back."""
    monkeypatch.setenv("GRADTUITY_BUCKET_RAMP", "3")
    r = _launch("allreduce")
    assert r.returncode == 0, r.stderr[-3000:]
    r = _launch("accumulate")
    assert r.returncode == 0, r.stderr[-3000:]


def test_launcher_stops_siblings_and_propagates_the_exit_code():
    t0 = time.monotonic()
    r = _launch("fail")
    assert r.returncode == 3
    assert time.monotonic() - t0 < 20          # rank 0 sleeps 30 s unless the launcher terminates it
